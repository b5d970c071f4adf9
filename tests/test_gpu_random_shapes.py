"""Seeded random shapes: the indexers' fast paths against their exact kernels, the attention kernel against the oracle.

The hand-picked shapes of test_gpu_indexers.py cover the cases each kernel was designed around; a
defect that depends on a remainder (a slice whose length modulo 256 is below 32 once left part of
a warp out of a vote) shows only on shapes nobody thought of. Every shape here is drawn from a
seeded generator, so a failure names a reproducible case. Ids must be bit-identical to the exact
kernels' (which the other tests pin to the oracle), no bounded wait may run out, no bound may be
violated."""
import os
import random

import pytest
import torch

pytestmark = pytest.mark.gpu
SCALE = int(os.environ.get("SPARSE_B200_RANDOM_SHAPES", "1"))      # multiplies the number of shapes (a longer hunt)


def sp():
    import sparse_attention_b200_b200 as m
    return m


def _summary_shapes(n, seed):
    rng = random.Random(seed)
    out = []
    while len(out) < n:
        r = rng.choice([1, 2, 4])
        g = rng.choice([1, 2, 4, 8, 16])
        if g * r > 64:
            continue
        hkv = rng.choice([1, 2, 4])
        b = rng.choice([1, 2])
        nt = rng.choice([rng.randint(16, 200), rng.randint(200, 1200), rng.randint(1200, 3000)])
        topk = rng.choice([4, 8, 16, 32, 64])
        if topk > nt:
            continue
        budget = 120_000_000 // (b * hkv * g * 128 * 128)      # query blocks that keep q under ~240 MB
        qt = min(rng.choice([rng.randint(1, 12), rng.randint(12, 80), rng.randint(80, 220)]), max(1, budget))
        out.append((b, hkv * g, hkv, qt * 128, nt * 128, r, topk))
    return out


@pytest.mark.parametrize("shape", _summary_shapes(28 * SCALE, 20250))
def test_summary_selector_random_shapes(shape):
    b, hq, hkv, sq, skv, r, topk = shape
    m = sp()
    gen = torch.Generator(device="cuda").manual_seed(hash(shape) % (2 ** 31))
    q = torch.randn((b, hq, sq, 128), device="cuda", generator=gen).to(torch.bfloat16)
    k = torch.randn((b, hkv, skv, 128), device="cuda", generator=gen)
    k += 0.5 * torch.randn((b, hkv, skv // 128, 1, 1), device="cuda", generator=gen).expand(-1, -1, -1, 128, 128) \
        .reshape(b, hkv, skv, 128)
    k = k.to(torch.bfloat16)
    fast = m.SummarySelector(q, k, r, topk=topk, keep_scores=False)
    ids = fast.run_fast().clone()
    exact = m.SummarySelector(q, k, r, topk=topk, keep_scores=False)
    exact.prepare()
    exact.score()
    torch.cuda.synchronize()
    m.device_status()
    assert torch.equal(ids, exact.ids)
    assert fast.bound_stats()[0] == 0


def _fp4_shapes(n, seed):
    rng = random.Random(seed)
    out = []
    while len(out) < n:
        hidx = rng.choice([1, 2, 4])
        hk = rng.choice([1, hidx])                   # one shared key head, or one per index head
        lq = 128 * rng.choice([1, 2, 3, 5, 8, 13, 32])
        pages = rng.choice([rng.randint(8, 64), rng.randint(64, 300), rng.randint(300, 700)])
        topk = rng.choice([4, 8, 16, 24, 64])
        if topk > pages:
            continue
        b = rng.choice([1, 2])
        out.append((b, hidx, hk, lq, pages * 128, topk))
    return out


@pytest.mark.parametrize("shape", _fp4_shapes(20 * SCALE, 777))
def test_fp4_indexer_random_shapes(shape):
    b, hidx, hk, lq, lkv, topk = shape
    m = sp()
    g = torch.Generator().manual_seed(hash(shape) % (2 ** 31))
    pages = lkv // 128
    qp = torch.randint(256, (b * lq, hidx, 64), dtype=torch.uint8, generator=g)
    kp = torch.randint(256, (b * pages, hk, 128, 64), dtype=torch.uint8, generator=g)
    choices = torch.tensor([0.25, 0.375, 0.5, 0.75, 1.0, 1.5, 2.0])
    qs = choices[torch.randint(7, (b * lq, hidx, 8), generator=g)].to(torch.float8_e4m3fn)
    ks = choices[torch.randint(7, (b * pages, hk, 128, 8), generator=g)].to(torch.float8_e4m3fn)
    inputs = m.prepare_fp4_inputs(qp.cuda(), kp.cuda(), qs.cuda(), ks.cuda(), batch_size=b, len_q=lq, len_kv=lkv)
    ids, ws = m.fp4_indexer_fast(inputs, topk=topk)
    ref = m.fp4_indexer(inputs, topk=topk)
    torch.cuda.synchronize()
    m.device_status()
    assert torch.equal(ids, ref)
    assert int(ws[12:16].view(torch.int32).item()) == 0          # violations of the tensor-core error bound


def _attention_shapes(n, seed):
    rng = random.Random(seed)
    out = []
    while len(out) < n:
        b = rng.choice([1, 2])
        hkv = rng.choice([1, 2, 3])
        g = rng.choice([1, 2, 3, 4, 8, 16])
        qb = rng.randint(1, 9)
        nb = rng.randint(1, 40)
        topk = rng.randint(1, min(nb, 12))
        if b * hkv * g * qb * topk > 1400:          # keeps the CPU oracle to a second or two per case
            continue
        out.append((b, hkv * g, hkv, qb * 128, nb * 128, topk, rng.choice(["full", "ragged"]), rng.randrange(1 << 30)))
    return out


@pytest.mark.parametrize("shape", _attention_shapes(16 * SCALE, 4242))
def test_q_centric_random_shapes(shape):
    """Random batch / head / group / block counts (odd group sizes, one query block, top-k = all blocks, ragged
    counts with empty lists) against the CPU oracle, tolerances of test_gpu_q_centric.py."""
    import oracle
    from oracle import inputs as gen
    b, hq, hkv, sq, skv, topk, counts_kind, seed = shape
    m = sp()
    q, k, v = gen.make_qkv(b, hq, hkv, sq, skv, seed=seed % 1000, k_block_offset=0.5)
    g = torch.Generator().manual_seed(seed)
    qb, nb = sq // 128, skv // 128
    ids = torch.stack([torch.randperm(nb, generator=g)[:topk] for _ in range(b * hkv * qb)]).to(torch.int32) \
        .reshape(b, hkv, qb, topk)
    counts = None
    if counts_kind == "ragged":
        counts = torch.randint(0, topk + 1, (b, hkv, qb), generator=g, dtype=torch.int32)
    ref_o, ref_l = oracle.gather_attention(q, k, v, ids, counts)
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full(q.shape[:3], float("nan"), device="cuda")
    m.attention_out(q.cuda(), k.cuda(), v.cuda(), ids.cuda(), out, None if counts is None else counts.cuda(), lse)
    torch.cuda.synchronize()
    m.device_status()
    o = out.float().cpu()
    assert torch.isfinite(o).all()
    d = (o - ref_o).abs()
    assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3
    fin = torch.isfinite(ref_l)
    l = lse.cpu()
    assert torch.equal(torch.isinf(l) & (l < 0), ~fin)
    assert torch.all((l[fin] - ref_l[fin]).abs() <= 1e-3 * ref_l[fin].abs().clamp_min(1.0))
    # the scatter launch (rows cut into 2-4 slices with destinations of their own) must write the same bits
    import ctypes
    from sparse_attention_b200_b200 import _lib
    tiles = b * hq * qb
    qc, kc, vc, idc = q.cuda(), k.cuda(), v.cuda(), ids.cuda()
    cc = None if counts is None else counts.cuda()
    plain, plain_l = torch.empty_like(out), torch.empty_like(lse)
    m.attention_out(qc, kc, vc, idc, plain, cc, plain_l, balance=False)      # (scatter launches never balance a last round)
    for owners in (2, 3, 4):
        if tiles % owners:
            continue
        per = tiles // owners * 128
        outs = [torch.full((per, 128), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(owners)]
        lses = [torch.full((per,), float("nan"), device="cuda") for _ in range(owners)]
        arr = ctypes.c_void_p * owners
        _lib.check(_lib.lib().sparse_b200_q_centric_scatter(
            _lib.ptr(qc), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(idc), _lib.ptr(cc), arr(*[t.data_ptr() for t in outs]),
            arr(*[t.data_ptr() for t in lses]), owners, b, hq, hkv, sq, skv, topk, _lib.current_stream()))
        torch.cuda.synchronize()
        m.device_status()
        assert torch.equal(torch.cat(outs).view(torch.int16), plain.reshape(-1, 128).view(torch.int16)), owners
        assert torch.equal(torch.cat(lses).view(torch.int32), plain_l.reshape(-1).view(torch.int32)), owners


def _token_shapes(n, seed):
    rng = random.Random(seed)
    layouts = random.Random(seed + 1)        # its own stream: the geometries stay those of the seed
    out = []
    while len(out) < n:
        b = rng.choice([1, 2])
        hkv = rng.choice([1, 2])
        g = rng.choice([1, 2, 4, 8, 16])
        sq = rng.choice([rng.randint(1, 40), rng.randint(40, 300)])
        nb = rng.choice([16, 17, 32, 40])
        topk = rng.choice([1, 4, 16, nb])
        if b * hkv * g * sq * topk > 160_000:
            continue
        out.append((b, hkv, g, sq, nb * 128, topk, rng.choice(["independent", "hot", "tile_shared", "identical"]),
                    rng.randrange(1 << 30), layouts.randrange(8)))
    return out


@pytest.mark.parametrize("shape", _token_shapes(14 * SCALE, 99))
def test_token_operator_random_shapes(shape):
    """The per-token KV-centric operator (reverse index, main, Combine) on random geometries: every group size the
    reference serves, token counts with tails, top-k from 1 to all blocks; the reverse index is audited by the CPU
    validator and the output compared with the masked-attention oracle (the reference's tolerances). The last
    field draws the layout: bit 0 q token-major, bit 1 partials token-major too (both only for 8 or 16 heads per
    group), bit 2 fp32 partials."""
    import oracle
    from tests.test_gpu_kv_token import make_selected, token_reference
    b, hkv, g, sq, skv, topk, kind, seed, layout = shape
    m = sp()
    q_tm = bool(layout & 1) and g in (8, 16)
    p_tm, f32 = q_tm and bool(layout & 2), bool(layout & 4)
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn((b, hkv * g, sq, 128), generator=gen).to(torch.bfloat16)
    k = torch.randn((b, hkv, skv, 128), generator=gen).to(torch.bfloat16)
    v = torch.randn((b, hkv, skv, 128), generator=gen).to(torch.bfloat16)
    selected = make_selected(b, hkv, sq, skv // 128, topk, kind, seed % 1000)
    ref_o, ref_l = token_reference(q, k, v, selected)
    p = m.PreparedTokens((q.permute(0, 2, 1, 3).contiguous() if q_tm else q).cuda(), k.cuda(), v.cuda(),
                         selected.cuda(), q_token_major=q_tm, partial_token_major=p_tm, partial_f32=f32)
    assert p.partial.dtype == (torch.float32 if f32 else torch.bfloat16)
    p.poison()
    out, lse = p.run()
    torch.cuda.synchronize()
    m.device_status()
    assert oracle.validate_reverse_plan(p.plan(), selected, skv // 128, g, ordered=False)
    assert torch.isfinite(p.partial.float()).all() and torch.isfinite(p.lses).all()
    torch.testing.assert_close(out.float().cpu(), ref_o, atol=0.02, rtol=0.02)
    torch.testing.assert_close(lse.cpu(), ref_l, atol=0.002, rtol=0.0002)
