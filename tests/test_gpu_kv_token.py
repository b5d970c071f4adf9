"""KV-centric operator for per-TOKEN selection lists (the reference's contract) through the
C ABI: GPU reverse index audited against the CPU builder, partials and merged output
against the masked-attention oracle. Cases after attention/kv_centric/validate_gpu.py:131-172
(G = 1..16, tails Sq = 9 / 129 / 257, patterns, zero_q, constant_v, large_qk) with the
reference's tolerances (O atol = rtol = 0.02, LSE atol 0.002 / rtol 0.0002)."""
import math

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def sp():
    import sparse_attention_b200_b200 as m
    return m


def make_selected(batch, hkv, sq, kv_blocks, topk, kind, seed):
    """Synthetic per-token selectors in the style of metadata.py:120-149."""
    gen = torch.Generator().manual_seed(seed)
    out = torch.empty((batch, hkv, sq, topk), dtype=torch.int32)
    for b in range(batch):
        for h in range(hkv):
            shared = torch.randperm(kv_blocks, generator=gen)[:topk]
            for qi in range(sq):
                if kind == "tile_shared":
                    if qi % 128 == 0:
                        shared = torch.randperm(kv_blocks, generator=gen)[:topk]
                    ids = shared
                elif kind == "identical":
                    ids = shared
                elif kind == "independent":
                    ids = torch.randperm(kv_blocks, generator=gen)[:topk]
                elif kind == "hot":
                    tail = torch.randperm(kv_blocks - 1, generator=gen)[:topk - 1] + 1
                    ids = torch.cat((torch.zeros(1, dtype=torch.int64), tail))
                    ids = torch.roll(ids, qi % topk)
                else:
                    raise ValueError(kind)
                out[b, h, qi] = ids.to(torch.int32)
    return out


def token_reference(q, k, v, selected):
    """Masked-attention oracle, per token (attention/kv_centric/reference.py:7-31 with free TopK)."""
    b, hq, sq, d = q.shape
    hkv, skv = k.shape[1:3]
    g = hq // hkv
    nb = skv // 128
    out = torch.empty(q.shape, dtype=torch.float32)
    lse = torch.empty(q.shape[:3], dtype=torch.float32)
    for bi in range(b):
        for h in range(hkv):
            mask = torch.zeros((sq, nb), dtype=torch.bool)
            mask.scatter_(1, selected[bi, h].long(), True)
            mask = mask.repeat_interleave(128, dim=1)
            s = q[bi, h * g:(h + 1) * g].float() @ k[bi, h].float().T / math.sqrt(d)
            s = s.masked_fill(~mask[None], -math.inf)
            out[bi, h * g:(h + 1) * g] = torch.softmax(s, -1) @ v[bi, h].float()
            lse[bi, h * g:(h + 1) * g] = torch.logsumexp(s, -1)
    return out, lse


SPECS = [
    # name, B, Hkv, G, Sq, Skv, TopK, pattern, transform
    ("g16_initial", 1, 1, 16, 256, 4096, 16, "independent", None),
    ("g1_batch_heads_tail", 2, 2, 1, 129, 4096, 16, "independent", None),
    ("g2_tail", 1, 2, 2, 17, 4096, 16, "independent", None),
    ("g4_batch_hot", 2, 2, 4, 9, 4096, 16, "hot", None),
    ("g8_tile_shared", 1, 2, 8, 257, 4096, 16, "tile_shared", None),
    ("g16_hot_chunks_empty_blocks", 1, 1, 16, 257, 4096, 16, "identical", None),
    ("g16_single_query", 1, 1, 16, 1, 4096, 16, "hot", None),
    ("g8_top4", 1, 2, 8, 64, 2048, 4, "independent", None),
    ("g4_top32", 1, 1, 4, 40, 8192, 32, "independent", None),
    ("g16_zero_q", 1, 1, 16, 9, 4096, 16, "independent", "zero_q"),
    ("g16_constant_v", 2, 2, 16, 9, 4096, 16, "independent", "constant_v"),
    ("g16_large_qk", 1, 1, 16, 17, 4096, 16, "independent", "large_qk"),
]


@pytest.mark.parametrize("spec", SPECS, ids=[s[0] for s in SPECS])
def test_token_operator(spec):
    name, b, hkv, g, sq, skv, topk, kind, transform = spec
    m = sp()
    gen = torch.Generator().manual_seed(31 + len(name))
    q = torch.randn((b, hkv * g, sq, 128), generator=gen).to(torch.bfloat16)
    k = torch.randn((b, hkv, skv, 128), generator=gen).to(torch.bfloat16)
    v = torch.randn((b, hkv, skv, 128), generator=gen).to(torch.bfloat16)
    selected = make_selected(b, hkv, sq, skv // 128, topk, kind, 7 + len(name))
    if transform == "zero_q":
        q.zero_()
    elif transform == "large_qk":
        q.mul_(2)
        k.mul_(2)
    elif transform == "constant_v":
        for bi in range(b):
            for hi in range(hkv):
                v[bi, hi].fill_(1 + bi * hkv + hi)
    ref_o, ref_l = token_reference(q, k, v, selected)
    p = m.PreparedTokens(q.cuda(), k.cuda(), v.cuda(), selected.cuda())
    p.poison()
    out, lse = p.run()
    torch.cuda.synchronize()
    m.device_status()
    # reverse index: exact edge coverage, audited by the CPU validator (edge order inside a row is free)
    plan = p.plan()
    assert oracle.validate_reverse_plan(plan, selected, skv // 128, g, ordered=False)
    cpu_plan = oracle.build_reverse_plan(selected, skv // 128, g)
    assert torch.equal(plan["row_ptr"], cpu_plan["row_ptr"])
    assert plan["tasks"].shape == cpu_plan["tasks"].shape
    assert torch.equal(plan["tasks"][:, [0, 1, 3]], cpu_plan["tasks"][:, [0, 1, 3]])
    # every partial slot written
    assert torch.isfinite(p.partial.float()).all() and torch.isfinite(p.lses).all()
    o = out.float().cpu()
    torch.testing.assert_close(o, ref_o, atol=0.02, rtol=0.02)
    torch.testing.assert_close(lse.cpu(), ref_l, atol=0.002, rtol=0.0002)
    d = (o - ref_o).abs()
    assert d.max() <= 2e-2 and d.mean() <= 2e-3
    # sampled partials against the per-block softmax
    for (bi, head, qi, rank) in ((0, 0, 0, 0), (b - 1, hkv * g - 1, sq - 1, topk - 1)):
        blk = int(selected[bi, head // g, qi, rank])
        kb, vb = k[bi, head // g, blk * 128:(blk + 1) * 128].float(), v[bi, head // g, blk * 128:(blk + 1) * 128].float()
        s = q[bi, head, qi].float() @ kb.T / math.sqrt(128)
        torch.testing.assert_close(p.partial[bi, head, qi, rank].float().cpu(), torch.softmax(s, -1) @ vb,
                                   atol=0.02, rtol=0.02)
        torch.testing.assert_close(p.lses[bi, head, qi, rank].cpu(), torch.logsumexp(s, -1), atol=0.002, rtol=0.0002)
    if transform == "constant_v":
        for bi in range(b):
            for hi in range(hkv):
                assert torch.allclose(o[bi, hi * g:(hi + 1) * g], torch.full((g, sq, 128), float(1 + bi * hkv + hi)),
                                      atol=2e-2)
    if transform == "zero_q":
        assert torch.allclose(lse.cpu(), torch.full(lse.shape, math.log(topk * 128.0)), atol=1e-3)


def test_token_operator_repeat_reorder_and_block_equivalence():
    m = sp()
    gen = torch.Generator().manual_seed(5)
    q = torch.randn((1, 16, 256, 128), generator=gen).to(torch.bfloat16)
    k = torch.randn((1, 1, 4096, 128), generator=gen).to(torch.bfloat16)
    v = torch.randn((1, 1, 4096, 128), generator=gen).to(torch.bfloat16)
    selected = make_selected(1, 1, 256, 32, 16, "tile_shared", 3)
    p = m.PreparedTokens(q.cuda(), k.cuda(), v.cuda(), selected.cuda())
    out, lse = p.run()
    a = out.clone()
    out2, _ = p.run()
    assert torch.equal(a, out2)                       # repeated identical inputs: bitwise equal
    p2 = m.PreparedTokens(q.cuda(), k.cuda(), v.cuda(), selected.flip(-1).contiguous().cuda())
    out3, lse3 = p2.run()
    torch.testing.assert_close(out3.float(), a.float(), atol=0.02, rtol=0.02)
    # tile-shared per-token lists == per-block lists through the block operator
    ids_blocks = selected[:, :, ::128].contiguous()
    ob, lb = m.kv_centric_attention(q.cuda(), k.cuda(), v.cuda(), ids_blocks.cuda(), nseg=4)
    torch.testing.assert_close(ob.float(), a.float(), atol=0.02, rtol=0.02)
    torch.testing.assert_close(lb, lse, atol=0.002, rtol=0.0002)
    bad = selected.clone()
    bad[0, 0, 3, 2] = 77
    p3 = m.PreparedTokens(q.cuda(), k.cuda(), v.cuda(), bad.cuda())
    p3.metadata()
    with pytest.raises(ValueError):
        p3.plan()
    m.device_status()


@pytest.mark.parametrize("g", [8, 16])
def test_token_major_q_gives_identical_results(g):
    """q handed over as [B,Sq,Hq,128] (the layout of the reference's TMA variants) must give
    bit-identical partials, LSEs and outputs to the head-major call."""
    import sparse_attention_b200_b200 as m
    gen = torch.Generator().manual_seed(91)
    b, hkv, sq, skv, topk = 2, 2, 300, 4096, 16
    q = torch.randn((b, hkv * g, sq, 128), generator=gen).to(torch.bfloat16).cuda()
    k = torch.randn((b, hkv, skv, 128), generator=gen).to(torch.bfloat16).cuda()
    v = torch.randn((b, hkv, skv, 128), generator=gen).to(torch.bfloat16).cuda()
    selected = make_selected(b, hkv, sq, skv // 128, topk, "independent", 5).cuda()
    head_major = m.PreparedTokens(q, k, v, selected)
    head_major.run()
    token_major = m.PreparedTokens(q.permute(0, 2, 1, 3).contiguous(), k, v, selected, q_token_major=True)
    token_major.poison()
    token_major.run()
    torch.cuda.synchronize()
    m.device_status()
    assert torch.equal(token_major.partial.view(torch.int16), head_major.partial.view(torch.int16))
    assert torch.equal(token_major.lses, head_major.lses)
    assert torch.equal(token_major.out.view(torch.int16), head_major.out.view(torch.int16))
    # partials token-major as well ([B,Sq,TopK,Hq,128], what the reference's main_tm_out writes and its
    # combine_tm_out reads): same partial rows in another place, the same merged output
    both = m.PreparedTokens(q.permute(0, 2, 1, 3).contiguous(), k, v, selected, q_token_major=True, partial_token_major=True)
    both.poison()
    both.run()
    torch.cuda.synchronize()
    m.device_status()
    assert torch.equal(both.partial.permute(0, 3, 1, 2, 4).contiguous().view(torch.int16), head_major.partial.view(torch.int16))
    assert torch.equal(both.lses, head_major.lses)
    assert torch.equal(both.out.view(torch.int16), head_major.out.view(torch.int16))
    assert torch.equal(both.out_lse, head_major.out_lse)
    with pytest.raises(m.SparseB200Error):
        m.PreparedTokens(torch.zeros((1, 8, 4, 128), dtype=torch.bfloat16, device="cuda"), k[:1, :1], v[:1, :1],
                         selected[:1, :1, :8].contiguous(), q_token_major=True)      # Hq/Hkv = 4


@pytest.mark.parametrize("g,topk,sq", [(1, 16, 130), (2, 5, 77), (4, 16, 257), (8, 16, 300), (16, 7, 129)])
def test_fp32_partials_round_to_the_bf16_ones(g, topk, sq):
    """The fp32-partial form of the main stage (the reference's control variants, api11.py:22-25): the same
    arithmetic with the last rounding left out, so its partials rounded to bf16 are the bf16 partials bit for bit,
    the LSEs are identical, and the merged output matches the masked-attention reference (every group size: the
    generic kernel below 8 heads per group, the pipelined one for 8 and 16; token-major for those as well)."""
    import sparse_attention_b200_b200 as m
    gen = torch.Generator().manual_seed(17 + g)
    b, hkv, skv = 2, 2, 2048
    q = torch.randn((b, hkv * g, sq, 128), generator=gen).to(torch.bfloat16)
    k = torch.randn((b, hkv, skv, 128), generator=gen).to(torch.bfloat16)
    v = torch.randn((b, hkv, skv, 128), generator=gen).to(torch.bfloat16)
    selected = make_selected(b, hkv, sq, skv // 128, topk, "independent", 3)
    ref_o, ref_l = token_reference(q, k, v, selected)
    q, k, v, selected = q.cuda(), k.cuda(), v.cuda(), selected.cuda()
    half = m.PreparedTokens(q, k, v, selected)
    half.run()
    full = m.PreparedTokens(q, k, v, selected, partial_f32=True)
    full.poison()
    full.run()
    torch.cuda.synchronize()
    m.device_status()
    assert full.partial.dtype == torch.float32 and torch.isfinite(full.partial).all()
    assert torch.equal(full.partial.to(torch.bfloat16).view(torch.int16), half.partial.view(torch.int16))
    assert torch.equal(full.lses, half.lses) and torch.equal(full.out_lse, half.out_lse)
    torch.testing.assert_close(full.out.float().cpu(), ref_o, atol=0.02, rtol=0.02)
    torch.testing.assert_close(full.out_lse.cpu(), ref_l, atol=0.002, rtol=0.0002)
    if g in (8, 16):
        tm = m.PreparedTokens(q.permute(0, 2, 1, 3).contiguous(), k, v, selected, q_token_major=True,
                              partial_token_major=True, partial_f32=True)
        tm.poison()
        tm.run()
        torch.cuda.synchronize()
        m.device_status()
        assert torch.equal(tm.partial.permute(0, 3, 1, 2, 4), full.partial)
        assert torch.equal(tm.out.view(torch.int16), full.out.view(torch.int16)) and torch.equal(tm.out_lse, full.out_lse)
