"""KV-centric operator (segment metadata + partial main + combine) through the
C ABI against the CPU oracle. Cases and tolerances after
attention/kv_centric/validate_gpu.py:12-13, 30-40, 43-172."""
import os

import numpy as np
import pytest
import torch

import oracle
from oracle import inputs as gen
from tests.golden import cases

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(__file__), "golden")


def sp():
    import sparse_attention_b200_b200 as m
    return m


def close(out, lse, ref_o, ref_l):
    o = out.float().cpu()
    assert torch.isfinite(o).all()
    d = (o - ref_o).abs()
    assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3, (d.max().item(), d.mean().item())
    torch.testing.assert_close(o, ref_o, atol=0.02, rtol=0.02)
    fin = torch.isfinite(ref_l)
    l = lse.cpu()
    torch.testing.assert_close(l[fin], ref_l[fin], atol=0.002, rtol=0.0002)


def test_combine_golden_and_extreme_lse():
    m = sp()
    fx = np.load(os.path.join(G, "combine.npz"))
    partial, lses = cases.combine_case()
    out, lse = m.combine(partial.cuda(), lses.cuda())
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float().cpu(), torch.from_numpy(fx["o"]), atol=0.02, rtol=0.02)
    torch.testing.assert_close(lse.cpu(), torch.from_numpy(fx["lse"]), atol=0.002, rtol=0.0002)
    # bf16 partials, -inf ranks and an all -inf row
    pb = partial.to(torch.bfloat16)
    l2 = lses.clone()
    l2[0, 0, 1, :] = -float("inf")
    l2[0, 1, 2, 3:] = -float("inf")
    pb2 = pb.clone()
    pb2[0, 1, 2, 3:] = float("nan")          # ignored ranks may hold anything
    out, lse = m.combine(pb2.cuda(), l2.cuda())
    ref_o, ref_l = oracle.combine_partials(torch.nan_to_num(pb2.float()), l2)
    assert torch.all(out[0, 0, 1] == 0) and lse[0, 0, 1].item() == -float("inf")
    fin = torch.isfinite(ref_l)
    torch.testing.assert_close(out.float().cpu()[fin], ref_o[fin], atol=0.02, rtol=0.02)
    torch.testing.assert_close(lse.cpu()[fin], ref_l[fin], atol=0.002, rtol=0.0002)


SPECS = [
    # name, B, Hkv, G, Sq, Skv, topk, pattern, nseg, partial, transform
    ("g16_initial", 1, 1, 16, 256, 4096, 16, "independent", 4, "f32", None),
    ("g1_batch_heads", 2, 2, 1, 384, 4096, 16, "unsorted", 4, "bf16", None),
    ("g2_reverse", 1, 2, 2, 256, 4096, 16, "reverse", 3, "f32", None),
    ("g4_batch", 2, 2, 4, 128, 4096, 16, "unsorted", 8, "bf16", None),
    ("g8_paired", 1, 2, 8, 512, 4096, 16, "paired", 2, "bf16", None),
    ("g16_top64", 1, 1, 16, 256, 16384, 64, "unsorted", 4, "bf16", None),
    ("g16_dense_equivalence", 1, 1, 16, 256, 2048, 16, "unsorted", 4, "f32", None),
    ("g16_one_segment", 1, 1, 16, 128, 2048, 4, "unsorted", 1, "f32", None),
    ("g16_zero_q", 1, 1, 16, 128, 4096, 16, "independent", 4, "f32", "zero_q"),
    ("g16_constant_v", 2, 2, 16, 128, 4096, 16, "independent", 4, "bf16", "constant_v"),
    ("g16_large_qk", 1, 1, 16, 256, 4096, 16, "independent", 4, "f32", "large_qk"),
    ("g16_dominant_block", 1, 1, 16, 256, 4096, 16, "independent", 4, "f32", "dominant_block"),
]


@pytest.mark.parametrize("spec", SPECS, ids=[s[0] for s in SPECS])
def test_operator_cases(spec):
    name, b, hkv, g, sq, skv, topk, pattern, nseg, partial, transform = spec
    m = sp()
    q, k, v = gen.make_qkv(b, hkv * g, hkv, sq, skv, seed=31 + len(name))
    ids = gen.make_ids(b, hkv, sq // 128, skv // 128, topk, 131 + len(name), pattern)
    if transform == "zero_q":
        q.zero_()
    elif transform == "large_qk":
        q.mul_(2)
        k.mul_(2)
    elif transform == "constant_v":
        for bi in range(b):
            for hi in range(hkv):
                v[bi, hi].fill_(1 + bi * hkv + hi)
    elif transform == "dominant_block":
        q.fill_(1)
        k.zero_()
        blk = int(ids[0, 0, 0, 3])
        ids[..., 3] = blk
        for t in range(sq // 128):         # keep ids distinct: move a clash elsewhere
            for bi in range(b):
                for hi in range(hkv):
                    row = ids[bi, hi, t]
                    free = [x for x in range(skv // 128) if x not in row.tolist()]
                    for j in range(topk):
                        if j != 3 and int(row[j]) == blk:
                            row[j] = free.pop()
        k[:, :, blk * 128:(blk + 1) * 128].fill_(4)
        for block in range(skv // 128):
            v[:, :, block * 128:(block + 1) * 128].fill_(block)
    ref_o, ref_l = oracle.gather_attention(q, k, v, ids)
    p = m.Prepared(q.cuda(), k.cuda(), v.cuda(), ids.cuda(), nseg=nseg, partial=partial)
    p.poison()
    out, lse = p.run()
    torch.cuda.synchronize()
    m.device_status()
    assert p.audit()["edges"] == ids.numel()
    # every partial slot was written (poisoned NaN overwritten)
    assert torch.isfinite(p.partial.float()).all() and not torch.isnan(p.lses).any()
    close(out, lse, ref_o, ref_l)
    # the metadata equals the oracle's segmentation, bit for bit
    seg_ids, seg_counts = oracle.split_kv_segments(ids, skv // 128, nseg)
    assert torch.equal(p.seg_counts.cpu(), seg_counts)
    live = torch.arange(topk)[None, None, None, None, :] < seg_counts[..., None]
    assert torch.equal(p.seg_ids.cpu()[live], seg_ids[live])
    # the device combine agrees with the oracle's merge of the device partials
    po = p.partial.float().cpu().permute(1, 2, 3, 0, 4)
    pl = p.lses.cpu().permute(1, 2, 3, 0)
    co, cl = oracle.combine_partials(po, pl)
    torch.testing.assert_close(out.float().cpu(), co, atol=0.01, rtol=0.01)
    torch.testing.assert_close(lse.cpu(), cl, atol=1e-4, rtol=1e-5)
    if transform == "constant_v":
        for bi in range(b):
            for hi in range(hkv):
                assert torch.allclose(out[bi, hi * g:(hi + 1) * g].float().cpu(),
                                      torch.full((g, sq, 128), float(1 + bi * hkv + hi)), atol=2e-2)
    if transform == "zero_q":
        assert torch.allclose(lse.cpu(), torch.full(lse.shape, float(np.log(topk * 128.0))), atol=1e-3)
    if name == "g16_dense_equivalence":
        dense = torch.softmax(q.float() @ k.float().transpose(-1, -2) / 128 ** 0.5, -1) @ v.float()
        close(out, lse, dense, ref_l)


def test_fused_entry_reorder_stream_and_repeat():
    m = sp()
    q, k, v = gen.make_qkv(1, 16, 1, 256, 4096, seed=31)
    ids = gen.make_ids(1, 1, 2, 32, 16, 131, "unsorted")
    ref_o, ref_l = oracle.gather_attention(q, k, v, ids)
    qc, kc, vc, ic = q.cuda(), k.cuda(), v.cuda(), ids.cuda()
    out, lse = m.kv_centric_attention(qc, kc, vc, ic, nseg=4, partial="bf16")
    close(out, lse, ref_o, ref_l)
    out2, _ = m.kv_centric_attention(qc, kc, vc, ic.flip(-1).contiguous(), nseg=4, partial="bf16")
    close(out2, lse, ref_o, ref_l)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        out3, _ = m.kv_centric_attention(qc, kc, vc, ic, nseg=4, partial="bf16")
    stream.synchronize()
    assert torch.equal(out3, out)
    out4, _ = m.kv_centric_attention(qc, kc, vc, ic, nseg=4, partial="bf16")
    assert torch.equal(out4, out)
    m.device_status()
    with pytest.raises(RuntimeError):
        m.kv_centric_attention(qc, kc, vc, ic, nseg=4, workspace=torch.empty(1024, dtype=torch.uint8, device="cuda"))


def test_counts_and_out_of_range_flag():
    m = sp()
    q, k, v = gen.make_qkv(1, 4, 2, 256, 1024, seed=3)
    ids = gen.make_ids(1, 2, 2, 8, 4, 5, "unsorted")
    counts = torch.tensor([[[4, 0], [1, 3]]], dtype=torch.int32)
    ref_o, ref_l = oracle.gather_attention(q, k, v, ids, counts)
    p = m.Prepared(q.cuda(), k.cuda(), v.cuda(), ids.cuda(), counts.cuda(), nseg=2, partial="f32")
    out, lse = p.run()
    close(out, lse, ref_o, ref_l)
    assert torch.all(out[0, 0:2, 128:] == 0) and torch.all(torch.isinf(lse[0, 0:2, 128:]))
    bad = ids.clone()
    bad[0, 0, 0, 0] = 99
    p = m.Prepared(q.cuda(), k.cuda(), v.cuda(), bad.cuda(), nseg=2)
    p.metadata()
    with pytest.raises(ValueError):
        p.audit()


@pytest.mark.parametrize("hq,hkv,partial", [(32, 32, "f32"), (32, 32, "bf16"), (16, 4, "f32")])
def test_many_items_per_cta_with_short_segment_lists(hq, hkv, partial):
    """More work items than SMs and segment lists of 0, 1, 2 ... blocks in a row: every
    persistent CTA walks several items whose streams end after different tile counts
    (a one-block list ends before its PV has been issued). Split + merge must equal the
    unsplit kernel and no bounded wait may give up."""
    m = sp()
    b, n, topk = 1, 4096, 16
    g = torch.Generator(device="cuda").manual_seed(17)
    q = torch.randn((b, hq, n, 128), device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn((b, hkv, n, 128), device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn((b, hkv, n, 128), device="cuda", generator=g).to(torch.bfloat16)
    nb = n // 128
    ids = torch.rand((b * hkv * nb, nb), device="cuda", generator=g).argsort(-1)[:, :topk].sort(-1).values \
        .int().reshape(b, hkv, nb, topk).contiguous()
    out, lse = m.attention(q, k, v, ids, return_lse=True)
    torch.cuda.synchronize()
    m.device_status()
    o2, l2 = m.kv_centric_attention(q, k, v, ids, nseg=4, partial=partial)
    torch.cuda.synchronize()
    m.device_status()
    assert (o2.float() - out.float()).abs().max().item() <= 2e-2
    assert torch.all((l2 - lse).abs() <= 1e-3 * lse.abs().clamp_min(1.0))
