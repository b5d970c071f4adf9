"""Q-centric kernel through the C ABI against the CPU oracle (B200 only).

Tolerances: O max-abs 2e-2 and mean-abs 2e-3 against the fp32 oracle, LSE
within 1e-3 relative (and inside the reference's own atol 0.002 / rtol 0.0002,
attention/kv_centric/validate_gpu.py:12-13). Cases follow the reference gate
list (attention/q_centric/progression_validation.py:82-104)."""
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


def check(out, lse, ref_o, ref_l, o_max=2e-2, o_mean=2e-3):
    o = out.float().cpu()
    assert torch.isfinite(o).all()
    d = (o - ref_o).abs()
    assert d.max().item() <= o_max, d.max().item()
    assert d.mean().item() <= o_mean, d.mean().item()
    if lse is not None:
        l = lse.cpu()
        fin = torch.isfinite(ref_l)
        assert torch.equal(torch.isinf(l) & (l < 0), ~fin)
        err = (l[fin] - ref_l[fin]).abs()
        assert torch.all(err <= 1e-3 * ref_l[fin].abs().clamp_min(1.0))
        assert torch.all(err <= 0.002 + 0.0002 * ref_l[fin].abs())
    return d.max().item()


def run(q, k, v, ids, counts=None):
    m = sp()
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full(q.shape[:3], float("nan"), device="cuda")
    m.attention_out(q.cuda(), k.cuda(), v.cuda(), ids.cuda(), out,
                    None if counts is None else counts.cuda(), lse)
    torch.cuda.synchronize()
    m.device_status()
    return out, lse


CASES = [
    # (B, Hq, Hkv, Sq, Skv), topk, pattern, scale
    ((1, 2, 2, 256, 128), 1, "independent", 1.0),
    ((1, 2, 2, 512, 512), 2, "reverse", 0.25),
    ((2, 4, 2, 256, 512), 3, "unsorted", 1.0),
    ((1, 8, 2, 512, 2048), 16, "reverse", 1.0),
    ((1, 16, 2, 512, 4096), 16, "unsorted", 2.0),
    ((1, 32, 2, 256, 4096), 16, "independent", 4.0),
    ((1, 2, 2, 512, 4096), 32, "reverse", 1.0),
    ((1, 4, 2, 128, 128), 1, "independent", 1.0),
    ((1, 8, 2, 384, 512), 3, "reverse", 1.0),
    ((1, 3, 3, 384, 512), 4, "unsorted", 1.0),      # odd tile count, MHA
    ((1, 6, 2, 256, 1024), 5, "unsorted", 1.0),     # odd group size 3
    ((2, 16, 16, 2048, 2048), 16, "independent", 1.0),
    ((2, 16, 1, 1024, 8192), 16, "paired", 1.0),
]


@pytest.mark.parametrize("shape,topk,pattern,scale", CASES)
def test_against_oracle(shape, topk, pattern, scale):
    b, hq, hkv, sq, skv = shape
    q, k, v = gen.make_qkv(b, hq, hkv, sq, skv, seed=1700 + topk, scale=scale)
    ids = gen.make_ids(b, hkv, sq // 128, skv // 128, topk, 2300 + topk, pattern)
    ref_o, ref_l = oracle.gather_attention(q, k, v, ids)
    out, lse = run(q, k, v, ids)
    check(out, lse, ref_o, ref_l)


def test_golden_fixtures():
    """Directly against the reference's stored outputs."""
    fx = np.load(os.path.join(G, "attention_masked.npz"))
    q, k, v, ids = cases.attention_masked_case()
    out, lse = run(q, k, v, ids)
    check(out, lse, torch.from_numpy(fx["o"]), torch.from_numpy(fx["lse"]))
    fx = np.load(os.path.join(G, "attention_gather.npz"))
    for i, (q, k, v, ids) in enumerate(cases.attention_gather_cases()):
        out, _ = run(q, k, v, ids)
        check(out, None, torch.from_numpy(fx[f"o{i}"]), None)


def test_config1_shape():
    """B=1, Hq=Hkv=8, N=4096, top-8, K with per-block offsets, masked oracle."""
    q, k, v = gen.make_qkv(1, 8, 8, 4096, 4096, seed=17, k_block_offset=0.5)
    ids = gen.make_ids(1, 8, 32, 32, 8, 1017, "unsorted")
    ref_o, ref_l = oracle.masked_attention(q, k, v, ids)
    out, lse = run(q, k, v, ids)
    check(out, lse, ref_o, ref_l)


def test_counts_and_empty_lists():
    q, k, v = gen.make_qkv(1, 4, 2, 512, 512, seed=5)
    ids = gen.make_ids(1, 2, 4, 4, 3, 6, "unsorted")
    counts = torch.tensor([[[3, 0, 1, 2], [2, 3, 0, 1]]], dtype=torch.int32)
    for hq in (4, 2):   # pair mode and split mode
        qq = q[:, :hq].contiguous()
        ref_o, ref_l = oracle.gather_attention(qq, k, v, ids, counts)
        out, lse = run(qq, k, v, ids, counts)
        check(out, lse, ref_o, ref_l)
        assert torch.all(out[0, :, 128:256][: hq // 2] == 0)


def test_analytic_cases():
    """validate_gpu.py:49-73: constant V gives the constant; zero Q gives the
    uniform softmax with LSE = ln(#keys); selecting every block equals dense."""
    q, k, v = gen.make_qkv(1, 16, 1, 256, 2048, seed=42)
    ids = gen.make_ids(1, 1, 2, 16, 16, 43, "unsorted")      # all 16 blocks
    vc = torch.full_like(v, 3.0)
    out, lse = run(q, k, vc, ids)
    assert torch.allclose(out.float().cpu(), torch.full(q.shape, 3.0), atol=2e-2)
    out, lse = run(torch.zeros_like(q), k, v, ids)
    assert torch.allclose(lse.cpu(), torch.full(q.shape[:3], float(np.log(2048.0))), atol=1e-3)
    assert torch.allclose(out.float().cpu(), v.float().mean(dim=2, keepdim=True).expand(1, 16, 256, 128)
                          .contiguous(), atol=2e-2)
    dense = torch.softmax(q.float() @ k.float().transpose(-1, -2) / 128 ** 0.5, -1) @ v.float()
    out, _ = run(q, k, v, ids)
    check(out, None, dense, None)


def test_out_api_repeat_bitwise_and_nondefault_stream():
    m = sp()
    q, k, v = gen.make_qkv(2, 16, 2, 1024, 4096, seed=601)
    ids = gen.make_ids(2, 2, 8, 32, 16, 601, "unsorted")
    qc, kc, vc, ic = q.cuda(), k.cuda(), v.cuda(), ids.cuda()
    a = m.attention(qc, kc, vc, ic)
    b = torch.full_like(qc, float("nan"))
    m.attention_out(qc, kc, vc, ic, b)
    assert torch.equal(a, b)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        c = m.attention(qc, kc, vc, ic)
    stream.synchronize()
    assert torch.equal(a, c)
    m.device_status()


def test_cuda_graph_replay_with_mutated_inputs():
    """progression_validation.py:118-140."""
    m = sp()
    q, k, v = gen.make_qkv(2, 16, 2, 1024, 4096, seed=601)
    ids = gen.make_ids(2, 2, 8, 32, 16, 601, "unsorted")
    qc, kc, vc, ic = q.cuda(), k.cuda(), v.cuda(), ids.cuda()
    out = torch.empty_like(qc)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            m.attention_out(qc, kc, vc, ic, out)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        m.attention_out(qc, kc, vc, ic, out)
        m.attention_out(qc, kc, vc, ic, out)
    torch.cuda.synchronize()
    for seed in (607, 613):
        with torch.cuda.stream(stream):
            qc.mul_(-0.75)
            vc.add_(0.0625)
            ic.copy_(gen.make_ids(2, 2, 8, 32, 16, seed, "unsorted"))
            out.fill_(float("nan"))
            graph.replay()
        stream.synchronize()
        ref_o, _ = oracle.gather_attention(qc.cpu(), kc.cpu(), vc.cpu(), ic.cpu())
        check(out, None, ref_o, None)
    m.device_status()


def test_rejected_inputs():
    """progression_validation.py:141-161."""
    m = sp()
    q, k, v = gen.make_qkv(1, 4, 2, 256, 512, seed=9)
    ids = gen.make_ids(1, 2, 2, 4, 2, 9)
    qc, kc, vc, ic = q.cuda(), k.cuda(), v.cuda(), ids.cuda()
    bad = [
        (qc, kc[:, :0], vc[:, :0], ic[:, :0]),
        (qc, kc, vc, ic[..., :0]),
        (qc.float(), kc, vc, ic),
        (qc.detach().requires_grad_(), kc, vc, ic),
        (qc, kc, vc, ic.repeat_interleave(2, dim=1)),
        (qc, kc, vc, ic.long()),
        (qc[:, :, :, :64], kc, vc, ic),
    ]
    for args in bad:
        with pytest.raises(RuntimeError):
            m.attention(*args)
    out = torch.empty_like(qc)
    with pytest.raises(RuntimeError):
        m.attention_out(qc, kc, vc, ic, qc)
    with pytest.raises(RuntimeError):
        m.attention_out(qc, kc, vc, ic, out[:, :, :128])
    # top-k larger than the number of KV blocks
    with pytest.raises(RuntimeError):
        m.attention(qc, kc, vc, torch.zeros((1, 2, 2, 5), dtype=torch.int32, device="cuda"))


def test_partial_segments_merge_to_whole():
    """KV-range segments through the partial entry point + oracle merge."""
    m = sp()
    q, k, v = gen.make_qkv(1, 8, 2, 512, 2048, seed=77)
    ids = gen.make_ids(1, 2, 4, 16, 8, 78, "unsorted")
    ref_o, ref_l = oracle.gather_attention(q, k, v, ids)
    seg_ids, seg_counts = oracle.split_kv_segments(ids, 16, 4)
    for dtype in (torch.float32, torch.bfloat16):
        partial = torch.full((4, 1, 8, 512, 128), float("nan"), dtype=dtype, device="cuda")
        plse = torch.full((4, 1, 8, 512), float("nan"), device="cuda")
        m.attention_partial_out(q.cuda(), k.cuda(), v.cuda(), seg_ids.cuda(), seg_counts.cuda(), partial, plse)
        torch.cuda.synchronize()
        m.device_status()
        po = partial.float().cpu().permute(1, 2, 3, 0, 4)
        pl = plse.cpu().permute(1, 2, 3, 0)
        o, l = oracle.combine_partials(po, pl)
        d = (o - ref_o).abs()
        assert d.max() <= 2e-2 and d.mean() <= 2e-3
        assert torch.all((l - ref_l).abs() <= 1e-3 * ref_l.abs().clamp_min(1.0))


def test_host_pipeline_matches_device_path():
    """Pinned host buffers in and out, chunks pipelined over three streams."""
    m = sp()
    q, k, v = gen.make_qkv(2, 8, 4, 512, 1024, seed=91)
    ids = gen.make_ids(2, 4, 4, 8, 3, 92, "unsorted")
    ref_o, ref_l = oracle.gather_attention(q, k, v, ids)
    hq_, hk_, hv_, hi_ = (t.pin_memory() for t in (q, k, v, ids))
    ho = torch.full(q.shape, float("nan"), dtype=torch.bfloat16).pin_memory()
    hl = torch.full(q.shape[:3], float("nan")).pin_memory()
    pipe = m.HostPipeline(2, 8, 4, 512, 1024, 3, "cuda:0", chunks=3)
    for _ in range(2):                      # second call reuses the staging buffers
        ho.fill_(float("nan"))
        pipe.run(hq_, hk_, hv_, hi_, ho, hl).synchronize()
        check(ho, hl, ref_o, ref_l)
    m.device_status()
    # fewer groups than chunks: a group's heads are split over chunks (K, V and the lists travel with
    # the first one), staged through caller-owned device buffers; changed inputs on the second call
    q, k, v = gen.make_qkv(1, 8, 1, 512, 1024, seed=93)
    ids = gen.make_ids(1, 1, 4, 8, 3, 94)
    hq_, hk_, hv_, hi_ = (t.clone().pin_memory() for t in (q, k, v, ids))
    ho = torch.empty(q.shape, dtype=torch.bfloat16).pin_memory()
    hl = torch.empty(q.shape[:3]).pin_memory()
    bufs = (torch.empty_like(q, device="cuda"), torch.empty_like(k, device="cuda"), torch.empty_like(v, device="cuda"),
            torch.empty_like(ids, device="cuda"), torch.empty_like(q, device="cuda"),
            torch.empty(q.shape[:3], device="cuda"))
    pipe = m.HostPipeline(1, 8, 1, 512, 1024, 3, "cuda:0", chunks=4, buffers=bufs)
    assert pipe.chunks == 4
    for shift in (0, 1):
        hk_.copy_(k.roll(shift * 128, dims=2))
        hv_.copy_(v.roll(shift * 128, dims=2))
        ref_o, ref_l = oracle.gather_attention(q, hk_.clone(), hv_.clone(), ids)
        ho.fill_(float("nan"))
        pipe.run(hq_, hk_, hv_, hi_, ho, hl).synchronize()
        check(ho, hl, ref_o, ref_l)
    t0 = pipe.run(hq_, hk_, hv_, hi_, ho, hl, copy_only=True)
    t0.synchronize()
    m.device_status()


@pytest.mark.parametrize("shape,topk,counts_kind", [
    ((2, 16, 1, 4096, 2048), 16, "full"),      # the reference's shape: 512 items = 3 rounds + 68 -> two pieces each
    ((1, 8, 2, 40 * 128, 4096), 16, "ragged"),      # 160 items: 1 round + 12 -> four pieces each, ragged counts
    ((1, 3, 3, 51 * 256, 2048), 8, "full"),    # split mode (group 1): 153 items, 5 left over, two pieces of four blocks
])
def test_balanced_last_round_matches_the_plain_call(shape, topk, counts_kind):
    """With a workspace the kernel cuts the items of a last, partly filled round into pieces and merges their
    partials: same result as the plain call up to the bf16 rounding of the partials, LSE to fp32 rounding, and
    inside the oracle tolerance; rows outside the last round are bit-identical."""
    m = sp()
    b, hq, hkv, sq, skv = shape
    q, k, v = gen.make_qkv(b, hq, hkv, sq, skv, seed=11, k_block_offset=0.5)
    ids = gen.make_ids(b, hkv, sq // 128, skv // 128, topk, 3, "unsorted")
    counts = None
    if counts_kind == "ragged":
        g = torch.Generator().manual_seed(4)
        counts = torch.randint(0, topk + 1, (b, hkv, sq // 128), generator=g, dtype=torch.int32)
    qc, kc, vc, ic = q.cuda(), k.cuda(), v.cuda(), ids.cuda()
    cc = None if counts is None else counts.cuda()
    plain = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
    plain_lse = torch.full(q.shape[:3], float("nan"), device="cuda")
    m.attention_out(qc, kc, vc, ic, plain, cc, plain_lse, balance=False)
    bal = torch.full_like(plain, float("nan"))
    bal_lse = torch.full_like(plain_lse, float("nan"))
    m.attention_out(qc, kc, vc, ic, bal, cc, bal_lse, balance=True)
    torch.cuda.synchronize()
    m.device_status()
    assert torch.isfinite(bal.float()).all()
    diff = (bal.float() - plain.float()).abs()
    changed = (diff > 0).reshape(b, hq, sq // 128, -1).any(-1)    # (head, query block) tiles that went through the merge
    assert 0 < int(changed.sum()) <= changed.numel() // 2         # the last round only
    assert diff.max().item() <= 2.0 ** -6 * max(1.0, plain.float().abs().max().item())
    fin = torch.isfinite(plain_lse)
    assert torch.equal(torch.isfinite(bal_lse), fin)
    assert torch.all((bal_lse[fin] - plain_lse[fin]).abs() <= 2e-6 * plain_lse[fin].abs().clamp_min(1.0))
    ref_o, ref_l = oracle.gather_attention(q, k, v, ids, counts)
    check(bal, bal_lse, ref_o, ref_l)
