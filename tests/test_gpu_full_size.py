"""Full-size configurations on the GPU, checked through properties that do not need a full
CPU run: sampled query blocks against the oracle, the KV-range split + log-sum-exp merge
against the unsplit kernel, sampled selection lists against the oracle's fixed arithmetic."""
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def sp():
    import sparse_attention_b200_b200 as m
    return m


def device_inputs(b, hq, hkv, n, seed, k_offset=0.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((b, hq, n, 128), device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn((b, hkv, n, 128), device="cuda", generator=g)
    if k_offset:
        k = (k.view(b, hkv, n // 128, 128, 128) + k_offset * torch.randn((b, hkv, n // 128, 1, 128), device="cuda",
                                                                        generator=g)).view(b, hkv, n, 128)
    k = k.to(torch.bfloat16)
    v = torch.randn((b, hkv, n, 128), device="cuda", generator=g).to(torch.bfloat16)
    return q, k, v


def test_config2_full_size_sampled_blocks_and_split_merge():
    """B=1, Hq=Hkv=32, N=32768, 16 sorted distinct blocks per list."""
    m = sp()
    b, h, n, topk = 1, 32, 32768, 16
    q, k, v = device_inputs(b, h, h, n, 17)
    nb = n // 128
    g = torch.Generator(device="cuda").manual_seed(1017)
    ids = torch.rand((b * h * nb, nb), device="cuda", generator=g).argsort(-1)[:, :topk].sort(-1).values \
        .int().reshape(b, h, nb, topk).contiguous()
    out, lse = m.attention(q, k, v, ids, return_lse=True)
    torch.cuda.synchronize()
    m.device_status()
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    # sampled (head, query block) pairs against the CPU oracle
    for head, qb in ((0, 0), (7, 255), (31, 128), (19, 77)):
        qs = q[:, head:head + 1, qb * 128:(qb + 1) * 128].cpu()
        ro, rl = oracle.gather_attention(qs, k[:, head:head + 1].cpu(), v[:, head:head + 1].cpu(),
                                         ids[:, head:head + 1, qb:qb + 1].cpu())
        d = (out[:, head:head + 1, qb * 128:(qb + 1) * 128].float().cpu() - ro).abs()
        assert d.max() <= 2e-2 and d.mean() <= 2e-3
        l = lse[:, head:head + 1, qb * 128:(qb + 1) * 128].cpu()
        assert torch.all((l - rl).abs() <= 1e-3 * rl.abs().clamp_min(1.0))
    # KV-range split (4 segments) + merge == unsplit kernel (property of the whole output)
    o2, l2 = m.kv_centric_attention(q, k, v, ids, nseg=4, partial="f32")
    torch.cuda.synchronize()
    assert (o2.float() - out.float()).abs().max().item() <= 2e-2
    assert torch.all((l2 - lse).abs() <= 1e-3 * lse.abs().clamp_min(1.0))
    # repeat: bitwise identical
    assert torch.equal(m.attention(q, k, v, ids), out)


def test_config3_full_size_indexer_sampled_lists_and_attention():
    """B=2, Hq=64, Hkv=8, N=65536, R4 top-32: tensor-core indexer == exact kernel everywhere,
    sampled lists == CPU oracle, attention on sampled blocks == oracle."""
    m = sp()
    b, hq, hkv, n, topk = 2, 64, 8, 65536, 32
    q, k, v = device_inputs(b, hq, hkv, n, 17, k_offset=0.5)
    fast = m.SummarySelector(q, k, 4, topk=topk, keep_scores=False)
    ids = fast.run_fast().clone()
    exact = m.SummarySelector(q, k, 4, topk=topk, keep_scores=True)
    exact.prepare()
    exact.score()
    torch.cuda.synchronize()
    m.device_status()
    assert torch.equal(ids, exact.ids)                      # every one of the 8192 lists, bit for bit
    assert torch.equal(fast.kd.view(torch.int16), exact.kd.view(torch.int16))
    # sampled (batch, kv head): full oracle for that head on the CPU (canonical arithmetic)
    for bi, kvh in ((0, 0), (1, 5)):
        qh = q[bi:bi + 1, kvh * 8:(kvh + 1) * 8, :1024].cpu()          # first 8 query blocks of the group
        kh = k[bi:bi + 1, kvh:kvh + 1].cpu()
        _, kd, scores, ref = oracle.summary_select(qh, kh, 4, topk)
        assert torch.equal(exact.kd[bi, kvh].cpu().view(torch.int16), kd[0, 0].view(torch.int16))
        assert torch.equal(ids[bi, kvh, :8].cpu(), ref[0, 0])
        assert torch.equal(exact.scores[bi, kvh, :8].cpu(), scores[0, 0])
    out, lse = m.attention(q, k, v, ids, return_lse=True)
    torch.cuda.synchronize()
    m.device_status()
    for bi, head, qb in ((0, 3, 0), (1, 63, 511)):
        kvh = head // 8
        ro, rl = oracle.gather_attention(q[bi:bi + 1, head:head + 1, qb * 128:(qb + 1) * 128].cpu(),
                                         k[bi:bi + 1, kvh:kvh + 1].cpu(), v[bi:bi + 1, kvh:kvh + 1].cpu(),
                                         ids[bi:bi + 1, kvh:kvh + 1, qb:qb + 1].cpu())
        d = (out[bi:bi + 1, head:head + 1, qb * 128:(qb + 1) * 128].float().cpu() - ro).abs()
        assert d.max() <= 2e-2 and d.mean() <= 2e-3
        l = lse[bi:bi + 1, head:head + 1, qb * 128:(qb + 1) * 128].cpu()
        assert torch.all((l - rl).abs() <= 1e-3 * rl.abs().clamp_min(1.0))


def test_config4_reduced_fp4_fast_equals_exact_and_kv_centric():
    """Configuration-4 flow at N = 32768 (the exact dp4a scorer needs 18 ms there): quantise,
    tensor-core NVFP4 indexer == exact scorer, KV-centric operator == Q-centric kernel."""
    m = sp()
    b, hq, hkv, n, topk = 1, 64, 4, 32768, 64
    q, k, v = device_inputs(b, hq, hkv, n, 23)
    qc, qs = m.quantize_queries(q, hkv)
    kc, ks = m.quantize_keys(k)
    inputs = m.prepare_fp4_inputs(qc, kc, qs, ks, batch_size=b, len_q=n, len_kv=n)
    ids_fast, _ = m.fp4_indexer_fast(inputs, topk=topk)
    ids_exact = m.fp4_indexer(inputs, topk=topk)
    torch.cuda.synchronize()
    assert torch.equal(ids_fast, ids_exact)
    o1, l1 = m.kv_centric_attention(q, k, v, ids_fast, nseg=4)
    o2, l2 = m.attention(q, k, v, ids_fast, return_lse=True)
    torch.cuda.synchronize()
    m.device_status()
    assert (o1.float() - o2.float()).abs().max().item() <= 2e-2
    assert torch.all((l1 - l2).abs() <= 1e-3 * l2.abs().clamp_min(1.0))
