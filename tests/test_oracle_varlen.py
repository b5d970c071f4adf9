"""CPU checks of the ragged / paged / causal NVFP4 scorer oracle (its parity is unpinned: the
reference's scorer for this contract is GPU-only). It must reduce to the dense oracle, which IS
pinned against the reference's fixtures, and masking must only ever remove keys."""
import torch

import oracle


def _inputs(seed, total_q, hq, total_pages, hk):
    g = torch.Generator().manual_seed(seed)
    qp = torch.randint(256, (total_q, hq, 64), dtype=torch.uint8, generator=g)
    kp = torch.randint(256, (total_pages, hk, 128, 64), dtype=torch.uint8, generator=g)
    ch = torch.tensor([0.25, 0.5, 1.0, 2.0])
    qs = ch[torch.randint(4, (total_q, hq, 8), generator=g)].to(torch.float8_e4m3fn)
    ks = ch[torch.randint(4, (total_pages, hk, 128, 8), generator=g)].to(torch.float8_e4m3fn)
    return qp, qs, kp, ks


def test_dense_batch_equals_the_dense_oracle():
    qp, qs, kp, ks = _inputs(1, 256, 2, 4, 2)
    dense = oracle.fp4_scores(qp, qs, kp, ks, 2, 128, 256)
    cu_q = torch.tensor([0, 128, 256], dtype=torch.int32)
    cu_k = torch.tensor([0, 256, 512], dtype=torch.int32)
    cu_p = torch.tensor([0, 2, 4], dtype=torch.int32)
    ragged = oracle.fp4_scores_varlen(qp, qs, kp, ks, cu_q, cu_k, cu_p, torch.arange(4, dtype=torch.int32), 256)
    assert torch.equal(dense, ragged)
    # a permuted page table with permuted pages gives the same scores
    perm = torch.tensor([2, 0, 3, 1])
    inv = torch.argsort(perm).to(torch.int32)
    again = oracle.fp4_scores_varlen(qp, qs, kp[perm], ks[perm], cu_q, cu_k, cu_p, inv, 256)
    assert torch.equal(dense, again)


def test_ragged_lengths_causal_mask_and_gqa():
    q_lens, k_lens = [70, 1, 130], [300, 129, 100]
    pages = [(k + 127) // 128 for k in k_lens]
    qp, qs, kp, ks = _inputs(2, sum(q_lens), 4, sum(pages), 2)
    cu = lambda xs: torch.tensor([0] + [sum(xs[:i + 1]) for i in range(len(xs))], dtype=torch.int32)
    idx = torch.arange(sum(pages), dtype=torch.int32)
    full = oracle.fp4_scores_varlen(qp, qs, kp, ks, cu(q_lens), cu(k_lens), cu(pages), idx, max(k_lens))
    caus = oracle.fp4_scores_varlen(qp, qs, kp, ks, cu(q_lens), cu(k_lens), cu(pages), idx, max(k_lens), causal=True)
    assert full.shape == (4, 3, sum(q_lens))
    assert torch.all(caus <= full)                          # masking only removes keys
    # request 1 (one query, 129 keys, offset 128): everything visible -> equal to the full scores
    assert torch.equal(caus[:, :, 70:71], full[:, :, 70:71])
    # request 2 has more queries than keys: offset -30, its first 30 queries see nothing
    assert torch.all(torch.isinf(caus[:, :, 71:71 + 30]))
    assert torch.all(torch.isfinite(caus[:, 0, 71 + 30:]))
    # pages past a request's keys stay -inf
    assert torch.all(torch.isinf(full[:, 2, 70:71])) and torch.all(torch.isinf(full[:, 1:, 71:]))
    # heads 0,1 read key head 0; heads 2,3 key head 1: swapping the key heads swaps the groups' scores
    swapped = oracle.fp4_scores_varlen(qp[:, [2, 3, 0, 1]], qs[:, [2, 3, 0, 1]], kp[:, [1, 0]], ks[:, [1, 0]],
                                       cu(q_lens), cu(k_lens), cu(pages), idx, max(k_lens))
    assert torch.equal(swapped[[2, 3, 0, 1]], full)
