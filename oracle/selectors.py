"""R1 / R4 block-summary selectors (CPU). Test infrastructure only.

Restates benchmarks/ch4_selectors/reference.py:28-38 (`summary_reference`)
and, for the kernel-side formulation, indexers/r1_r4/gpu_ops.py:6-49
(pool_blocks, descriptor_dot, reduce_topk), generalised to any number of KV
heads (the max runs over the query heads of ONE KV-head group), any TopK and
any number of KV blocks.

Canonical arithmetic (what makes the ids reproducible bit for bit):
  descriptor = bf16_rne( (x_0 + x_1 + ... + x_{n-1}) * (1/n) ), fp32 adds in
               token order, n = 128/R tokens per representative;
  raw(m, j)  = ( ... ((qd_0*kd_0) + qd_1*kd_1) + ... + qd_127*kd_127 ) in fp32,
               feature order (every product of two bf16 values is exact in fp32,
               so fused and unfused multiply-add agree), then * fp32(128**-0.5);
  score      = max over (group heads, R query reps, R key reps) of raw;
  ids        = TopK by (score descending, block id ascending), emitted in that
               order (the stable argsort of reference.py:37).
The reference computes the same quantities with torch.mean / torch.bmm, whose
summation order is unspecified; it agrees with the canonical order to fp32
rounding (scores) and, on every case its own gate uses, exactly (ids).
"""
import numpy as np
import torch

BLOCK = 128
SCALE = np.float32(128.0 ** -0.5)


@torch.no_grad()
def pool_descriptors(x, r):
    """[B,H,S,128] bf16 -> [B,H,S/128,R,128] bf16 (gpu_ops.py:6-16,
    reference.py:32-33) with the canonical sequential fp32 sum."""
    b, h, s, d = x.shape
    n = BLOCK // r
    xf = x.float().reshape(b, h, s // BLOCK, r, n, d)
    acc = torch.zeros((b, h, s // BLOCK, r, d), dtype=torch.float32)
    for t in range(n):
        acc = acc + xf[..., t, :]
    return (acc * (1.0 / n)).to(torch.bfloat16)


@torch.no_grad()
def _raw_scores(qd, kd):
    """qd [M,128] bf16, kd [N,128] bf16 -> [M,N] fp32, sequential over features."""
    a, bm = qd.float(), kd.float()
    acc = torch.zeros((a.shape[0], bm.shape[0]), dtype=torch.float32)
    for f in range(a.shape[1]):
        acc = acc + a[:, f:f + 1] * bm[:, f][None, :]
    return acc * float(SCALE)


@torch.no_grad()
def summary_scores(q, k, r):
    """-> (qd, kd, scores[B,Hkv,Sq/128,Skv/128] fp32)."""
    b, hq, sq, _ = q.shape
    hkv, skv = k.shape[1:3]
    g = hq // hkv
    qt, nt = sq // BLOCK, skv // BLOCK
    qd, kd = pool_descriptors(q, r), pool_descriptors(k, r)
    scores = torch.empty((b, hkv, qt, nt), dtype=torch.float32)
    for bi in range(b):
        for h in range(hkv):
            raw = _raw_scores(qd[bi, h * g:(h + 1) * g].reshape(g * qt * r, 128),
                              kd[bi, h].reshape(nt * r, 128))
            scores[bi, h] = raw.reshape(g, qt, r, nt, r).amax(dim=(0, 2, 4))
    return qd, kd, scores


def stable_topk(scores, topk):
    """Score-descending, lower index first among equals (reference.py:37;
    indexers/fp4/reference.py:15-17)."""
    return torch.argsort(scores, dim=-1, descending=True, stable=True)[..., :topk] \
        .to(torch.int32).contiguous()


@torch.no_grad()
def summary_select(q, k, r, topk):
    qd, kd, scores = summary_scores(q, k, r)
    return qd, kd, scores, stable_topk(scores, topk)
