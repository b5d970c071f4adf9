"""NVFP4 indexer oracle (CPU). Test infrastructure only.

Data contract (indexers/fp4/fp4.py:37-60): a 128-feature index vector is 64
bytes of packed e2m1 codes (low nibble = even feature,
indexers/fp4/fp4_reference.py:7-10) plus eight e4m3 scales, one per 16
features. Query index vectors are [B*Sq, Hidx, 64]; key index vectors are
paged [B*Skv/128, Hk, 128, 64] with Hk = 1 (shared, the reference's layout) or
Hk = Hidx.

Canonical score arithmetic (exact until the last step, so any evaluation order
inside a 16-feature group gives the same bits):
  t_g   = (sum_{i in group g} qv_i * kv_i) * (qs_g * ks_g)      exact in fp32
  dot   = ((t_0 + t_1) + t_2) + ... + t_7                        fp32, in order
The reference oracle (fp4_reference.py:17-35) multiplies dequantised fp32
vectors with torch.matmul (order unspecified) and agrees to fp32 rounding; its
own gate uses rtol 1e-4 / atol 1e-3 (benchmarks/ch4_selectors/harness.py:38).

bf16 -> NVFP4 quantisation is NOT in the reference (parity unpinned). Rule:
  scale_g = e4m3_rne(amax_g / 6), saturating at 448;
  code_i  = nearest e2m1 value to x_i / scale_g (fp32 division), ties to the
            even code, saturating at +-6; scale_g == 0 gives code 0.
"""
import numpy as np
import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# decision thresholds between consecutive magnitudes and which way a tie goes
# (True: tie rounds up to the higher code). Even codes are 0,2,4,6.
_MID = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
_TIE_UP = np.array([False, True, False, True, False, True, False])


def _e2m1_codes(mag):
    """fp32 magnitudes -> codes 0..7, round-to-nearest, ties to even code."""
    mag = np.asarray(mag, dtype=np.float32)
    code = np.zeros(mag.shape, dtype=np.uint8)
    for i in range(7):
        up = (mag > _MID[i]) | ((mag == _MID[i]) & _TIE_UP[i])
        code = np.where(up, np.uint8(i + 1), code)
    return code


@torch.no_grad()
def quantize_nvfp4(x):
    """[..., 128] bf16/fp32 -> (packed uint8 [..., 64], scales float8_e4m3fn [..., 8])."""
    xf = x.float()
    lead = xf.shape[:-1]
    grp = xf.reshape(*lead, 8, 16)
    amax = grp.abs().amax(dim=-1)
    scale = (amax / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    sf = scale.float()
    safe = torch.where(sf > 0, sf, torch.ones_like(sf))
    ratio = (grp / safe.unsqueeze(-1)).numpy()
    code = _e2m1_codes(np.abs(ratio))
    code = np.where(sf.unsqueeze(-1).numpy() > 0, code, 0).astype(np.uint8)
    sign = (np.signbit(ratio) & (code > 0)).astype(np.uint8) << 3
    nib = (code | sign).reshape(*lead, 64, 2)
    packed = (nib[..., 0] | (nib[..., 1] << 4)).astype(np.uint8)
    return torch.from_numpy(packed), scale


@torch.no_grad()
def group_mean(x, heads_out):
    """[B,H,S,128] -> fp32 [B,heads_out,S,128]: mean of each group of H/heads_out
    consecutive heads, summed in head order then divided (IEEE fp32)."""
    b, h, s, d = x.shape
    g = h // heads_out
    xf = x.float().reshape(b, heads_out, g, s, d)
    acc = torch.zeros((b, heads_out, s, d), dtype=torch.float32)
    for i in range(g):
        acc = acc + xf[:, :, i]
    return acc / float(g) if g > 1 else acc


def quantize_queries(q, hidx):
    """q [B,Hq,Sq,128] -> (codes [B*Sq,hidx,64], scales [B*Sq,hidx,8]), token-major."""
    b, _, sq, _ = q.shape
    m = group_mean(q, hidx).permute(0, 2, 1, 3).reshape(b * sq, hidx, 128)
    return quantize_nvfp4(m)


def quantize_keys(k):
    """k [B,Hkv,Skv,128] -> paged (codes [B*Skv/128,Hkv,128,64], scales [...,8])."""
    b, h, skv, _ = k.shape
    paged = k.float().reshape(b, h, skv // 128, 128, 128).permute(0, 2, 1, 3, 4).reshape(b * skv // 128, h, 128, 128)
    return quantize_nvfp4(paged)


@torch.no_grad()
def dequantize_nvfp4(packed, scales):
    """fp4_reference.py:4-14."""
    codes = torch.stack((packed & 15, packed >> 4), dim=-1).reshape(*packed.shape[:-1], 128).long()
    mags = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    values = mags[codes & 7] * torch.where((codes & 8) != 0, -1.0, 1.0)
    return values * scales.float().repeat_interleave(16, dim=-1)


def _int_codes(packed):
    """packed -> signed integers 2*value in [-12, 12], [..., 128] int32."""
    codes = torch.stack((packed & 15, packed >> 4), dim=-1).reshape(*packed.shape[:-1], 128).long()
    mags2 = torch.tensor([0, 1, 2, 3, 4, 6, 8, 12], dtype=torch.int32)
    return mags2[codes & 7] * torch.where((codes & 8) != 0, -1, 1).to(torch.int32)


@torch.no_grad()
def _canonical_dots(qp, qs, kp, ks):
    """qp [M,64] u8, qs [M,8] e4m3, kp [N,64], ks [N,8] -> [M,N] fp32 canonical."""
    qi = _int_codes(qp).float().reshape(-1, 8, 16)
    ki = _int_codes(kp).float().reshape(-1, 8, 16)
    qsf, ksf = qs.float(), ks.float()
    acc = None
    for g in range(8):
        isum = qi[:, g] @ ki[:, g].T                  # exact small integers (x4)
        t = (isum * 0.25) * (qsf[:, g:g + 1] * ksf[:, g][None, :])
        acc = t if acc is None else acc + t
    return acc


@torch.no_grad()
def fp4_scores(qp, qs, kp, ks, batch_size, len_q, len_kv):
    """Per-query block scores, fp4_reference.py:17-35 layout:
    [Hidx, Skv/128, B*Sq] fp32 = max over the 128 keys of a page."""
    hidx = qp.shape[1]
    hk = kp.shape[1]
    tiles = len_kv // 128
    out = torch.empty((hidx, tiles, batch_size * len_q), dtype=torch.float32)
    for b in range(batch_size):
        for h in range(hidx):
            kh = h if hk > 1 else 0
            keys_p = kp[b * tiles:(b + 1) * tiles, kh].reshape(len_kv, 64)
            keys_s = ks[b * tiles:(b + 1) * tiles, kh].reshape(len_kv, 8)
            s0 = b * len_q
            for first in range(0, len_q, 512):
                end = min(first + 512, len_q)
                dots = _canonical_dots(qp[s0 + first:s0 + end, h], qs[s0 + first:s0 + end, h],
                                       keys_p, keys_s)
                out[h, :, s0 + first:s0 + end] = dots.reshape(end - first, tiles, 128).amax(-1).T
    return out


def fp4_scores_varlen(qp, qs, kp, ks, cu_seqlens_q, cu_seqlens_k, cu_page_offsets, kv_indices, max_seqlen_k,
                      causal=False, qo_offset=None):
    """Ragged batch over a paged key cache, optionally causal (PARITY UNPINNED: the vendored scorer
    is GPU-only; this restates its documented contract, indexers/fp4/vendor_minimax_msa/
    fp4_indexer_interface.py:745-811, with the canonical arithmetic of _canonical_dots).
    qp [total_q,Hq,64], qs [total_q,Hq,8], kp [total_pages,Hk,128,64], ks [total_pages,Hk,128,8];
    request b: queries cu_seqlens_q[b]..cu_seqlens_q[b+1], k_len keys in logical pages
    kv_indices[cu_page_offsets[b] + t]; query head h reads key head h // (Hq // Hk); causal: key j is
    visible to query i when j <= i + offset, offset = k_len - q_len unless qo_offset[b] is given
    (src/sm100/fp4_indexer.py:525-529). Returns fp32 [Hq, ceil(max_seqlen_k/128), total_q] = max over
    the visible keys of each page, -inf where there is none."""
    total_q, hq = qp.shape[0], qp.shape[1]
    hk = kp.shape[1]
    tiles = (int(max_seqlen_k) + 127) // 128
    out = torch.full((hq, tiles, total_q), -float("inf"), dtype=torch.float32)
    batch = len(cu_seqlens_q) - 1
    for b in range(batch):
        q0, q1 = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        k_len = int(cu_seqlens_k[b + 1]) - int(cu_seqlens_k[b])
        q_len = q1 - q0
        if q_len <= 0 or k_len <= 0:
            continue
        pages = (k_len + 127) // 128
        phys = [int(kv_indices[int(cu_page_offsets[b]) + t]) for t in range(pages)]
        offset = (int(qo_offset[b]) if qo_offset is not None else k_len - q_len) if causal else None
        qi = torch.arange(q_len)[:, None]
        kj = torch.arange(pages * 128)[None, :]
        visible = kj < k_len
        if causal:
            visible = visible & (kj <= qi + offset)
        else:
            visible = visible.expand(q_len, -1)
        for h in range(hq):
            kh = h // (hq // hk)
            keys_p = torch.stack([kp[i, kh] for i in phys]).reshape(pages * 128, 64)
            keys_s = torch.stack([ks[i, kh] for i in phys]).reshape(pages * 128, 8)
            dots = _canonical_dots(qp[q0:q1, h], qs[q0:q1, h], keys_p, keys_s)
            dots = torch.where(visible, dots, torch.tensor(-float("inf")))
            out[h, :pages, q0:q1] = dots.reshape(q_len, pages, 128).amax(-1).T
    return out


def fp4_tile_scores(scores, batch_size, len_q):
    """indexers/fp4/reference.py:8-13: max over the 128 queries of a tile ->
    [B, Hidx, Sq/128, Skv/128]."""
    heads, tiles, _ = scores.shape
    return scores.reshape(heads, tiles, batch_size, len_q // 128, 128).amax(-1).permute(2, 0, 3, 1).contiguous()


def fp4_select(scores, batch_size, len_q, topk):
    """indexers/fp4/reference.py:4-17 with a free TopK."""
    from .selectors import stable_topk
    return stable_topk(fp4_tile_scores(scores, batch_size, len_q), topk)
