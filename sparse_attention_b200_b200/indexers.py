"""Host-side mirrors of the reference indexers, bound to the C ABI.

SummarySelector   indexers/r1_r4/block_selectors.py:9-45 (prepare / score+topk / run)
quantize_*        bf16 -> NVFP4 index vectors (no counterpart in the reference)
fp4_block_scores  indexers/fp4/fp4.py:122-134
tile_topk(_out)   indexers/fp4/__init__.py:24-38, indexers/fp4/wrapper.cpp:16-72
fp4_indexer       indexers/fp4/fp4.py:137-146
indexed_attention indexers/fp4/pipeline.py:49-65
"""
import ctypes

import torch

from . import _lib


class SummarySelector:
    """R1 / R4 selector for q [B,Hq,Sq,128], k [B,Hkv,Skv,128] (bf16, CUDA).
    ids [B,Hkv,Sq/128,topk] are score-descending, ties to the lower block id."""

    def __init__(self, q, k, representatives, topk=16, keep_scores=True):
        b, hq, sq, d = q.shape
        if d != 128 or sq % 128 or k.shape[0] != b or k.shape[3] != 128 or k.shape[2] % 128:
            raise ValueError("D128 and complete 128-token blocks only")
        hkv = k.shape[1]
        if hq % hkv or representatives not in (1, 2, 4) or (hq // hkv) * representatives > 64:
            raise ValueError("Hq must be a multiple of Hkv; R in (1,2,4); group size x R <= 64")
        for t in (q, k):
            if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()):
                raise ValueError("q and k must be contiguous bf16 CUDA tensors")
        self.q, self.k, self.r, self.b, self.hq, self.hkv = q, k, representatives, b, hq, hkv
        self.qt, self.nt, self.topk = sq // 128, k.shape[2] // 128, topk
        if not 0 < topk <= self.nt:
            raise ValueError("topk must be in [1, number of KV blocks]")
        r = representatives
        self.qd = torch.empty((b, hq, self.qt, r, 128), dtype=torch.bfloat16, device=q.device)
        self.kd = torch.empty((b, hkv, self.nt, r, 128), dtype=torch.bfloat16, device=q.device)
        self.scores = torch.empty((b, hkv, self.qt, self.nt), dtype=torch.float32, device=q.device) \
            if keep_scores else None
        self.ids = torch.empty((b, hkv, self.qt, topk), dtype=torch.int32, device=q.device)
        # workspace of the tensor-core path: key abs-max and largest squared key norm per (batch, KV head)
        # + fallback counter, bound-violation counter, largest error / bound (sparse_b200_indexer_summary_aux_bytes)
        self.aux = torch.zeros(2 * b * hkv + 3, dtype=torch.int32, device=q.device)
        self.name = f"mean{r}_bf16"

    def prepare(self):
        L = _lib.lib()
        with torch.cuda.device(self.q.device):
            st = _lib.current_stream()
            _lib.check(L.sparse_b200_pool_blocks(_lib.ptr(self.q), _lib.ptr(self.qd), self.b, self.hq,
                                                 self.qt * 128, self.r, st))
            _lib.check(L.sparse_b200_pool_blocks(_lib.ptr(self.k), _lib.ptr(self.kd), self.b, self.hkv,
                                                 self.nt * 128, self.r, st))

    def score(self):
        """Scores and top-k are one fused kernel here (the raw matrix is never stored)."""
        with torch.cuda.device(self.q.device):
            _lib.check(_lib.lib().sparse_b200_summary_select(
                _lib.ptr(self.qd), _lib.ptr(self.kd), _lib.ptr(self.scores), _lib.ptr(self.ids), self.b, self.hq,
                self.hkv, self.qt, self.nt, self.r, self.topk, _lib.current_stream()))

    def topk_stage(self):
        return self.ids

    def run_fast(self):
        """Same ids through the tensor-core pre-filter + exact re-scoring (no scores output)."""
        with torch.cuda.device(self.q.device):
            _lib.check(_lib.lib().sparse_b200_indexer_summary_fast(
                _lib.ptr(self.q), _lib.ptr(self.k), _lib.ptr(self.qd), _lib.ptr(self.kd), _lib.ptr(self.aux),
                _lib.ptr(self.ids), self.b, self.hq, self.hkv, self.qt * 128, self.nt * 128, self.r, self.topk,
                _lib.current_stream()))
        return self.ids

    def fallback_lists(self):
        """Lists of the last run_fast() that needed the exact fallback (synchronising)."""
        return int(self.aux[2 * self.b * self.hkv].item())

    def bound_stats(self):
        """(re-scored candidates whose tensor-core score was further than the error bound from the exact one,
        largest observed |tensor-core - exact| / bound) of the last run_fast() (synchronising)."""
        tail = self.aux[2 * self.b * self.hkv + 1:].cpu()
        return int(tail[0]), float(tail[1:2].view(torch.float32))

    def run(self):
        if self.scores is None:
            return self.run_fast()
        with torch.cuda.device(self.q.device):
            _lib.check(_lib.lib().sparse_b200_indexer_summary(
                _lib.ptr(self.q), _lib.ptr(self.k), _lib.ptr(self.qd), _lib.ptr(self.kd), _lib.ptr(self.scores),
                _lib.ptr(self.ids), self.b, self.hq, self.hkv, self.qt * 128, self.nt * 128, self.r, self.topk,
                _lib.current_stream()))
        return self.ids


def summary_indexed_attention_out(selector, v, out, lse=None):
    """selector.run_fast() + attention on the current stream as ONE C call; ids land in selector.ids."""
    s = selector
    with torch.cuda.device(s.q.device):
        _lib.check(_lib.lib().sparse_b200_indexed_attention_summary(
            _lib.ptr(s.q), _lib.ptr(s.k), _lib.ptr(v), _lib.ptr(s.qd), _lib.ptr(s.kd), _lib.ptr(s.aux),
            _lib.ptr(s.ids), _lib.ptr(out), _lib.ptr(lse), s.b, s.hq, s.hkv, s.qt * 128, s.nt * 128, s.r, s.topk,
            _lib.current_stream()))
    return out


# ---------------------------------------------------------------- NVFP4
def quantize_queries(q, hidx):
    """q [B,Hq,Sq,128] bf16 -> (codes [B*Sq,hidx,64] u8, scales [B*Sq,hidx,8] e4m3):
    index vector h = mean over the Hq/hidx heads of group h."""
    b, hq, sq, _ = q.shape
    if hq % hidx:
        raise ValueError("Hq must be a multiple of the index head count")
    codes = torch.empty((b * sq, hidx, 64), dtype=torch.uint8, device=q.device)
    scales = torch.empty((b * sq, hidx, 8), dtype=torch.float8_e4m3fn, device=q.device)
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().sparse_b200_nvfp4_quantize(_lib.ptr(q), _lib.ptr(codes), _lib.ptr(scales), b, hidx,
                                                         hq // hidx, sq, 0, _lib.current_stream()))
    return codes, scales


def quantize_keys(k):
    """k [B,Hkv,Skv,128] bf16 -> paged (codes [B*Skv/128,Hkv,128,64], scales [...,128,8])."""
    b, hkv, skv, _ = k.shape
    codes = torch.empty((b * skv // 128, hkv, 128, 64), dtype=torch.uint8, device=k.device)
    scales = torch.empty((b * skv // 128, hkv, 128, 8), dtype=torch.float8_e4m3fn, device=k.device)
    with torch.cuda.device(k.device):
        _lib.check(_lib.lib().sparse_b200_nvfp4_quantize(_lib.ptr(k), _lib.ptr(codes), _lib.ptr(scales), b, hkv, 1,
                                                         skv, 1, _lib.current_stream()))
    return codes, scales


def prepare_fp4_inputs(q_fp4, k_fp4, q_scale, k_scale, *, batch_size, len_q, len_kv):
    """Validated bundle with the reference's keys (indexers/fp4/fp4.py:37-85). No
    scale reordering is needed: the scorer reads the public layout directly."""
    if batch_size <= 0 or len_q <= 0 or len_q % 128 or len_kv <= 0 or len_kv % 128:
        raise ValueError("B must be positive; Sq and Skv positive multiples of 128")
    if q_fp4.ndim != 3 or q_fp4.shape[0] != batch_size * len_q or q_fp4.shape[2] != 64:
        raise ValueError("Qidx must be [B*Sq,Hidx,64]")
    hidx = q_fp4.shape[1]
    pages = batch_size * (len_kv // 128)
    if k_fp4.ndim != 4 or k_fp4.shape[0] != pages or k_fp4.shape[1] not in (1, hidx) \
            or tuple(k_fp4.shape[2:]) != (128, 64):
        raise ValueError("Kidx must be [pages,1 or Hidx,128,64]")
    expected = (("Qidx", q_fp4, (batch_size * len_q, hidx, 64), torch.uint8),
                ("Kidx", k_fp4, tuple(k_fp4.shape), torch.uint8),
                ("Q scales", q_scale, (batch_size * len_q, hidx, 8), torch.float8_e4m3fn),
                ("K scales", k_scale, (*k_fp4.shape[:3], 8), torch.float8_e4m3fn))
    for name, t, shape, dtype in expected:
        if not t.is_cuda or t.device != q_fp4.device or t.dtype != dtype or tuple(t.shape) != shape \
                or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous {dtype} {shape} on Qidx's CUDA device")
    return {"q": q_fp4, "k": k_fp4, "q_scale": q_scale, "k_scale": k_scale, "batch_size": batch_size,
            "hkv": hidx, "hk": k_fp4.shape[1], "len_q": len_q, "len_kv": len_kv}


def fp4_block_scores(inputs, exact=True):
    """fp32 [Hidx, KV_tiles, B*Sq] scores (max over the keys of each page). exact=False: straight off the NVFP4
    tensor cores (the dense batch handed to the ragged scorer as B equal requests over pages in order)."""
    b, h, lq, lkv = inputs["batch_size"], inputs["hkv"], inputs["len_q"], inputs["len_kv"]
    if not exact:
        dev = inputs["q"].device
        if "cu_q" not in inputs:          # the reference's prepare_fp4_inputs keeps the same index tensors (fp4.py:78-82)
            req = torch.arange(b + 1, device=dev, dtype=torch.int32)
            inputs.update(cu_q=req * lq, cu_k=req * lkv, cu_pages=req * (lkv // 128),
                          page_indices=torch.arange(b * (lkv // 128), device=dev, dtype=torch.int32))
        return fp4_block_scores_varlen(inputs["q"], inputs["k"], inputs["q_scale"], inputs["k_scale"], inputs["cu_q"],
                                       inputs["cu_k"], inputs["cu_pages"], max_seqlen_q=lq, max_seqlen_k=lkv,
                                       kv_indices=inputs["page_indices"], exact=False)
    scores = torch.empty((h, lkv // 128, b * lq), dtype=torch.float32, device=inputs["q"].device)
    with torch.cuda.device(scores.device):
        _lib.check(_lib.lib().sparse_b200_fp4_scores(
            _lib.ptr(inputs["q"]), _lib.ptr(inputs["q_scale"]), _lib.ptr(inputs["k"]), _lib.ptr(inputs["k_scale"]),
            _lib.ptr(scores), None, b, h, inputs["hk"], lq, lkv, _lib.current_stream()))
    return scores


def fp4_block_scores_varlen(q_fp4, k_fp4, q_scale, k_scale, cu_seqlens_q, cu_seqlens_k, cu_page_offsets, *,
                            max_seqlen_q, max_seqlen_k, kv_indices, causal=False, qo_offset=None, exact=True):
    """Ragged batch over a paged key cache, optionally causal: fp32 [Hq, ceil(max_seqlen_k/128), total_q]
    (max over the visible keys of each page, -inf where none), the public-layout form of
    fp4_indexer_block_scores (indexers/fp4/vendor_minimax_msa/fp4_indexer_interface.py:745-811).
    exact=True: canonical group-ordered arithmetic (bit-reproducible); exact=False: straight off the NVFP4
    tensor cores, as the reference's scorer (finite scores within its gate tolerance of the exact ones)."""
    if q_fp4.ndim != 3 or q_fp4.shape[2] != 64 or k_fp4.ndim != 4 or tuple(k_fp4.shape[2:]) != (128, 64):
        raise ValueError("q_fp4 must be [total_q,Hq,64] and k_fp4 [total_pages,Hk,128,64]")
    total_q, hq = int(q_fp4.shape[0]), int(q_fp4.shape[1])
    total_pages, hk = int(k_fp4.shape[0]), int(k_fp4.shape[1])
    if hq % hk:
        raise ValueError("num_qo_heads must be divisible by num_kv_heads")
    if qo_offset is not None and not causal:
        raise ValueError("qo_offset is only valid when causal=True")
    batch = int(cu_seqlens_q.numel()) - 1
    dev = q_fp4.device
    checks = (("q_fp4", q_fp4, torch.uint8, None), ("k_fp4", k_fp4, torch.uint8, None),
              ("q_scale", q_scale, torch.float8_e4m3fn, (total_q, hq, 8)),
              ("k_scale", k_scale, torch.float8_e4m3fn, (total_pages, hk, 128, 8)),
              ("cu_seqlens_q", cu_seqlens_q, torch.int32, (batch + 1,)),
              ("cu_seqlens_k", cu_seqlens_k, torch.int32, (batch + 1,)),
              ("cu_page_offsets", cu_page_offsets, torch.int32, (batch + 1,)),
              ("kv_indices", kv_indices, torch.int32, None)) + \
        ((("qo_offset", qo_offset, torch.int32, (batch,)),) if qo_offset is not None else ())
    for name, t, dtype, shape in checks:
        if not t.is_cuda or t.device != dev or t.dtype != dtype or not t.is_contiguous() \
                or (shape is not None and tuple(t.shape) != shape):
            raise ValueError(f"{name} must be a contiguous {dtype} CUDA tensor" + (f" of shape {shape}" if shape else ""))
    tiles = (int(max_seqlen_k) + 127) // 128
    scores = torch.empty((hq, tiles, total_q), dtype=torch.float32, device=dev)
    entry = _lib.lib().sparse_b200_fp4_scores_varlen if exact else _lib.lib().sparse_b200_fp4_scores_varlen_fast
    with torch.cuda.device(dev):
        _lib.check(entry(
            _lib.ptr(q_fp4), _lib.ptr(q_scale), _lib.ptr(k_fp4), _lib.ptr(k_scale), _lib.ptr(cu_seqlens_q),
            _lib.ptr(cu_seqlens_k), _lib.ptr(cu_page_offsets), _lib.ptr(kv_indices), _lib.ptr(qo_offset),
            _lib.ptr(scores), batch, hq, hk, total_q, total_pages, int(max_seqlen_q), int(max_seqlen_k),
            int(bool(causal)), _lib.current_stream()))
    return scores


def tile_topk_out(scores, selected, *, batch_size, len_q):
    if not (scores.is_cuda and scores.dtype == torch.float32 and scores.is_contiguous() and scores.ndim == 3):
        raise _lib.SparseB200Error("scores must be contiguous float32 [Hkv,KV_tiles,B*Sq] on CUDA")
    heads, tiles, total = scores.shape
    if batch_size <= 0 or len_q <= 0 or len_q % 128 or total != batch_size * len_q:
        raise _lib.SparseB200Error("B*Sq must match the score matrix; Sq a positive multiple of 128")
    topk = int(selected.shape[-1])
    if selected.dtype != torch.int32 or not selected.is_contiguous() \
            or tuple(selected.shape) != (batch_size, heads, len_q // 128, topk) or selected.device != scores.device:
        raise _lib.SparseB200Error("selected must be contiguous int32 [B,Hkv,Sq/128,TopK] on the scores' device")
    with torch.cuda.device(scores.device):
        _lib.check(_lib.lib().sparse_b200_tile_topk(_lib.ptr(scores), _lib.ptr(selected), batch_size, heads, len_q,
                                                    tiles, topk, _lib.current_stream()))
    return selected


def tile_topk(scores, *, batch_size, len_q, topk=16):
    selected = torch.empty((batch_size, scores.shape[0], len_q // 128, topk), dtype=torch.int32,
                           device=scores.device)
    return tile_topk_out(scores, selected, batch_size=batch_size, len_q=len_q)


def fp4_indexer(inputs, selected=None, topk=16, tile_scores=None):
    """Scoring + max over the query tile + top-k; only ids (and tile scores) touch memory."""
    b, h, lq, lkv = inputs["batch_size"], inputs["hkv"], inputs["len_q"], inputs["len_kv"]
    dev = inputs["q"].device
    if selected is None:
        selected = torch.empty((b, h, lq // 128, topk), dtype=torch.int32, device=dev)
    if tile_scores is None:
        tile_scores = torch.empty((b, h, lq // 128, lkv // 128), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().sparse_b200_indexer_fp4(
            _lib.ptr(inputs["q"]), _lib.ptr(inputs["q_scale"]), _lib.ptr(inputs["k"]), _lib.ptr(inputs["k_scale"]),
            _lib.ptr(tile_scores), _lib.ptr(selected), b, h, inputs["hk"], lq, lkv, int(selected.shape[-1]),
            _lib.current_stream()))
    return selected


def fp4_indexer_fast(inputs, selected=None, topk=16, workspace=None):
    """Same ids as fp4_indexer through the NVFP4 tensor-core pre-filter + exact re-scoring.
    Returns (selected, workspace); the int32 words 1 and 3 of the workspace count the tiles that took
    the exact path and the violations of the error bound since the workspace was zeroed."""
    b, h, lq, lkv = inputs["batch_size"], inputs["hkv"], inputs["len_q"], inputs["len_kv"]
    dev = inputs["q"].device
    L = _lib.lib()
    L.sparse_b200_indexer_fp4_workspace_bytes.restype = ctypes.c_int64
    need = L.sparse_b200_indexer_fp4_workspace_bytes(b, h, inputs["hk"], lq, lkv)
    if workspace is None:
        workspace = torch.zeros(need, dtype=torch.uint8, device=dev)    # its leading counters accumulate over calls
    if selected is None:
        selected = torch.empty((b, h, lq // 128, topk), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(L.sparse_b200_indexer_fp4_fast(
            _lib.ptr(inputs["q"]), _lib.ptr(inputs["q_scale"]), _lib.ptr(inputs["k"]), _lib.ptr(inputs["k_scale"]),
            _lib.ptr(workspace), ctypes.c_int64(workspace.numel()), _lib.ptr(selected), b, h, inputs["hk"], lq, lkv,
            int(selected.shape[-1]), _lib.current_stream()))
    return selected, workspace


class Fp4Pipeline:
    """quantise -> NVFP4 tensor-core indexer -> top-k -> Q-centric attention as ONE C call on the
    current stream, every buffer owned here and reused (nothing is allocated per call; capturable
    in a CUDA graph after one eager call). One index head per KV head: the index vector of a
    (token, KV head) is the NVFP4 of the mean of the group's query heads.
    inputs=None: q and k are quantised inside every run(); inputs=<prepare_fp4_inputs bundle>: the
    prepared codes are used as they are (the reference's timing, indexers/fp4/pipeline.py:49-65)."""

    def __init__(self, q, k, v, topk=16, inputs=None):
        b, hq, sq, _ = q.shape
        hkv, skv = k.shape[1:3]
        dev = q.device
        self.q, self.k, self.v, self.topk = q, k, v, int(topk)
        self.dims = (b, hq, hkv, sq, skv)
        if inputs is None:
            self.quantize = 1
            self.qc = torch.empty((b * sq, hkv, 64), dtype=torch.uint8, device=dev)
            self.qs = torch.empty((b * sq, hkv, 8), dtype=torch.float8_e4m3fn, device=dev)
            self.kc = torch.empty((b * skv // 128, hkv, 128, 64), dtype=torch.uint8, device=dev)
            self.ks = torch.empty((b * skv // 128, hkv, 128, 8), dtype=torch.float8_e4m3fn, device=dev)
        else:
            if inputs["batch_size"] != b or inputs["hkv"] != hkv or inputs["hk"] != hkv or inputs["len_q"] != sq \
                    or inputs["len_kv"] != skv:
                raise ValueError("indexer inputs must match attention shapes (one index head per KV head)")
            self.quantize = 0
            self.qc, self.qs, self.kc, self.ks = inputs["q"], inputs["q_scale"], inputs["k"], inputs["k_scale"]
        L = _lib.lib()
        L.sparse_b200_indexer_fp4_workspace_bytes.restype = ctypes.c_int64
        self.ws = torch.zeros(L.sparse_b200_indexer_fp4_workspace_bytes(b, hkv, hkv, sq, skv), dtype=torch.uint8, device=dev)
        self.ids = torch.empty((b, hkv, sq // 128, self.topk), dtype=torch.int32, device=dev)

    def run(self, out, lse=None):
        b, hq, hkv, sq, skv = self.dims
        with torch.cuda.device(self.q.device):
            _lib.check(_lib.lib().sparse_b200_indexed_attention_fp4(
                _lib.ptr(self.q), _lib.ptr(self.k), _lib.ptr(self.v), _lib.ptr(self.qc), _lib.ptr(self.qs),
                _lib.ptr(self.kc), _lib.ptr(self.ks), _lib.ptr(self.ws), ctypes.c_int64(self.ws.numel()),
                _lib.ptr(self.ids), _lib.ptr(out), _lib.ptr(lse), b, hq, hkv, sq, skv, self.topk, self.quantize,
                _lib.current_stream()))
        return out

    def stats(self):
        """(tiles that took the exact path, bound violations, largest |tensor-core - exact| / bound)
        of the last run (synchronising)."""
        w = self.ws[:20].cpu()
        return int(w[4:8].view(torch.int32)), int(w[12:16].view(torch.int32)), float(w[16:20].view(torch.float32))


def indexed_attention(q, k, v, inputs, topk=16):
    """(O, selected): NVFP4 tensor-core indexer then Q-centric attention on the same stream, one C call
    (indexers/fp4/pipeline.py:49-65)."""
    pipe = Fp4Pipeline(q, k, v, topk=topk, inputs=inputs)
    out = torch.empty_like(q)
    pipe.run(out)
    return out, pipe.ids
