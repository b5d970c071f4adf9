"""Host-side mirror of the reference Q-centric operator
(attention/q_centric/progression.py:40-46 `stage_functions`,
attention/q_centric/progression_attention.cpp:19-125 `attention` / `attention_out`),
bound to the C ABI. Same argument meaning and the same rejected inputs; adds
the optional `counts` and `lse` arguments."""
import ctypes

import torch

from . import _lib


def _validate(q, k, v, ids, out=None, counts=None, lse=None):
    def bad(msg):
        raise _lib.SparseB200Error(msg)
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        bad("q, k, and v must be CUDA tensors")
    if not (q.device == k.device == v.device):
        bad("q, k, and v must be on the same CUDA device")
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        bad("q, k, and v must be bfloat16")
    if q.requires_grad or k.requires_grad or v.requires_grad:
        bad("This attention implementation is forward-only")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        bad("q, k, and v must be contiguous")
    if not (q.dim() == 4 and k.dim() == 4 and v.dim() == 4):
        bad("q must be [B,Hq,Sq,128], k/v must be [B,Hkv,Skv,128]")
    if not (q.shape[0] == k.shape[0] == v.shape[0]) or k.shape[1] != v.shape[1] or k.shape[2] != v.shape[2]:
        bad("q, k, and v batch / head / length dimensions must match")
    if q.shape[0] <= 0 or k.shape[1] <= 0:
        bad("batch and KV heads must be positive")
    if q.shape[1] < k.shape[1] or q.shape[1] % k.shape[1]:
        bad("Hq must be a multiple of and at least Hkv")
    if not (q.shape[3] == k.shape[3] == v.shape[3] == 128):
        bad("head dimension must be 128")
    if not (ids.is_cuda and ids.device == q.device and ids.dtype == torch.int32 and ids.is_contiguous()):
        bad("selected_indices must be a contiguous int32 CUDA tensor on q's device")
    if ids.dim() != 4 or ids.shape[0] != q.shape[0] or ids.shape[1] != k.shape[1] \
            or ids.shape[2] * 128 != q.shape[2]:
        bad("selected_indices must be [B,Hkv,Sq/128,TopK]")
    if out is not None:
        if not (out.is_cuda and out.device == q.device and out.dtype == q.dtype
                and out.shape == q.shape and out.is_contiguous()):
            bad("output must match q shape, dtype, device, and contiguous layout")
        for t in (q, k, v, ids):
            if out.untyped_storage().data_ptr() == t.untyped_storage().data_ptr():
                bad("output must not alias inputs")
    if counts is not None and not (counts.is_cuda and counts.dtype == torch.int32 and counts.is_contiguous()
                                   and tuple(counts.shape) == tuple(ids.shape[:3])):
        bad("block counts must be contiguous int32 [B,Hkv,Sq/128] on q's device")
    if lse is not None and not (lse.is_cuda and lse.dtype == torch.float32 and lse.is_contiguous()
                                and tuple(lse.shape) == tuple(q.shape[:3])):
        bad("lse must be contiguous float32 [B,Hq,Sq] on q's device")


_WORKSPACES = {}


def _workspace(device):
    """Scratch of the balanced last round, one per (device, stream): allocated at the first call."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None:
        import ctypes
        fn = _lib.lib().sparse_b200_q_centric_workspace_bytes
        fn.restype = ctypes.c_int64
        with torch.cuda.device(device):
            ws = torch.empty(int(fn()), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def attention_out(q, k, v, ids, out, counts=None, lse=None, balance=True):
    """out <- block-sparse attention on the current stream. balance: let the kernel split the work items of a
    last, partly filled round (a per-stream scratch buffer is allocated at the first call; no allocation
    afterwards); False is the plain entry, which never allocates."""
    _validate(q, k, v, ids, out, counts, lse)
    b, hq, sq, _ = q.shape
    hkv, skv = k.shape[1:3]
    with torch.cuda.device(q.device):
        if not balance:
            _lib.check(_lib.lib().sparse_b200_q_centric(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ids), _lib.ptr(counts), _lib.ptr(out), _lib.ptr(lse),
                b, hq, hkv, sq, skv, int(ids.shape[3]), _lib.current_stream()))
            return
        import ctypes
        ws = _workspace(q.device)
        _lib.check(_lib.lib().sparse_b200_q_centric_ws(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ids), _lib.ptr(counts), _lib.ptr(out), _lib.ptr(lse),
            _lib.ptr(ws), ctypes.c_int64(ws.numel()), b, hq, hkv, sq, skv, int(ids.shape[3]), _lib.current_stream()))


def attention(q, k, v, ids, counts=None, return_lse=False):
    _validate(q, k, v, ids, None, counts)
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device) if return_lse else None
    attention_out(q, k, v, ids, out, counts, lse)
    return (out, lse) if return_lse else out


def attention_partial_out(q, k, v, seg_ids, seg_counts, partial, partial_lse):
    """KV-range-segmented lists -> partial (O, LSE) per segment (see kv_centric.py)."""
    nseg = seg_ids.shape[0]
    _validate(q, k, v, seg_ids[0])
    b, hq, sq, _ = q.shape
    hkv, skv = k.shape[1:3]
    if partial.dtype not in (torch.float32, torch.bfloat16) or tuple(partial.shape) != (nseg, b, hq, sq, 128):
        raise _lib.SparseB200Error("partial must be [nseg,B,Hq,Sq,128] float32 or bfloat16")
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().sparse_b200_q_centric_partial(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(seg_ids), _lib.ptr(seg_counts), _lib.ptr(partial),
            _lib.ptr(partial_lse), nseg, int(partial.dtype == torch.float32), b, hq, hkv, sq, skv,
            int(seg_ids.shape[-1]), _lib.current_stream()))


def stage_functions(version="b200"):
    """(attention, attention_out) pair, the shape of the reference's
    progression.stage_functions; every version name maps to the one kernel."""
    return attention, attention_out
