"""Host-side mirror of the reference KV-centric operator
(attention/kv_centric/optimization_round11/api11.py:50-92 `Prepared` with its
metadata() / main() / combine() / run() stages), bound to the C ABI.

Differences the block-list contract brings: selections are per query BLOCK
([B,Hkv,Sq/128,TopK], any TopK) and q stays head-major [B,Hq,Sq,128]; the
reverse index is by KV range (nseg ranges) instead of by single block, so the
partial buffers are nseg x the output instead of TopK x."""
import torch

from . import _lib
from .q_centric import _validate

PARTIAL_DTYPE = {"f32": torch.float32, "bf16": torch.bfloat16}


def default_segments(kv_blocks, topk):
    """Few ranges keep the partial traffic low; enough ranges keep a range's K/V in L2."""
    return max(1, min(4, kv_blocks, topk))


class Prepared:
    """q [B,Hq,Sq,128], k/v [B,Hkv,Skv,128] bf16, selected [B,Hkv,Sq/128,TopK] int32 (CUDA)."""

    def __init__(self, q, k, v, selected, counts=None, nseg=None, partial="bf16"):
        _validate(q, k, v, selected, None, counts)
        if partial not in PARTIAL_DTYPE:
            raise ValueError("partial must be 'f32' or 'bf16'")
        b, hq, sq, d = q.shape
        hkv, skv = k.shape[1:3]
        self.q, self.k, self.v, self.selected, self.counts = q, k, v, selected, counts
        self.topk = int(selected.shape[-1])
        self.kv_blocks = skv // 128
        self.nseg = default_segments(self.kv_blocks, self.topk) if nseg is None else int(nseg)
        if not 1 <= self.nseg <= self.kv_blocks:
            raise ValueError("nseg must be in [1, kv_blocks]")
        dev = q.device
        self.seg_ids = torch.empty((self.nseg, b, hkv, sq // 128, self.topk), dtype=torch.int32, device=dev)
        self.seg_counts = torch.empty((self.nseg, b, hkv, sq // 128), dtype=torch.int32, device=dev)
        self.error = torch.zeros(1, dtype=torch.int32, device=dev)
        self.partial = torch.empty((self.nseg, b, hq, sq, d), dtype=PARTIAL_DTYPE[partial], device=dev)
        self.lses = torch.empty((self.nseg, b, hq, sq), dtype=torch.float32, device=dev)
        self.out = torch.empty((b, hq, sq, d), dtype=torch.bfloat16, device=dev)
        self.out_lse = torch.empty((b, hq, sq), dtype=torch.float32, device=dev)

    def poison(self):
        for t in (self.partial, self.lses, self.out, self.out_lse):
            t.fill_(float("nan"))

    def metadata(self):
        b, hkv, qb, _ = self.selected.shape
        self.error.zero_()
        with torch.cuda.device(self.q.device):
            _lib.check(_lib.lib().sparse_b200_split_kv_segments(
                _lib.ptr(self.selected), _lib.ptr(self.counts), _lib.ptr(self.seg_ids), _lib.ptr(self.seg_counts),
                _lib.ptr(self.error), b, hkv, qb, self.topk, self.kv_blocks, self.nseg, _lib.current_stream()))

    def main(self):
        from .q_centric import attention_partial_out
        attention_partial_out(self.q, self.k, self.v, self.seg_ids, self.seg_counts, self.partial, self.lses)

    def combine(self):
        rows = self.out_lse.numel()
        with torch.cuda.device(self.q.device):
            _lib.check(_lib.lib().sparse_b200_combine(
                _lib.ptr(self.partial), int(self.partial.dtype == torch.float32), _lib.ptr(self.lses),
                _lib.ptr(self.out), _lib.ptr(self.out_lse), rows, self.nseg, 1, _lib.current_stream()))

    def core(self):
        self.main()
        self.combine()

    def run(self):
        self.metadata()
        self.core()
        return self.out, self.out_lse

    def audit(self):
        """Synchronous check of the id-range error word (tests only)."""
        status = int(self.error.item())
        if status:
            raise ValueError(f"selected validation failed on the GPU: flag={status} (1 = id out of range)")
        return {"segments": self.nseg, "edges": int(self.seg_counts.sum().item())}


def kv_centric_attention(q, k, v, selected, counts=None, nseg=None, partial="bf16", workspace=None):
    """One call through the fused C entry (metadata + main + combine, caller workspace)."""
    _validate(q, k, v, selected, None, counts)
    b, hq, sq, _ = q.shape
    hkv, skv = k.shape[1:3]
    topk = int(selected.shape[-1])
    nseg = default_segments(skv // 128, topk) if nseg is None else int(nseg)
    f32 = int(partial == "f32")
    L = _lib.lib()
    L.sparse_b200_kv_centric_workspace_bytes.restype = __import__("ctypes").c_int64
    need = L.sparse_b200_kv_centric_workspace_bytes(b, hq, hkv, sq, topk, nseg, f32)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    import ctypes
    with torch.cuda.device(q.device):
        _lib.check(L.sparse_b200_kv_centric(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(selected), _lib.ptr(counts), _lib.ptr(out), _lib.ptr(lse),
            _lib.ptr(workspace), ctypes.c_int64(workspace.numel()), nseg, f32, b, hq, hkv, sq, skv, topk,
            _lib.current_stream()))
    return out, lse


def combine(partial, lses):
    """Reference-layout merge: partial [..., R, 128], lses [..., R]
    (load_extension().combine of attention/kv_centric/validate_gpu.py:36)."""
    import ctypes
    ranks = partial.shape[-2]
    rows = lses.numel() // ranks
    out = torch.empty((*partial.shape[:-2], 128), dtype=torch.bfloat16, device=partial.device)
    lse = torch.empty(partial.shape[:-2], dtype=torch.float32, device=partial.device)
    partial, lses = partial.contiguous(), lses.contiguous()   # keep any copies alive across the call
    with torch.cuda.device(partial.device):
        _lib.check(_lib.lib().sparse_b200_combine(
            _lib.ptr(partial), int(partial.dtype == torch.float32), _lib.ptr(lses),
            _lib.ptr(out), _lib.ptr(lse), ctypes.c_int64(rows), ranks, 0, _lib.current_stream()))
    return out, lse
