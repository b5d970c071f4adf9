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


class PreparedTokens:
    """Per-TOKEN selections, the reference's own contract (api11.py:50-92, gpu_plan.py:19-45):
    q [B,Hq,Sq,128], k/v [B,Hkv,Skv,128] bf16, selected [B,Hkv,Sq,TopK] int32 (CUDA), any TopK.
    metadata() builds the reverse index and the task list on the GPU, main() writes one
    normalised partial per (query, head, rank), combine() merges the TopK partials.
    q_token_major=True: q is [B,Sq,Hq,128], the layout of the reference's TMA variants (groups of
    8 or 16 heads only); outputs stay head-major. partial_f32=True keeps the partials in fp32 (the
    reference's control variants -2 and 0, api11.py:22-25) instead of bf16."""

    def __init__(self, q, k, v, selected, q_token_major=False, partial_token_major=False, partial_f32=False):
        import ctypes
        if not (q.is_cuda and q.dtype == torch.bfloat16 and q.is_contiguous() and q.dim() == 4 and q.shape[3] == 128):
            raise _lib.SparseB200Error("q must be contiguous bf16 [B,Hq,Sq,128] (or [B,Sq,Hq,128]) on CUDA")
        self.q_token_major = bool(q_token_major)
        # partials [B,Sq,TopK,Hq,128] as the reference's main_tm_out writes them (needs q token-major too)
        self.partial_token_major = bool(partial_token_major)
        self.partial_f32 = bool(partial_f32)
        if self.partial_token_major and not self.q_token_major:
            raise _lib.SparseB200Error("token-major partials go with token-major q")
        q_arg = q
        if self.q_token_major:
            q = q.permute(0, 2, 1, 3)          # a head-major VIEW for the shape checks below; q_arg is what runs
        for t in (k, v):
            if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and t.dim() == 4
                    and t.shape[3] == 128 and t.device == q.device):
                raise _lib.SparseB200Error("k and v must be contiguous bf16 [B,Hkv,Skv,128] on q's device")
        b, hq, sq, d = q.shape
        hkv, skv = k.shape[1:3]
        if k.shape != v.shape or k.shape[0] != b or hq % hkv or skv % 128:
            raise _lib.SparseB200Error("QKV/GQA geometry")
        if selected.dtype != torch.int32 or not selected.is_contiguous() or selected.device != q.device \
                or selected.dim() != 4 or tuple(selected.shape[:3]) != (b, hkv, sq):
            raise _lib.SparseB200Error("selected must be contiguous int32 [B,Hkv,Sq,TopK] on q's device")
        if self.q_token_major and hq // hkv not in (8, 16):
            raise _lib.SparseB200Error("the token-major layout needs Hq/Hkv of 8 or 16")
        self.q, self.k, self.v, self.selected = q_arg, k, v, selected
        self.b, self.hq, self.hkv, self.sq, self.skv = b, hq, hkv, sq, skv
        self.g, self.topk, self.kv_blocks = hq // hkv, int(selected.shape[3]), skv // 128
        self.rows = b * hkv * self.kv_blocks
        self.edges = selected.numel()
        L = _lib.lib()
        L.sparse_b200_kv_token_max_tasks.restype = ctypes.c_int64
        self.max_tasks = int(L.sparse_b200_kv_token_max_tasks(b, hkv, sq, self.topk, self.kv_blocks, self.g))
        if self.max_tasks <= 0:
            raise _lib.SparseB200Error("invalid routing geometry")
        dev = q.device

        def ints(n):
            return torch.empty(n, device=dev, dtype=torch.int32)
        self.counts, self.cursors = ints(self.rows + 1), ints(self.rows + 1)
        self.row_ptr, self.task_ptr = ints(self.rows + 1), ints(self.rows + 1)
        self.qids, self.ranks = ints(self.edges), ints(self.edges)
        self.tasks = torch.zeros((self.max_tasks, 4), device=dev, dtype=torch.int32)
        self.error = ints(1)
        self.partial = torch.empty((b, sq, self.topk, hq, d) if self.partial_token_major else (b, hq, sq, self.topk, d),
                                   device=dev, dtype=torch.float32 if self.partial_f32 else torch.bfloat16)
        self.lses = torch.empty((b, hq, sq, self.topk), device=dev, dtype=torch.float32)
        self.out = torch.empty((b, hq, sq, d), device=dev, dtype=torch.bfloat16)
        self.out_lse = torch.empty((b, hq, sq), device=dev, dtype=torch.float32)

    def poison(self):
        for t in (self.partial, self.lses, self.out, self.out_lse):
            t.fill_(float("nan"))

    def metadata(self):
        with torch.cuda.device(self.q.device):
            _lib.check(_lib.lib().sparse_b200_kv_token_metadata(
                _lib.ptr(self.selected), _lib.ptr(self.counts), _lib.ptr(self.cursors), _lib.ptr(self.row_ptr),
                _lib.ptr(self.qids), _lib.ptr(self.ranks), _lib.ptr(self.task_ptr), _lib.ptr(self.tasks),
                _lib.ptr(self.error), self.b, self.hkv, self.sq, self.topk, self.kv_blocks, self.g,
                _lib.current_stream()))

    def main(self):
        with torch.cuda.device(self.q.device):
            layout = int(self.q_token_major) | int(self.partial_token_major) << 1 | int(self.partial_f32) << 2
            _lib.check(_lib.lib().sparse_b200_kv_token_main_layout(
                _lib.ptr(self.q), _lib.ptr(self.k), _lib.ptr(self.v), _lib.ptr(self.tasks), _lib.ptr(self.task_ptr),
                _lib.ptr(self.qids), _lib.ptr(self.ranks), _lib.ptr(self.partial), _lib.ptr(self.lses),
                self.b, self.hq, self.hkv, self.sq, self.skv, self.topk, layout, _lib.current_stream()))

    def combine(self):
        import ctypes
        with torch.cuda.device(self.q.device):
            if self.partial_token_major:
                _lib.check(_lib.lib().sparse_b200_combine_tm(
                    _lib.ptr(self.partial), int(self.partial_f32), _lib.ptr(self.lses), _lib.ptr(self.out),
                    _lib.ptr(self.out_lse), self.b, self.hq, self.sq, self.topk, _lib.current_stream()))
                return
            _lib.check(_lib.lib().sparse_b200_combine(
                _lib.ptr(self.partial), int(self.partial_f32), _lib.ptr(self.lses), _lib.ptr(self.out),
                _lib.ptr(self.out_lse), ctypes.c_int64(self.out_lse.numel()), self.topk, 0, _lib.current_stream()))

    def core(self):
        self.main()
        self.combine()

    def run(self):
        self.metadata()
        self.core()
        return self.out, self.out_lse

    def plan(self):
        """Host copy of the device plan (synchronising; tests compare it with the CPU builder)."""
        status = int(self.error.item())
        if status:
            raise ValueError(f"GPU selected validation failed: flag={status} (1 = id out of range)")
        ntasks = int(self.task_ptr[-1].item())
        return {"row_ptr": self.row_ptr.cpu(), "query_ids": self.qids.cpu(), "ranks": self.ranks.cpu(),
                "tasks": self.tasks[:ntasks].cpu()}


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
