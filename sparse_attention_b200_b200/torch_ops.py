"""The reference's torch operator names, served by libsparse_b200.so.

`register()` defines the operator libraries the reference's Python loaders look for, so that its
own modules pick these kernels up unchanged (its loaders build their extension only when the
operator is not registered yet, attention/q_centric/progression.py:29-36):

  xomtention_progression::attention / attention_out
      (attention/q_centric/progression_attention.cpp:19-125; `variant` selects nothing here: one kernel)
  xomtention_tile_topk::tile_topk / tile_topk_out
      (indexers/fp4/wrapper.cpp:16-80; 16 ids per list as there)
  xomtention_kvopt11::metadata_temp_bytes / metadata_out / main_out / combine_out / main_tm_out /
      combine_tm_out (attention/kv_centric/optimization_round11/wrapper11.cpp:29-171): the head-major
      chain (variants -2 = fp32 partials, -1 = bf16) and the token-major pair (variants 0 = fp32
      partials, 1 and 2 = bf16; Hq/Hkv of 8 or 16). metadata_out takes the reference's chunk sizes; the
      main kernels always work on tasks of at most 128 / group_size queries, which metadata_out keeps
      in storage of its own next to the grouped list it hands back.

Each operator validates like the reference (RuntimeError on rejected inputs), runs on the current
CUDA stream of the tensors' device, allocates only where the reference's does (`attention`,
`tile_topk`), and is capturable in a CUDA graph. Nothing here is needed by the package itself.
"""
import ctypes

import torch

from . import _lib
from .q_centric import attention as _attention, attention_out as _attention_out
from .indexers import tile_topk_out as _tile_topk_out

_REGISTERED = {}


def _fail(msg):
    raise _lib.SparseB200Error(msg)


def _register_progression():
    lib = torch.library.Library("xomtention_progression", "DEF")
    lib.define("attention(Tensor q, Tensor k, Tensor v, Tensor selected_indices, int variant) -> Tensor")
    lib.define("attention_out(Tensor q, Tensor k, Tensor v, Tensor selected_indices, Tensor(a!) output, int variant) -> ()")

    def attention(q, k, v, selected_indices, variant):
        return _attention(q, k, v, selected_indices)

    def attention_out(q, k, v, selected_indices, output, variant):
        _attention_out(q, k, v, selected_indices, output)

    lib.impl("attention", attention, "CUDA")
    lib.impl("attention_out", attention_out, "CUDA")
    return lib


def _register_tile_topk():
    lib = torch.library.Library("xomtention_tile_topk", "DEF")
    lib.define("tile_topk(Tensor scores, int batch_size, int len_q) -> Tensor")
    lib.define("tile_topk_out(Tensor scores, Tensor(a!) selected, int batch_size, int len_q) -> ()")

    def tile_topk(scores, batch_size, len_q):
        if scores.dim() != 3 or len_q <= 0 or len_q % 128:
            _fail("scores must be contiguous [Hkv, KV_tiles, B*Sq]; len_q a positive multiple of 128")
        selected = torch.empty((batch_size, scores.shape[0], len_q // 128, 16), dtype=torch.int32, device=scores.device)
        return _tile_topk_out(scores, selected, batch_size=batch_size, len_q=len_q)

    def tile_topk_out(scores, selected, batch_size, len_q):
        if selected.dim() != 4 or selected.shape[-1] != 16:
            _fail("selected must have shape [B, Hkv, Sq/128, 16]")
        if selected.untyped_storage().data_ptr() == scores.untyped_storage().data_ptr():
            _fail("selected must not alias scores")
        _tile_topk_out(scores, selected, batch_size=batch_size, len_q=len_q)

    lib.impl("tile_topk", tile_topk, "CUDA")
    lib.impl("tile_topk_out", tile_topk_out, "CUDA")
    return lib


def _ints(anchor, *tensors):
    for t in tensors:
        if not (t.is_cuda and t.device == anchor.device and t.dtype == torch.int32 and t.is_contiguous()) \
                or t.requires_grad:
            _fail("same CUDA device, int32 and contiguous layout required")


def _register_kvopt11():
    lib = torch.library.Library("xomtention_kvopt11", "DEF")
    lib.define("metadata_temp_bytes(int rows) -> int")
    lib.define("metadata_out(Tensor selected, Tensor(a!) counts, Tensor(b!) row_ptr, Tensor(c!) cursors, "
               "Tensor(d!) qids, Tensor(e!) ranks, Tensor(f!) chunks, Tensor(g!) task_ptr, Tensor(h!) tasks, "
               "Tensor(i!) error, Tensor(j!) temp, int kv_blocks, int group_size, int chunk_size) -> ()")
    lib.define("main_out(Tensor q, Tensor k, Tensor v, Tensor tasks, Tensor qids, Tensor ranks, Tensor(a!) partial, "
               "Tensor(b!) lses, int variant) -> ()")
    lib.define("combine_out(Tensor partial, Tensor lses, Tensor(a!) out, Tensor(b!) out_lse) -> ()")
    lib.define("main_tm_out(Tensor q, Tensor k, Tensor v, Tensor tasks, Tensor qids, Tensor ranks, Tensor(a!) partial, "
               "Tensor(b!) lses, int variant) -> ()")
    lib.define("combine_tm_out(Tensor partial, Tensor lses, Tensor(a!) out, Tensor(b!) out_lse) -> ()")
    # the task count travels from metadata_out to main_out on the device: task_ptr[rows] of the last build
    state = {}
    private = {}

    def metadata_temp_bytes(rows):
        if not 0 < rows < 2 ** 31 - 2:
            _fail("metadata row count")
        return 16                     # no scratch is used; a token size keeps callers' allocation code unchanged

    def metadata_out(selected, counts, row_ptr, cursors, qids, ranks, chunks, task_ptr, tasks, error, temp,
                     kv_blocks, group_size, chunk_size):
        _ints(selected, selected, counts, row_ptr, cursors, qids, ranks, chunks, task_ptr, tasks, error)
        if selected.dim() != 4:
            _fail("selected [B,Hkv,Sq,TopK]")
        if chunk_size not in (1, 4, 8, 16) or group_size not in (1, 2, 4, 8, 16):
            _fail("invalid routing geometry")
        b, hkv, sq, topk = selected.shape
        rows = b * hkv * kv_blocks
        for t in (counts, row_ptr, chunks, task_ptr):
            if t.dim() != 1 or t.numel() != rows + 1:
                _fail("scan buffers must hold rows + 1 ints")
        if cursors.numel() < rows or qids.numel() != selected.numel() or ranks.shape != qids.shape or error.numel() != 1:
            _fail("cursors / edge storage / status shapes")
        L = _lib.lib()
        L.sparse_b200_kv_token_max_tasks.restype = ctypes.c_int64
        bound = L.sparse_b200_kv_token_max_tasks(b, hkv, sq, topk, kv_blocks, group_size)
        cap = 128 // group_size * chunk_size
        edges = selected.numel()
        if tasks.dim() != 2 or tasks.shape[1] != 4 or tasks.shape[0] < min(edges, -(-edges // cap) + rows):
            _fail("bounded tasks: [min(E, ceil(E / (128 / group_size * chunk_size)) + rows), 4]")
        # The kernels of this library take tasks of at most 128 / group_size queries. With a larger chunk_size
        # that list lives in storage of the shim (allocated once per geometry), and the caller's tensors get the
        # grouped list the reference's planner would have written (same edges, tasks of up to chunk_size times as
        # many queries), which its audit reads.
        own = chunk_size == 1
        key = (selected.device, rows, int(bound))
        if own:
            run_tasks, run_task_ptr = tasks, task_ptr
        else:
            if key not in private:
                private[key] = (torch.zeros((int(bound), 4), dtype=torch.int32, device=selected.device),
                                torch.empty(rows + 1, dtype=torch.int32, device=selected.device))
            run_tasks, run_task_ptr = private[key]
        # counts / cursors are scratch of rows + 1 ints in the C ABI: `chunks` serves as the cursors
        with torch.cuda.device(selected.device):
            _lib.check(L.sparse_b200_kv_token_metadata(
                _lib.ptr(selected), _lib.ptr(counts), _lib.ptr(chunks), _lib.ptr(row_ptr), _lib.ptr(qids), _lib.ptr(ranks),
                _lib.ptr(run_task_ptr), _lib.ptr(run_tasks), _lib.ptr(error), b, hkv, sq, topk, kv_blocks, group_size,
                _lib.current_stream()))
            if not own:                          # grouped list for the caller, on the device, no synchronisation
                per_row = row_ptr[1:] - row_ptr[:-1]
                n_tasks = (per_row + (cap - 1)) // cap
                ends = torch.cumsum(n_tasks, 0)
                task_ptr[0] = 0
                task_ptr[1:] = ends
                chunks.copy_(task_ptr)
                t = torch.arange(tasks.shape[0], device=selected.device, dtype=torch.int64)
                row = torch.searchsorted(ends.to(torch.int64), t, right=True).clamp_(max=rows - 1)
                local = t - (ends[row].to(torch.int64) - n_tasks[row].to(torch.int64))
                valid = (t < ends[-1].to(torch.int64)).to(torch.int32)
                start = row_ptr[row].to(torch.int64) + local * cap
                count = torch.minimum(per_row[row].to(torch.int64) - local * cap, torch.full_like(local, cap))
                tasks.copy_(torch.stack([row // kv_blocks, row % kv_blocks, start, count], 1).to(torch.int32) * valid[:, None])
        state[tasks.data_ptr()] = (run_tasks, run_task_ptr)

    def main_out(q, k, v, tasks, qids, ranks, partial, lses, variant):
        # wrapper11.cpp:66-70: -2 = fp32 partials, -1 = bf16 partials
        if variant not in (-2, -1):
            _fail("main_out serves the head-major variants (-2, -1); the token-major ones use main_tm_out")
        f32 = variant == -2
        for t in (q, k, v):
            if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()) or t.requires_grad:
                _fail("q, k and v must be contiguous bf16 CUDA tensors (forward only)")
        if not (partial.is_cuda and partial.is_contiguous() and
                partial.dtype == (torch.float32 if f32 else torch.bfloat16)) or partial.requires_grad:
            _fail("partial must be a contiguous CUDA tensor of the variant's type (fp32 for -2, bf16 for -1)")
        _ints(q, tasks, qids, ranks)
        if q.dim() != 4 or k.dim() != 4 or k.shape != v.shape or q.shape[3] != 128 or k.shape[3] != 128:
            _fail("QKV rank/shape")
        b, hq, sq, _ = q.shape
        hkv, skv = k.shape[1:3]
        topk = qids.numel() // max(1, b * hkv * sq)
        if tuple(partial.shape) != (b, hq, sq, topk, 128) or tuple(lses.shape) != (b, hq, sq, topk) \
                or lses.dtype != torch.float32:
            _fail("partials must be [B,Hq,Sq,TopK,128] and [B,Hq,Sq,TopK] fp32")
        built = state.get(tasks.data_ptr())
        if built is None:
            _fail("main_out needs the task list of a preceding metadata_out on the same tasks tensor")
        run_tasks, task_ptr = built
        with torch.cuda.device(q.device):
            _lib.check(_lib.lib().sparse_b200_kv_token_main_layout(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(run_tasks), _lib.ptr(task_ptr), _lib.ptr(qids),
                _lib.ptr(ranks), _lib.ptr(partial), _lib.ptr(lses), b, hq, hkv, sq, skv, topk, 4 if f32 else 0,
                _lib.current_stream()))

    def combine_out(partial, lses, out, out_lse):
        if partial.dtype not in (torch.float32, torch.bfloat16) or not partial.is_contiguous() or not lses.is_contiguous():
            _fail("partial dtype / layout")
        if out.dim() != 4 or out.shape[3] != 128 or tuple(out_lse.shape) != tuple(out.shape[:3]) \
                or out.dtype != torch.bfloat16 or out_lse.dtype != torch.float32:
            _fail("output")
        ranks = partial.shape[-2]
        if tuple(partial.shape) != (*out.shape[:3], ranks, 128) or tuple(lses.shape) != (*out.shape[:3], ranks):
            _fail("Combine input")
        with torch.cuda.device(out.device):
            _lib.check(_lib.lib().sparse_b200_combine(
                _lib.ptr(partial), int(partial.dtype == torch.float32), _lib.ptr(lses), _lib.ptr(out), _lib.ptr(out_lse),
                ctypes.c_int64(out_lse.numel()), ranks, 0, _lib.current_stream()))

    def main_tm_out(q, k, v, tasks, qids, ranks, partial, lses, variant):
        # wrapper11.cpp:94-118: q [B,Sq,Hq,128], partial [B,Sq,TopK,Hq,128], lses [B,Hq,Sq,TopK]; variant 0 has
        # fp32 partials, 1 and 2 bf16 ones
        if variant not in (0, 1, 2):
            _fail("main_tm_out serves the token-major variants (0, 1, 2)")
        f32 = variant == 0
        for t in (q, k, v):
            if not (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()) or t.requires_grad:
                _fail("q, k and v must be contiguous bf16 CUDA tensors (forward only)")
        if not (partial.is_cuda and partial.is_contiguous() and
                partial.dtype == (torch.float32 if f32 else torch.bfloat16)) or partial.requires_grad:
            _fail("partial must be a contiguous CUDA tensor of the variant's type (fp32 for 0, bf16 for 1 and 2)")
        _ints(q, tasks, qids, ranks)
        if q.dim() != 4 or k.dim() != 4 or k.shape != v.shape or q.shape[3] != 128 or k.shape[3] != 128:
            _fail("QKV rank/shape")
        b, sq, hq, _ = q.shape
        hkv, skv = k.shape[1:3]
        if hkv <= 0 or hq % hkv or hq // hkv not in (8, 16):
            _fail("GQA ratio (the token-major operators serve Hq/Hkv of 8 and 16)")
        topk = qids.numel() // max(1, b * hkv * sq)
        if tuple(partial.shape) != (b, sq, topk, hq, 128) or tuple(lses.shape) != (b, hq, sq, topk) \
                or lses.dtype != torch.float32:
            _fail("token-major partials")
        built = state.get(tasks.data_ptr())
        if built is None:
            _fail("main_tm_out needs the task list of a preceding metadata_out on the same tasks tensor")
        run_tasks, task_ptr = built
        with torch.cuda.device(q.device):
            _lib.check(_lib.lib().sparse_b200_kv_token_main_layout(
                _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(run_tasks), _lib.ptr(task_ptr), _lib.ptr(qids),
                _lib.ptr(ranks), _lib.ptr(partial), _lib.ptr(lses), b, hq, hkv, sq, skv, topk, 7 if f32 else 3,
                _lib.current_stream()))

    def combine_tm_out(partial, lses, out, out_lse):
        if partial.dtype not in (torch.float32, torch.bfloat16) or not partial.is_contiguous() or not lses.is_contiguous():
            _fail("partial dtype / layout")
        if out.dim() != 4 or out.shape[3] != 128 or tuple(out_lse.shape) != tuple(out.shape[:3]) \
                or out.dtype != torch.bfloat16 or out_lse.dtype != torch.float32:
            _fail("output")
        b, h, s, _ = out.shape
        ranks = lses.shape[-1]
        if tuple(partial.shape) != (b, s, ranks, h, 128) or tuple(lses.shape) != (b, h, s, ranks):
            _fail("token-major Combine input")
        with torch.cuda.device(out.device):
            _lib.check(_lib.lib().sparse_b200_combine_tm(
                _lib.ptr(partial), int(partial.dtype == torch.float32), _lib.ptr(lses), _lib.ptr(out), _lib.ptr(out_lse),
                b, h, s, ranks, _lib.current_stream()))

    lib.impl("metadata_temp_bytes", metadata_temp_bytes, "CompositeExplicitAutograd")
    lib.impl("metadata_out", metadata_out, "CUDA")
    lib.impl("main_out", main_out, "CUDA")
    lib.impl("combine_out", combine_out, "CUDA")
    lib.impl("main_tm_out", main_tm_out, "CUDA")
    lib.impl("combine_tm_out", combine_tm_out, "CUDA")
    return lib


_BUILDERS = {"xomtention_progression": _register_progression, "xomtention_tile_topk": _register_tile_topk,
             "xomtention_kvopt11": _register_kvopt11}


def register(namespaces=tuple(_BUILDERS)):
    """Defines the operator libraries (once per process). Fails if a namespace is already defined,
    e.g. by the reference's own extension loaded into the same process."""
    for name in namespaces:
        if name not in _REGISTERED:
            _REGISTERED[name] = _BUILDERS[name]()
    return {name: getattr(torch.ops, name) for name in namespaces}
