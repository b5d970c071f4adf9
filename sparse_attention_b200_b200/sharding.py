"""Multi-GPU sharding of the hot path: one process per GPU, torch.distributed for the plumbing.

Two ways to shard (no TMA multicast anywhere; a peer's memory is touched only by this package's own kernels,
with plain loads and stores, in the `PeerExchange` forms below):

* by (batch, KV-head group): groups are independent in the indexer, in the
  attention kernel and in Combine, so ranks need no data-path collective
  (`group_range`, `group_view`);
* by KV range (long contexts): `kv_ranks` ranks share the same heads, each owns a
  contiguous range of KV blocks and the K/V rows of that range. A rank filters every
  selection list to its range, runs the same attention kernel and gets a normalised
  partial (O_r, L_r) for EVERY query; one exchange step then moves the slice of rows
  a rank owns from every peer into local memory (NCCL send/recv), and the local
  Combine kernel merges them by log-sum-exp (`KVSplit`); `KVSplit.run_pipelined` does it in chunks of head
  pairs, the exchange of one chunk under the attention of the next.

`PeerExchange` + `KVSplit.run_peer` are the fused form of that exchange + Combine on one machine: every
rank keeps its partial in memory the other ranks have mapped (CUDA IPC), flags tell when a partial is
complete, and the merge kernel reads the peers' rows with plain loads over NVLink (no copy step, no
NCCL call on the data path, no multicast; every cross-GPU wait is bounded). `KVSplit.run_scatter` goes one
step further: the attention kernel itself stores every finished tile into the exchange memory of the rank
that merges it, so the transfer runs under the computation and the merge is local.

The reference has no multi-GPU path; this module adds the one the 1 Mi-token
configuration needs.
"""
import torch
import torch.distributed as dist


def group_range(n_groups, world, rank):
    """Contiguous, balanced range [start, stop) of (batch, KV-head) groups for `rank`."""
    base, extra = divmod(n_groups, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def group_view(q, k, v, ids, start, stop, counts=None):
    """Views of the groups [start, stop): the rank's problem has batch = #groups,
    Hq = group size, Hkv = 1. No copy: a group is contiguous in every tensor."""
    b, hq, sq, d = q.shape
    hkv, skv = k.shape[1:3]
    g = hq // hkv
    qv = q.view(b * hkv, g, sq, d)[start:stop]
    kv = k.view(b * hkv, 1, skv, d)[start:stop]
    vv = v.view(b * hkv, 1, skv, d)[start:stop]
    iv = ids.view(b * hkv, 1, ids.shape[2], ids.shape[3])[start:stop]
    cv = None if counts is None else counts.view(b * hkv, 1, counts.shape[2])[start:stop]
    return qv, kv, vv, iv, cv


def kv_block_range(kv_blocks, kv_ranks, kv_rank):
    """KV blocks [lo, hi) owned by a rank: ceil(kv_blocks / kv_ranks) wide, the same
    split the segment-metadata kernel makes."""
    width = (kv_blocks + kv_ranks - 1) // kv_ranks
    lo = min(kv_rank * width, kv_blocks)
    return lo, min(lo + width, kv_blocks)


def exchange_rows(send, group=None):
    """send: [R, rows_per_rank, ...] (slice j goes to rank j of `group`). Returns
    recv [R, rows_per_rank, ...] where slice i came from rank i. Point-to-point
    send/recv, so it runs on NCCL (GPU tensors) and on gloo (CPU tensors)."""
    world = dist.get_world_size(group)
    me = dist.get_rank(group)
    recv = torch.empty_like(send)
    recv[me].copy_(send[me])
    ops = []
    for peer in range(world):
        if peer == me:
            continue
        gp = dist.get_global_rank(group, peer) if group is not None else peer
        ops.append(dist.P2POp(dist.isend, send[peer], gp, group))
        ops.append(dist.P2POp(dist.irecv, recv[peer], gp, group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return recv


def _gpu_filter(ids, counts, kv_blocks, kv_ranks, kv_rank):
    """Lists restricted to this rank's KV range, ids rebased to the local K/V slice."""
    from . import _lib
    b, hkv, qb, topk = ids.shape
    seg_ids = torch.empty((kv_ranks, b, hkv, qb, topk), dtype=torch.int32, device=ids.device)
    seg_counts = torch.empty((kv_ranks, b, hkv, qb), dtype=torch.int32, device=ids.device)
    err = torch.zeros(1, dtype=torch.int32, device=ids.device)
    with torch.cuda.device(ids.device):
        _lib.check(_lib.lib().sparse_b200_split_kv_segments(
            _lib.ptr(ids), _lib.ptr(counts), _lib.ptr(seg_ids), _lib.ptr(seg_counts), _lib.ptr(err),
            b, hkv, qb, topk, kv_blocks, kv_ranks, _lib.current_stream()))
    lo, _ = kv_block_range(kv_blocks, kv_ranks, kv_rank)
    return (seg_ids[kv_rank] - lo).clamp_(min=0), seg_counts[kv_rank]


def _gpu_attention(q, k, v, ids, counts):
    from .q_centric import attention_out
    out = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
    attention_out(q, k, v, ids, out, counts, lse)
    return out, lse


def _gpu_combine(partial, lses):
    """partial [R, rows, 128] bf16/fp32, lses [R, rows] -> (bf16 [rows,128], fp32 [rows])."""
    from . import _lib
    import ctypes
    ranks, rows = lses.shape
    out = torch.empty((rows, 128), dtype=torch.bfloat16, device=partial.device)
    lse = torch.empty((rows,), dtype=torch.float32, device=partial.device)
    with torch.cuda.device(partial.device):
        _lib.check(_lib.lib().sparse_b200_combine(
            _lib.ptr(partial), int(partial.dtype == torch.float32), _lib.ptr(lses), _lib.ptr(out), _lib.ptr(lse),
            ctypes.c_int64(rows), ranks, 1, _lib.current_stream()))
    return out, lse


class KVSplit:
    """KV-range split of one (set of) head group(s) over the ranks of `group`.

    q [B,Hq,Sq,128] (same on every rank of the group), k_local / v_local
    [B,Hkv,Skv/R,128] (this rank's KV rows), ids [B,Hkv,Sq/128,TopK] GLOBAL block ids.
    `run` returns this rank's slice of the merged result: rows [r*rows/R, (r+1)*rows/R)
    of the flattened [B*Hq*Sq] axis, as (O [rows/R,128] bf16, LSE [rows/R] fp32).
    The three stage functions can be replaced (the CPU tests inject the oracle)."""

    def __init__(self, group=None, filter_fn=_gpu_filter, attention_fn=_gpu_attention, combine_fn=_gpu_combine):
        self.group = group
        self.ranks = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.filter_fn, self.attention_fn, self.combine_fn = filter_fn, attention_fn, combine_fn

    def partial(self, q, k_local, v_local, ids, kv_blocks, counts=None):
        ids_r, counts_r = self.filter_fn(ids, counts, kv_blocks, self.ranks, self.rank)
        return self.attention_fn(q, k_local, v_local, ids_r, counts_r)

    def merge(self, o_r, l_r):
        rows = l_r.numel()
        if rows % self.ranks:
            raise ValueError("B*Hq*Sq must be divisible by the number of KV ranks")
        per = rows // self.ranks
        o_all = exchange_rows(o_r.reshape(self.ranks, per, 128), self.group)
        l_all = exchange_rows(l_r.reshape(self.ranks, per), self.group)
        return self.combine_fn(o_all, l_all)

    def run(self, q, k_local, v_local, ids, kv_blocks, counts=None):
        o_r, l_r = self.partial(q, k_local, v_local, ids, kv_blocks, counts)
        return self.merge(o_r, l_r)

    def run_peer(self, exchange, q, k_local, v_local, ids, kv_blocks, counts=None):
        """Same result as `run`, bit for bit, without the send/recv step: the attention kernel writes this
        rank's partial into `exchange` (a PeerExchange of B*Hq*Sq rows made by every rank of the group), and
        the merge kernel reads this rank's slice of rows from every rank's exchange memory. GPU only."""
        from .q_centric import attention_out
        rows = q.shape[0] * q.shape[1] * q.shape[2]
        if rows != exchange.rows or exchange.ranks != self.ranks or exchange.rank != self.rank:
            raise ValueError("the exchange was made for another geometry or group")
        ids_r, counts_r = self.filter_fn(ids, counts, kv_blocks, self.ranks, self.rank)
        exchange.begin()                                   # every reader of the previous partial has finished
        attention_out(q, k_local, v_local, ids_r, exchange.o.view(q.shape), counts_r, exchange.lse.view(q.shape[:3]))
        exchange.publish()                                 # my partial of this step is complete
        return exchange.merge()

    def run_scatter(self, exchange, q, k_local, v_local, ids, kv_blocks, counts=None):
        """Same result again, with the transfer inside the attention kernel: every finished 128-row tile of this
        rank's partial is stored (TMA store, LSE with plain stores) straight into the memory of the rank that
        merges it, under the remaining computation; the merge then reads local memory only. Up to 4 KV ranks;
        B*Hq*Sq / ranks must be whole 128-row tiles. GPU only. (A scatter launch never cuts the items of a short
        last round into pieces as `attention_out(balance=True)` may on launches of a few rounds; where that
        applies the rows of that round can differ from `run` in the last bf16 bit.)"""
        import ctypes
        from . import _lib
        rows = q.shape[0] * q.shape[1] * q.shape[2]
        if rows != exchange.rows or exchange.ranks != self.ranks or exchange.rank != self.rank:
            raise ValueError("the exchange was made for another geometry or group")
        if self.ranks > 4 or exchange.per % 128:
            raise ValueError("the scatter form serves up to 4 KV ranks and slices of whole 128-row tiles")
        ids_r, counts_r = self.filter_fn(ids, counts, kv_blocks, self.ranks, self.rank)
        b, hq, sq, _ = q.shape
        hkv, skv = k_local.shape[1:3]
        exchange.begin()
        with torch.cuda.device(q.device):
            _lib.check(_lib.lib().sparse_b200_q_centric_scatter(
                _lib.ptr(q), _lib.ptr(k_local), _lib.ptr(v_local), _lib.ptr(ids_r), _lib.ptr(counts_r),
                exchange.slot_out, exchange.slot_lse, self.ranks, b, hq, hkv, sq, skv, int(ids_r.shape[-1]),
                _lib.current_stream()))
        exchange.publish()
        return exchange.merge(slots=True)

    # ------------------------------------------------------------------ pipelined form
    def chunks(self, q, heads_per_chunk=2):
        """(group, first head, heads) chunks of q [B,Hq,Sq,128] seen as [groups, G, Sq, 128] with Hkv = 1 per
        group (the layout of a rank's problem); chunk c is merged on rank c % R."""
        groups, g = q.shape[0], q.shape[1]
        hpc = heads_per_chunk if g % heads_per_chunk == 0 else g
        return [(grp, h0, hpc) for grp in range(groups) for h0 in range(0, g, hpc)]

    def run_pipelined(self, q, k_local, v_local, ids, kv_blocks, counts=None, heads_per_chunk=2):
        """Same merge, chunk by chunk: q [groups, G, Sq, 128] with one KV head per group (k_local / v_local
        [groups, 1, Skv/R, 128], ids [groups, 1, Sq/128, TopK]). The attention of chunk c + 1 runs on the
        current stream while the partials of chunk c travel to the chunk's owner (rank c % R) on a side
        stream; the owner merges what it received with its own partial. Returns {chunk index: (O
        [heads*Sq, 128] bf16, LSE [heads*Sq] fp32)} for the chunks this rank owns; `self.chunks(q)` names them.
        On CPU tensors (gloo) everything runs in order."""
        if k_local.shape[1] != 1 or ids.shape[1] != 1:
            raise ValueError("run_pipelined takes the per-group layout: one KV head per leading index")
        on_gpu = q.is_cuda
        ids_r, counts_r = self.filter_fn(ids, counts, kv_blocks, self.ranks, self.rank)
        plan = self.chunks(q, heads_per_chunk)
        cur = torch.cuda.current_stream(q.device) if on_gpu else None
        side = self._side_stream(q.device) if on_gpu else None
        if on_gpu:
            side.wait_stream(cur)
        received, own, sent = {}, {}, []
        for c, (grp, h0, nh) in enumerate(plan):
            o_c, l_c = self.attention_fn(q[grp:grp + 1, h0:h0 + nh], k_local[grp:grp + 1], v_local[grp:grp + 1],
                                         ids_r[grp:grp + 1], counts_r[grp:grp + 1])
            o_c, l_c = o_c.reshape(-1, 128), l_c.reshape(-1)
            owner = c % self.ranks
            ready = None
            if on_gpu:
                ready = torch.cuda.Event()
                ready.record(cur)
            ctx = torch.cuda.stream(side) if on_gpu else _NullContext()
            with ctx:
                if on_gpu:
                    side.wait_event(ready)
                ops = []
                if owner == self.rank:
                    own[c] = (o_c, l_c)
                    bufs = []
                    for peer in range(self.ranks):
                        if peer == self.rank:
                            continue
                        gp = dist.get_global_rank(self.group, peer) if self.group is not None else peer
                        bo, bl = torch.empty_like(o_c), torch.empty_like(l_c)
                        ops += [dist.P2POp(dist.irecv, bo, gp, self.group), dist.P2POp(dist.irecv, bl, gp, self.group)]
                        bufs.append((peer, bo, bl))
                    received[c] = bufs
                else:
                    gp = dist.get_global_rank(self.group, owner) if self.group is not None else owner
                    ops += [dist.P2POp(dist.isend, o_c, gp, self.group), dist.P2POp(dist.isend, l_c, gp, self.group)]
                    sent.append((o_c, l_c))            # keep the buffers alive until the transfers have run
                if ops:
                    for req in dist.batch_isend_irecv(ops):
                        req.wait()
        if on_gpu:
            cur.wait_stream(side)
        out = {}
        for c, (o_c, l_c) in own.items():
            parts = sorted([(self.rank, o_c, l_c)] + received[c], key=lambda t: t[0])     # fixed rank order
            out[c] = self.combine_fn(torch.stack([p[1] for p in parts]), torch.stack([p[2] for p in parts]))
        return out

    def _side_stream(self, device):
        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=device)
        return self._side


class PeerExchange:
    """Exchange memory of one rank for `KVSplit.run_peer`: partial O [rows, 128] bf16, partial LSE [rows] fp32 and
    two rows of flag words (ready[R], done[R]), allocated by the library, mapped by every other rank of `group`
    (all ranks of the group must be processes on one machine whose GPUs have peer access). Collective: every rank
    of the group constructs it at the same point. `wait_ms` bounds every wait on a flag another GPU writes; when it
    runs out the kernel records a status code (`device_status()` raises) instead of hanging."""

    def __init__(self, rows, device, group=None, wait_ms=4000):
        import ctypes
        from . import _lib
        self.group, self.ranks, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        if rows % self.ranks:
            raise ValueError("B*Hq*Sq must be divisible by the number of KV ranks")
        if self.ranks not in (1, 2, 4, 8):
            raise ValueError("the peer merge serves 1, 2, 4 or 8 KV ranks")
        self.rows, self.per, self.device, self.wait_ms, self.epoch = rows, rows // self.ranks, torch.device(device), wait_ms, 0
        self.o_bytes = rows * 256
        self.lse_off = self.o_bytes
        self.flag_off = (self.lse_off + rows * 4 + 255) // 256 * 256
        self.bytes = self.flag_off + 256
        L = _lib.lib()
        base, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            # every failure below is first told to the whole group, then raised by every rank alike
            rc = L.sparse_b200_peer_alloc(ctypes.c_int64(self.bytes), ctypes.byref(base), handle)
            problem = None if rc == 0 else \
                f"rank {self.rank} cannot allocate exchange memory: {L.sparse_b200_last_error().decode()}"
            self.base = base.value if rc == 0 else None
            handles = [None] * self.ranks
            dist.all_gather_object(handles, handle.raw if rc == 0 else None, group=group)
            self.bases = []
            for r, h in enumerate(handles):
                if problem or any(x is None for x in handles):
                    break
                if r == self.rank:
                    self.bases.append(self.base)
                    continue
                peer = ctypes.c_void_p()
                rc = L.sparse_b200_peer_open(ctypes.create_string_buffer(h, 64), ctypes.byref(peer))
                if rc != 0:
                    problem = f"rank {self.rank} cannot map the memory of rank {r}: {L.sparse_b200_last_error().decode()}"
                    break
                self.bases.append(peer.value)
            problems = [None] * self.ranks
            dist.all_gather_object(problems, problem, group=group)      # all ranks go on, or none
            if any(problems):
                for r, b in enumerate(self.bases):
                    if r != self.rank:
                        L.sparse_b200_peer_close(ctypes.c_void_p(b))
                dist.barrier(group=group)
                if self.base is not None:
                    L.sparse_b200_peer_free(ctypes.c_void_p(self.base))
                self.base = None
                raise _lib.SparseB200Error("; ".join(p for p in problems if p))
        self.o = _wrap(self.base, (rows, 128), torch.bfloat16, self.device, self)
        self.lse = _wrap(self.base + self.lse_off, (rows,), torch.float32, self.device, self)
        self.flags = _wrap(self.base + self.flag_off, (2, 32), torch.int32, self.device, self)
        # flag words: ready[j] at flag_off + 4*j, done[j] at flag_off + 128 + 4*j (j = the rank that writes it)
        arr = ctypes.c_void_p * self.ranks
        self._ready_targets = arr(*[b + self.flag_off + 4 * self.rank for b in self.bases])
        self._done_targets = arr(*[b + self.flag_off + 128 + 4 * self.rank for b in self.bases])
        self._parts = arr(*[b + self.rank * self.per * 256 for b in self.bases])
        self._lses = arr(*[b + self.lse_off + self.rank * self.per * 4 for b in self.bases])
        # scatter form: the same memory seen as R slots of `per` rows, slot r = what rank r computed for MY rows.
        # slot_out[j] / slot_lse[j]: where this rank's rows of owner j go (slot `rank` of rank j's memory); the R
        # slots of my own memory are one rank-major [R, per, 128] / [R, per] pair for the merge
        self.slot_out = arr(*[b + self.rank * self.per * 256 for b in self.bases])
        self.slot_lse = arr(*[b + self.lse_off + self.rank * self.per * 4 for b in self.bases])
        self.out = torch.empty((self.per, 128), dtype=torch.bfloat16, device=self.device)
        self.out_lse = torch.empty((self.per,), dtype=torch.float32, device=self.device)

    def begin(self):
        """Opens a step: waits (on the stream) until every rank has finished reading the previous partial."""
        import ctypes
        from . import _lib
        self.epoch += 1
        if self.epoch > 1:
            with torch.cuda.device(self.device):
                _lib.check(_lib.lib().sparse_b200_peer_wait(
                    ctypes.c_void_p(self.base + self.flag_off + 128), self.ranks, self.epoch - 1, self.wait_ms,
                    _lib.current_stream()))

    def publish(self):
        from . import _lib
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().sparse_b200_peer_signal(self._ready_targets, self.ranks, self.epoch,
                                                          _lib.current_stream()))

    def merge(self, slots=False):
        """Merged rows [rank*rows/R, (rank+1)*rows/R) -> (O [rows/R, 128] bf16, LSE [rows/R] fp32); then tells every
        rank that this rank has finished reading. slots=False: every rank's memory holds its whole partial and the
        kernel loads this rank's rows from each of them; slots=True (after a scatter launch): the R partials of this
        rank's rows lie in its own memory."""
        import ctypes
        from . import _lib
        with torch.cuda.device(self.device):
            L = _lib.lib()
            if slots:
                # the R partials of my rows are local and rank-major: wait for the ready flags, then the ordinary
                # Combine kernel (two rows per thread group in flight: it runs at the memory roof)
                _lib.check(L.sparse_b200_peer_wait(ctypes.c_void_p(self.base + self.flag_off), self.ranks, self.epoch,
                                                   self.wait_ms, _lib.current_stream()))
                _lib.check(L.sparse_b200_combine(
                    ctypes.c_void_p(self.base), 0, ctypes.c_void_p(self.base + self.lse_off), _lib.ptr(self.out),
                    _lib.ptr(self.out_lse), ctypes.c_int64(self.per), self.ranks, 1, _lib.current_stream()))
                _lib.check(L.sparse_b200_peer_signal(self._done_targets, self.ranks, self.epoch, _lib.current_stream()))
                return self.out, self.out_lse
            _lib.check(L.sparse_b200_combine_peer(
                self._parts, self._lses,
                ctypes.c_void_p(self.base + self.flag_off), self.epoch, self.wait_ms,
                _lib.ptr(self.out), _lib.ptr(self.out_lse), ctypes.c_int64(self.per), self.ranks, _lib.current_stream()))
            _lib.check(L.sparse_b200_peer_signal(self._done_targets, self.ranks, self.epoch, _lib.current_stream()))
        return self.out, self.out_lse

    def close(self):
        """Collective: all ranks have finished their steps (synchronises, then unmaps and frees)."""
        from . import _lib
        import ctypes
        if self.base is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        L = _lib.lib()
        with torch.cuda.device(self.device):
            for r, b in enumerate(self.bases):
                if r != self.rank:
                    L.sparse_b200_peer_close(ctypes.c_void_p(b))
            dist.barrier(group=self.group)
            self.o = self.lse = self.flags = None
            L.sparse_b200_peer_free(ctypes.c_void_p(self.base))
        self.base = None


class _Raw:
    def __init__(self, ptr, shape, typestr, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2}


def _wrap(ptr, shape, dtype, device, owner):
    """torch tensor over library-owned device memory (no copy; `owner` must outlive it)."""
    if dtype == torch.bfloat16:         # no typestr for bf16: wrap as int16 and reinterpret
        return torch.as_tensor(_Raw(ptr, shape, "<i2", owner), device=device).view(torch.bfloat16)
    typestr = {torch.float32: "<f4", torch.int32: "<i4"}[dtype]
    return torch.as_tensor(_Raw(ptr, shape, typestr, owner), device=device)


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
