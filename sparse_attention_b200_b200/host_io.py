"""Attention on HOST (pinned) buffers: the copies in, the kernel and the copies out of
independent chunks run on three CUDA streams, so the PCIe link works in both directions
while the GPU computes. A chunk is some query heads of one (batch, KV-head) group: the
group's K / V rows and selection lists travel with its first chunk. The device staging
buffers are owned by the caller-visible `HostPipeline` object (or handed in by the caller)
and reused from call to call.

The reference has no host-buffer path (its operators take CUDA tensors); this is the
entry a caller with host-resident q/k/v uses, and what the end-to-end benchmark times."""
import torch

from .q_centric import attention_out


class HostPipeline:
    """chunks: target number of chunks over the whole problem (rounded to whole groups, or to
    an even number of heads inside a group when there are fewer groups than chunks).
    buffers: optional (q, k, v, ids, out, lse) device tensors to stage through instead of
    allocating new ones."""

    def __init__(self, b, hq, hkv, sq, skv, topk, device, chunks=4, buffers=None):
        n_groups = b * hkv
        g = hq // hkv
        self.shape = (b, hq, hkv, sq, skv, topk)
        self.device = torch.device(device)
        self.g = g
        dev = self.device
        if buffers is None:
            self.q = torch.empty((b, hq, sq, 128), dtype=torch.bfloat16, device=dev)
            self.k = torch.empty((b, hkv, skv, 128), dtype=torch.bfloat16, device=dev)
            self.v = torch.empty((b, hkv, skv, 128), dtype=torch.bfloat16, device=dev)
            self.ids = torch.empty((b, hkv, sq // 128, topk), dtype=torch.int32, device=dev)
            self.out = torch.empty((b, hq, sq, 128), dtype=torch.bfloat16, device=dev)
            self.lse = torch.empty((b, hq, sq), dtype=torch.float32, device=dev)
        else:
            self.q, self.k, self.v, self.ids, self.out, self.lse = buffers
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        # chunk = (group, first head, heads): whole groups when there are enough of them, else an even
        # number of heads (two heads of a group share each K/V tile in the kernel) of one group
        per_group = 1
        if chunks > n_groups and g % 2 == 0:
            per_group = max(1, min(g // 2, chunks // n_groups))
            while (g // 2) % per_group:
                per_group -= 1
        hpc = g // per_group
        if per_group == 1 and chunks < n_groups:
            # several groups per chunk
            per_chunk = -(-n_groups // max(1, chunks))
            self.plan = [(a, min(n_groups, a + per_chunk), 0, g) for a in range(0, n_groups, per_chunk)]
        else:
            self.plan = [(grp, grp + 1, h0, hpc) for grp in range(n_groups) for h0 in range(0, g, hpc)]
        self.chunks = len(self.plan)
        self.done_run = [None] * self.chunks     # compute of the previous call finished with chunk c's inputs
        self.done_out = [None] * self.chunks     # copy-out of the previous call finished with chunk c's outputs

    def _views(self, q, k, v, ids, out, lse, chunk):
        bsz, hq, hkv, sq, skv, topk = self.shape
        a, b_, h0, nh = chunk
        g = self.g
        qv = q.view(bsz * hkv, g, sq, 128)[a:b_, h0:h0 + nh]
        ov = out.view(bsz * hkv, g, sq, 128)[a:b_, h0:h0 + nh]
        lv = lse.view(bsz * hkv, g, sq)[a:b_, h0:h0 + nh]
        kv = k.view(bsz * hkv, 1, skv, 128)[a:b_]
        vv = v.view(bsz * hkv, 1, skv, 128)[a:b_]
        iv = ids.view(bsz * hkv, 1, sq // 128, topk)[a:b_]
        return qv, kv, vv, iv, ov, lv

    def run(self, q_host, k_host, v_host, ids_host, out_host, lse_host, copy_only=False):
        """All host tensors pinned and shaped like their device twins. Asynchronous: returns
        an event that completes when out_host / lse_host are filled. copy_only skips the kernel
        (the transfer time of the same buffers alone: what the host link allows)."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        for c, chunk in enumerate(self.plan):
            dq, dk, dv, di, do, dl = self._views(self.q, self.k, self.v, self.ids, self.out, self.lse, chunk)
            hq_, hk_, hv_, hi_, ho_, hl_ = self._views(q_host, k_host, v_host, ids_host, out_host, lse_host, chunk)
            first_of_group = chunk[2] == 0
            with torch.cuda.stream(self.s_in):
                if self.done_run[c] is not None:
                    self.s_in.wait_event(self.done_run[c])
                dq.copy_(hq_, non_blocking=True)
                if first_of_group:          # later chunks of the group find K, V and the lists in place (stream order)
                    # the previous call's kernels of every chunk of this group have finished reading K, V, lists
                    for c2, other in enumerate(self.plan):
                        if c2 != c and other[0] == chunk[0] and self.done_run[c2] is not None:
                            self.s_in.wait_event(self.done_run[c2])
                    dk.copy_(hk_, non_blocking=True)
                    dv.copy_(hv_, non_blocking=True)
                    di.copy_(hi_, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ready)
                if self.done_out[c] is not None:
                    self.s_run.wait_event(self.done_out[c])
                if not copy_only:
                    attention_out(dq, dk, dv, di, do, None, dl)
                ran = torch.cuda.Event()
                ran.record(self.s_run)
                self.done_run[c] = ran
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ran)
                ho_.copy_(do, non_blocking=True)
                hl_.copy_(dl, non_blocking=True)
                out_ev = torch.cuda.Event()
                out_ev.record(self.s_out)
                self.done_out[c] = out_ev
        cur.wait_stream(self.s_out)
        done = torch.cuda.Event()
        done.record(cur)
        return done
