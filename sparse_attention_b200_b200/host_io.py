"""Attention on HOST (pinned) buffers: the copies in, the kernel and the copies out of
independent (batch, KV-head group) chunks run on three CUDA streams, so the PCIe link
works in both directions while the GPU computes. The device staging buffers are owned
by the caller-visible `HostPipeline` object and reused from call to call.

The reference has no host-buffer path (its operators take CUDA tensors); this is the
entry a caller with host-resident q/k/v uses, and what the end-to-end benchmark times."""
import torch

from . import sharding
from .q_centric import attention_out


class HostPipeline:
    def __init__(self, b, hq, hkv, sq, skv, topk, device, chunks=4):
        n_groups = b * hkv
        self.chunks = max(1, min(chunks, n_groups))
        self.shape = (b, hq, hkv, sq, skv, topk)
        self.device = torch.device(device)
        g = hq // hkv
        dev = self.device
        self.q = torch.empty((b, hq, sq, 128), dtype=torch.bfloat16, device=dev)
        self.k = torch.empty((b, hkv, skv, 128), dtype=torch.bfloat16, device=dev)
        self.v = torch.empty((b, hkv, skv, 128), dtype=torch.bfloat16, device=dev)
        self.ids = torch.empty((b, hkv, sq // 128, topk), dtype=torch.int32, device=dev)
        self.out = torch.empty((b, hq, sq, 128), dtype=torch.bfloat16, device=dev)
        self.lse = torch.empty((b, hq, sq), dtype=torch.float32, device=dev)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        self.ranges = [sharding.group_range(n_groups, self.chunks, c) for c in range(self.chunks)]
        self.done_run = [None] * self.chunks     # compute of the previous call finished with chunk c's inputs
        self.done_out = [None] * self.chunks     # copy-out of the previous call finished with chunk c's outputs
        self.g = g

    def _views(self, q, k, v, ids, out, lse, a, b_):
        bsz, hq, hkv, sq, skv, topk = self.shape
        qv, kv, vv, iv, _ = sharding.group_view(q, k, v, ids, a, b_)
        ov = out.view(bsz * hkv, self.g, sq, 128)[a:b_]
        lv = lse.view(bsz * hkv, self.g, sq)[a:b_]
        return qv, kv, vv, iv, ov, lv

    def run(self, q_host, k_host, v_host, ids_host, out_host, lse_host):
        """All host tensors pinned and shaped like their device twins. Asynchronous: returns
        an event that completes when out_host / lse_host are filled."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        for c, (a, b_) in enumerate(self.ranges):
            dq, dk, dv, di, do, dl = self._views(self.q, self.k, self.v, self.ids, self.out, self.lse, a, b_)
            hq_, hk_, hv_, hi_, ho_, hl_ = self._views(q_host, k_host, v_host, ids_host, out_host, lse_host, a, b_)
            with torch.cuda.stream(self.s_in):
                if self.done_run[c] is not None:
                    self.s_in.wait_event(self.done_run[c])
                dq.copy_(hq_, non_blocking=True)
                dk.copy_(hk_, non_blocking=True)
                dv.copy_(hv_, non_blocking=True)
                di.copy_(hi_, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(ready)
                if self.done_out[c] is not None:
                    self.s_run.wait_event(self.done_out[c])
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
