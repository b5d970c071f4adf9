#!/usr/bin/env python
"""Headline benchmark: block-sparse attention forward, selected-block TFLOP/s.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (N = 1): B=1, Hq=Hkv=32, N=32768, d=128, bf16, 16 distinct sorted KV
blocks of 128 per (head, query block), seeded synthetic data. With N > 1 every
rank runs one such shard (independent heads, no collective): weak scaling.
A step is one pass of the Q-centric kernel over the whole shard.

value   = selected-block FLOPs of all ranks / device time (inputs resident in HBM)
e2e     = same metric with HOST (pinned) q, k, v, block_idx copied in and out,
          lse copied back inside the timed region, through the C ABI
roofline= tensor-pipe roofline of the attention kernel against the measured
          BF16 peak of this pool
cpu_baseline = the CPU oracle's gather formulation of the reference's
          masked-attention computation, timed on a bounded sample
`--impl reference` times that CPU path alone, on all host cores.
"""
import argparse
import json
import os
import random
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sparse-attn fwd TFLOPS (selected blocks) & % BF16 tensor peak; indexer ms"
WORKLOAD = {"name": "q_centric_mha_32k", "B": 1, "Hq": 32, "Hkv": 32, "N": 32768, "topk": 16}
# DRAM bytes per launch of the attention kernel on this workload
# (dram__bytes_read.sum + dram__bytes_write.sum, Nsight Compute capture
# summarised in profiles/q_centric_kernel_mha_32k.md).
NCU_TRAFFIC_BYTES = 1.090e9


def flops(w):
    return 4.0 * w["B"] * w["Hq"] * w["N"] * (w["topk"] * 128) * 128


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json, burst bf16)"
    return 1590.0, 6650.0, "fallback (earlier measurement on this pool)"


def make_ids(w, seed):
    import torch
    rng = random.Random(seed)
    nb = w["N"] // 128
    rows = [sorted(rng.sample(range(nb), w["topk"])) for _ in range(w["B"] * w["Hkv"] * nb)]
    return torch.tensor(rows, dtype=torch.int32).reshape(w["B"], w["Hkv"], nb, w["topk"])


class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [x for x in sm if x >= 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_sample(w, budget_s=20.0, max_heads=32):
    """Oracle gather path (the reference's torch computation) on whole heads of
    the workload until the time budget is used. Returns (TFLOP/s, description)."""
    import torch
    import oracle
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(17)
    n, topk = w["N"], w["topk"]
    nb = n // 128
    per_block = 4.0 * 128 * (topk * 128) * 128
    done_blocks, t_total, heads = 0, 0.0, 0
    ids_all = make_ids({**w, "B": 1, "Hkv": max_heads}, 1017)
    while heads < max_heads and t_total < budget_s:
        q = torch.randn((1, 1, n, 128), generator=g).to(torch.bfloat16)
        k = torch.randn((1, 1, n, 128), generator=g).to(torch.bfloat16)
        v = torch.randn((1, 1, n, 128), generator=g).to(torch.bfloat16)
        ids = ids_all[:, heads:heads + 1].contiguous()
        blocks = range(nb)
        t0 = time.perf_counter()
        oracle.gather_attention(q, k, v, ids, q_blocks=blocks)
        t_total += time.perf_counter() - t0
        done_blocks += nb
        heads += 1
    tf = done_blocks * per_block / t_total / 1e12
    return tf, f"{heads} of {w['B'] * w['Hq']} (batch, head) slices x all {nb} query blocks, gather path, {t_total:.1f} s"


def run_reference(args):
    """CPU arm: rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    w = WORKLOAD
    cores = os.cpu_count() or 1
    times, tfs, sample = [], [], ""
    for step in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        tf, sample = cpu_sample(w, budget_s=2.0, max_heads=2)
        if step >= args.warmup:
            times.append(time.perf_counter() - t0)
            tfs.append(tf)
    value = statistics.mean(tfs)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(times),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic (seeded N(0,1) q/k/v, uniform sorted block lists)",
            "config": {"workload": w["name"], **{k: v for k, v in w.items() if k != "name"}},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": "per step: " + sample + f" (host has {cores} cores)"},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_e2e(args, sp, q, k, v, ids, ids_host, out, lse, barrier):
    """Host (pinned) buffers in and out through the C ABI, copies inside the timed region."""
    import torch
    hq_, hk_, hv_ = (t.cpu().pin_memory() for t in (q, k, v))
    hids = ids_host.pin_memory()
    hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    hlse = torch.empty(lse.shape, dtype=lse.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (hq_, hk_, hv_, hids))
    d2h = sum(t.numel() * t.element_size() for t in (hout, hlse))

    def e2e_step():
        q.copy_(hq_, non_blocking=True)
        k.copy_(hk_, non_blocking=True)
        v.copy_(hv_, non_blocking=True)
        ids.copy_(hids, non_blocking=True)
        sp.attention_out(q, k, v, ids, out, None, lse)
        hout.copy_(out, non_blocking=True)
        hlse.copy_(lse, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1) / e2e_steps
    return e2e_ms, e2e_steps, h2d, d2h


def run_ours(args):
    import torch
    import torch.distributed as dist
    import sparse_attention_b200_b200 as sp

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = WORKLOAD
    b, hq, hkv, n, topk = w["B"], w["Hq"], w["Hkv"], w["N"], w["topk"]
    gen = torch.Generator(device=dev).manual_seed(17 + rank)
    q = torch.randn((b, hq, n, 128), device=dev, generator=gen).to(torch.bfloat16)
    k = torch.randn((b, hkv, n, 128), device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn((b, hkv, n, 128), device=dev, generator=gen).to(torch.bfloat16)
    ids_host = make_ids(w, 1017 + rank)
    ids = ids_host.to(dev)
    out = torch.empty_like(q)
    lse = torch.empty((b, hq, n), device=dev, dtype=torch.float32)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        sp.attention_out(q, k, v, ids, out, None, lse)

    sampler = ClockSampler(local_rank)
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    sp.device_status()
    clocks = sampler.stop() if rank == 0 else None

    e2e_ms, e2e_steps, h2d, d2h = float("nan"), 0, 0, 0
    if not args.kernel_only:
        e2e_ms, e2e_steps, h2d, d2h = run_e2e(args, sp, q, k, v, ids, ids_host, out, lse, barrier)
    sp.device_status()
    times = torch.tensor([ms_total, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = times.tolist()
    ms_step = ms_total / args.steps
    total_flops = flops(w) * world
    value = total_flops / (ms_step * 1e-3) / 1e12
    e2e_value = total_flops / (e2e_ms * 1e-3) / 1e12

    if rank == 0:
        peak_tf, peak_gbs, peak_src = measured_peaks()
        achieved = flops(w) / (ms_step * 1e-3) / 1e12      # one launch on one GPU
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic (seeded N(0,1) q/k/v, 16 distinct sorted KV blocks per list)",
                "config": {"workload": w["name"], "B": b, "Hq": hq, "Hkv": hkv, "N": n, "d": 128, "topk": topk,
                           "block": 128, "sharding": f"{world} x independent (batch, KV-head group) shards",
                           "l2": "inputs (1.07 GB per GPU) exceed the 126 MB L2; no flush between steps"},
                "pct_bf16_peak": 100.0 * achieved / peak_tf,
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                             "frac": achieved / peak_tf, "traffic": NCU_TRAFFIC_BYTES, "peak_source": peak_src,
                             "kernel": "q_centric_kernel<bf16 out>", "launches_timed": args.steps},
                "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_ms, "steps": e2e_steps},
                "gpu_launches": args.steps, "clocks": clocks}
        if world == 1 and not args.kernel_only:
            tf, sample = cpu_sample(w)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                                    "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident timing only (used for profiler captures): no e2e, no CPU baseline")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
