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
NCU_TRAFFIC_BYTES = 1.145e9


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
    """SM clock and throttle reasons sampled while the timed region runs: NVML polled every 2 ms from
    a thread (read-only queries), so that even a 20 ms region gets several samples; nvidia-smi every
    200 ms when the NVML binding is missing."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = ((0x4, "sw_power_cap"), (0x8, "hw_slowdown"), (0x20, "sw_thermal_slowdown"),
               (0x40, "hw_thermal_slowdown"))

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.thread = None
        self.samples = []
        self.stop_flag = False
        self.max_mhz = None

    def _nvml_loop(self, nvml, handle):
        while not self.stop_flag:
            try:
                sm = nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)
                try:
                    mask = nvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except Exception:
                    mask = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((float(sm), int(mask), time.time()))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        try:
            import threading
            import pynvml as nvml
            import torch
            nvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(self.gpu).uuid)
            try:
                handle = nvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                handle = nvml.nvmlDeviceGetHandleByIndex(self.gpu)
            self.max_mhz = float(nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nvml, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self, window=None):
        """window = (t0, t1) host times of the timed region: its samples are reported; the samples
        of the whole sampling period (timed region + probe loop) are summarised beside them."""
        if self.thread is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)

            def summary(samples):
                sm = [x[0] for x in samples]
                reasons = set()
                for _, mask, _t in samples:
                    for bit, name in self.REASONS:
                        if mask & bit:
                            reasons.add(name)
                busy = [x for x in sm if x >= 0.5 * max(sm)] if sm else []
                return (statistics.median(busy) if busy else None), sorted(reasons), len(sm)
            inside = [x for x in self.samples if window and window[0] <= x[2] <= window[1]]
            all_mhz, all_reasons, all_n = summary(self.samples)
            if inside:
                mhz, reasons, n = summary(inside)
            else:
                mhz, reasons, n = all_mhz, all_reasons, all_n
            return {"sm_mhz": mhz, "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": n,
                    "source": "nvml, 2 ms period",
                    "window": "timed region" if inside else "timed region + 0.3 s of the same launches",
                    "probe": {"sm_mhz": all_mhz, "reasons": all_reasons, "samples": all_n,
                              "what": "timed region + 0.3 s of the same launches (sustained load)"}}
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
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvidia-smi, 200 ms period"}


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

    b, hq, sq, _ = q.shape
    hkv, skv = k.shape[1:3]
    pipe = sp.HostPipeline(b, hq, hkv, sq, skv, ids.shape[-1], q.device, chunks=8)

    def e2e_step():
        pipe.run(hq_, hk_, hv_, hids, hout, hlse)

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
    t_region0 = time.time()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    t_region1 = time.time()
    ms_total = e0.elapsed_time(e1)
    sp.device_status()
    # An NVML query takes longer than one launch, so a short timed region yields one or two
    # samples: keep issuing the very same launches (untimed) for 0.3 s with the sampler running.
    t_probe = time.time()
    while time.time() - t_probe < 0.3:
        for _ in range(10):
            step()
        torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop((t_region0, t_region1)) if rank == 0 else None

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
        line["e2e"]["how"] = ("pinned host q,k,v,block_idx in, out+lse back, 8 head chunks pipelined over three "
                              "streams through the C ABI (HostPipeline)")
        if world == 1 and not args.kernel_only:
            tf, sample = cpu_sample(w)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                                    "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- other configurations
CONFIGS = {
    # name: B, Hq, Hkv, N, topk, indexer, operator
    "c1": dict(B=1, Hq=8, Hkv=8, N=4096, topk=8, indexer="r1", op="q_centric", k_offset=0.5),
    "c3": dict(B=2, Hq=64, Hkv=8, N=65536, topk=32, indexer="r4", op="q_centric", k_offset=0.5),
    "c4": dict(B=1, Hq=64, Hkv=4, N=131072, topk=64, indexer="fp4", op="kv_centric", k_offset=0.0),
    "c5": dict(B=1, Hq=64, Hkv=8, N=1048576, topk=64, indexer="r4", op="q_centric", k_offset=0.5),
}


def fill_normal_bf16(t, gen, k_offset=0.0):
    """N(0,1) in place, generated head by head (a 1 Mi-token tensor does not fit twice in fp32);
    optionally adds a per-128-row-block offset ~ N(0, k_offset) (the K families of configurations 1, 3, 5)."""
    import torch
    flat = t.view(-1, t.shape[-2], t.shape[-1])
    for h in range(flat.shape[0]):
        rows = flat.shape[1]
        for r0 in range(0, rows, 1 << 18):
            r1 = min(rows, r0 + (1 << 18))
            x = torch.randn((r1 - r0, 128), device=t.device, generator=gen)
            if k_offset:
                off = torch.randn(((r1 - r0) // 128, 1, 128), device=t.device, generator=gen) * k_offset
                x = (x.view(-1, 128, 128) + off).view(-1, 128)
            flat[h, r0:r1] = x.to(torch.bfloat16)


def timed(fn, steps, warmup, barrier):
    import torch
    for _ in range(warmup):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier()
    return e0.elapsed_time(e1) / steps


def reference_kv_centric(q, k, v, selected, ours, steps, barrier):
    """The reference's own round-11 KV-centric operator (variant tma16_bf16: token-major Q, bf16
    partials; attention/kv_centric/optimization_round11/api11.py:50-92), prebuilt unmodified by
    baseline/build_reference_kernels.py in the git-ignored baseline/_ref/, timed on the same tensors
    with the same protocol. Its Q layout [B,Sq,Hq,D] is made once outside the timing, as in the
    reference's benchmark. Returns None when it is not built here."""
    import torch
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "kv_centric",
                        "optimization_round11")
    lib = os.path.join(root, "build", "xomtention_kvopt11.so")
    if not os.path.exists(lib) or tuple(selected.shape[1:]) != (1, q.shape[2], 16) or q.shape[1] != 16:
        return None
    sys.path.insert(0, root)
    import api11
    torch.ops.load_library(lib)
    api11._OPS = torch.ops.xomtention_kvopt11
    api11.old_plan.load_extension = lambda: api11._OPS
    q_tm = q.permute(0, 2, 1, 3).contiguous()
    ref = api11.Prepared(q_tm, k, v, selected, variant=api11.VARIANTS["tma16_bf16"])
    stages = {"metadata_ms": timed(ref.metadata, steps, 3, barrier), "main_ms": timed(ref.main, steps, 3, barrier),
              "combine_ms": timed(ref.combine, steps, 3, barrier)}
    rounds = []
    for _ in range(3):                      # interleaved with ours: same thermal state for both
        rounds.append((timed(ref.run, steps, 3, barrier), timed(ours.run, steps, 3, barrier)))
    diff = (ref.out.float() - ours.out.float()).abs().max().item()
    lse_diff = (ref.out_lse - ours.out_lse).abs().max().item()
    return {"variant": "tma16_bf16", "ms": min(r[0] for r in rounds), "ours_ms_interleaved": min(r[1] for r in rounds),
            "stages": stages, "max_abs_diff_out": diff, "max_abs_diff_lse": lse_diff}


def run_kv_token(args):
    """The reference's own KV-centric benchmark shape (B8, Hq16, Hkv1, Sq = Skv = 4096, TopK 16,
    per-TOKEN independent lists; benchmarks/ch5_kv_centric/round11_final/RESULTS_RU.md:9-13)
    through the per-token operator: metadata, main, combine."""
    import torch
    import sparse_attention_b200_b200 as sp
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    B, Hq, Hkv, S, topk = 8, 16, 1, args.n or 4096, 16
    gen = torch.Generator(device=dev).manual_seed(17)
    q = torch.randn((B, Hq, S, 128), device=dev, generator=gen).to(torch.bfloat16)
    k = torch.randn((B, Hkv, S, 128), device=dev, generator=gen).to(torch.bfloat16)
    v = torch.randn((B, Hkv, S, 128), device=dev, generator=gen).to(torch.bfloat16)
    selected = torch.rand((B * Hkv * S, S // 128), device=dev, generator=gen).argsort(-1)[:, :topk] \
        .int().reshape(B, Hkv, S, topk).contiguous()
    prep = sp.PreparedTokens(q, k, v, selected)

    def barrier():
        torch.cuda.synchronize()
    stages = {"metadata_ms": timed(prep.metadata, args.steps, 3, barrier),
              "main_ms": timed(prep.main, args.steps, 3, barrier),
              "combine_ms": timed(prep.combine, args.steps, 3, barrier)}
    ms = timed(prep.run, args.steps, 3, barrier)
    sp.device_status()
    # the same operator with q handed over token-major [B,Sq,Hq,128], the layout the reference's TMA
    # variants take (the copy is made once outside the timing, as in the reference's benchmark)
    prep_tm = sp.PreparedTokens(q.permute(0, 2, 1, 3).contiguous(), k, v, selected, q_token_major=True)
    prep_tm.metadata()
    token_major = {"main_ms": timed(prep_tm.main, args.steps, 3, barrier), "ms": timed(prep_tm.run, args.steps, 3, barrier),
                   "identical_output": bool(torch.equal(prep_tm.out, prep.out))}
    sp.device_status()
    same_box = reference_kv_centric(q, k, v, selected, prep, args.steps, barrier)
    fl = 4.0 * B * Hq * S * (topk * 128) * 128
    peak_tf, peak_gbs, peak_src = measured_peaks()
    value = fl / (ms * 1e-3) / 1e12
    print(json.dumps({"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": 3, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "bf16", "data": "synthetic (seeded N(0,1), independent per-token lists)",
                      "config": {"workload": "kv_token_reference_shape", "B": B, "Hq": Hq, "Hkv": Hkv, "Sq": S, "Skv": S,
                                 "topk": topk}, "stages_rank0": stages,
                      "reference_published": {"ms": 1.503, "tflops": 365.8, "variant": "tma16_bf16",
                                              "source": "benchmarks/ch5_kv_centric/round11_final/RESULTS_RU.md:12"},
                      "ours_q_token_major": token_major, "reference_same_box": same_box,
                      "roofline": {"bound": "tensor", "achieved": value, "peak": peak_tf, "unit": "TFLOP/s",
                                   "frac": value / peak_tf, "traffic": None, "peak_source": peak_src,
                                   "kernel": "kv_token_kernel + combine_kernel"}}), flush=True)


REFCMP_SHAPES = [
    # (name, B, Hq, Hkv, Sq, Skv, topk): the reference's own benchmark shapes
    # (benchmarks/ch4_q_centric sweep: B2, Hq16, Hkv1, Sq4096, TopK16, Skv 2048..16384), GQA 4:1,
    # and this repository's headline MHA configuration.
    ("ref_gqa16_skv2048", 2, 16, 1, 4096, 2048, 16),
    ("ref_gqa16_skv4096", 2, 16, 1, 4096, 4096, 16),
    ("ref_gqa16_skv8192", 2, 16, 1, 4096, 8192, 16),
    ("ref_gqa16_skv16384", 2, 16, 1, 4096, 16384, 16),
    ("gqa4_32k", 1, 32, 8, 32768, 32768, 16),
    ("mha_32k", 1, 32, 32, 32768, 32768, 16),
]


def run_refcmp(args):
    """Same-box comparator: the reference's own Q-centric kernels (p02 = Q-position pairing,
    variant 1; p03 = head pairing, variant 2; attention/q_centric/progression.py:40-58), compiled
    unmodified by baseline/build_reference_kernels.py into the git-ignored baseline/_ref/, timed
    next to this repository's kernel with one protocol: same tensors, same lists, CUDA events
    around back-to-back launches, arms interleaved in rounds and the best round kept per arm.
    Prints one JSON line per shape; when the reference library is absent, one `unavailable` line."""
    import torch
    import sparse_attention_b200_b200 as sp
    lib = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "xomtention_progression.so")
    if not os.path.exists(lib):
        print(json.dumps({"workload": "refcmp", "unavailable": "baseline/_ref/xomtention_progression.so not built "
                          "(python baseline/build_reference_kernels.py)"}), flush=True)
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    torch.ops.load_library(lib)
    ref_out = torch.ops.xomtention_progression.attention_out

    def barrier():
        torch.cuda.synchronize()
    for name, B, Hq, Hkv, Sq, Skv, topk in REFCMP_SHAPES:
        gen = torch.Generator(device=dev).manual_seed(23)
        q = torch.randn((B, Hq, Sq, 128), device=dev, generator=gen).to(torch.bfloat16)
        k = torch.randn((B, Hkv, Skv, 128), device=dev, generator=gen).to(torch.bfloat16)
        v = torch.randn((B, Hkv, Skv, 128), device=dev, generator=gen).to(torch.bfloat16)
        # the reference's "independent" pattern: a fresh random subset per list, ascending
        # (attention/q_centric/progression_validation.py:21-41)
        ids = torch.rand((B * Hkv * (Sq // 128), Skv // 128), device=dev, generator=gen).argsort(-1)[:, :topk] \
            .sort(-1).values.int().reshape(B, Hkv, Sq // 128, topk).contiguous()
        outs = {"ours": torch.empty_like(q), "p02": torch.empty_like(q), "p03": torch.empty_like(q)}
        arms = {"ours": lambda: sp.attention_out(q, k, v, ids, outs["ours"]),
                "p02": lambda: ref_out(q, k, v, ids, outs["p02"], 1)}
        if Hq // Hkv >= 2:
            arms["p03"] = lambda: ref_out(q, k, v, ids, outs["p03"], 2)
        best = {a: float("inf") for a in arms}
        for rnd in range(3):
            for a, fn in arms.items():
                best[a] = min(best[a], timed(fn, args.steps, 3, barrier))
        sp.device_status()
        fl = 4.0 * B * Hq * Sq * (topk * 128) * 128
        diff = {a: (outs[a].float() - outs["ours"].float()).abs().max().item() for a in arms if a != "ours"}
        ref_best = min(v_ for a, v_ in best.items() if a != "ours")
        print(json.dumps({"workload": "refcmp", "shape": {"name": name, "B": B, "Hq": Hq, "Hkv": Hkv, "Sq": Sq,
                                                          "Skv": Skv, "topk": topk},
                          "us": {a: round(t * 1e3, 2) for a, t in best.items()},
                          "tflops": {a: round(fl / (t * 1e-3) / 1e12, 1) for a, t in best.items()},
                          "ours_over_best_reference": round(ref_best / best["ours"], 4),
                          "max_abs_diff_vs_ours": diff, "steps": args.steps, "rounds": 3,
                          "protocol": "back-to-back launches, no L2 flush, best of 3 interleaved rounds"}), flush=True)
        del q, k, v, ids, outs


# The reference's published selector benchmark (benchmarks/ch4_selectors/RESULTS.md:7-15), microseconds:
# Skv -> selector -> (selector only, selector -> p03 pipeline)
REFSEL_PUBLISHED = {4096: {"R1": (20.73, 155.72), "R4": (47.84, 175.00), "FP4": (17.66, 154.67)},
                    8192: {"R1": (22.01, 154.33), "R4": (53.55, 178.44), "FP4": (28.92, 162.50)},
                    16384: {"R1": (22.09, 154.50), "R4": (60.73, 187.04), "FP4": (48.38, 180.43)}}


def graph_time_us(fn, replays=20):
    """Median-free protocol of the reference's selector benchmark: capture one call in a CUDA
    graph, replay it back to back, CUDA events around the replays; best of three rounds."""
    import torch
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    best = float("inf")
    for _ in range(3):
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / replays * 1e3)
    return best


def run_refsel(args):
    """This repository's selectors on the reference's own selector benchmark shapes (B2, Hq16, Hkv1,
    Sq 4096, Skv 4096 / 8192 / 16384, TopK 16; benchmarks/ch4_selectors/RESULTS.md): selector alone
    and selector -> attention as one CUDA graph, next to the reference's published microseconds.
    FP4 starts, as there, from prepared quantised inputs (quantisation excluded)."""
    import torch
    import sparse_attention_b200_b200 as sp
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    B, Hq, Hkv, Sq, topk = 2, 16, 1, 4096, 16
    # the reference's own Triton selectors (indexers/r1_r4/block_selectors.py:9-55), copied unmodified
    # into the git-ignored baseline/_ref/r1_r4, when present: same tensors, same protocol
    ref_sel = None
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "r1_r4")
    if os.path.isdir(ref_dir):
        try:
            sys.path.insert(0, ref_dir)
            import block_selectors as ref_sel
        except Exception as e:          # Triton missing or unusable on this box
            print(json.dumps({"workload": "refsel", "reference_same_box": f"unavailable: {e}"}), flush=True)
            ref_sel = None
    for Skv in (4096, 8192, 16384):
        gen = torch.Generator(device=dev).manual_seed(29)
        q = torch.randn((B, Hq, Sq, 128), device=dev, generator=gen).to(torch.bfloat16)
        k = (torch.randn((B, Hkv, Skv, 128), device=dev, generator=gen)
             + 0.5 * torch.randn((B, Hkv, Skv // 128, 1, 128), device=dev, generator=gen)
             .expand(B, Hkv, Skv // 128, 128, 128).reshape(B, Hkv, Skv, 128)).to(torch.bfloat16)
        v = torch.randn((B, Hkv, Skv, 128), device=dev, generator=gen).to(torch.bfloat16)
        out = torch.empty_like(q)
        row = {"workload": "refsel", "shape": {"B": B, "Hq": Hq, "Hkv": Hkv, "Sq": Sq, "Skv": Skv, "topk": topk},
               "us": {}, "reference_published_us": {}, "protocol": "CUDA-graph replays, best of 3 rounds x 20"}
        for name, r in (("R1", 1), ("R4", 4)):
            sel = sp.SummarySelector(q, k, r, topk=topk, keep_scores=False)
            exact = sp.SummarySelector(q, k, r, topk=topk, keep_scores=True)
            t_sel = graph_time_us(sel.run_fast)
            t_exact = graph_time_us(exact.run)
            t_pipe = graph_time_us(lambda: sp.summary_indexed_attention_out(sel, v, out))
            torch.cuda.synchronize()
            assert torch.equal(sel.ids, exact.ids)
            row["us"][name] = {"selector": round(t_sel, 2), "selector_exact_kernels": round(t_exact, 2),
                               "selector_to_attention": round(t_pipe, 2), "fallback_lists": sel.fallback_lists()}
            pub = REFSEL_PUBLISHED[Skv][name]
            row["reference_published_us"][name] = {"selector": pub[0], "selector_to_p03": pub[1]}
            if ref_sel is not None:
                rs = ref_sel.SummarySelector(q, k, r)
                t_ref = graph_time_us(rs.run)
                torch.cuda.synchronize()
                same = (rs.ids == sel.ids).all(-1).float().mean().item()
                row.setdefault("reference_same_box_us", {})[name] = {"selector": round(t_ref, 2),
                                                                      "lists_with_identical_ids": round(same, 4)}
        qc, qs = sp.quantize_queries(q, Hkv)
        kc, ks = sp.quantize_keys(k)
        inputs = sp.prepare_fp4_inputs(qc, kc, qs, ks, batch_size=B, len_q=Sq, len_kv=Skv)
        ids_fast, ws = sp.fp4_indexer_fast(inputs, topk=topk)
        ids_exact = sp.fp4_indexer(inputs, topk=topk)
        tile_scores = torch.empty((B, Hkv, Sq // 128, Skv // 128), dtype=torch.float32, device=dev)
        t_sel = graph_time_us(lambda: sp.fp4_indexer_fast(inputs, selected=ids_fast, workspace=ws))
        t_exact = graph_time_us(lambda: sp.fp4_indexer(inputs, selected=ids_exact, tile_scores=tile_scores))

        def fp4_pipe():
            sp.fp4_indexer_fast(inputs, selected=ids_fast, workspace=ws)
            sp.attention_out(q, k, v, ids_fast, out)
        t_pipe = graph_time_us(fp4_pipe)
        torch.cuda.synchronize()
        assert torch.equal(ids_fast, ids_exact)
        row["us"]["FP4"] = {"selector": round(t_sel, 2), "selector_exact_kernels": round(t_exact, 2),
                            "selector_to_attention": round(t_pipe, 2)}
        pub = REFSEL_PUBLISHED[Skv]["FP4"]
        row["reference_published_us"]["FP4"] = {"selector": pub[0], "selector_to_p03": pub[1]}
        row["us"]["attention_only"] = round(graph_time_us(lambda: sp.attention_out(q, k, v, ids_fast, out)), 2)
        sp.device_status()
        print(json.dumps(row), flush=True)
        del q, k, v, out


def run_config(args):
    """Configurations 1, 3, 4, 5: indexer -> lists -> attention operator, stage by stage.
    With N > 1 ranks the (batch, KV-head) groups are dealt to the ranks (strong scaling, no
    collective); --kv-split R additionally splits the KV range R ways inside each head shard
    and merges partial (O, LSE) over NCCL."""
    import torch
    import torch.distributed as dist
    import sparse_attention_b200_b200 as sp
    from sparse_attention_b200_b200 import sharding

    cfg = dict(CONFIGS[args.workload])
    if args.n:                       # shorter sequence of the same configuration (profiler captures)
        cfg["N"] = args.n
        cfg["topk"] = min(cfg["topk"], args.n // 128)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    kvs = max(1, args.kv_split)
    head_shards = world // kvs
    shard, kv_rank = rank // kvs, rank % kvs
    kv_group = None
    if kvs > 1:
        for s_ in range(head_shards):
            g_ = dist.new_group(list(range(s_ * kvs, (s_ + 1) * kvs)))
            if s_ == shard:
                kv_group = g_

    B, Hq, Hkv, N, topk = cfg["B"], cfg["Hq"], cfg["Hkv"], cfg["N"], cfg["topk"]
    G = Hq // Hkv
    g0, g1 = sharding.group_range(B * Hkv, head_shards, shard)
    ng = g1 - g0                                    # this rank's problem: batch ng, Hq G, Hkv 1
    gen = torch.Generator(device=dev).manual_seed(17 + shard)
    q = torch.empty((ng, G, N, 128), dtype=torch.bfloat16, device=dev)
    k = torch.empty((ng, 1, N, 128), dtype=torch.bfloat16, device=dev)
    v = torch.empty((ng, 1, N, 128), dtype=torch.bfloat16, device=dev)
    fill_normal_bf16(q, gen)
    fill_normal_bf16(k, gen, cfg["k_offset"])
    fill_normal_bf16(v, gen)
    nb = N // 128

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stages = {}
    steps, warmup = args.steps, max(args.warmup, 3)
    # ---------------- indexer
    if cfg["indexer"] in ("r1", "r4"):
        r = 1 if cfg["indexer"] == "r1" else 4
        sel = sp.SummarySelector(q, k, r, topk=topk, keep_scores=False)
        stages["indexer_pool_ms"] = timed(sel.prepare, steps, warmup, barrier)
        if N <= 131072:      # the exact CUDA-core selector is only timed where it takes milliseconds
            stages["indexer_select_exact_ms"] = timed(sel.score, min(steps, 3), 1, barrier)
        stages["indexer_ms"] = timed(sel.run_fast, steps, warmup, barrier)     # pool + tensor-core select
        stages["indexer_fallback_lists"] = sel.fallback_lists()
        ids = sel.ids
        pool_bytes = (q.numel() + k.numel()) * 2 * (1 + r / 128.0)
        stages["indexer_pool_gbs"] = pool_bytes / stages["indexer_pool_ms"] / 1e6
        stages["indexer_gbs"] = pool_bytes / stages["indexer_ms"] / 1e6
        stages["indexer_score_flop"] = 2.0 * ng * (G * nb * r) * (nb * r) * 128
    else:
        hidx = 1                                   # one index vector per (token, KV head) = mean of the group
        qc = qs = kc = ks = None

        def quant():
            nonlocal qc, qs, kc, ks
            qc, qs = sp.quantize_queries(q, hidx)
            kc, ks = sp.quantize_keys(k)
        stages["quantize_ms"] = timed(quant, steps, warmup, barrier)
        inputs = sp.prepare_fp4_inputs(qc, kc, qs, ks, batch_size=ng, len_q=N, len_kv=N)
        ids = torch.empty((ng, 1, nb, topk), dtype=torch.int32, device=dev)
        tile_scores = torch.empty((ng, 1, nb, nb), dtype=torch.float32, device=dev)
        stages["indexer_exact_ms"] = timed(lambda: sp.fp4_indexer(inputs, ids, tile_scores=tile_scores),
                                           1, 1, barrier)
        ws = sp.fp4_indexer_fast(inputs, ids)[1]
        stages["indexer_ms"] = timed(lambda: sp.fp4_indexer_fast(inputs, ids, workspace=ws), min(steps, 3), 1, barrier)
        stages["indexer_fallback_tiles"] = int(ws[4:8].view(torch.int32).item())
    # ---------------- attention
    fl_local = 4.0 * ng * G * N * (topk * 128) * 128
    if kvs > 1:
        lo, hi = sharding.kv_block_range(nb, kvs, kv_rank)
        k_loc = k[:, :, lo * 128:hi * 128].contiguous()
        v_loc = v[:, :, lo * 128:hi * 128].contiguous()
        split = sharding.KVSplit(kv_group)
        res = {}

        def attn():
            res["o"], res["l"] = split.run(q, k_loc, v_loc, ids, nb)
        fl_local /= kvs
    elif cfg["op"] == "kv_centric":
        prep = sp.Prepared(q, k, v, ids, nseg=args.segments, partial="bf16")
        stages["kv_metadata_ms"] = timed(prep.metadata, steps, warmup, barrier)
        stages["kv_main_ms"] = timed(prep.main, steps, warmup, barrier)
        stages["kv_combine_ms"] = timed(prep.combine, steps, warmup, barrier)
        rows = ng * G * N
        comb_bytes = rows * (args.segments * (256 + 4) + 256 + 4)
        stages["kv_combine_gbs"] = comb_bytes / stages["kv_combine_ms"] / 1e6
        attn = prep.run
    else:
        out = torch.empty_like(q)
        lse = torch.empty((ng, G, N), dtype=torch.float32, device=dev)

        def attn():
            sp.attention_out(q, k, v, ids, out, None, lse)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_attn = timed(attn, steps, warmup, barrier)
    clocks = sampler.stop() if rank == 0 else None
    sp.device_status()
    t = torch.tensor([ms_attn, stages.get("indexer_ms", 0.0)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_attn, ms_idx = t.tolist()
    total_flops = 4.0 * B * Hq * N * (topk * 128) * 128
    if rank == 0:
        peak_tf, peak_gbs, peak_src = measured_peaks()
        value = total_flops / (ms_attn * 1e-3) / 1e12
        per_gpu = value / world
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": ms_attn, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded N(0,1), K block offsets per config)",
                "config": {"workload": args.workload, **{kk: vv for kk, vv in cfg.items()}, "d": 128,
                           "sharding": f"{head_shards} head-group shard(s) x {kvs} KV range(s)",
                           "kv_segments": args.segments if cfg["op"] == "kv_centric" else None},
                "pct_bf16_peak": 100.0 * per_gpu / peak_tf, "indexer_ms": ms_idx,
                "stages_rank0": stages,
                "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak_tf, "unit": "TFLOP/s",
                             "frac": per_gpu / peak_tf, "traffic": None, "peak_source": peak_src,
                             "kernel": "q_centric_kernel", "hbm_peak_gbs": peak_gbs},
                "clocks": clocks}
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
    ap.add_argument("--workload", default="c2", choices=["c2", "kvtoken", "refcmp", "refsel"] + sorted(CONFIGS),
                    help="c2 (default) is the headline workload; c1/c3/c4/c5 run indexer + operator stage by stage")
    ap.add_argument("--kv-split", type=int, default=1, help="KV ranges per head shard (c5 only, needs --gpus >= 2)")
    ap.add_argument("--n", type=int, default=0, help="override the token count of c1/c3/c4/c5 (small profiler cases)")
    ap.add_argument("--segments", type=int, default=4, help="KV-range segments of the KV-centric operator (c4)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "kvtoken":
        run_kv_token(args)
    elif args.workload == "refcmp":
        run_refcmp(args)
    elif args.workload == "refsel":
        run_refsel(args)
    elif args.workload != "c2":
        run_config(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
