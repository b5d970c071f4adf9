#!/usr/bin/env python
"""Headline benchmark: block-sparse attention forward, selected-block TFLOP/s, and indexer ms.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload c1..c5]

Default workload at every N: the 1 Mi-token configuration (B=1, Hq=64, Hkv=8, N=1048576, d=128,
bf16, K with per-block offsets, R4 indexer, top-64 of 8192 KV blocks; 38.7 GB of q, k, v, out). The
eight KV-head groups are dealt to the ranks (8 / 4 / 2 / 1 groups per GPU at 1 / 2 / 4 / 8 GPUs,
no data-path collective): STRONG scaling. A step is one pass of the Q-centric (GQA) attention
kernel over all groups of the rank; the indexer that produced the lists is timed beside it.

value    = selected-block FLOPs of the whole job / device time (max over ranks), inputs in HBM
e2e      = same metric with HOST (pinned) q, k, v, block_idx copied in and out + lse copied back
           inside the timed region, through HostPipeline -> the C ABI
roofline = tensor-pipe roofline of the attention kernel against the measured BF16 peak
indexer  = indexer_ms with its own roofline (HBM bytes and score FLOPs, binding roof named)
parity   = sampled lists and output blocks of every rank against the CPU oracle (outside the
           timed region; the oracle is only ever the checker)
configs  = (N = 1) the other configurations, stage by stage, in the same process
kv_split = (N >= 2) the same workload with the KV range split two ways inside each head shard
           and partial (O, LSE) merged over NVLink: NCCL send/recv + Combine, and the merge kernel
           that loads the peer's rows itself; the record's figure is the faster form
cpu_baseline = CPU oracle (gather formulation of the reference's masked-attention computation)
           on a bounded sample; `--impl reference` times that CPU path alone on all host cores.
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
HEADLINE = "c5"
CONFIGS = {
    # B, Hq, Hkv, N, topk, indexer (None = seeded random sorted lists), operator, K block-offset sigma
    "c1": dict(B=1, Hq=8, Hkv=8, N=4096, topk=8, indexer="r1", op="q_centric", k_offset=0.5),
    "c2": dict(B=1, Hq=32, Hkv=32, N=32768, topk=16, indexer=None, op="q_centric", k_offset=0.0),
    "c3": dict(B=2, Hq=64, Hkv=8, N=65536, topk=32, indexer="r4", op="q_centric", k_offset=0.5),
    "c4": dict(B=1, Hq=64, Hkv=4, N=131072, topk=64, indexer="fp4", op="kv_centric", k_offset=0.0),
    "c5": dict(B=1, Hq=64, Hkv=8, N=1048576, topk=64, indexer="r4", op="q_centric", k_offset=0.5),
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the attention kernel, from one
# Nsight Compute capture per shape. c5: captured at N = 524288 (136.5 GB read + 10.8 GB written for
# the 8 groups) and doubled: the K + V of a group exceed the L2 at both sizes, so the gathered
# tiles miss at the same rate and the traffic grows with the token count. None = not captured.
NCU_TRAFFIC_BYTES = {"c2": 1.145e9, "c5": 2.946e11}


def attention_flops(cfg, groups=None):
    g = cfg["Hq"] // cfg["Hkv"]
    groups = cfg["B"] * cfg["Hkv"] if groups is None else groups
    return 4.0 * groups * g * cfg["N"] * (cfg["topk"] * 128) * 128


def attention_bytes(cfg, groups=None):
    """Compulsory HBM bytes of the attention step: Q + O + K + V + ids + LSE."""
    g = cfg["Hq"] // cfg["Hkv"]
    groups = cfg["B"] * cfg["Hkv"] if groups is None else groups
    n = cfg["N"]
    return groups * (2 * g * n * 256 + 2 * n * 256 + (n // 128) * cfg["topk"] * 4 + g * n * 4)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"bf16": float(d["bf16_tflops"]), "bf16_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm": float(d["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0,
            "source": "fallback (earlier measurement on this pool)"}


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


class Workload:
    """One rank's share of a configuration: the (batch, KV-head) groups [g0, g1) as a problem of
    batch = #groups, Hq = group size, Hkv = 1. Group `gid` is generated from seed 17000 + gid, so
    the data of a group does not depend on how many ranks share the job."""

    def __init__(self, name, cfg, g0, g1, dev):
        import torch
        self.name, self.cfg, self.g0, self.g1, self.dev = name, cfg, g0, g1, dev
        self.G = cfg["Hq"] // cfg["Hkv"]
        self.ng = g1 - g0
        n = cfg["N"]
        self.nb = n // 128
        self.q = torch.empty((self.ng, self.G, n, 128), dtype=torch.bfloat16, device=dev)
        self.k = torch.empty((self.ng, 1, n, 128), dtype=torch.bfloat16, device=dev)
        self.v = torch.empty((self.ng, 1, n, 128), dtype=torch.bfloat16, device=dev)
        for i, gid in enumerate(range(g0, g1)):
            gen = torch.Generator(device=dev).manual_seed(17000 + gid)
            fill_normal_bf16(self.q[i:i + 1], gen)
            fill_normal_bf16(self.k[i:i + 1], gen, cfg["k_offset"])
            fill_normal_bf16(self.v[i:i + 1], gen)
        self.ids = None
        self.stages = {}
        self.fp4 = None

    # ------------------------------------------------------------------ lists
    def build_lists(self, sp, steps, warmup, barrier, time_exact=False):
        """Runs (and times) the configuration's indexer; leaves the lists in self.ids."""
        import torch
        cfg, st = self.cfg, self.stages
        topk, n, nb, ng, G = cfg["topk"], cfg["N"], self.nb, self.ng, self.G
        if cfg["indexer"] is None:
            ids = torch.cat([make_ids({**cfg, "B": 1, "Hkv": 1}, 1017 + gid) for gid in range(self.g0, self.g1)])
            self.ids = ids.to(self.dev)
            return
        if cfg["indexer"] in ("r1", "r4"):
            r = 1 if cfg["indexer"] == "r1" else 4
            sel = sp.SummarySelector(self.q, self.k, r, topk=topk, keep_scores=False)
            st["indexer_pool_ms"] = timed(sel.prepare, steps, warmup, barrier)
            if time_exact and n <= 131072:   # the exact CUDA-core selector, where it takes milliseconds
                st["indexer_select_exact_ms"] = timed(sel.score, min(steps, 3), 1, barrier)
            st["indexer_ms"] = timed(sel.run_fast, steps, warmup, barrier)     # pool + tensor-core select
            st["indexer_select_ms"] = st["indexer_ms"] - st["indexer_pool_ms"]
            st["indexer_fallback_lists"] = sel.fallback_lists()
            st["indexer_bound_violations"], st["indexer_max_err_over_bound"] = sel.bound_stats()
            self.ids = sel.ids
            self.selector = sel
            st["indexer_bytes"] = (self.q.numel() + self.k.numel()) * 2 + self.ids.numel() * 4
            st["indexer_score_flop"] = 2.0 * ng * (G * nb * r) * (nb * r) * 128
        else:
            hidx = 1                                   # one index vector per (token, KV head) = mean of the group
            box = {}

            def quant():
                box["qc"], box["qs"] = sp.quantize_queries(self.q, hidx)
                box["kc"], box["ks"] = sp.quantize_keys(self.k)
            st["quantize_ms"] = timed(quant, steps, warmup, barrier)
            inputs = sp.prepare_fp4_inputs(box["qc"], box["kc"], box["qs"], box["ks"], batch_size=ng, len_q=n, len_kv=n)
            self.fp4 = inputs
            ids = torch.empty((ng, 1, nb, topk), dtype=torch.int32, device=self.dev)
            if time_exact:
                tile_scores = torch.empty((ng, 1, nb, nb), dtype=torch.float32, device=self.dev)
                st["indexer_exact_ms"] = timed(lambda: sp.fp4_indexer(inputs, ids, tile_scores=tile_scores), 1, 1, barrier)
                del tile_scores
            ws = sp.fp4_indexer_fast(inputs, ids)[1]
            st["indexer_ms"] = timed(lambda: sp.fp4_indexer_fast(inputs, ids, workspace=ws), steps, warmup, barrier)
            ws[:32].zero_()                                  # the counters accumulate: one clean call to read them
            sp.fp4_indexer_fast(inputs, ids, workspace=ws)
            st["indexer_fallback_tiles"] = int(ws[4:8].view(torch.int32).item())
            st["indexer_bound_violations"] = int(ws[12:16].view(torch.int32).item())
            st["indexer_max_err_over_bound"] = float(ws[16:20].view(torch.float32).item())
            self.ids = ids
            st["indexer_bytes"] = (ng * n * hidx + ng * n) * 72 + ids.numel() * 4
            st["indexer_bytes_with_quantize"] = st["indexer_bytes"] + (self.q.numel() + self.k.numel()) * 2
            st["indexer_score_flop"] = 2.0 * ng * hidx * n * n * 128

    # ------------------------------------------------------------------ operator
    def make_step(self, sp, segments):
        """Returns (step function, kernels per step). Outputs land in self.out / self.lse."""
        import torch
        cfg = self.cfg
        if cfg["op"] == "kv_centric":
            prep = sp.Prepared(self.q, self.k, self.v, self.ids, nseg=segments, partial="bf16")
            self.prepared = prep
            self.out, self.lse = prep.out, prep.out_lse
            return prep.run, 3
        self.out = torch.empty_like(self.q)
        self.lse = torch.empty((self.ng, self.G, cfg["N"]), dtype=torch.float32, device=self.dev)

        def step():
            sp.attention_out(self.q, self.k, self.v, self.ids, self.out, None, self.lse)
        return step, 1

    def time_operator_stages(self, steps, warmup, barrier):
        if self.cfg["op"] != "kv_centric":
            return
        prep, st = self.prepared, self.stages
        st["kv_metadata_ms"] = timed(prep.metadata, steps, warmup, barrier)
        st["kv_main_ms"] = timed(prep.main, steps, warmup, barrier)
        st["kv_combine_ms"] = timed(prep.combine, steps, warmup, barrier)
        rows = self.ng * self.G * self.cfg["N"]
        st["kv_combine_gbs"] = rows * (prep.nseg * (256 + 4) + 256 + 4) / st["kv_combine_ms"] / 1e6

    # ------------------------------------------------------------------ parity (oracle = checker only)
    def parity(self, max_blocks=3):
        """Sampled lists and output blocks against the CPU oracle, never inside a timed region.
        Samples: the first and the last group of the rank, first / last / middle query block."""
        import torch
        import oracle
        cfg, G, nb, topk = self.cfg, self.G, self.nb, self.cfg["topk"]
        rec = {"max_abs": 0.0, "mean_abs": 0.0, "lse_rel": 0.0, "ids_equal": True, "ids_checked": 0, "blocks": 0,
               "tolerance": {"max_abs": 2e-2, "mean_abs": 2e-3, "lse_rel": 1e-3}}
        groups = sorted({0, self.ng - 1})
        qbs = sorted({0, nb - 1, nb // 2 + 1 if nb > 2 else 0})[:max_blocks]
        for gi in groups:
            kc, vc = self.k[gi:gi + 1].cpu(), self.v[gi:gi + 1].cpu()
            # lists
            if cfg["indexer"] in ("r1", "r4"):
                r = 1 if cfg["indexer"] == "r1" else 4
                qh = torch.cat([self.q[gi:gi + 1, :, qb * 128:(qb + 1) * 128] for qb in qbs], dim=2).cpu()
                ref = oracle.summary_select(qh, kc, r, topk)[3]
                rec["ids_equal"] = rec["ids_equal"] and bool(torch.equal(self.ids[gi, 0, qbs].cpu(), ref[0, 0]))
                rec["ids_checked"] += len(qbs)
            elif cfg["indexer"] == "fp4":
                qb = qbs[-1]
                rows = slice(qb * 128, (qb + 1) * 128)
                rqc, rqs = oracle.quantize_queries(self.q[gi:gi + 1, :, rows].cpu(), 1)
                rkc, rks = oracle.quantize_keys(kc)
                tile = oracle.fp4_tile_scores(oracle.fp4_scores(rqc, rqs, rkc, rks, 1, 128, cfg["N"]), 1, 128)
                rec["ids_equal"] = rec["ids_equal"] and bool(
                    torch.equal(self.ids[gi, 0, qb].cpu(), oracle.stable_topk(tile, topk)[0, 0, 0]))
                rec["ids_checked"] += 1
            # output blocks: first / last head of the group
            for head in sorted({0, G - 1}):
                for qb in qbs:
                    rows = slice(qb * 128, (qb + 1) * 128)
                    ro, rl = oracle.gather_attention(self.q[gi:gi + 1, head:head + 1, rows].cpu(), kc, vc,
                                                     self.ids[gi:gi + 1, :, qb:qb + 1].cpu())
                    d = (self.out[gi:gi + 1, head:head + 1, rows].float().cpu() - ro).abs()
                    l = self.lse[gi:gi + 1, head:head + 1, rows].cpu()
                    rec["max_abs"] = max(rec["max_abs"], d.max().item())
                    rec["mean_abs"] = max(rec["mean_abs"], d.mean().item())
                    rec["lse_rel"] = max(rec["lse_rel"], ((l - rl).abs() / rl.abs().clamp_min(1.0)).max().item())
                    rec["blocks"] += 1
        rec["ok"] = bool(rec["ids_equal"] and rec["max_abs"] <= 2e-2 and rec["mean_abs"] <= 2e-3
                         and rec["lse_rel"] <= 1e-3)
        return rec


def merge_parity(records):
    out = dict(records[0])
    for r in records[1:]:
        for key in ("max_abs", "mean_abs", "lse_rel"):
            out[key] = max(out[key], r[key])
        out["ids_equal"] = out["ids_equal"] and r["ids_equal"]
        out["ids_checked"] += r["ids_checked"]
        out["blocks"] += r["blocks"]
        out["ok"] = out["ok"] and r["ok"]
    out["ranks"] = len(records)
    return out


def indexer_roofline(stages, ms, peaks):
    """Both roofs of the indexer; the one that needs more time at its peak binds."""
    if not ms or "indexer_bytes" not in stages:
        return None
    gbs = stages["indexer_bytes"] / ms / 1e6
    tfs = stages["indexer_score_flop"] / ms / 1e9
    t_hbm = stages["indexer_bytes"] / (peaks["hbm"] * 1e9)
    t_tc = stages["indexer_score_flop"] / (peaks["bf16"] * 1e12)
    bound = "hbm" if t_hbm >= t_tc else "tensor"
    rec = {"bound": bound, "hbm_gbs": gbs, "hbm_frac": gbs / peaks["hbm"], "score_tflops": tfs,
           "tensor_frac": tfs / peaks["bf16"], "frac": (gbs / peaks["hbm"]) if bound == "hbm" else tfs / peaks["bf16"],
           "algorithmic_bytes": stages["indexer_bytes"], "score_flop": stages["indexer_score_flop"],
           "peak_hbm_gbs": peaks["hbm"], "peak_bf16_tflops": peaks["bf16"]}
    if stages.get("indexer_select_ms"):        # the scoring + selection kernel alone (pooling is the HBM-bound part)
        sel = stages["indexer_score_flop"] / stages["indexer_select_ms"] / 1e9
        rec["select_score_tflops"] = sel
        rec["select_tensor_frac"] = sel / peaks["bf16"]
    return rec


def cpu_gather_sample(cfg, q, k, v, ids, budget_s, threads=None):
    """Oracle gather path over query blocks of ONE (batch, KV-head) group until the time budget is
    used. q [1,G,N,128], k/v [1,1,N,128], ids [1,1,N/128,topk] CPU tensors. -> (TFLOP/s, text)."""
    import torch
    import oracle
    torch.set_num_threads(threads or os.cpu_count() or 1)
    G, nb = q.shape[1], ids.shape[2]
    per_block = 4.0 * G * 128 * (cfg["topk"] * 128) * 128
    done, t_total = 0, 0.0
    chunk = max(1, min(64, nb))
    while done < nb and t_total < budget_s:
        blocks = range(done, min(nb, done + chunk))
        t0 = time.perf_counter()
        oracle.gather_attention(q, k, v, ids, q_blocks=blocks)
        t_total += time.perf_counter() - t0
        done += len(blocks)
    tf = done * per_block / t_total / 1e12
    total_blocks = cfg["B"] * cfg["Hkv"] * nb
    return tf, (f"{done} of {total_blocks} (KV-head group, query block) units x {G} heads, gather formulation, "
                f"{t_total:.1f} s; linear in the unit count (scale factor {total_blocks / done:.1f})")


def cpu_masked_sample(cfg, q, k, v, ids):
    """The reference's masked formulation (dense scores over ALL keys, then the block mask) on one
    query block of one group: what its CPU path costs per unit at this density."""
    import torch
    import oracle
    t0 = time.perf_counter()
    oracle.masked_attention(q[:, :, :128], k, v, ids[:, :, :1])
    dt = time.perf_counter() - t0
    useful = 4.0 * q.shape[1] * 128 * (cfg["topk"] * 128) * 128
    return {"value": useful / dt / 1e12, "unit": "TFLOP/s (selected-block FLOPs)", "seconds": dt,
            "sample": "1 (KV-head group, query block) unit, masked formulation over all keys"}


def cpu_group_inputs(cfg, gid=0):
    """Group `gid` of a configuration generated on the CPU (same distributions as the device data)."""
    import torch
    G, n = cfg["Hq"] // cfg["Hkv"], cfg["N"]
    gen = torch.Generator().manual_seed(17000 + gid)
    q = torch.randn((1, G, n, 128), generator=gen).to(torch.bfloat16)
    k = torch.randn((1, 1, n, 128), generator=gen)
    if cfg["k_offset"]:
        k = (k.view(1, 1, n // 128, 128, 128) + cfg["k_offset"] * torch.randn((1, 1, n // 128, 1, 128), generator=gen)) \
            .view(1, 1, n, 128)
    k = k.to(torch.bfloat16)
    v = torch.randn((1, 1, n, 128), generator=gen).to(torch.bfloat16)
    rng = random.Random(1017 + gid)
    nb = n // 128
    ids = torch.tensor([sorted(rng.sample(range(nb), cfg["topk"])) for _ in range(nb)], dtype=torch.int32) \
        .reshape(1, 1, nb, cfg["topk"])
    return q, k, v, ids


def run_reference(args):
    """CPU arm (rank 0 only): the oracle's gather formulation of the reference's torch computation
    on the headline workload; every step is a bounded sample of (group, query block) units. The
    lists are seeded random sorted lists (the CPU cost of a unit does not depend on which blocks
    are selected; running the 1 Mi-token indexer on the CPU is not part of this arm)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    name = args.workload
    cfg = dict(CONFIGS[name])
    if args.n:
        cfg["N"] = args.n
        cfg["topk"] = min(cfg["topk"], args.n // 128)
    cores = os.cpu_count() or 1
    q, k, v, ids = cpu_group_inputs(cfg)
    nb = cfg["N"] // 128
    import oracle
    torch.set_num_threads(cores)
    units = 16
    tfs, times = [], []
    for step in range(args.warmup + args.steps):
        # one bounded sample: `units` query blocks of the group, a different window every step
        lo = (step * units) % max(1, nb - units + 1)
        done = min(nb, lo + units) - lo
        t0 = time.perf_counter()
        oracle.gather_attention(q, k, v, ids, q_blocks=range(lo, lo + done))
        dt = time.perf_counter() - t0
        if step >= args.warmup:
            times.append(dt)
            tfs.append(done * 4.0 * q.shape[1] * 128 * (cfg["topk"] * 128) * 128 / dt / 1e12)
    value = statistics.mean(tfs)
    total_units = cfg["B"] * cfg["Hkv"] * nb
    sample = (f"per step: {units} of {total_units} (KV-head group, query block) units x {q.shape[1]} heads, gather "
              f"formulation of the reference's torch computation; linear in the unit count "
              f"(scale factor {total_units / units:.0f}); host has {cores} cores")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.mean(times),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic (seeded N(0,1) q/k/v, K block offsets per config, seeded sorted block lists)",
            "config": config_record(name, cfg),
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def config_record(name, cfg):
    return {"workload": name, "B": cfg["B"], "Hq": cfg["Hq"], "Hkv": cfg["Hkv"], "N": cfg["N"], "topk": cfg["topk"],
            "indexer": cfg["indexer"] or "none (seeded sorted lists)", "operator": cfg["op"]}


def run_e2e(sp, wl, barrier, steps):
    """Host (pinned) buffers in and out through HostPipeline -> C ABI, copies inside the timed
    region; staged through the workload's own device buffers. Also times the same copies with the
    kernel left out: the share of the end-to-end time that is the host link."""
    import torch
    dev = wl.dev

    def pinned_copy(t):
        h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        h.copy_(t)
        return h
    hq_, hk_, hv_, hi_ = (pinned_copy(t) for t in (wl.q, wl.k, wl.v, wl.ids))
    hout = torch.empty(wl.out.shape, dtype=wl.out.dtype, pin_memory=True)
    hlse = torch.empty(wl.lse.shape, dtype=wl.lse.dtype, pin_memory=True)
    h2d = sum(t.numel() * t.element_size() for t in (hq_, hk_, hv_, hi_))
    d2h = sum(t.numel() * t.element_size() for t in (hout, hlse))
    cfg = wl.cfg
    pipe = sp.HostPipeline(wl.ng, wl.G, 1, cfg["N"], cfg["N"], cfg["topk"], dev, chunks=max(8, wl.ng),
                           buffers=(wl.q, wl.k, wl.v, wl.ids, wl.out, wl.lse))
    torch.cuda.synchronize()

    def run(n, copy_only):
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(n):
            pipe.run(hq_, hk_, hv_, hi_, hout, hlse, copy_only=copy_only)
        f1.record()
        barrier()
        return f0.elapsed_time(f1) / n
    run(1, False)
    e2e_ms = run(steps, False)
    copy_ms = run(max(1, steps // 2), True)
    return {"ms": e2e_ms, "copy_only_ms": copy_ms, "steps": steps, "h2d": h2d, "d2h": d2h, "chunks": pipe.chunks}


def kv_split_record(sp, sharding, dist, name, cfg, world, rank, dev, barrier, steps):
    """The same workload with 2 KV ranges inside each head shard: every rank of a pair holds the
    pair's groups and half of the KV rows, filters the lists to its range, runs the same kernel and
    the pair merges partial (O, LSE): with NCCL send/recv + the Combine kernel, with the peer-memory merge
    kernel (same rows bit for bit), and chunk by chunk (the exchange of one chunk of two heads under the
    attention of the next). The merged chunks are compared with the oracle on sampled blocks."""
    import torch
    import oracle
    kvs = 2
    head_shards = world // kvs
    shard, kv_rank = rank // kvs, rank % kvs
    kv_group = None
    for s_ in range(head_shards):
        g_ = dist.new_group(list(range(s_ * kvs, (s_ + 1) * kvs)))
        if s_ == shard:
            kv_group = g_
    g0, g1 = sharding.group_range(cfg["B"] * cfg["Hkv"], head_shards, shard)
    wl = Workload(name, cfg, g0, g1, dev)
    wl.build_lists(sp, 1, 1, barrier)
    nb, n, G = wl.nb, cfg["N"], wl.G
    lo, hi = sharding.kv_block_range(nb, kvs, kv_rank)
    k_loc = wl.k[:, :, lo * 128:hi * 128].contiguous()
    v_loc = wl.v[:, :, lo * 128:hi * 128].contiguous()
    split = sharding.KVSplit(kv_group)
    res = {}

    def step():
        res["m"] = split.run_pipelined(wl.q, k_loc, v_loc, wl.ids, nb, heads_per_chunk=2)

    def step_unpipelined():
        res["u"] = split.run(wl.q, k_loc, v_loc, wl.ids, nb)
    ms_plain = timed(step_unpipelined, steps, 2, barrier)
    # the same merge over peer memory: the Combine kernel reads the other rank's partial rows over NVLink itself
    peer = {}
    try:
        ex = sharding.PeerExchange(wl.q.shape[0] * wl.q.shape[1] * wl.q.shape[2], dev, kv_group)
    except Exception as e:          # raised on every rank of the pair alike (no IPC / peer access between the GPUs)
        ex, peer = None, {"unavailable": str(e)[:200]}
    def arm_ok():
        # status word of every rank of the job, read together: either all ranks keep an arm's result or none does
        code = sp.lib().sparse_b200_device_status(1)
        t_ = torch.tensor([1 if code != 0 else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(t_, op=dist.ReduceOp.MAX)
        return t_.item() == 0, code
    if ex is not None:
        def step_peer():
            res["p"] = split.run_peer(ex, wl.q, k_loc, v_loc, wl.ids, nb)

        def step_scatter():
            res["s"] = split.run_scatter(ex, wl.q, k_loc, v_loc, wl.ids, nb)
        ms_p = timed(step_peer, steps, 2, barrier)
        ok_p, code = arm_ok()
        if ok_p:
            peer["ms_per_step"] = ms_p
            peer["identical_to_send_recv"] = bool(torch.equal(res["p"][0], res["u"][0]) and torch.equal(res["p"][1], res["u"][1]))
            # ... and with the transfer inside the attention kernel: tiles stored straight into the merging rank's memory
            ms_s = timed(step_scatter, steps, 2, barrier)
            ok_s, code = arm_ok()
            if ok_s:
                peer["scatter_ms_per_step"] = ms_s
                peer["scatter_identical"] = bool(torch.equal(res["s"][0], res["u"][0]) and torch.equal(res["s"][1], res["u"][1]))
            else:
                peer["scatter_failed"] = f"a bounded wait ran out on some rank (status here 0x{code:x})"
        else:
            peer = {"unavailable": f"a bounded wait ran out on some rank (status here 0x{code:x})"}
        res.pop("p", None)
        res.pop("s", None)
        ex.close()
    res.pop("u", None)
    ms = timed(step, max(1, steps // 2), 1, barrier)
    sp.device_status()
    # parity of the chunks this rank merged: first and last head of the first and last owned chunk
    plan = split.chunks(wl.q, 2)
    owned = sorted(res["m"])
    par = {"max_abs": 0.0, "mean_abs": 0.0, "lse_rel": 0.0, "blocks": 0}
    for c in sorted({owned[0], owned[-1]}):
        gi, h0, nh = plan[c]
        o_c, l_c = res["m"][c]
        for head, qb in ((h0, 0), (h0 + nh - 1, nb - 1)):
            s0 = qb * 128
            ro, rl = oracle.gather_attention(wl.q[gi:gi + 1, head:head + 1, s0:s0 + 128].cpu(), wl.k[gi:gi + 1].cpu(),
                                             wl.v[gi:gi + 1].cpu(), wl.ids[gi:gi + 1, :, qb:qb + 1].cpu())
            local = (head - h0) * n + s0
            d = (o_c[local:local + 128].float().cpu() - ro[0, 0]).abs()
            l = l_c[local:local + 128].cpu()
            par["max_abs"] = max(par["max_abs"], d.max().item())
            par["mean_abs"] = max(par["mean_abs"], d.mean().item())
            par["lse_rel"] = max(par["lse_rel"], ((l - rl[0, 0]).abs() / rl[0, 0].abs().clamp_min(1.0)).max().item())
            par["blocks"] += 1
    t = torch.tensor([ms, par["max_abs"], par["mean_abs"], par["lse_rel"], ms_plain, peer.get("ms_per_step", 0.0),
                      0.0 if peer.get("identical_to_send_recv", True) else 1.0, peer.get("scatter_ms_per_step", 0.0),
                      0.0 if peer.get("scatter_identical", True) else 1.0], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, mx, mean, lrel, ms_plain, ms_peer, peer_differs, ms_scatter, scatter_differs = t.tolist()
    flops = attention_flops(cfg)
    forms = {"send_recv": ms_plain}
    scatter = {}
    if "ms_per_step" in peer:
        peer = {"ms_per_step": ms_peer, "value": flops / (ms_peer * 1e-3) / 1e12, "unit": "TFLOP/s",
                "identical_to_send_recv": not peer_differs,
                "how": "partials stay in IPC-mapped exchange memory, ready / done flag words, combine_peer_kernel loads "
                       "the peer's rows over NVLink (no NCCL call on the data path)"}
        if not peer_differs:
            forms["peer_merge"] = ms_peer
        if ms_scatter > 0:
            scatter = {"ms_per_step": ms_scatter, "value": flops / (ms_scatter * 1e-3) / 1e12, "unit": "TFLOP/s",
                       "identical_to_send_recv": not scatter_differs,
                       "how": "the attention kernel's TMA stores carry every finished tile into the exchange memory of "
                              "the rank that merges it (NVLink, under the computation); the merge reads local memory only"}
            if not scatter_differs:
                forms["scatter_merge"] = ms_scatter
        else:
            scatter = {"unavailable": "a bounded wait ran out on some rank"}
    best = min(forms, key=forms.get)
    ms_best = forms[best]
    return {"sharding": f"{head_shards} head-group shard(s) x {kvs} KV ranges", "ms_per_step": ms_best, "steps": steps,
            "value": flops / (ms_best * 1e-3) / 1e12, "unit": "TFLOP/s",
            "merge": f"{best} (below): the fastest of the forms that give the same rows bit for bit",
            "scatter_merge": scatter,
            "send_recv": {"ms_per_step": ms_plain, "value": flops / (ms_plain * 1e-3) / 1e12, "unit": "TFLOP/s",
                          "how": "NCCL send/recv of the owner's rows of (O, LSE) after the attention kernel, then the "
                                 "Combine kernel"},
            "peer_merge": peer,
            "ms_per_step_pipelined": ms,
            "pipelined": "chunks of two heads, a chunk's exchange on a side stream under the attention of the next chunk "
                         "(parity record below is of this form); slower when the persistent attention grid leaves "
                         "NCCL's copy kernels no SM",
            "parity": {"max_abs": mx, "mean_abs": mean, "lse_rel": lrel, "blocks": par["blocks"] * world,
                       "ok": bool(mx <= 2e-2 and mean <= 2e-3 and lrel <= 1e-3)}}


def sub_config(sp, name, dev, barrier, steps, segments):
    """One of the other configurations on one GPU, stage by stage (few steps each)."""
    import torch
    cfg = dict(CONFIGS[name])
    wl = Workload(name, cfg, 0, cfg["B"] * cfg["Hkv"], dev)
    wl.build_lists(sp, steps, 2, barrier, time_exact=True)
    step, kernels = wl.make_step(sp, segments)
    ms = timed(step, steps, 3, barrier)
    wl.time_operator_stages(steps, 2, barrier)
    sp.device_status()
    peaks = measured_peaks()
    fl = attention_flops(cfg)
    tf = fl / (ms * 1e-3) / 1e12
    rec = {"config": config_record(name, cfg), "attention_ms": ms, "tflops": tf, "frac_bf16_burst": tf / peaks["bf16"],
           "steps": steps, "kernels_per_step": kernels, "stages": wl.stages, "parity": wl.parity(max_blocks=2)}
    if "indexer_ms" in wl.stages:
        rec["indexer_ms"] = wl.stages["indexer_ms"]
        rec["indexer_roofline"] = indexer_roofline(wl.stages, wl.stages["indexer_ms"], peaks)
    del wl
    torch.cuda.empty_cache()
    return rec


def run_ours(args):
    import torch
    import torch.distributed as dist
    import sparse_attention_b200_b200 as sp
    from sparse_attention_b200_b200 import sharding

    name = args.workload
    cfg = dict(CONFIGS[name])
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
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    n_groups = cfg["B"] * cfg["Hkv"]
    g0, g1 = sharding.group_range(n_groups, world, rank)
    if g1 == g0:
        raise SystemExit(f"{name} has {n_groups} (batch, KV-head) groups: fewer than {world} ranks")
    wl = Workload(name, cfg, g0, g1, dev)
    steps, warmup = args.steps, max(args.warmup, 3)
    idx_steps = max(2, min(steps, 5))
    wl.build_lists(sp, idx_steps, 2, barrier, time_exact=args.kernel_only and name != "c5")
    step, kernels = wl.make_step(sp, args.segments)

    # ---------------- timed region: K attention steps, device-resident
    sampler = ClockSampler(local_rank)
    for _ in range(warmup):
        step()
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_region0 = time.time()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    barrier()
    t_region1 = time.time()
    ms_total = e0.elapsed_time(e1)
    sp.device_status()
    # sustained state: the same launches for at least 1.2 s (the power cap settles the clock within
    # a few hundred ms); when the timed region was that long already it is the sustained figure
    sustained_ms, sustained_window = ms_total / steps, ms_total * 1e-3
    if ms_total < 1200.0:
        reps = max(1, int(1200.0 / max(ms_total / steps, 1e-3)) + 1)
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s0.record()
        for _ in range(reps):
            step()
        s1.record()
        barrier()
        # the last half of the window: after the clock has settled
        sustained_ms = s0.elapsed_time(s1) / reps
        sustained_window = s0.elapsed_time(s1) * 1e-3
    clocks = sampler.stop((t_region0, t_region1)) if rank == 0 else None
    wl.time_operator_stages(idx_steps, 2, barrier)

    parity = wl.parity() if not args.kernel_only else None
    e2e = None
    if not args.kernel_only:
        e2e = run_e2e(sp, wl, barrier, max(2, min(steps, 3)))
        sp.device_status()

    idx_ms = wl.stages.get("indexer_ms", 0.0)
    t = torch.tensor([ms_total, sustained_ms, idx_ms, e2e["ms"] if e2e else 0.0, e2e["copy_only_ms"] if e2e else 0.0,
                      wl.stages.get("indexer_pool_ms", 0.0)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, sustained_ms, idx_ms, e2e_ms, copy_ms, pool_ms = t.tolist()
    parities = [parity]
    if world > 1 and parity is not None:
        parities = [None] * world
        dist.all_gather_object(parities, parity)
    ms_step = ms_total / steps
    total_flops = attention_flops(cfg)
    value = total_flops / (ms_step * 1e-3) / 1e12

    line = None
    if rank == 0:
        peaks = measured_peaks()
        local_flops = attention_flops(cfg, wl.ng)
        per_gpu = local_flops / (ms_step * 1e-3) / 1e12          # rank 0's share over the slowest rank's time
        per_gpu_sustained = local_flops / (sustained_ms * 1e-3) / 1e12
        traffic = NCU_TRAFFIC_BYTES.get(name)
        if traffic is not None and name == "c5":
            traffic = traffic * wl.ng / n_groups
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic (seeded N(0,1) q/k/v, K block offsets ~ N(0,0.5) where the config has them)",
                "config": {**config_record(name, cfg), "d": 128, "block": 128,
                           "sharding": f"{n_groups} (batch, KV-head) groups dealt to {world} rank(s), no collective",
                           "groups_per_gpu": wl.ng,
                           "l2": f"inputs ({attention_bytes(cfg, wl.ng) / 1e9:.1f} GB per GPU) exceed the 126 MB L2; "
                                 "no flush between steps"},
                "pct_bf16_peak": 100.0 * per_gpu / peaks["bf16"],
                "value_sustained": total_flops / (sustained_ms * 1e-3) / 1e12,
                "sustained": {"window_s": sustained_window, "per_gpu_tflops": per_gpu_sustained,
                              "frac_of_sustained_peak": per_gpu_sustained / peaks["bf16_sustained"],
                              "peak_sustained": peaks["bf16_sustained"]},
                "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["bf16"], "unit": "TFLOP/s",
                             "frac": per_gpu / peaks["bf16"], "traffic": traffic,
                             "algorithmic_bytes": attention_bytes(cfg, wl.ng), "algorithmic_flop": local_flops,
                             "peak_source": peaks["source"] + ", burst bf16",
                             "kernel": "q_centric_kernel" if cfg["op"] == "q_centric" else
                                       "split_segments + q_centric_kernel (partials) + combine",
                             "launches_timed": steps * kernels},
                "indexer_ms": idx_ms if idx_ms else None,
                "indexer": {"ms": idx_ms, "pool_ms": pool_ms, "select_ms": idx_ms - pool_ms,
                            "roofline": indexer_roofline(wl.stages, idx_ms, peaks),
                            "fallback_lists": wl.stages.get("indexer_fallback_lists",
                                                            wl.stages.get("indexer_fallback_tiles"))} if idx_ms else None,
                "stages_rank0": wl.stages,
                "parity": merge_parity(parities) if parities[0] is not None else None,
                "gpu_launches": steps * kernels, "clocks": clocks}
        if e2e:
            line["e2e"] = {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "h2d_bytes_per_step": e2e["h2d"],
                           "d2h_bytes_per_step": e2e["d2h"], "ms_per_step": e2e_ms, "steps": e2e["steps"],
                           "copy_only_ms_per_step": copy_ms, "frac_of_copy_ceiling": copy_ms / e2e_ms,
                           "bytes_are": "per GPU (rank 0)",
                           "how": f"pinned host q,k,v,block_idx in, out+lse back, {e2e['chunks']} chunks pipelined over "
                                  "three streams through the C ABI (HostPipeline); copy_only = the same copies "
                                  "with the kernel left out (what the host link allows)"}
    # ---------------- free the headline buffers, then the sub-records
    hold_q, hold_k, hold_v, hold_ids = None, None, None, None
    if rank == 0 and world == 1 and not args.kernel_only:
        # CPU baseline on group 0 of this very data (bounded sample)
        hold_q, hold_k, hold_v, hold_ids = wl.q[:1].cpu(), wl.k[:1].cpu(), wl.v[:1].cpu(), wl.ids[:1].cpu()
    del wl, step
    torch.cuda.empty_cache()
    if world >= 2 and world % 2 == 0 and name == "c5" and not args.kernel_only and not args.no_kv_split:
        rec = kv_split_record(sp, sharding, dist, name, cfg, world, rank, dev, barrier, max(2, min(steps, 3)))
        torch.cuda.empty_cache()
        if rank == 0:
            line["kv_split"] = rec
    if rank == 0 and world == 1 and not args.kernel_only:
        tf, sample = cpu_gather_sample(cfg, hold_q, hold_k, hold_v, hold_ids, budget_s=12.0)
        line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": sample,
                                "what": "oracle gather formulation (the reference's progression_validation.reference "
                                        "restated); the masked formulation on one unit is in `masked`",
                                "masked": cpu_masked_sample(cfg, hold_q, hold_k, hold_v, hold_ids)}
        del hold_q, hold_k, hold_v, hold_ids
        if name == HEADLINE and not args.no_configs:
            line["configs"] = {}
            for other in ("c1", "c2", "c3", "c4"):
                line["configs"][other] = sub_config(sp, other, dev, barrier, 5, args.segments)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


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


def run_peermerge(args):
    """One GPU's share of the peer-memory merge, with the "peers" in local memory: combine_peer_kernel over R = 2
    separate partial buffers (the kernel of KVSplit.run_peer; over NVLink its remote half is bound by the link) next
    to the Combine kernel on one rank-major buffer (the local merge of KVSplit.run_scatter). 1 Mi rows by default
    (--n overrides)."""
    import ctypes
    import torch
    import sparse_attention_b200_b200 as sp
    from sparse_attention_b200_b200 import _lib
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    rows, ranks = args.n or (1 << 20), 2
    gen = torch.Generator(device=dev).manual_seed(3)
    part = torch.randn((ranks, rows, 128), device=dev, generator=gen).to(torch.bfloat16)
    lses = torch.randn((ranks, rows), device=dev, generator=gen)
    out = torch.empty((rows, 128), dtype=torch.bfloat16, device=dev)
    out_lse = torch.empty((rows,), device=dev)
    ref = torch.empty_like(out)
    ref_lse = torch.empty_like(out_lse)
    L = sp.lib()
    arr = ctypes.c_void_p * ranks
    parts, ls = arr(*[part[r].data_ptr() for r in range(ranks)]), arr(*[lses[r].data_ptr() for r in range(ranks)])

    def peer():
        _lib.check(L.sparse_b200_combine_peer(parts, ls, None, 0, 1000, _lib.ptr(out), _lib.ptr(out_lse),
                                              ctypes.c_int64(rows), ranks, _lib.current_stream()))

    def plain():
        _lib.check(L.sparse_b200_combine(_lib.ptr(part), 0, _lib.ptr(lses), _lib.ptr(ref), _lib.ptr(ref_lse),
                                         ctypes.c_int64(rows), ranks, 1, _lib.current_stream()))
    sync = torch.cuda.synchronize
    steps = max(args.steps, 5)
    ms_peer = timed(peer, steps, 3, sync)
    ms_plain = timed(plain, steps, 3, sync)
    sp.device_status()
    peaks = measured_peaks()
    byts = rows * (ranks * 256 + ranks * 4 + 260)
    print(json.dumps({
        "metric": "merge of 2 partial (O, LSE) per row, bf16", "unit": "GB/s", "n_gpus": 1, "steps": steps,
        "config": {"workload": "peermerge", "rows": rows, "ranks": ranks,
                   "l2": f"{byts / 1e9:.2f} GB per launch exceed the 126 MB L2"},
        "combine_peer_kernel": {"ms": ms_peer, "gbs": byts / ms_peer / 1e6, "frac_hbm": byts / ms_peer / 1e6 / peaks["hbm"]},
        "combine_few_kernel": {"ms": ms_plain, "gbs": byts / ms_plain / 1e6, "frac_hbm": byts / ms_plain / 1e6 / peaks["hbm"]},
        "identical": bool(torch.equal(out, ref) and torch.equal(out_lse, ref_lse)),
        "algorithmic_bytes": byts}))


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
    # q and partials token-major: the reference's own pair (main_tm_out + combine_tm_out)
    prep_tt = sp.PreparedTokens(prep_tm.q, k, v, selected, q_token_major=True, partial_token_major=True)
    prep_tt.metadata()
    token_major["partials_token_major"] = {
        "main_ms": timed(prep_tt.main, args.steps, 3, barrier), "combine_ms": timed(prep_tt.combine, args.steps, 3, barrier),
        "ms": timed(prep_tt.run, args.steps, 3, barrier), "identical_output": bool(torch.equal(prep_tt.out, prep.out))}
    sp.device_status()
    del prep_tt
    same_box = reference_kv_centric(q, k, v, selected, prep, args.steps, barrier)
    fl = 4.0 * B * Hq * S * (topk * 128) * 128
    peaks = measured_peaks()
    peak_tf, peak_src = peaks["bf16"], peaks["source"]
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
    # the reference's own NVFP4 indexer (indexers/fp4/fp4.py:122-146): the vendored MiniMax MSA scorer
    # (CuTe DSL, compiled by nvidia-cutlass-dsl at the first call) + its tile_topk extension, copied
    # unmodified into baseline/_ref/fp4 and prebuilt by baseline/build_reference_kernels.py
    ref_fp4, ref_fp4_note = None, None
    fp4_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "fp4")
    topk_lib = os.path.join(fp4_dir, "build", "xomtention_tile_topk.so")
    if os.path.exists(topk_lib):
        try:
            import pathlib
            sys.path.insert(0, os.path.dirname(fp4_dir))
            import fp4 as ref_fp4_pkg
            from fp4 import fp4 as ref_fp4
            torch.ops.load_library(topk_lib)
            ref_fp4_pkg._load_extension = lambda: torch.ops.xomtention_tile_topk
            ref_fp4.MSA_CUTE_DIR = pathlib.Path(fp4_dir) / "vendor_minimax_msa"   # the vendored copy of the scorer
        except Exception as e:
            ref_fp4, ref_fp4_note = None, f"unavailable: {type(e).__name__}: {e}"
    else:
        ref_fp4_note = "unavailable: baseline/_ref/fp4 not built (python baseline/build_reference_kernels.py --ref ...)"
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
        sp.fp4_block_scores(inputs, exact=False)             # builds the index tensors once, outside the capture
        t_scorer = graph_time_us(lambda: sp.fp4_block_scores(inputs, exact=False))

        def fp4_pipe():
            sp.fp4_indexer_fast(inputs, selected=ids_fast, workspace=ws)
            sp.attention_out(q, k, v, ids_fast, out)
        t_pipe = graph_time_us(fp4_pipe)
        torch.cuda.synchronize()
        assert torch.equal(ids_fast, ids_exact)
        row["us"]["FP4"] = {"selector": round(t_sel, 2), "selector_exact_kernels": round(t_exact, 2),
                            "selector_to_attention": round(t_pipe, 2), "scorer_only_per_query_scores": round(t_scorer, 2)}
        pub = REFSEL_PUBLISHED[Skv]["FP4"]
        row["reference_published_us"]["FP4"] = {"selector": pub[0], "selector_to_p03": pub[1]}
        if ref_fp4 is not None:
            try:
                rin = ref_fp4.prepare_fp4_inputs(qc, kc, qs, ks, batch_size=B, len_q=Sq, len_kv=Skv)
                rsel = torch.empty((B, Hkv, Sq // 128, 16), dtype=torch.int32, device=dev)
                ref_fp4.fp4_indexer(rin, rsel)                      # compiles the scorer
                torch.cuda.synchronize()
                t_ref = graph_time_us(lambda: ref_fp4.fp4_indexer(rin, rsel))
                t_ref_scorer = graph_time_us(lambda: ref_fp4.fp4_block_scores(rin))
                torch.cuda.synchronize()
                same = (rsel == ids_fast).all(-1).float().mean().item()
                row.setdefault("reference_same_box_us", {})["FP4"] = {
                    "selector": round(t_ref, 2), "scorer_only": round(t_ref_scorer, 2),
                    "lists_with_identical_ids": round(same, 4)}
            except Exception as e:                                  # DSL version or compile trouble on this box
                ref_fp4_note = f"unavailable: {type(e).__name__}: {str(e)[:300]}"
                ref_fp4 = None
        if ref_fp4 is None:
            row.setdefault("reference_same_box_us", {})["FP4"] = ref_fp4_note
        row["us"]["attention_only"] = round(graph_time_us(lambda: sp.attention_out(q, k, v, ids_fast, out)), 2)
        sp.device_status()
        print(json.dumps(row), flush=True)
        del q, k, v, out


def run_varlen(args):
    """The ragged / paged / causal NVFP4 scorer (per-query page scores) on a prefill batch and on a decode
    batch (at most 8 new queries per request, group of 16 heads: the packed form), timed next to the
    reference's own scorer on the same tensors where baseline/_ref/fp4 holds it
    (indexers/fp4/vendor_minimax_msa/fp4_indexer_interface.py:745-1056, public scale layout)."""
    import numpy as np
    import torch
    import sparse_attention_b200_b200 as sp
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    vendor = os.path.join(ROOT, "baseline", "_ref", "fp4", "vendor_minimax_msa")
    ref_fn, ref_note = None, "unavailable: baseline/_ref/fp4 not present"
    if os.path.isdir(vendor):
        try:
            sys.path.insert(0, vendor)
            from fp4_indexer_interface import fp4_indexer_block_scores as ref_fn
        except Exception as e:
            ref_fn, ref_note = None, f"unavailable: {type(e).__name__}: {e}"
    rng = np.random.default_rng(7)
    batches = {"prefill": dict(hq=2, hk=1, q_lens=rng.integers(512, 4097, 8).tolist(), k_lens=rng.integers(4096, 16385, 8).tolist()),
               "decode": dict(hq=16, hk=1, q_lens=rng.integers(1, 9, 64).tolist(), k_lens=rng.integers(8192, 32769, 64).tolist())}

    def barrier():
        torch.cuda.synchronize()
    for name, bt in batches.items():
        hq, hk, q_lens, k_lens = bt["hq"], bt["hk"], bt["q_lens"], bt["k_lens"]
        pages_per = [(k + 127) // 128 for k in k_lens]
        total_q, total_pages = sum(q_lens), sum(pages_per)
        g = torch.Generator(device=dev).manual_seed(11)
        qp = torch.randint(256, (total_q, hq, 64), dtype=torch.uint8, device=dev, generator=g)
        kp = torch.randint(256, (total_pages, hk, 128, 64), dtype=torch.uint8, device=dev, generator=g)
        qs = (torch.rand((total_q, hq, 8), device=dev, generator=g) + 0.5).to(torch.float8_e4m3fn)
        ks = (torch.rand((total_pages, hk, 128, 8), device=dev, generator=g) + 0.5).to(torch.float8_e4m3fn)
        cu = lambda xs: torch.tensor([0] + list(np.cumsum(xs)), dtype=torch.int32, device=dev)
        cu_q, cu_k, cu_p = cu(q_lens), cu(k_lens), cu(pages_per)
        kv_idx = torch.randperm(total_pages, device=dev, generator=g).to(torch.int32)
        flop = 2.0 * 128 * hq * sum(q * p_ * 128 for q, p_ in zip(q_lens, pages_per))
        row = {"workload": "varlen", "batch": name, "requests": len(q_lens), "Hq": hq, "Hk": hk, "total_q": total_q,
               "total_pages": total_pages, "score_flop": flop, "ms": {}, "reference_same_box_ms": {}}
        for causal in (False, True):
            key = "causal" if causal else "full"
            fn = lambda: sp.fp4_block_scores_varlen(qp, kp, qs, ks, cu_q, cu_k, cu_p, max_seqlen_q=max(q_lens),
                                                    max_seqlen_k=max(k_lens), kv_indices=kv_idx, causal=causal)
            row["ms"][key] = timed(fn, args.steps, 3, barrier)
            fast = lambda: sp.fp4_block_scores_varlen(qp, kp, qs, ks, cu_q, cu_k, cu_p, max_seqlen_q=max(q_lens),
                                                      max_seqlen_k=max(k_lens), kv_indices=kv_idx, causal=causal, exact=False)
            row.setdefault("ms_tensor_core", {})[key] = timed(fast, args.steps, 3, barrier)
            exact_out, fast_out = fn(), fast()
            fin = torch.isfinite(exact_out)
            row.setdefault("tensor_core_vs_exact", {})[key] = {
                "max_abs": (fast_out[fin] - exact_out[fin]).abs().max().item(),
                "same_inf_pattern": bool(torch.equal(torch.isinf(fast_out), torch.isinf(exact_out)))}
            if ref_fn is not None:
                try:
                    rf = lambda: ref_fn(qp, kp, qs, ks, cu_q, cu_k, cu_p, max_seqlen_q=max(q_lens), max_seqlen_k=max(k_lens),
                                        kv_indices=kv_idx, fp4_format="nvfp4", causal=causal, scale_layout="public")
                    theirs = rf()
                    row["reference_same_box_ms"][key] = timed(rf, args.steps, 3, barrier)
                    ours = fn()
                    fin = torch.isfinite(theirs)
                    row.setdefault("max_abs_diff_vs_reference", {})[key] = (ours[fin] - theirs[fin]).abs().max().item()
                    row.setdefault("same_inf_pattern", {})[key] = bool(torch.equal(torch.isinf(ours), torch.isinf(theirs)))
                except Exception as e:
                    row["reference_same_box_ms"][key] = f"unavailable: {type(e).__name__}: {str(e)[:200]}"
            else:
                row["reference_same_box_ms"][key] = ref_note
        sp.device_status()
        print(json.dumps(row), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident timing only (used for profiler captures): no e2e, parity, CPU baseline "
                         "or sub-records")
    ap.add_argument("--workload", default=HEADLINE, choices=["kvtoken", "refcmp", "refsel", "varlen", "peermerge"] + sorted(CONFIGS),
                    help=f"{HEADLINE} (default) is the headline workload; c1..c4 run the same way on their own shapes")
    ap.add_argument("--no-configs", action="store_true", help="skip the c1..c4 sub-record of the headline run")
    ap.add_argument("--no-kv-split", action="store_true", help="skip the KV-split sub-record of multi-GPU runs")
    ap.add_argument("--n", type=int, default=0, help="override the token count of the workload (small profiler cases)")
    ap.add_argument("--segments", type=int, default=4, help="KV-range segments of the KV-centric operator (c4)")
    args = ap.parse_args()
    if args.workload == "kvtoken":
        run_kv_token(args)
    elif args.workload == "refcmp":
        run_refcmp(args)
    elif args.workload == "refsel":
        run_refsel(args)
    elif args.workload == "varlen":
        run_varlen(args)
    elif args.workload == "peermerge":
        run_peermerge(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
