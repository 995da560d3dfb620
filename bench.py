#!/usr/bin/env python
"""Benchmark of the compressed-KV decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (default): the Llama-3.1-8B-shaped decode configuration -- 32 layers, 32 query
heads, 8 KV heads, head_dim 128, KIVI 4-bit keys (per channel) and values (per token),
group 32, a 128-token bf16 residual window, batch 16, context 32768, bf16 activations,
K/V ~ N(0,1) with 4 outlier channels per head scaled x20. A "step" is one decode step of the
attention path: for each layer, fused dequant + attention of one new query token over that
layer's packed cache (no model weights are involved).

Scaling across GPUs is STRONG: the one batch of 16 sequences is partitioned over the ranks by
(batch, kv head) unit (128 units -> 128/N per GPU; `veloxquant_mlx_b200.sharding`). Attention
needs no collective; each layer's output rows are delivered to every rank by the attention
kernel's merge step itself (stores to peer-mapped buffers + an arrival flag with a bounded
wait), or with `--gather nccl` by an NCCL all-gather on a side stream. The per-step kernel
sequence is captured once into a CUDA graph and replayed.

One JSON line is printed by rank 0. `value` is KV GB/s: algorithmic bytes of packed codes,
scales, zero-points, residual window, queries and outputs that one step of the WHOLE batch
must move, divided by the step time (max over ranks; median over repeated blocks of
`--steps` steps). `e2e` is the same metric through the cache interface with host buffers
(query and new K/V token copied in, output copied out, every step; the run crosses
quantize-on-append flushes). `extra` carries further figures measured in the same run: the
same shape at 2 bits, quantize-on-append throughput, the Qwen2.5-32B-shaped prefill + decode
configuration, the weak-scaling (replicated batch) figure, `quantize_vq` and RaBitQ.
`--impl reference` times the CPU oracle (a NumPy restatement of the reference's path; the
reference's own MLX code cannot be installed on this box) on a bounded sample.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fused dequant-SDPA decode KV GB/s"
UNIT = "GB/s"


# ----------------------------------------------------------------------------- workload
def workload(args):
    w = dict(name="llama3.1-8b-decode-kivi4", layers=32, H_q=32, H_kv=8, D=128, bits=4, group=32,
             residual=128, batch=16, ctx=32768, dtype="bf16")
    if args.workload == "c1":
        w.update(name="kivi2-single-layer", layers=1, bits=2, batch=1, ctx=4096, dtype="f16")
    elif args.workload == "c5":
        w.update(name="qwen2.5-32b-decode-kivi2", layers=64, H_q=40, bits=2, batch=4, ctx=16384 + 256)
    for k in ("layers", "batch", "ctx", "bits"):
        v = getattr(args, k)
        if v is not None:
            w[k] = v
    w["n_quant"] = max(0, (w["ctx"] - w["residual"]) // w["group"]) * w["group"]
    w["n_res"] = w["ctx"] - w["n_quant"]
    return w


def config_of(w, n_gpus):
    """The `config` object of the JSON line; both arms print the same keys and values."""
    units = w["batch"] * w["H_kv"]
    return {"workload": w["name"], **{k: w[k] for k in ("layers", "batch", "ctx", "bits", "group", "residual", "H_q", "H_kv", "D")},
            "global_batch": w["batch"],
            "parallelism": f"{units} (batch, kv head) units block-partitioned over {n_gpus} GPU(s)",
            "l2": "inputs larger than L2: each layer's packed KV is read once per step and the layers are distinct buffers"}


def algorithmic_bytes_per_layer(w, batch=None, bits=None, n_quant=None, n_res=None):
    """Bytes one layer's attend must move: packed codes + fp32 params + residual + q + out."""
    B = w["batch"] if batch is None else batch
    b = w["bits"] if bits is None else bits
    D, g = w["D"], w["group"]
    Sq = w["n_quant"] if n_quant is None else n_quant
    R = w["n_res"] if n_res is None else n_res
    per_head = (Sq * D * b // 8 + (Sq // g) * D * 8) + (Sq * D * b // 8 + Sq * (D // g) * 8) + 2 * R * D * 2
    return B * (w["H_kv"] * per_head + 2 * w["H_q"] * D * 2)


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons (NVML in-process, else nvidia-smi) while the timed
    region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.nvml = None

    def _start_nvml(self):
        import pynvml

        pynvml.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        phys = self.gpu_index
        if vis:
            ids = [v for v in vis.split(",") if v.strip()]
            if self.gpu_index < len(ids) and ids[self.gpu_index].strip().isdigit():
                phys = int(ids[self.gpu_index])
        h = pynvml.nvmlDeviceGetHandleByIndex(phys)
        self.nvml = {"sm": [], "power": [], "reasons": set(), "stop": False,
                     "max": pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)}
        bits = {"hw_slowdown": pynvml.nvmlClocksEventReasonHwSlowdown,
                "hw_thermal_slowdown": pynvml.nvmlClocksEventReasonHwThermalSlowdown,
                "sw_thermal_slowdown": pynvml.nvmlClocksEventReasonSwThermalSlowdown,
                "sw_power_cap": pynvml.nvmlClocksEventReasonSwPowerCap}

        def poll():
            while not self.nvml["stop"]:
                try:
                    self.nvml["sm"].append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                    self.nvml["power"].append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
                    r = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                    for nm, bit in bits.items():
                        if r & bit:
                            self.nvml["reasons"].add(nm)
                except Exception:
                    pass
                time.sleep(0.02)

        self.thread = threading.Thread(target=poll, daemon=True)
        self.thread.start()

    def start(self):
        try:
            self._start_nvml()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    @staticmethod
    def _summary(sm, mx, power, reasons, source):
        out = {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
               "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons),
               "source": source}
        if sm:
            # samples binned by SM clock (100 MHz bins): how long the run spent at which clock
            bins = {}
            for v in sm:
                key = int(v // 100) * 100
                bins[key] = bins.get(key, 0) + 1
            out["sm_mhz_bins"] = {f"{k}-{k + 99}": n for k, n in sorted(bins.items())}
        return out

    def stop(self):
        if self.nvml is not None:
            self.nvml["stop"] = True
            self.thread.join(timeout=2)
            return self._summary(self.nvml["sm"], float(self.nvml["max"]), self.nvml["power"], self.nvml["reasons"], "nvml")
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return self._summary(sm, max(mx) if mx else None, power, reasons, "nvidia-smi")


def ncu_traffic(w):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the attend kernel, read from
    the data file kept beside the ncu summary of that capture (same per-layer shape as the
    default workload); None for shapes that were not captured."""
    path = os.path.join(ROOT, "profiles", "kivi_attend_mma_llama8b_decode.traffic.json")
    try:
        rec = json.load(open(path))
    except (OSError, ValueError):
        return None
    shape = [w["batch"], w["ctx"], w["H_kv"], w["H_q"], w["D"], w["group"], w["residual"]]
    if rec.get("shape") != shape:
        return None
    per_bits = rec.get("dram_bytes_per_launch", {}).get(str(w["bits"]))
    return None if per_bits is None else int(per_bits["read"]) + int(per_bits["write"])


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["bf16_tflops"]), "measured (burst)"
    except Exception:
        return 1590.0, "fallback"


# ----------------------------------------------------------------------------- CPU oracle arm
def cpu_reference_sample(w, seconds_budget=20.0, seed=0):
    """Time the oracle (NumPy restatement of the reference's KIVI quantize + attend) on a
    bounded sample of the workload: one layer, one sequence of the batch. Returns (GB/s by the
    same algorithmic-bytes formula, sample description, cores, seconds per run)."""
    from oracle import kivi as ok

    rng = np.random.default_rng(seed)
    H_kv, H_q, D, g, b = w["H_kv"], w["H_q"], w["D"], w["group"], w["bits"]
    Sq, R = w["n_quant"], w["n_res"]
    levels = (1 << b) - 1
    k = rng.standard_normal((1, H_kv, Sq + R, D)).astype(np.float16)
    v = rng.standard_normal((1, H_kv, Sq + R, D)).astype(np.float16)
    q = rng.standard_normal((1, H_q, 1, D)).astype(np.float16)
    kc, ks, kz = ok.quant_keys(k[:, :, :Sq], g, levels)
    vc, vs, vz = ok.quant_values(v[:, :, :Sq], g, levels)
    scale = 1.0 / math.sqrt(D)
    ok.reference_attend(q, kc, ks, kz, vc, vs, vz, g, scale, k_res=k[:, :, Sq:], v_res=v[:, :, Sq:])  # warm-up
    times = []
    t_start = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_start < seconds_budget and len(times) < 50):
        t0 = time.perf_counter()
        ok.reference_attend(q, kc, ks, kz, vc, vs, vz, g, scale, k_res=k[:, :, Sq:], v_res=v[:, :, Sq:])
        times.append(time.perf_counter() - t0)
    t = float(np.median(times))
    nbytes = algorithmic_bytes_per_layer(w, batch=1)
    sample = (f"1 layer x 1 sequence of the batch ({H_kv} kv heads, {Sq}+{R} tokens), median of "
              f"{len(times)} runs of oracle.kivi.reference_attend (NumPy, BLAS threads); MLX unavailable on this box")
    return nbytes / t / 1e9, sample, os.cpu_count(), t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = workload(args)
    per_step_budget = 8.0
    vals = []
    for _ in range(args.warmup):
        cpu_reference_sample(w, seconds_budget=0.0)
    t_all = 0.0
    sample = ""
    cores = os.cpu_count()
    for _ in range(args.steps):
        gbs, sample, cores, t = cpu_reference_sample(w, seconds_budget=per_step_budget / 4)
        vals.append(gbs)
        t_all += t
    value = float(np.median(vals))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * t_all / max(args.steps, 1), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": config_of(w, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- our arm
def synth_kv(torch, shape, device, seed, dtype):
    """Seeded synthetic K and V: N(0,1) with 4 outlier channels scaled x20."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    ch = torch.randperm(shape[-1], generator=gen, device=device)[:4]
    kv = []
    for _ in range(2):
        x = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        x[..., ch] *= 20.0
        kv.append(x.to(dtype))
        del x
    return kv


def new_cache(w, bits=None):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    return KVCacheFactory.create(KVCacheConfig(
        method="kivi", head_dim=w["D"], bit_width_inlier=w["bits"] if bits is None else bits,
        kivi_group_size=w["group"], residual_length=w["residual"], fused_sdpa_memory_bound=True))


def build_cache(torch, w, shape_bh, device, seed, dtype, bits=None):
    """One layer's cache, filled by a prefill append of seeded synthetic K/V: quantize-on-write
    through the public cache interface (packed codes + fp32 params + residual window)."""
    k, v = synth_kv(torch, (*shape_bh, w["ctx"], w["D"]), device, seed, dtype)
    cache = new_cache(w, bits)
    cache.update_and_fetch(k, v)
    assert cache._n_quantized == w["n_quant"] and cache.offset == w["ctx"]
    return cache


class Timer:
    """Blocks of `steps` steps, each bracketed by barrier + synchronize and CUDA events on the
    launching stream; per block the max over ranks; the result is the list of ms per step."""

    def __init__(self, torch, dist, world, device):
        self.torch, self.dist, self.world, self.device = torch, dist, world, device

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def blocks(self, fn, steps, n_blocks):
        torch = self.torch
        out = []
        for _ in range(n_blocks):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            self.barrier()
            t = torch.tensor([e0.elapsed_time(e1)], device=self.device, dtype=torch.float64)
            if self.world > 1:
                self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            out.append(float(t.item()) / steps)
        return out


def stats(ms_list):
    return {"median": float(np.median(ms_list)), "min": float(np.min(ms_list)), "max": float(np.max(ms_list)),
            "blocks": len(ms_list)}


def capture(torch, fn):
    """fn captured into a CUDA graph (after a warm-up on a side stream); returns the replay."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    torch.cuda.synchronize()
    return g


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    from veloxquant_mlx_b200 import kernels as vk
    from veloxquant_mlx_b200 import sharding

    w = workload(args)
    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    L, B, H_q, H_kv, D = w["layers"], w["batch"], w["H_q"], w["H_kv"], w["D"]
    hpk = H_q // H_kv
    scale = 1.0 / math.sqrt(D)
    timer = Timer(torch, dist, world, device)
    notes = []

    # ---- the partition: this rank's (batch, kv head) units ----------------------------------
    plan = sharding.plan_shards(B, H_kv, world, rank)
    if world == 1:
        shape_bh, q_shape = (B, H_kv), (B, H_q, 1, D)
    else:
        shape_bh, q_shape = (plan.size, 1), (plan.size, hpk, 1, D)
    frac_local = plan.size / plan.units  # share of the whole problem this rank attends

    gather_mode = "none" if world == 1 else args.gather
    px = None
    if gather_mode == "peer":
        try:
            px = sharding.PeerExchange(plan, L, hpk, D, dtype, device)
            ok = torch.tensor([1], device=device)
        except Exception as e:  # the benchmark still has to produce its line
            notes.append(f"peer exchange unavailable on rank {rank}: {e}")
            ok = torch.tensor([0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            px = None
            gather_mode = "nccl"
            notes.append("fell back to the NCCL all-gather")

    caches = [build_cache(torch, w, shape_bh, device, 1000 * l + rank, dtype) for l in range(L)]
    gen = torch.Generator(device=device)
    gen.manual_seed(7 + rank)
    qs = [torch.randn(q_shape, generator=gen, device=device, dtype=torch.float32).to(dtype) for _ in range(L)]
    outs = [torch.empty(q_shape, device=device, dtype=dtype) for _ in range(L)]
    comm_stream = torch.cuda.Stream(device) if gather_mode == "nccl" else None
    gathered = [torch.empty((B, H_q, 1, D), device=device, dtype=dtype) for _ in range(L)] if gather_mode == "nccl" else None
    torch.cuda.synchronize()

    def nccl_gather(l, src=None):
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(comm_stream):
            comm_stream.wait_event(ev)
            sharding.gather_layer_output(outs[l] if src is None else src, plan, out=gathered[l])

    def make_step(with_gather=True):
        def step():
            for l in range(L):
                g = px.layer(l) if (px is not None and with_gather) else None
                # (the queries and caches of this loop are static: nothing the kernel reads is
                # written by the work right before it, which is what overlap_previous requires)
                caches[l].fused_sdpa(qs[l], scale, out=outs[l], overlap_previous=True, gather=g)
                if g is not None:
                    px.wait(l)
                elif gather_mode == "nccl" and with_gather:
                    nccl_gather(l)
            if gather_mode == "nccl" and with_gather:
                torch.cuda.current_stream().wait_stream(comm_stream)
        return step

    step = make_step()
    for _ in range(max(args.warmup, 3)):
        step()
    timer.barrier()
    vk.attend_status()
    run = step
    graphed = False
    if gather_mode != "nccl" and not args.no_graph:
        try:
            run = capture(torch, step).replay
            graphed = True
        except Exception as e:
            notes.append(f"graph capture failed, timing eager launches: {e}")
            run = step
    for _ in range(max(args.warmup, 3)):
        run()
    timer.barrier()

    # timed region: >= 1 s of GPU work in blocks of `steps` steps (at least 5 blocks, at most 40)
    probe = timer.blocks(run, args.steps, 1)[0]
    n_blocks = int(min(40, max(5, math.ceil(1000.0 / max(probe * args.steps, 1e-3)))))
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_blocks = timer.blocks(run, args.steps, n_blocks)
    clocks = sampler.stop() if rank == 0 else None
    ms_step = float(np.median(ms_blocks))
    vk.attend_status()

    # the collective's share: the same step without publishing / gathering the outputs
    gather_info = None
    if world > 1:
        bare = make_step(with_gather=False)
        bare_run = bare
        if graphed:
            try:
                bare_run = capture(torch, bare).replay
            except Exception:
                bare_run = bare
        for _ in range(3):
            bare_run()
        ms_bare = float(np.median(timer.blocks(bare_run, args.steps, max(5, n_blocks // 2))))
        gather_info = {"mode": gather_mode, "ms_per_step_without_gather": ms_bare,
                       "share_of_step": max(0.0, 1.0 - ms_bare / ms_step),
                       "bytes_per_rank_per_layer": plan.size * hpk * D * outs[0].element_size()}
        if px is not None:
            # the gathered tensors must hold every rank's rows: compare with an NCCL all-gather
            worst = 0.0
            for l in (0, L - 1):
                ref = sharding.gather_layer_output(outs[l], plan)
                worst = max(worst, float((px.output(l).float() - ref.float()).abs().max().item()))
            gather_info["max_abs_diff_vs_nccl_allgather"] = worst

    # ---- extras measured in the same run -----------------------------------------------------
    extra = {}
    peak, peak_kind = measured_peak()
    if not args.no_extras:
        extra = run_extras(torch, dist, timer, w, plan, world, rank, device, dtype, px, args, peak)

    # ---- end-to-end arm (after the kernel arm, so the cache contents above stay fixed)
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(torch, dist, timer, w, plan, world, device, dtype, caches, outs, px, gather_mode, nccl_gather,
                      comm_stream, q_shape, shape_bh, args)
    vk.attend_status()

    if rank == 0:
        bytes_layer = algorithmic_bytes_per_layer(w)
        bytes_step = bytes_layer * L
        value = bytes_step / (ms_step * 1e-3) / 1e9
        per_launch_s = ms_step * 1e-3 / L
        achieved = frac_local * bytes_layer / per_launch_s / 1e9
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            gbs, sample, cores, _ = cpu_reference_sample(w, seconds_budget=15.0)
            cpu = {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        if clocks and clocks.get("sm_mhz"):
            clocks["ms_per_step_x_sm_mhz"] = ms_step * clocks["sm_mhz"]
        launches_per_layer = 1 + (1 if px is not None else 0)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": config_of(w, world),
            "ms_per_step_blocks": stats(ms_blocks),
            "tokens_per_s": B / (ms_step * 1e-3),
            "pct_of_hbm_peak": 100.0 * (value / world) / peak,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind + " (burst copy)", "traffic": ncu_traffic(w) if world == 1 else None,
                         "kernel": f"kivi_attend_mma_kernel<{w['bits']}> (one launch per layer: packed groups, residual rows and the split merge; duration = step time / layers)",
                         "algorithmic_bytes_per_launch": int(frac_local * bytes_layer)},
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gather": gather_info,
            "extra": extra,
            "launch": {"cuda_graph": graphed, "overlap_previous": True},
            "gpu_launches": launches_per_layer * L * args.steps,  # one attend kernel (+ arrival wait when sharded) per layer
            "clocks": clocks,
            "notes": notes,
        }
        print(json.dumps(line), flush=True)
    if px is not None:
        px.close()
    if world > 1:
        dist.destroy_process_group()


def run_e2e(torch, dist, timer, w, plan, world, device, dtype, caches, outs, px, gather_mode, nccl_gather, comm_stream,
            q_shape, shape_bh, args):
    """End-to-end step through the cache interface with HOST buffers: per layer the query and the
    new token's K/V come from pinned host memory, the token is appended (and, every `group`
    steps, the group that aged out of the residual window is quantized into the packed store),
    attention runs over the packed cache, and the layer's output goes back to pinned host memory.
    The copies run on their own streams in chunks of four layers: one pinned staging buffer per
    chunk (query, key, value of its layers back to back) with its device twin and an event;
    uploads are issued one chunk ahead of the compute launches; the compute stream waits for the
    event of the chunk it is about to run, the download stream for the chunk's last attention."""
    L, D = w["layers"], w["D"]
    scale = 1.0 / math.sqrt(D)
    kv_shape = (*shape_bh, 1, D)
    n_q = int(np.prod(q_shape))
    n_kv = int(np.prod(kv_shape))
    per_layer = n_q + 2 * n_kv
    CH = 4
    chunks = [list(range(c, min(c + CH, L))) for c in range(0, L, CH)]
    host_in = [torch.empty(len(ch) * per_layer, dtype=dtype).pin_memory() for ch in chunks]
    dev_in = [torch.empty(len(ch) * per_layer, device=device, dtype=dtype) for ch in chunks]
    for t in host_in:
        t.copy_(torch.randn(t.numel(), dtype=torch.float32).to(dtype))
    dq, dk, dv = [], [], []
    for ci, ch in enumerate(chunks):
        for j in range(len(ch)):
            base = j * per_layer
            dq.append(dev_in[ci][base:base + n_q].view(q_shape))
            dk.append(dev_in[ci][base + n_q:base + n_q + n_kv].view(kv_shape))
            dv.append(dev_in[ci][base + n_q + n_kv:base + per_layer].view(kv_shape))
    # the layers of a chunk write their outputs into one device buffer, downloaded as a whole
    dev_out = [torch.empty((len(ch), *q_shape), device=device, dtype=dtype) for ch in chunks]
    host_out = [torch.empty((len(ch), *q_shape), dtype=dtype).pin_memory() for ch in chunks]
    e2e_outs = [dev_out[ci][j] for ci, ch in enumerate(chunks) for j in range(len(ch))]
    h2d_bytes = sum(t.numel() * t.element_size() for t in dev_in)
    d2h_bytes = sum(t.numel() * t.element_size() for t in dev_out)
    up_stream, down_stream = torch.cuda.Stream(device), torch.cuda.Stream(device)
    ev_in = [torch.cuda.Event() for _ in chunks]
    ev_done = [torch.cuda.Event() for _ in chunks]

    def upload(ci):
        with torch.cuda.stream(up_stream):
            dev_in[ci].copy_(host_in[ci], non_blocking=True)
            ev_in[ci].record(up_stream)

    def e2e_step():
        main = torch.cuda.current_stream()
        up_stream.wait_stream(main)  # the previous step is done with the staging buffers
        upload(0)
        for ci, ch in enumerate(chunks):
            if ci + 1 < len(chunks):
                upload(ci + 1)
            main.wait_event(ev_in[ci])
            for l in ch:
                # (the new token and the query come from the upload stream, never from the kernels
                # right before these calls: both may start under the previous layer's attention)
                caches[l].update_and_fetch(dk[l], dv[l], overlap_previous=True)
                caches[l].fused_sdpa(dq[l], scale, out=e2e_outs[l], overlap_previous=True,
                                     gather=px.layer(l) if px is not None else None)
                if px is not None:
                    px.wait(l)
                if gather_mode == "nccl":
                    nccl_gather(l, e2e_outs[l])
            ev_done[ci].record(main)
            with torch.cuda.stream(down_stream):
                down_stream.wait_event(ev_done[ci])
                host_out[ci].copy_(dev_out[ci], non_blocking=True)
        if gather_mode == "nccl":
            main.wait_stream(comm_stream)
        main.wait_stream(down_stream)
        torch.cuda.synchronize()  # the host reads this step's outputs

    g = w["group"]
    # warm up until 10 steps before the next flush, so that every block of >= 10 steps that
    # follows crosses quantize-on-append flushes at a known step
    n_warm = 3
    while (caches[0].offset + n_warm + 10) % g:
        n_warm += 1
    for _ in range(n_warm):
        e2e_step()
    timer.barrier()
    n_steps = max(args.steps, g) * 2  # two flush periods at least
    per_step = []
    flush_steps = []
    timer.barrier()
    alloc0 = torch.cuda.memory_stats(device).get("allocation.all.allocated", 0)
    t_all0 = time.perf_counter()
    for i in range(n_steps):
        nq_before = caches[0]._n_quantized
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_step()
        e1.record()
        torch.cuda.synchronize()
        per_step.append(e0.elapsed_time(e1))
        if caches[0]._n_quantized != nq_before:
            flush_steps.append(i)
    alloc1 = torch.cuda.memory_stats(device).get("allocation.all.allocated", 0)
    wall_ms = (time.perf_counter() - t_all0) * 1e3 / n_steps
    timer.barrier()
    t = torch.tensor([float(np.mean(per_step)), float(np.median(per_step)),
                      float(np.mean([per_step[i] for i in flush_steps])) if flush_steps else 0.0],
                     device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    mean_ms, median_ms, flush_ms = (float(x) for x in t.tolist())
    bytes_step = algorithmic_bytes_per_layer(w, n_quant=caches[0]._n_quantized, n_res=caches[0]._n_res) * L
    return {
        "value": bytes_step / (mean_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": mean_ms,
        "ms_per_step_median": median_ms, "flush_step_ms": flush_ms, "steps_timed": n_steps,
        "flush_steps_in_timed_region": len(flush_steps), "wall_ms_per_step": wall_ms,
        "tokens_per_s": w["batch"] / (mean_ms * 1e-3),
        "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
        "torch_allocations_in_timed_region": int(alloc1 - alloc0),
        "path": "KIVIKVCache.update_and_fetch(new token; quantize-on-append flush every group) + "
                "KIVIKVCache.fused_sdpa per layer; pinned host buffers, uploads and downloads in chunks of 4 "
                "layers on their own streams; value = mean over all timed steps, flush steps included",
    }


def run_extras(torch, dist, timer, w, plan, world, rank, device, dtype, px, args, peak):
    """Further figures of the same run (each a few seconds at most)."""
    from veloxquant_mlx_b200 import kernels as vk

    extra = {}
    L, B, H_q, H_kv, D = w["layers"], w["batch"], w["H_q"], w["H_kv"], w["D"]
    hpk = H_q // H_kv
    scale = 1.0 / math.sqrt(D)

    def graph_time(fn, steps, blocks=5):
        try:
            run = capture(torch, fn).replay
        except Exception:
            run = fn
        for _ in range(3):
            run()
        return float(np.median(timer.blocks(run, steps, blocks)))

    if world == 1 and w["name"] == "llama3.1-8b-decode-kivi4" and w["bits"] == 4:
        # -- the same shape with 2-bit codes (the width the >= 70 % of HBM target is quoted on)
        c2 = [build_cache(torch, w, (B, H_kv), device, 5000 + l, dtype, bits=2) for l in range(L)]
        q2 = [torch.randn((B, H_q, 1, D), device=device, dtype=torch.float32).to(dtype) for _ in range(L)]
        o2 = [torch.empty((B, H_q, 1, D), device=device, dtype=dtype) for _ in range(L)]

        def step2():
            for l in range(L):
                c2[l].fused_sdpa(q2[l], scale, out=o2[l], overlap_previous=True)

        try:
            run2 = capture(torch, step2).replay
        except Exception:
            run2 = step2
        for _ in range(3):
            run2()
        blocks2 = timer.blocks(run2, args.steps, 10)
        ms, ms_best = float(np.median(blocks2)), float(min(blocks2))
        bl = algorithmic_bytes_per_layer(w, bits=2)
        extra["kivi2"] = {"workload": "the default shape with 2-bit codes", "ms_per_step": ms,
                          "value": bl * L / (ms * 1e-3) / 1e9, "unit": UNIT,
                          "frac": bl * L / (ms * 1e-3) / 1e9 / peak, "tokens_per_s": B / (ms * 1e-3),
                          "algorithmic_bytes_per_launch": bl,
                          # (the fastest of the ten blocks: the first ones run before the power cap pulls the clock down)
                          "best_block_ms_per_step": ms_best, "best_block_frac": bl * L / (ms_best * 1e-3) / 1e9 / peak}
        del c2, q2, o2
        torch.cuda.empty_cache()

        # -- quantize-on-append: one layer's prefill block, K (per channel) and V (per token)
        k, v = synth_kv(torch, (B, H_kv, w["ctx"], D), device, 99, dtype)
        n = k.numel()
        for bits in (4, 2):
            for axis, name, x in ((-2, "keys", k), (-1, "values", v)):
                codes, sc, zr = vk.kivi_quantize(x, axis, w["group"], bits)
                ms = graph_time(lambda: vk.kivi_quantize_into(x, axis, w["group"], bits, codes=codes, scale=sc, zero=zr), 5)
                nb = n * x.element_size() + n * bits // 8 + (n // w["group"]) * 8
                extra[f"quantize_{name}_{bits}bit"] = {"shape": list(x.shape), "us": ms * 1e3, "GBps": nb / (ms * 1e-3) / 1e9,
                                                       "frac": nb / (ms * 1e-3) / 1e9 / peak, "bytes": nb}
        del k, v
        torch.cuda.empty_cache()

        # -- quantize_vq (the dense contraction): config 2 and a long one
        from veloxquant_mlx_b200 import vecinfer as vi
        tpeak, tkind = measured_tensor_peak()
        for S in (4096, 65536):
            keys = torch.randn(8, S, 128, device=device).to(torch.float16)
            cb = torch.randn(256, 8, device=device)
            ms = graph_time(lambda: vi.quantize_vq(keys, cb, 8, index_dtype=torch.uint8), 5)
            # the other searches on the same input: tcgen05 with the two-pass epilogue, warp-level MMAs
            other = {}
            for name, mode in (("tcgen05_two_pass", 4), ("mma_sync", 2)):
                vk.tune("vq_search", mode)
                other[name + "_us"] = graph_time(lambda: vi.quantize_vq(keys, cb, 8, index_dtype=torch.uint8), 5) * 1e3
            vk.tune("vq_search", 0)
            fl = 2 * 8 * S * 16 * 256 * 8
            # tensor-pipe time of the two 128 x 256 x 16 MMAs per 128 rows at the measured dense peak
            mma_fl = 2 * 8 * S * 16 * 256 * 32
            extra[f"quantize_vq_S{S}"] = {"shape": [8, S, 128], "us": ms * 1e3, "useful_TFLOPs": fl / (ms * 1e-3) / 1e12,
                                          "frac_of_bf16_peak": fl / (ms * 1e-3) / 1e12 / tpeak, "peak_kind": tkind,
                                          "issued_mma_frac_of_peak": mma_fl / (ms * 1e-3) / 1e12 / tpeak, **other}
        vk.quantize_status()

        # -- VecInfer config 2: decode attention over the VQ key codes (dense fp16 values, 32 query heads)
        from veloxquant_mlx_b200 import vecinfer as vi
        kx = torch.randn(1, 8, 4096, D, device=device, dtype=torch.float16)
        cbk = torch.randn(256, 8, device=device)
        kix = vi.quantize_vq(kx, cbk, 8, index_dtype=torch.uint8)
        qx = torch.randn(1, 32, 1, D, device=device, dtype=torch.float16)
        ms = graph_time(lambda: vi.fused_sdpa_vq(qx, kix, cbk, kx, None, D ** -0.5), 20)
        nb = kix.numel() + kx.numel() * 2
        extra["vq_attend_config2"] = {"shape": [1, 8, 4096, D], "us": ms * 1e3, "GBps": nb / (ms * 1e-3) / 1e9,
                                      "note": "8.9 MB: bound by per-CTA set-up (lookup tables) and load latency, not by HBM"}
        del kx, kix, qx
        # ... and at a serving shape (batch 8, 16 384 keys): the staged tensor-core kernel with the score table in shared memory
        kx = torch.randn(8, 8, 16384, D, device=device, dtype=torch.float16)
        kix = vi.quantize_vq(kx, cbk, 8, index_dtype=torch.uint8)
        qx = torch.randn(8, 32, 1, D, device=device, dtype=torch.float16)
        ms = graph_time(lambda: vi.fused_sdpa_vq(qx, kix, cbk, kx, None, D ** -0.5), 10)
        nb = kix.numel() + kx.numel() * 2
        extra["vq_attend_serving"] = {"shape": [8, 8, 16384, D], "us": ms * 1e3, "GBps": nb / (ms * 1e-3) / 1e9, "frac": nb / (ms * 1e-3) / 1e9 / peak}
        # ... and with the values as codebook indices too (what VecInferKVCache stores: 32 bytes per key)
        vix = torch.randint(0, 256, (8, 8, 16384, 16), device=device, dtype=torch.uint8)
        ms = graph_time(lambda: vi.fused_sdpa_vq(qx, kix, cbk, vix, cbk, D ** -0.5), 10)
        extra["vq_attend_serving_coded_values"] = {"shape": [8, 8, 16384, D], "us": ms * 1e3, "keys_per_us": 8 * 8 * 16384 / (ms * 1e3),
                                                    "note": "33.5 MB: bound by the expansion of the value tile and the table gathers, not by HBM"}
        del kx, kix, qx, vix

        # -- TurboQuant-RVQ: quantize+pack and unpack+decode of 1 Mi rotated keys
        from veloxquant_mlx_b200 import rvq
        Nr = 8 * 8 * 16384
        tq = rvq.TurboQuantRVQ(D, 2, use_hadamard=True)
        yr = (torch.randn(Nr, D, device=device) / D ** 0.5).to(torch.float16)
        cb1, cb2 = tq._codebook1, tq._codebook2
        ms = graph_time(lambda: rvq.rvq_quant_pack(yr, cb1.centroids, cb1.boundaries, cb2.boundaries, 2), 5)
        nb = Nr * D * 2 + 2 * Nr * rvq.n_words_for(D, 2) * 4
        extra["rvq_quant_pack_2bit"] = {"rows": Nr, "us": ms * 1e3, "GBps": nb / (ms * 1e-3) / 1e9, "frac": nb / (ms * 1e-3) / 1e9 / peak}
        pk1, pk2 = rvq.rvq_quant_pack(yr, cb1.centroids, cb1.boundaries, cb2.boundaries, 2)
        nrm = torch.ones(Nr, device=device, dtype=torch.bfloat16)
        dg = tq._rot(device)
        ms = graph_time(lambda: rvq.rvq_unpack_decode(pk1, pk2, nrm, cb1.centroids, cb2.centroids, dg, 2, D), 5)
        nb += Nr * 2
        extra["rvq_unpack_decode_2bit"] = {"rows": Nr, "us": ms * 1e3, "GBps": nb / (ms * 1e-3) / 1e9, "frac": nb / (ms * 1e-3) / 1e9 / peak}
        del yr, pk1, pk2, nrm

        # -- SKVQ: clipped group quantize + pack (five clip factors searched / one) and unpack + dequantize, 1 Mi rows
        from veloxquant_mlx_b200 import skvq
        xs = torch.randn(64, 16384, D, device=device, dtype=torch.float16)
        nb = xs.numel() * 2 + xs.numel() // 2 + 2 * (xs.numel() // 32) * 4
        sk_out = skvq.quantize_pack(xs, 4, 32)
        for name, alphas in (("skvq_quant_pack_4bit_search5", skvq.DEFAULT_ALPHA_GRID), ("skvq_quant_pack_4bit_fixed", (0.94,))):
            ms = graph_time(lambda: skvq.quantize_pack(xs, 4, 32, alphas, out=sk_out), 5)
            extra[name] = {"rows": 64 * 16384, "us": ms * 1e3, "GBps": nb / (ms * 1e-3) / 1e9, "frac": nb / (ms * 1e-3) / 1e9 / peak}
        ms = graph_time(lambda: skvq.unpack_dequant(*sk_out, 4, 32, 16384, torch.float16, out=xs), 5)
        extra["skvq_unpack_dequant_4bit"] = {"rows": 64 * 16384, "us": ms * 1e3, "GBps": nb / (ms * 1e-3) / 1e9, "frac": nb / (ms * 1e-3) / 1e9 / peak}
        del xs, sk_out

        # -- RaBitQ config 4: encode and attend
        from veloxquant_mlx_b200 import rabitq as rq
        Br, Hr, Sr = 8, 8, 16384
        keys = torch.randn(Br * Hr * Sr, D, device=device, dtype=torch.float16)
        diag = torch.from_numpy(rq.make_hadamard_diagonal(D)).to(device)
        ms = graph_time(lambda: rq.rabitq_encode(keys, diag), 5)
        nb = keys.numel() * 2 + keys.shape[0] * (D // 8 + 4)
        extra["rabitq_encode"] = {"rows": keys.shape[0], "us": ms * 1e3, "GBps": nb / (ms * 1e-3) / 1e9, "frac": nb / (ms * 1e-3) / 1e9 / peak}
        bits_, mag = rq.rabitq_encode(keys, diag)
        vv = torch.randn(Br, Hr, Sr, D, device=device, dtype=torch.float16)
        qq = torch.randn(Br, 32, 1, D, device=device, dtype=torch.float16)
        qsc = torch.full((Br, 32, 1), 0.01, device=device)
        ms = graph_time(lambda: rq.rabitq_fused_attend(qq, qsc, bits_.view(Br, Hr, Sr, D // 8), mag.view(Br, Hr, Sr), None, vv, None), 5)
        nb = Br * Hr * Sr * (D // 8 + 4 + 2 * D)
        extra["rabitq_attend"] = {"shape": [Br, Hr, Sr, D], "us": ms * 1e3, "GBps": nb / (ms * 1e-3) / 1e9, "frac": nb / (ms * 1e-3) / 1e9 / peak}
        del keys, vv, bits_, mag
        torch.cuda.empty_cache()

    if world > 1 and w["name"] == "llama3.1-8b-decode-kivi4":
        # -- weak scaling (secondary): every rank attends a whole batch of its own, no exchange
        cw = [build_cache(torch, w, (B, H_kv), device, 9000 + 1000 * l + rank, dtype) for l in range(L)]
        qw = [torch.randn((B, H_q, 1, D), device=device, dtype=torch.float32).to(dtype) for _ in range(L)]
        ow = [torch.empty((B, H_q, 1, D), device=device, dtype=dtype) for _ in range(L)]

        def stepw():
            for l in range(L):
                cw[l].fused_sdpa(qw[l], scale, out=ow[l], overlap_previous=True)

        ms = graph_time(stepw, args.steps, 10)
        bl = algorithmic_bytes_per_layer(w)
        extra["weak_scaling"] = {"what": "replicated mode: every rank attends its own batch of 16, no output exchange",
                                 "global_batch": world * B, "ms_per_step": ms,
                                 "value": world * bl * L / (ms * 1e-3) / 1e9, "unit": UNIT,
                                 "tokens_per_s": world * B / (ms * 1e-3)}
        del cw, qw, ow
        torch.cuda.empty_cache()

    if w["name"] == "llama3.1-8b-decode-kivi4" and not args.no_c5:
        extra["qwen32b_prefill_decode"] = run_c5(torch, dist, timer, plan.world, rank, device, dtype, args)
    return extra


def run_c5(torch, dist, timer, world, rank, device, dtype, args):
    """The Qwen2.5-32B-shaped configuration: 64 layers, 40 query heads, 8 KV heads, batch 4, a
    16384-token prompt quantized on write (KIVI 2-bit), then 256 decode steps (append + attend)
    over the packed cache, the 32 (batch, kv head) units partitioned over the ranks."""
    from veloxquant_mlx_b200 import kernels as vk
    from veloxquant_mlx_b200 import sharding

    class A:  # the c5 workload through the same helper
        workload, layers, batch, ctx, bits = "c5", args.c5_layers, None, 16384, None

    w = workload(A)
    L, B, H_q, H_kv, D = w["layers"], w["batch"], w["H_q"], w["H_kv"], w["D"]
    hpk = H_q // H_kv
    plan = sharding.plan_shards(B, H_kv, world, rank)
    shape_bh = (B, H_kv) if world == 1 else (plan.size, 1)
    q_shape = (B, H_q, 1, D) if world == 1 else (plan.size, hpk, 1, D)
    scale = 1.0 / math.sqrt(D)
    S = 16384
    k, v = synth_kv(torch, (*shape_bh, S, D), device, 77 + rank, dtype)
    # a first, untimed pass over all layers: it pays the kernels' first launches and leaves the
    # device memory of 64 packed caches in torch's caching allocator, as a warmed-up server has it
    caches = [new_cache(w) for _ in range(L)]
    for l in range(L):
        caches[l].update_and_fetch(k, v)
    torch.cuda.synchronize()
    del caches
    caches = [new_cache(w) for _ in range(L)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    timer.barrier()
    e0.record()
    for l in range(L):
        caches[l].update_and_fetch(k, v)
    e1.record()
    timer.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    prefill_ms = float(t.item())
    n = B * H_kv * S * D  # elements of K (and of V) per layer, whole batch
    prefill_bytes = L * 2 * (n * 2 + n * w["bits"] // 8 + (n // w["group"]) * 8)
    del k, v
    px = None
    if world > 1 and args.gather == "peer":
        try:
            px = sharding.PeerExchange(plan, L, hpk, D, dtype, device)
            ok = torch.tensor([1], device=device)
        except Exception:
            ok = torch.tensor([0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            px = None
    n_dec = args.c5_decode_steps
    qs = [torch.randn(q_shape, device=device, dtype=torch.float32).to(dtype) for _ in range(L)]
    kn = torch.randn((*shape_bh, 1, D), device=device, dtype=torch.float32).to(dtype)
    vn = torch.randn((*shape_bh, 1, D), device=device, dtype=torch.float32).to(dtype)
    outs = [torch.empty(q_shape, device=device, dtype=dtype) for _ in range(L)]

    def dec_step():
        for l in range(L):
            caches[l].update_and_fetch(kn, vn, overlap_previous=True)
            caches[l].fused_sdpa(qs[l], scale, out=outs[l], overlap_previous=True, gather=px.layer(l) if px is not None else None)
            if px is not None:
                px.wait(l)

    for _ in range(3):
        dec_step()
    ms = timer.blocks(dec_step, n_dec - 3, 1)[0]
    vk.attend_status()
    ctx_end = caches[0].offset
    wq = dict(w, ctx=ctx_end)
    wq["n_quant"], wq["n_res"] = caches[0]._n_quantized, caches[0]._n_res
    bl = algorithmic_bytes_per_layer(wq)

    # The attention of the same step as the device sees it: the 64 launches (and, sharded, the
    # exchange) captured once and replayed, as in the default workload's timed region.
    def attend_step():
        for l in range(L):
            caches[l].fused_sdpa(qs[l], scale, out=outs[l], overlap_previous=True, gather=px.layer(l) if px is not None else None)
            if px is not None:
                px.wait(l)

    try:
        replay = capture(torch, attend_step).replay
        for _ in range(3):
            replay()
        graph_ms = float(np.median(timer.blocks(replay, 10, 5)))
    except Exception:
        graph_ms = None
    vk.attend_status()
    if px is not None:
        px.close()
    return {"workload": w["name"], "layers": L, "batch": B, "prompt": S, "decode_steps": n_dec, "bits": w["bits"],
            "prefill_ms": prefill_ms, "prefill_quantize_GBps": prefill_bytes / (prefill_ms * 1e-3) / 1e9,
            "prefill_tokens_per_s": B * S / (prefill_ms * 1e-3),
            "decode_ms_per_step": ms, "decode_tokens_per_s": B / (ms * 1e-3),
            "decode_value": bl * L / (ms * 1e-3) / 1e9, "unit": UNIT,
            "attend_graph_ms_per_step": graph_ms,
            "attend_graph_value": None if not graph_ms else bl * L / (graph_ms * 1e-3) / 1e9,
            "units_per_rank": plan.size, "gather": "peer" if px is not None else ("none" if world == 1 else "not gathered"),
            "note": "decode steps are eager launches through update_and_fetch + fused_sdpa (about 1.3 ms of host time per step on "
                    "an idle host, close to the device time: a busy host makes the loop host-bound); "
                    "attend_graph_*: the step's 64 attention launches (+ exchange) captured into a CUDA graph"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=["c3", "c1", "c5"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--bits", type=int, default=None)
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="how a layer's output rows reach every rank when N > 1")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of graph replays")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-c5", action="store_true")
    ap.add_argument("--c5-layers", type=int, default=64)
    ap.add_argument("--c5-decode-steps", type=int, default=256)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
