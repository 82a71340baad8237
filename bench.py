#!/usr/bin/env python
"""Fused-MoE layer benchmark (one JSON line on stdout).

Workload: the Mixtral-8x7B-shaped bf16 MoE layer (H=4096, I=14336, E=8, top-2,
weights randn*0.02, routing softmax(randn) -> top-2 -> renormalise), seeded
synthetic data.  One step = one fused-MoE call over a batch of M tokens
(default M=4096); `value` is tokens/s with everything resident in HBM, `e2e`
the same through the public Python entry point with pinned-host inputs and
outputs copied inside the timed region.  With --gpus N every rank runs its own
replica of the layer on its own M tokens (weak scaling, no collective).

At every N the line also carries `config.expert_parallel`: the DeepSeek-V3-shaped FP8 layer
(256 experts, zipf-skewed routing) at a fixed global batch of 4096 tokens -- on one GPU at N = 1,
with the experts partitioned over the ranks at N > 1 (strong scaling).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference | reference-gpu]

`--impl reference` times the CPU restatement of the reference's algorithm on the host cores (the
reference has no CPU implementation); `--impl reference-gpu` times the reference's own Triton
operator on the GPU through baseline/ref_shim.py (context only: not the reference arm).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT, ROOT / "flaggems-sglang_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import torch  # noqa: E402

WORKLOADS = {
    # name: (H, I, E, topk, dtype string)
    "mixtral": (4096, 14336, 8, 2, "bf16"),
    "qwen3-30b-a3b": (2048, 768, 128, 8, "bf16"),
    "reference-bench": (1280, 3072, 64, 8, "bf16"),
    # FP8 e4m3 weights with 128x128 block scales, zipf-skewed routing; with --gpus N the
    # experts are partitioned over the ranks (expert parallelism) and M is the global batch
    "deepseek-v3": (7168, 2048, 256, 8, "fp8"),
    "deepseek-v3-e32": (7168, 2048, 32, 8, "fp8"),        # 32-expert slice of the same layer (small profiling case)
    # int4 AWQ w4a16: uint4 group-128 weights with zero points, fp16 activations
    "mixtral-awq": (4096, 14336, 8, 2, "int4"),
}
SWEEP_M = {"mixtral": [1, 16, 128, 1024, 4096], "qwen3-30b-a3b": [1, 8, 32, 64, 128, 256],
           "reference-bench": [1, 4, 17, 64, 1024, 2048, 4096], "deepseek-v3": [1, 64, 512, 4096],
           "deepseek-v3-e32": [1, 64, 512], "mixtral-awq": [1, 32, 256, 2048]}

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the
# ncu capture summarised under profiles/ (None until such a capture exists for the workload).
NCU_TRAFFIC = {("mixtral", 4096): {"kernel": "moe_gemm_tc_kernel<gate/up>", "bytes": 2189100000,
                                   "source": "profiles/moe_gemm_tc_mixtral_m4096_launch_list.md"}}


def load_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


def algorithmic_work(h, i, k, m, experts_hit, bytes_w=2):
    """bytes = D*(3*H*I*b_w + S_e) + M*H*(b_x + b_out); flops = 6*M*k*H*I.
    S_e = per-expert scale bytes (FP8: one fp32 per 128x128 block)."""
    s_e = 0
    if bytes_w == 1:
        s_e = 3 * h * i // (128 * 128) * 4
    elif bytes_w == 0.5:
        s_e = 3 * h * i // 128 * 2.5            # fp16 scale + packed uint4 zero per group and output row
    return int(experts_hit * (3 * h * i * bytes_w + s_e) + m * h * 4), 6 * m * k * h * i


class Layer:
    """The benchmarked MoE layer on one rank: weights (all experts, or this rank's
    share under expert parallelism) and the forward call."""

    def __init__(self, workload, dev, rank, world):
        import flaggems_sglang_b200 as F
        from flaggems_sglang_b200.testing import make_weights
        self.F = F
        self.h, self.i, self.e, self.k, self.dt = WORKLOADS[workload]
        self.fp8 = self.dt == "fp8"
        self.int4 = self.dt == "int4"
        self.act_dtype = torch.float16 if self.int4 else torch.bfloat16
        self.ep = self.fp8 and world > 1
        self.world = world
        self.ep_collective = None
        e_ids = range(self.e)
        self.placement = None
        if self.ep:
            # Load-balanced expert placement from the layer's own traffic statistics: a calibration batch
            # (other tokens, same router bias) counts the tokens per expert, the experts are dealt out heaviest
            # first to the least loaded rank.  The timed batch is not the calibration batch.
            from flaggems_sglang_b200 import ep
            from flaggems_sglang_b200.testing import make_tokens
            assert self.e % world == 0
            _, _, cal_ids = make_tokens(8192, 64, self.e, self.k, seed=1234, skew=True, bias_seed=0)
            load = torch.bincount(cal_ids.flatten().long(), minlength=self.e).tolist()
            self.placement = ep.plan_placement(self.e, world, load if not os.environ.get("B200MOE_EP_CONTIGUOUS") else None)
            e_ids = ep.local_experts(self.placement, rank)
        if self.fp8:
            from flaggems_sglang_b200.quant import quantize_fp8_block
            qs = [[], [], [], []]
            for ei in e_ids:                      # expert by expert keeps the bf16 temporaries small
                a, b = make_weights(self.h, self.i, self.e, device=dev, seed=0, expert_ids=[ei])
                aq, as_ = quantize_fp8_block(a)
                bq, bs_ = quantize_fp8_block(b)
                for lst, t in zip(qs, (aq, as_, bq, bs_)):
                    lst.append(t)
            self.w13, self.s13, self.w2, self.s2 = (torch.cat(l, dim=0).contiguous() for l in qs)
            self.kw = dict(use_fp8_w8a8=True, w13_scale=self.s13, w2_scale=self.s2)
            if self.ep:
                self.kw.update(placement=self.placement, mode=os.environ.get("B200MOE_EP_MODE") or None)
                if self.kw["mode"] in ("allgather", "alltoall"):
                    self.kw["placement"] = None
            self.bytes_w = 1
        elif self.int4:
            from flaggems_sglang_b200.quant import quantize_awq, repack_awq_for_kernel
            qs = [[], [], [], []]
            for ei in e_ids:
                a, b = make_weights(self.h, self.i, self.e, dtype=torch.float16, device=dev, seed=0, expert_ids=[ei])
                p1, z1 = repack_awq_for_kernel(*quantize_awq(a.transpose(1, 2).contiguous()))
                p2, z2 = repack_awq_for_kernel(*quantize_awq(b.transpose(1, 2).contiguous()))
                for lst, t in zip(qs, (p1, z1, p2, z2)):
                    lst.append(t)
            self.w13, z13, self.w2, z2 = (torch.cat(l, dim=0).contiguous() for l in qs)
            self.kw = dict(use_int4_w4a16=True, w13_sz=z13, w2_sz=z2)
            self.bytes_w = 0.5
        else:
            self.w13, self.w2 = make_weights(self.h, self.i, self.e, device=dev, seed=0)
            self.kw = {}
            self.bytes_w = 2

    def tokens(self, m, dev, seed):
        from flaggems_sglang_b200.testing import make_tokens
        return make_tokens(m, self.h, self.e, self.k, dtype=self.act_dtype, device=dev, seed=seed, skew=self.fp8,
                           bias_seed=0 if self.fp8 else None)

    def forward(self, x, tw, ids):
        if self.ep:
            from flaggems_sglang_b200 import ep
            out = ep.ep_fused_experts(x, self.w13, self.w2, tw, ids, **self.kw)
            self.ep_collective = ep.last_collective()
            return out
        return self.F.fused_experts(x, self.w13, self.w2, tw, ids, **self.kw)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while timed regions run; every sample
    carries its host time so that a region can be given its own median."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None      # samples: (perf_counter, MHz)
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append((time.perf_counter(), nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def median_between(self, t0, t1):
        v = [mhz for (t, mhz) in self.samples if t0 <= t <= t1]
        return statistics.median(v) if v else None

    def summary(self):
        v = [mhz for (_, mhz) in self.samples]
        return {"sm_mhz": statistics.median(v) if v else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(v)}


def physical_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ------------------------------------------------------------------ CPU arm (oracle)
def workload_string(name, h, i, e, k, m):
    return f"{name} H{h} I{i} E{e} top{k} M{m} per GPU, layer-layout weights"


def cpu_arm(args, h, i, e, k, m, steps, warmup, budget_s=12.0, keep=None):
    """Times the CPU per-expert-loop restatement (oracle/moe.py) on a bounded
    sample of the workload: the first m_cpu tokens of the batch.  `keep` (a dict) receives the
    fp32 host weights so that the caller can reuse them for its output check."""
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    from oracle import moe as OM
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen_dev = "cuda" if torch.cuda.is_available() else "cpu"
    w13, w2 = make_weights(h, i, e, device=gen_dev, seed=0)
    w13f, w2f = w13.cpu().float(), w2.cpu().float()
    del w13, w2
    if keep is not None:
        keep["w13f"], keep["w2f"] = w13f, w2f
    x, tw, ids = make_tokens(m, h, e, k, device="cpu", seed=0)
    m_cpu = min(m, 64)
    t0 = time.perf_counter()
    OM.fused_experts(x[:m_cpu], w13f, w2f, tw[:m_cpu], ids[:m_cpu])
    t = time.perf_counter() - t0
    # grow the sample towards the time budget per step
    per_step = budget_s / max(1, steps + warmup)
    while m_cpu < m and t * 2.5 < per_step:
        m_cpu = min(m, m_cpu * 2)
        t0 = time.perf_counter()
        OM.fused_experts(x[:m_cpu], w13f, w2f, tw[:m_cpu], ids[:m_cpu])
        t = time.perf_counter() - t0
    for _ in range(warmup):
        OM.fused_experts(x[:m_cpu], w13f, w2f, tw[:m_cpu], ids[:m_cpu])
    t0 = time.perf_counter()
    for _ in range(steps):
        OM.fused_experts(x[:m_cpu], w13f, w2f, tw[:m_cpu], ids[:m_cpu])
    el = time.perf_counter() - t0
    return {"value": m_cpu * steps / el, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"first {m_cpu} of {m} tokens per step, {steps} steps, fp32 torch per-expert loop, "
                      f"weights pre-converted to fp32", "ms_per_step": el / steps * 1e3, "m_cpu": m_cpu}


def run_reference(args, rank, world):
    """CPU arm: rank 0 alone runs it, whatever N is (one host, one set of cores), so the line says
    n_gpus 1 when launched under N ranks: its value does not grow with N."""
    h, i, e, k, dt = WORKLOADS[args.workload]
    if rank != 0:
        return
    res = cpu_arm(args, h, i, e, k, args.M, max(1, args.steps), max(0, args.warmup), budget_s=60.0)
    line = {
        "impl": "reference", "metric": "fused_moe_tokens_per_s", "value": res["value"], "unit": "tokens/s",
        "n_gpus": 1 if world > 1 else args.gpus, "launched_ranks": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": {"workload": workload_string(args.workload, h, i, e, k, args.M),
                   "note": "the reference has no CPU implementation of this path; this arm times the CPU "
                           "restatement of its algorithm (oracle/moe.py) on the host cores of rank 0 only"},
        "cpu_baseline": {"value": res["value"], "unit": "tokens/s", "cores": res["cores"], "kind": "port",
                         "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_reference_gpu(args):
    """The reference's own Triton operator (src/flaggems_sglang/ops/fused_moe.py:133-216) on this
    GPU, through the import shim: CUDA-event median of >= 20 calls after >= 5 warm-ups for every M
    of the workload's sweep.  Context for the bf16 rows; not the reference arm."""
    sys.path.insert(0, str(ROOT / "baseline"))
    h, i, e, k, dt = WORKLOADS[args.workload]
    line = {"impl": "reference-gpu", "workload": args.workload, "shape": {"H": h, "I": i, "E": e, "topk": k},
            "dtype": dt, "rows": []}
    if dt != "bf16":
        line["unavailable"] = "the reference rejects quantised weights (fused_moe.py:154-169)"
        print(json.dumps(line), flush=True)
        return
    try:
        from ref_shim import load_reference
        ref, to_routing = load_reference()
    except Exception as ex:  # noqa: BLE001
        line["unavailable"] = f"reference not importable here: {ex!r}"[:300]
        print(json.dumps(line), flush=True)
        return
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    dev = torch.device("cuda:0")
    scale = 0.1 if args.workload == "reference-bench" else 0.02
    w13, w2 = make_weights(h, i, e, device=dev, seed=0, scale=scale)
    w1_op = w13.transpose(1, 2).contiguous()       # the reference's layout [E, H, 2I] / [E, I, H]
    del w13
    w2_op = w2.transpose(1, 2).contiguous()
    del w2
    n_calls = max(20, args.steps)
    for m in SWEEP_M[args.workload]:
        row = {"M": m}
        try:
            x, tw, ids = make_tokens(m, h, e, k, device=dev, seed=0)
            rd, gi, si = to_routing(tw, ids.long(), e)
            call = lambda: ref.triton_kernel_fused_experts(x, w1_op, w2_op, rd, gi, si)
            for _ in range(max(5, args.warmup)):
                call()
            torch.cuda.synchronize()
            times = []
            for _ in range(n_calls):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                call()
                e1.record()
                e1.synchronize()
                times.append(e0.elapsed_time(e1))
            row.update(us=statistics.median(times) * 1e3, us_min=min(times) * 1e3, calls=n_calls,
                       tokens_per_s=m / (statistics.median(times) / 1e3))
        except Exception as ex:  # noqa: BLE001
            row["unavailable"] = repr(ex)[:300]
        line["rows"].append(row)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def time_calls(fn, steps, warmup, barrier=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        fn()
    ev1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return ev0.elapsed_time(ev1)  # ms


def time_regions(fn, steps, warmup, barrier, dist, dev, clocks, min_total_s=1.0, max_regions=64):
    """Regions of exactly `steps` calls, each bracketed by barrier + synchronize and timed with CUDA
    events on the launching stream (maximum over ranks), repeated until at least `min_total_s` of
    device time has been measured.  The number of regions follows from the first region's
    (rank-maximum) time, so every rank runs the same number.  Returns [{ms, sm_mhz}]."""
    for _ in range(warmup):
        fn()
    regions, target = [], None
    while target is None or len(regions) < target:
        torch.cuda.synchronize()
        if barrier:
            barrier()
        torch.cuda.synchronize()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        if barrier:
            barrier()
        ms = ev0.elapsed_time(ev1)
        if dist:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        regions.append({"ms": ms, "sm_mhz": clocks.median_between(t0, t1) if clocks else None})
        if target is None:
            target = max(1, min(max_regions, int(min_total_s * 1e3 / max(ms, 1e-3)) + 1))
    return regions


def time_graph_replays(fn, steps, warmup=3):
    """Captures one call of `fn` in a CUDA graph and times replays (device time per
    replay in ms), the way a serving stack issues decode steps; returns None if the
    capture fails."""
    try:
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return time_calls(g.replay, steps, warmup) / steps
    except Exception as ex:  # noqa: BLE001
        sys.stderr.write(f"[bench] CUDA graph capture failed: {ex!r}\n")
        return None


def expert_parallel_leg(args, dev, rank, local_rank, world, dist, barrier):
    """DeepSeek-V3-shaped FP8 layer, one fixed global batch of 4096 tokens (seed 0, zipf-skewed routing over all
    256 experts) whatever N is: on one GPU at N = 1, experts partitioned over the ranks and each rank bringing its
    contiguous share of the tokens at N > 1.  Device-timed like the headline (regions of `steps` calls, median)."""
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200 import _lib
    name, m_global = "deepseek-v3", 4096
    h, i, e, k, dt = WORKLOADS[name]
    layer = Layer(name, dev, rank, world)
    gx, gtw, gids = layer.tokens(m_global, dev, 0)
    m = m_global // world
    x, tw, ids = (t[rank * m:(rank + 1) * m].contiguous() for t in (gx, gtw, gids))
    del gx, gtw
    step = lambda: layer.forward(x, tw, ids)
    steps = max(5, min(args.steps, 20))
    out_first = step()
    torch.cuda.synchronize()
    _ep_check_status(F)                       # a broken exchange shows here, after one call, not after a timed region
    with ClockSampler(physical_index(local_rank)) as clocks:
        regions = time_regions(step, steps, 3, barrier, dist, dev, clocks, min_total_s=0.5)
    _ep_check_status(F)
    # this rank's rows of the result against the one-GPU operator's bits are checked in tests; here: finite and repeatable
    again = step()
    torch.cuda.synchronize()
    repeatable = bool(torch.equal(out_first, again)) and bool(torch.isfinite(again.float()).all())
    # the global batch's output, rank-major = token order: expert parallelism stores the same pair rows and sums
    # them in the same order as one GPU does, so this digest must be the same at every N
    if dist:
        parts = [torch.empty_like(again) for _ in range(world)]
        dist.all_gather(parts, again.contiguous())
        whole = torch.cat(parts)
    else:
        whole = again
    import hashlib
    digest = hashlib.sha256(whole.contiguous().view(torch.int16).cpu().numpy().tobytes()).hexdigest()[:16]
    med = statistics.median(r["ms"] for r in regions)
    # time inside this package's local operator (alignment to output conversion), from events the library records
    lib = _lib.lib()
    _lib.check(lib.b200moe_profile_begin(steps), "profile_begin")
    for _ in range(steps):
        step()
    g1, g2, tot, loc, calls = C.c_double(), C.c_double(), C.c_double(), C.c_double(), C.c_int()
    _lib.check(lib.b200moe_profile_end(C.byref(g1), C.byref(g2), C.byref(tot), C.byref(loc), C.byref(calls)),
               "profile_end")
    n = max(1, calls.value)
    local_ms = loc.value / n
    if dist:
        t = torch.tensor([local_ms, g1.value / n + g2.value / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        local_ms, gemms_ms = float(t[0]), float(t[1])
    else:
        gemms_ms = g1.value / n + g2.value / n
    _, names = _lib.launch_stats()
    hit = int(torch.unique(gids).numel())
    b, f = algorithmic_work(h, i, k, m_global, hit, 1)
    ms_step = med / steps
    per_rank_pairs = None
    if layer.placement is not None:
        dest = (layer.placement.to(gids.device).long()[gids.long()] >> 16)
        per_rank_pairs = torch.bincount(dest.flatten(), minlength=world).tolist()
    res = {"placement": ("contiguous" if os.environ.get("B200MOE_EP_CONTIGUOUS") else
                         "load-balanced from a calibration batch (8192 other tokens, same router bias)") if world > 1 else None,
           "pairs_per_rank": per_rank_pairs, "repeatable_bits": repeatable, "output_sha256_16": digest,
           "workload": f"{name} H{h} I{i} E{e} top{k}, FP8 e4m3 128x128 block scales, zipf(1.1) routing skew, "
                       f"global M {m_global} (seed 0), {e // world} experts and {m} tokens per rank",
           "collective": layer.ep_collective if world > 1 else "none (one GPU)",
           "ms_per_step": ms_step, "tokens_per_s": m_global / (ms_step / 1e3), "steps": steps,
           "regions_ms": [round(r["ms"], 4) for r in regions],
           "local_op_ms": local_ms, "gemms_ms": gemms_ms, "comm_and_glue_ms": max(0.0, ms_step - local_ms),
           "kernels_last_call": names, "experts_hit": hit, "hbm_roofline_frac_whole_job":
               (b / (load_peaks()["hbm_gbs"] * 1e9)) / world / (ms_step / 1e3),
           "clocks": clocks.summary()}
    del layer
    torch.cuda.empty_cache()
    return res


def expert_parallel_emulated(args, dev):
    """`--ep-emulate N`: one process drives N ranks' heaps on ONE GPU, phase by phase in one stream (all
    dispatches, all computes, all combines), at the sizes of the real N-rank run.  For profiling one rank's
    share of the expert-parallel call where a single GPU is at hand (never a multi-rank run under a profiler).
    All ranks share one weight shard, so the timing is right and the numbers are not."""
    from flaggems_sglang_b200 import ep
    from flaggems_sglang_b200.quant import quantize_fp8_block
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    world = args.ep_emulate
    h, i, e, k, _ = WORKLOADS["deepseek-v3"]
    m_global = 4096
    _, _, cal = make_tokens(8192, 64, e, k, seed=1234, skew=True, bias_seed=0)
    placement = ep.plan_placement(e, world, torch.bincount(cal.flatten().long(), minlength=e).tolist())
    x, tw, ids = make_tokens(m_global, h, e, k, device=dev, seed=0, skew=True, bias_seed=0)
    m = m_global // world
    parts = [[], [], [], []]
    for ei in range(e // world):
        a, b = make_weights(h, i, e, device=dev, seed=0, expert_ids=[ei])
        for lst, t in zip(parts, (*quantize_fp8_block(a), *quantize_fp8_block(b))):
            lst.append(t)
    w13q, s13, w2q, s2 = (torch.cat(p).contiguous() for p in parts)
    ctxs = ep.EpContext.emulate(world, m, h, i, k, e // world, e, dev)
    outs = [torch.empty(m, h, dtype=x.dtype, device=dev) for _ in range(world)]
    toks = [tuple(t[r * m:(r + 1) * m].contiguous() for t in (x, tw, ids)) for r in range(world)]

    def call():
        for phase in (1, 2, 4):
            for r in range(world):
                ctxs[r].forward(toks[r][0], w13q, w2q, s13, s2, toks[r][1], toks[r][2], placement, phases=phase,
                                out=outs[r])

    for _ in range(max(1, args.warmup)):
        call()
    torch.cuda.synchronize()
    for c in ctxs:
        c.check_status()
    ms = time_calls(call, max(1, args.steps), 0) / max(1, args.steps)
    from flaggems_sglang_b200 import _lib
    print(json.dumps({"ep_emulated_ranks": world, "ms_per_call_all_ranks": ms, "ms_per_rank": ms / world,
                      "kernels_last_forward": _lib.launch_stats()[1]}), flush=True)
    ep.EpContext.close_emulated(ctxs)


def _ep_check_status(F):
    F.check_status()
    from flaggems_sglang_b200 import ep
    for ctx in ep._contexts.values():
        ctx.check_status()


def run_ours(args, rank, local_rank, world):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200 import _lib

    h, i, e, k, dt = WORKLOADS[args.workload]
    dev = torch.device(f"cuda:{local_rank}")
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    lib = _lib.lib()
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=dev)
    barrier = (lambda: dist.barrier()) if dist else None

    if args.ep_emulate:
        expert_parallel_emulated(args, dev)
        return
    if args.ep_only:
        leg = expert_parallel_leg(args, dev, rank, local_rank, world, dist, barrier)
        if rank == 0:
            print(json.dumps({"ep_only": True, "n_gpus": world, "expert_parallel": leg}), flush=True)
        if dist:
            from flaggems_sglang_b200 import ep
            ep.close_contexts()
            dist.destroy_process_group()
        return

    layer = Layer(args.workload, dev, rank, world)
    # expert parallelism: M is the global batch, split evenly; otherwise every rank has its own M tokens
    m = args.M // world if layer.ep else args.M
    m = max(m, 1)

    def make_step(mm, seed):
        x, tw, ids = layer.tokens(mm, dev, seed)
        return x, tw, ids, (lambda: layer.forward(x, tw, ids))

    # ---- headline: device-resident inputs; regions of `steps` calls until >= 1 s is timed, median region
    x, tw, ids, step = make_step(m, rank)
    warm = max(3, args.warmup)
    with ClockSampler(physical_index(local_rank)) as clocks:
        launches0, _ = _lib.launch_stats()
        regions = time_regions(step, args.steps, warm, barrier, dist, dev, clocks, min_total_s=args.min_seconds)
        launches1, kernel_names = _lib.launch_stats()
    F.check_status()
    ms = statistics.median(r["ms"] for r in regions)
    ms_per_step = ms / args.steps
    value = world * m * args.steps / (ms / 1e3)
    launches_per_step = (launches1 - launches0) // (len(regions) * args.steps + warm)

    # ---- per-kernel timing (same call, CUDA events recorded inside the library on the same stream)
    _lib.check(lib.b200moe_profile_begin(args.steps), "profile_begin")
    for _ in range(args.steps):
        step()
    g1, g2, tot, calls = C.c_double(), C.c_double(), C.c_double(), C.c_int()
    _lib.check(lib.b200moe_profile_end(C.byref(g1), C.byref(g2), C.byref(tot), None, C.byref(calls)), "profile_end")
    n_calls = max(1, calls.value)
    g1_ms, g2_ms, tot_ms = g1.value / n_calls, g2.value / n_calls, tot.value / n_calls

    if layer.ep:
        all_ids = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(all_ids, ids)
        e_loc = e // world
        gids = torch.cat(all_ids)
        hit = int(torch.unique(gids[(gids // e_loc) == rank]).numel())   # experts of this rank that got tokens
        m_eff, slots = m * world, int(((gids // e_loc) == rank).sum())
    else:
        hit = int(torch.unique(ids).numel())
        m_eff, slots = m, m * k
    bw = layer.bytes_w
    bytes_alg, flops_alg = algorithmic_work(h, i, k, m_eff if not layer.ep else slots // k, hit, bw)
    # dominant kernel: the gate/up grouped GEMM (2/3 of the weights and of the flops)
    g1_flops = 4 * slots * h * i
    g1_bytes = hit * 2 * h * i * bw + slots * h * bw + slots * i * bw
    # The kernel is timed inside regions that add up to >= 1 s: the board runs at its power cap, and the
    # matching denominator is the driver's sustained cuBLAS figure (the burst figure is given beside it).
    sustained = args.min_seconds >= 0.5
    tensor_peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    t_tensor = g1_flops / (tensor_peak * 1e12)
    t_hbm = g1_bytes / (peaks["hbm_gbs"] * 1e9)
    g1_bytes = int(g1_bytes)
    if bw == 1:
        t_tensor = 0.0          # FP8 dense peak is not among the measured peaks; this layer is HBM-bound at every M
    if t_tensor >= t_hbm:
        ach = g1_flops / (g1_ms / 1e3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": tensor_peak, "unit": "TFLOP/s",
                "frac": ach / tensor_peak, "peak_kind": "bf16_tflops_sustained (long step under the power cap)"
                if sustained else "bf16_tflops (burst)", "frac_of_burst_peak": ach / peaks["bf16_tflops"]}
    else:
        ach = g1_bytes / (g1_ms / 1e3) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"]}
    gemm1_name = next((n for n in kernel_names if "gate/up" in n), None)
    traffic = NCU_TRAFFIC.get((args.workload, m))
    if traffic is not None and traffic["kernel"] != gemm1_name:
        traffic = None                      # the capture on record is of another kernel than the one that ran
    roof.update({"traffic": traffic["bytes"] if traffic else None,
                 "traffic_source": traffic["source"] if traffic else None,
                 "kernel": f"{gemm1_name} (gate/up projection + activation)",
                 "peak_source": peaks["source"], "kernel_ms": g1_ms, "gemm2_ms": g2_ms, "call_ms": tot_ms,
                 "note": "kernel_ms and gemm2_ms come from CUDA events recorded between the kernels of a call; those "
                         "records serialise what programmatic dependent launch otherwise overlaps, so kernel_ms + "
                         "gemm2_ms can exceed ms_per_step and the fraction is a lower bound",
                 "algorithmic_bytes": g1_bytes, "algorithmic_flops": g1_flops})

    # ---- end to end: pinned host -> device, public entry point, device -> pinned host
    hx, htw, hids = x.cpu().pin_memory(), tw.cpu().pin_memory(), ids.cpu().pin_memory()
    hout = torch.empty(m, h, dtype=x.dtype).pin_memory()
    dx, dtw, dids = torch.empty_like(x), torch.empty_like(tw), torch.empty_like(ids)

    def e2e_step():
        dx.copy_(hx, non_blocking=True)
        dtw.copy_(htw, non_blocking=True)
        dids.copy_(hids, non_blocking=True)
        out = layer.forward(dx, dtw, dids)
        hout.copy_(out, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 20))

    def timed_host(fn_loop):
        torch.cuda.synchronize()
        if barrier:
            barrier()
        t0 = time.perf_counter()
        fn_loop()
        torch.cuda.synchronize()
        dt_ = time.perf_counter() - t0
        if dist:
            t = torch.tensor([dt_], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt_ = float(t.item())
        return dt_

    for _ in range(3):
        e2e_step()
    serial_s = min(timed_host(lambda: [e2e_step() for _ in range(e2e_steps)]) for _ in range(3))
    e2e_s, e2e_mode = serial_s, "serial: copy in, call, copy out on one stream"

    if not layer.ep:
        # The same steps as a serving loop issues them: step i+1's inputs travel while step i computes and
        # step i-1's result travels back (three streams, two buffers each).  Every step still copies its own
        # inputs from pinned host memory and its own result back inside the timed region.
        s_in, s_run, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        bufs = [(torch.empty_like(x), torch.empty_like(tw), torch.empty_like(ids)) for _ in range(2)]
        houts = [torch.empty(m, h, dtype=x.dtype).pin_memory() for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_run = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]

        def pipelined(n):
            for it in range(n):
                b = it & 1
                with torch.cuda.stream(s_in):
                    if it >= 2:
                        s_in.wait_event(ev_run[b])       # the call that last read these input buffers
                    bx, btw, bids = bufs[b]
                    bx.copy_(hx, non_blocking=True)
                    btw.copy_(htw, non_blocking=True)
                    bids.copy_(hids, non_blocking=True)
                    ev_in[b].record(s_in)
                with torch.cuda.stream(s_run):
                    s_run.wait_event(ev_in[b])
                    out = layer.forward(bx, btw, bids)
                    ev_run[b].record(s_run)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_run[b])
                    if it >= 2:
                        s_out.wait_event(ev_out[b])
                    houts[b].copy_(out, non_blocking=True)
                    out.record_stream(s_out)
                    ev_out[b].record(s_out)

        for st_ in (s_in, s_run, s_out):
            st_.wait_stream(torch.cuda.current_stream(dev))
        pipelined(4)
        pipe_s = min(timed_host(lambda: pipelined(e2e_steps)) for _ in range(3))
        F.check_status()
        if not torch.equal(houts[(e2e_steps - 1) & 1], hout):
            # split reductions merge with fp32 atomics and may flip a last bit; anything larger means the pipeline raced
            d = (houts[(e2e_steps - 1) & 1].float() - hout.float()).abs().max().item()
            assert d <= 0.05 * max(1.0, hout.float().abs().max().item()), f"pipelined e2e result differs by {d}"
        if pipe_s < serial_s:
            e2e_s, e2e_mode = pipe_s, "pipelined: copies of neighbouring steps overlap the call (3 streams, 2 buffers)"
    e2e = {"value": world * m * e2e_steps / e2e_s, "unit": "tokens/s",
           "h2d_bytes_per_step": hx.numel() * 2 + htw.numel() * 4 + hids.numel() * 4,
           "d2h_bytes_per_step": hout.numel() * 2, "steps": e2e_steps, "ms_per_step": e2e_s / e2e_steps * 1e3,
           "mode": e2e_mode, "serial_ms_per_step": serial_s / e2e_steps * 1e3, "best_of": 3}

    # ---- sweep over the configuration's other M values (rank 0 of a single-GPU run only)
    sweep = []
    if world == 1 and not args.no_sweep:
        for mm in SWEEP_M[args.workload]:
            _, _, ids_m, st = make_step(mm, 0)
            n = max(5, min(args.steps, 30))
            with ClockSampler(physical_index(local_rank)) as ck:
                reg = time_regions(st, n, 3, None, None, dev, ck, min_total_s=0.25)
            t_eager = statistics.median(r["ms"] for r in reg) / n
            t_graph = time_graph_replays(st, n)
            t_ms = min(t_eager, t_graph) if t_graph else t_eager
            hit_m = int(torch.unique(ids_m).numel())
            b, f = algorithmic_work(h, i, k, mm, hit_m, bw)
            t_tc = 0.0 if bw == 1 else f / (peaks["bf16_tflops"] * 1e12)
            t_tc_sus = 0.0 if bw == 1 else f / (peaks["bf16_tflops_sustained"] * 1e12)
            t_roof = max(b / (peaks["hbm_gbs"] * 1e9), t_tc)
            sweep.append({"M": mm, "us": t_ms * 1e3, "us_eager": t_eager * 1e3,
                          "us_cuda_graph": t_graph * 1e3 if t_graph else None,
                          "tokens_per_s": mm / (t_ms / 1e3), "experts_hit": hit_m,
                          "gbs": b / (t_ms / 1e3) / 1e9, "tflops": f / (t_ms / 1e3) / 1e12,
                          "bound": "hbm" if b / (peaks["hbm_gbs"] * 1e9) >= t_tc else "tensor",
                          "roofline_frac": t_roof / (t_ms / 1e3),
                          "roofline_frac_sustained_peak": max(b / (peaks["hbm_gbs"] * 1e9), t_tc_sus) / (t_ms / 1e3),
                          "regions": len(reg),
                          "sm_mhz": ck.summary()["sm_mhz"], "clock_reasons": ck.summary()["reasons"],
                          "kernels": _lib.launch_stats()[1]})
        F.check_status()

    # ---- the timed call's output against the CPU oracle, once (rank 0 of a single-GPU bf16 run)
    cpu, check = None, {"checked": False}
    if rank == 0 and world == 1 and not args.no_cpu and not layer.fp8 and not layer.int4:
        from oracle import moe as OM
        out_dev = step().float().cpu()
        hx_, htw_, hids_ = x.cpu(), tw.cpu(), ids.cpu()
        del x, tw, ids
        keep = {}
        cpu = cpu_arm(args, h, i, e, k, m, 3, 1, budget_s=15.0, keep=keep)
        cpu = {kk: cpu[kk] for kk in ("value", "unit", "cores", "kind", "sample")}
        ref = OM.fused_experts(hx_, keep["w13f"], keep["w2f"], htw_, hids_).float()
        err = (out_dev - ref).abs()
        check = {"checked": True, "against": "oracle/moe.py on the same seeded inputs, whole output",
                 "frac_within_1e-2": float((err <= 1e-2 + 1e-2 * ref.abs()).float().mean()),
                 "max_err": float(err.max()), "max_ref": float(ref.abs().max()),
                 "bit_equal_frac": float((out_dev == ref).float().mean())}
        del keep, ref, err

    ep_leg = None
    if not args.no_ep_leg and args.workload == "mixtral":
        ep_leg = expert_parallel_leg(args, dev, rank, local_rank, world, dist, barrier)

    if rank == 0:
        line = {
            "metric": "fused_moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong" if WORKLOADS[args.workload][4] == "fp8" and world > 1 else "weak",
            "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": workload_string(args.workload, h, i, e, k, m),
                       "l2": "expert weights (GBs) exceed the 126 MB L2; no flush between steps",
                       "timing": f"{len(regions)} regions of {args.steps} steps (>= {args.min_seconds:g} s of device time "
                                 f"in total), value from the median region",
                       "parallelism": ("single GPU" if world == 1 else
                                       f"{world} independent replicas (no collective)" if not layer_is_ep(args.workload, world)
                                       else f"expert parallel over {world} ranks, global M {m * world}"),
                       "expert_parallel": ep_leg},
            "regions": [{"ms_per_step": r["ms"] / args.steps, "sm_mhz": r["sm_mhz"]} for r in regions],
            "clocks": clocks.summary(), "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "launches_per_step": {"kernels": launches_per_step, "names": kernel_names,
                                  "source": "counted by the library (b200moe_launch_stats)",
                                  "resident_cta_pairs": lib.b200moe_debug_resident_cta_pairs() or None},
            "roofline": roof, "cpu_baseline": cpu, "check": check, "sweep": sweep,
            "whole_call": {"algorithmic_bytes": bytes_alg, "algorithmic_flops": flops_alg, "experts_hit": hit},
        }
        print(json.dumps(line), flush=True)
    if dist:
        from flaggems_sglang_b200 import ep
        ep.close_contexts()
        dist.destroy_process_group()


def layer_is_ep(workload, world):
    return WORKLOADS[workload][4] == "fp8" and world > 1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--workload", default="mixtral", choices=sorted(WORKLOADS))
    ap.add_argument("--M", type=int, default=4096)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-ep-leg", action="store_true", help="skip the expert-parallel DeepSeek-V3 leg")
    ap.add_argument("--ep-only", action="store_true", help="development: run only the expert-parallel leg")
    ap.add_argument("--ep-emulate", type=int, default=0, metavar="N",
                    help="profiling aid: N emulated ranks of the expert-parallel leg on one GPU")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="device time to accumulate over timed regions")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.impl == "reference-gpu":
        if rank == 0:
            run_reference_gpu(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused-MoE path has no CPU fallback "
                         "(use --impl reference for the CPU restatement)")
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
