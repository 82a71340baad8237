#!/usr/bin/env python
"""Fused-MoE layer benchmark (one JSON line on stdout).

Workload: the Mixtral-8x7B-shaped bf16 MoE layer (H=4096, I=14336, E=8, top-2,
weights randn*0.02, routing softmax(randn) -> top-2 -> renormalise), seeded
synthetic data.  One step = one fused-MoE call over a batch of M tokens
(default M=4096); `value` is tokens/s with everything resident in HBM, `e2e`
the same through the public Python entry point with pinned-host inputs and
outputs copied inside the timed region.  With --gpus N every rank runs its own
replica of the layer on its own M tokens (weak scaling, no collective).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
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
}
SWEEP_M = {"mixtral": [1, 16, 128, 1024, 4096], "qwen3-30b-a3b": [1, 8, 32, 64, 128, 256],
           "reference-bench": [1, 4, 17, 64, 1024, 2048, 4096]}

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the
# ncu capture summarised under profiles/ (None until such a capture exists for the workload).
NCU_TRAFFIC_BYTES = {}


def load_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


def algorithmic_work(h, i, k, m, experts_hit, bytes_w=2):
    """bytes = D*3*H*I*b_w + M*H*(b_x + b_out); flops = 6*M*k*H*I."""
    return experts_hit * 3 * h * i * bytes_w + m * h * 4, 6 * m * k * h * i


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
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

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ------------------------------------------------------------------ CPU arm (oracle)
def cpu_arm(args, h, i, e, k, m, steps, warmup, budget_s=12.0):
    """Times the CPU per-expert-loop restatement (oracle/moe.py) on a bounded
    sample of the workload: the first m_cpu tokens of the batch."""
    from flaggems_sglang_b200.testing import make_tokens, make_weights
    from oracle import moe as OM
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen_dev = "cuda" if torch.cuda.is_available() else "cpu"
    w13, w2 = make_weights(h, i, e, device=gen_dev, seed=0)
    w13f, w2f = w13.cpu().float(), w2.cpu().float()
    del w13, w2
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
    h, i, e, k, dt = WORKLOADS[args.workload]
    if rank != 0:
        return
    res = cpu_arm(args, h, i, e, k, args.M, max(1, args.steps), max(0, args.warmup), budget_s=60.0)
    line = {
        "impl": "reference", "metric": "fused_moe_tokens_per_s", "value": res["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
        "config": {"workload": f"{args.workload} H{h} I{i} E{e} top{k} M{args.M}",
                   "note": "the reference has no CPU implementation of this path; this arm times the CPU "
                           "restatement of its algorithm (oracle/moe.py) on the host cores"},
        "cpu_baseline": {"value": res["value"], "unit": "tokens/s", "cores": res["cores"], "kind": "port",
                         "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
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


def run_ours(args, rank, local_rank, world):
    import flaggems_sglang_b200 as F
    from flaggems_sglang_b200 import _lib
    from flaggems_sglang_b200.testing import make_tokens, make_weights

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

    w13, w2 = make_weights(h, i, e, device=dev, seed=0)
    m = args.M

    def make_step(mm, seed):
        x, tw, ids = make_tokens(mm, h, e, k, device=dev, seed=seed)
        return x, tw, ids, (lambda: F.fused_experts(x, w13, w2, tw, ids))

    # ---- headline: device-resident inputs
    x, tw, ids, step = make_step(m, rank)
    with ClockSampler(physical_index(local_rank)) as clocks:
        ms = time_calls(step, args.steps, max(3, args.warmup), barrier)
    F.check_status()
    if dist:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = world * m * args.steps / (ms / 1e3)

    # ---- per-kernel timing (same call, CUDA events recorded inside the library on the same stream)
    _lib.check(lib.b200moe_profile_begin(args.steps), "profile_begin")
    for _ in range(args.steps):
        step()
    g1, g2, tot, calls = C.c_double(), C.c_double(), C.c_double(), C.c_int()
    _lib.check(lib.b200moe_profile_end(C.byref(g1), C.byref(g2), C.byref(tot), C.byref(calls)), "profile_end")
    n_calls = max(1, calls.value)
    g1_ms, g2_ms, tot_ms = g1.value / n_calls, g2.value / n_calls, tot.value / n_calls

    hit = int(torch.unique(ids).numel())
    bytes_alg, flops_alg = algorithmic_work(h, i, k, m, hit)
    # dominant kernel: the gate/up grouped GEMM (2/3 of the weights and of the flops)
    g1_flops = 4 * m * k * h * i
    g1_bytes = hit * 2 * h * i * 2 + m * k * h * 2 + m * k * i * 2
    t_tensor = g1_flops / (peaks["bf16_tflops"] * 1e12)
    t_hbm = g1_bytes / (peaks["hbm_gbs"] * 1e9)
    if t_tensor >= t_hbm:
        ach = g1_flops / (g1_ms / 1e3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": ach / peaks["bf16_tflops"]}
    else:
        ach = g1_bytes / (g1_ms / 1e3) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"]}
    roof.update({"traffic": NCU_TRAFFIC_BYTES.get((args.workload, m)), "kernel": "moe_gemm_tc_kernel<0> (gate/up + SiLU*mul)",
                 "peak_source": peaks["source"], "kernel_ms": g1_ms, "gemm2_ms": g2_ms, "call_ms": tot_ms,
                 "algorithmic_bytes": g1_bytes, "algorithmic_flops": g1_flops})

    # ---- end to end: pinned host -> device, public entry point, device -> pinned host
    hx, htw, hids = x.cpu().pin_memory(), tw.cpu().pin_memory(), ids.cpu().pin_memory()
    hout = torch.empty(m, h, dtype=x.dtype).pin_memory()
    dx, dtw, dids = torch.empty_like(x), torch.empty_like(tw), torch.empty_like(ids)

    def e2e_step():
        dx.copy_(hx, non_blocking=True)
        dtw.copy_(htw, non_blocking=True)
        dids.copy_(hids, non_blocking=True)
        out = F.fused_experts(dx, w13, w2, dtw, dids)
        hout.copy_(out, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if dist:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": world * m * e2e_steps / e2e_s, "unit": "tokens/s",
           "h2d_bytes_per_step": hx.numel() * 2 + htw.numel() * 4 + hids.numel() * 4,
           "d2h_bytes_per_step": hout.numel() * 2, "steps": e2e_steps, "ms_per_step": e2e_s / e2e_steps * 1e3}

    # ---- sweep over the configuration's other M values (rank 0 of a single-GPU run only)
    sweep = []
    if world == 1 and not args.no_sweep:
        for mm in SWEEP_M[args.workload]:
            _, _, ids_m, st = make_step(mm, 0)
            n = max(5, min(args.steps, 30))
            t_ms = time_calls(st, n, 3) / n
            hit_m = int(torch.unique(ids_m).numel())
            b, f = algorithmic_work(h, i, k, mm, hit_m)
            t_roof = max(b / (peaks["hbm_gbs"] * 1e9), f / (peaks["bf16_tflops"] * 1e12))
            sweep.append({"M": mm, "us": t_ms * 1e3, "tokens_per_s": mm / (t_ms / 1e3), "experts_hit": hit_m,
                          "gbs": b / (t_ms / 1e3) / 1e9, "tflops": f / (t_ms / 1e3) / 1e12,
                          "bound": "hbm" if b / (peaks["hbm_gbs"] * 1e9) >= f / (peaks["bf16_tflops"] * 1e12) else "tensor",
                          "roofline_frac": t_roof / (t_ms / 1e3)})
        F.check_status()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        del x, tw, ids
        cpu = cpu_arm(args, h, i, e, k, m, 3, 1, budget_s=15.0)
        cpu = {kk: cpu[kk] for kk in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {
            "metric": "fused_moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dt, "data": "synthetic",
            "config": {"workload": f"{args.workload} H{h} I{i} E{e} top{k} M{m} per GPU, layer-layout weights",
                       "l2": "expert weights (2.8 GB for mixtral) exceed the 126 MB L2; no flush between steps",
                       "parallelism": "single GPU" if world == 1 else f"{world} independent replicas (no collective)"},
            "clocks": clocks.summary(), "e2e": e2e,
            "gpu_launches": 5 * args.steps, "launches_per_step": {"kernels": 5, "memsets": 1},
            "roofline": roof, "cpu_baseline": cpu, "sweep": sweep,
            "whole_call": {"algorithmic_bytes": bytes_alg, "algorithmic_flops": flops_alg, "experts_hit": hit},
        }
        print(json.dumps(line), flush=True)
    if dist:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixtral", choices=sorted(WORKLOADS))
    ap.add_argument("--M", type=int, default=4096)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused-MoE path has no CPU fallback "
                         "(use --impl reference for the CPU restatement)")
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
