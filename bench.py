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
NCU_TRAFFIC_BYTES = {("mixtral", 4096): 2201926400}   # profiles/moe_gemm_tc_mixtral_m4096_launch_list.md


def load_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        d = json.loads(f.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


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
        e_ids = range(self.e)
        if self.ep:
            assert self.e % world == 0
            e_loc = self.e // world
            e_ids = range(rank * e_loc, (rank + 1) * e_loc)
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
        return make_tokens(m, self.h, self.e, self.k, dtype=self.act_dtype, device=dev, seed=seed, skew=self.fp8)

    def forward(self, x, tw, ids):
        if self.ep:
            from flaggems_sglang_b200.ep import ep_fused_experts
            return ep_fused_experts(x, self.w13, self.w2, tw, ids, **self.kw)
        return self.F.fused_experts(x, self.w13, self.w2, tw, ids, **self.kw)


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

    layer = Layer(args.workload, dev, rank, world)
    # expert parallelism: M is the global batch, split evenly; otherwise every rank has its own M tokens
    m = args.M // world if layer.ep else args.M
    m = max(m, 1)

    def make_step(mm, seed):
        x, tw, ids = layer.tokens(mm, dev, seed)
        return x, tw, ids, (lambda: layer.forward(x, tw, ids))

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
    t_tensor = g1_flops / (peaks["bf16_tflops"] * 1e12)
    t_hbm = g1_bytes / (peaks["hbm_gbs"] * 1e9)
    g1_bytes = int(g1_bytes)
    if bw == 1:
        t_tensor = 0.0          # FP8 dense peak is not among the measured peaks; this layer is HBM-bound at every M
    if t_tensor >= t_hbm:
        ach = g1_flops / (g1_ms / 1e3) / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": ach / peaks["bf16_tflops"]}
    else:
        ach = g1_bytes / (g1_ms / 1e3) / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"]}
    roof.update({"traffic": NCU_TRAFFIC_BYTES.get((args.workload, m)),
                 "kernel": ("moe_gemm_fp8_kernel<0>" if bw == 1 else "moe_gemm_tc_kernel<0>") + " (gate/up + SiLU*mul)"
                           + (", int4 dequant warps" if bw == 0.5 else ""),
                 "peak_source": peaks["source"], "kernel_ms": g1_ms, "gemm2_ms": g2_ms, "call_ms": tot_ms,
                 "algorithmic_bytes": g1_bytes, "algorithmic_flops": g1_flops})

    # ---- this package's kernels launched by one call (mirrors the choices in csrc/api.cu; NCCL's own kernels
    # in the expert-parallel runs are not counted)
    m_loc = m * world if layer.ep else m          # tokens the local operator sees
    p_loc = m_loc * k
    kernel_names = []
    if layer.ep and bw == 1:
        kernel_names.append("group_quant_fp8 (own tokens, before the all-gather)")
    kernel_names += (["align_count", "align_scan", "align_place"] if p_loc >= 8192 else ["align_block"])
    bt = lib.b200moe_pick_block_tokens(C.byref(_lib.Cfg(C.sizeof(_lib.Cfg), m_loc, h, i, e // world if layer.ep else e, k,
                                                        _lib.DTYPE_FP16 if bw == 0.5 else _lib.DTYPE_BF16,
                                                        {2: _lib.W_16BIT, 1: _lib.W_FP8_BLOCK, 0.5: _lib.W_INT4_AWQ}[bw],
                                                        _lib.LAYOUT_LAYER, 0, 0, 0, 1.0, 0)))
    pair_rows = False
    if bw == 1:
        if layer.ep:
            kernel_names.append("gather_rows (FP8 rows + scales)")
        elif p_loc >= 2048 and k > 1:
            kernel_names += ["group_quant_fp8 (once per token)", "gather_rows (FP8 rows + scales)"]
        else:
            kernel_names.append("group_quant_fp8 (gather + quantise)")
        tokm = bt == 128
        pair_rows = tokm and (p_loc // 128) * ((h + 255) // 256) >= 2 * 148
        kernel_names += ["moe_gemm_fp8_tokm<gate/up>", "moe_gemm_fp8_tokm<down>"] if tokm else \
                        ["moe_gemm_fp8<gate/up>", "moe_gemm_fp8<down>"]
    elif bw == 0.5:
        if bt <= 32:
            kernel_names += ["group_split_i8", "moe_gemm_w4<gate/up>", "moe_gemm_w4<down>"]
        else:
            kernel_names += ["gather_rows", "moe_gemm_tc<gate/up, int4 operands>", "moe_gemm_tc<down, int4 operands>"]
    else:
        kernel_names += ["gather_rows", "moe_gemm_tc<gate/up>", "moe_gemm_tc<down>"]
    kernel_names.append("finalize_pairs" if pair_rows else "finalize")

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
        dt = time.perf_counter() - t0
        if dist:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        return dt

    for _ in range(3):
        e2e_step()
    serial_s = timed_host(lambda: [e2e_step() for _ in range(e2e_steps)])
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
            for i in range(n):
                b = i & 1
                with torch.cuda.stream(s_in):
                    if i >= 2:
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
                    if i >= 2:
                        s_out.wait_event(ev_out[b])
                    houts[b].copy_(out, non_blocking=True)
                    out.record_stream(s_out)
                    ev_out[b].record(s_out)

        for st_ in (s_in, s_run, s_out):
            st_.wait_stream(torch.cuda.current_stream(dev))
        pipelined(4)
        pipe_s = timed_host(lambda: pipelined(e2e_steps))
        F.check_status()
        if not torch.equal(houts[(e2e_steps - 1) & 1], hout):
            # fp32 atomics may flip a last bit; anything larger means the pipeline raced
            d = (houts[(e2e_steps - 1) & 1].float() - hout.float()).abs().max().item()
            assert d <= 0.05 * max(1.0, hout.float().abs().max().item()), f"pipelined e2e result differs by {d}"
        if pipe_s < serial_s:
            e2e_s, e2e_mode = pipe_s, "pipelined: copies of neighbouring steps overlap the call (3 streams, 2 buffers)"
    e2e = {"value": world * m * e2e_steps / e2e_s, "unit": "tokens/s",
           "h2d_bytes_per_step": hx.numel() * 2 + htw.numel() * 4 + hids.numel() * 4,
           "d2h_bytes_per_step": hout.numel() * 2, "steps": e2e_steps, "ms_per_step": e2e_s / e2e_steps * 1e3,
           "mode": e2e_mode, "serial_ms_per_step": serial_s / e2e_steps * 1e3}

    # ---- sweep over the configuration's other M values (rank 0 of a single-GPU run only)
    sweep = []
    if world == 1 and not args.no_sweep:
        for mm in SWEEP_M[args.workload]:
            _, _, ids_m, st = make_step(mm, 0)
            n = max(5, min(args.steps, 30))
            t_eager = time_calls(st, n, 3) / n
            t_graph = time_graph_replays(st, n)
            t_ms = min(t_eager, t_graph) if t_graph else t_eager
            hit_m = int(torch.unique(ids_m).numel())
            b, f = algorithmic_work(h, i, k, mm, hit_m, bw)
            t_tc = 0.0 if bw == 1 else f / (peaks["bf16_tflops"] * 1e12)
            t_roof = max(b / (peaks["hbm_gbs"] * 1e9), t_tc)
            sweep.append({"M": mm, "us": t_ms * 1e3, "us_eager": t_eager * 1e3,
                          "us_cuda_graph": t_graph * 1e3 if t_graph else None,
                          "tokens_per_s": mm / (t_ms / 1e3), "experts_hit": hit_m,
                          "gbs": b / (t_ms / 1e3) / 1e9, "tflops": f / (t_ms / 1e3) / 1e12,
                          "bound": "hbm" if b / (peaks["hbm_gbs"] * 1e9) >= t_tc else "tensor",
                          "roofline_frac": t_roof / (t_ms / 1e3)})
        F.check_status()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and not layer.fp8 and not layer.int4:
        del x, tw, ids
        cpu = cpu_arm(args, h, i, e, k, m, 3, 1, budget_s=15.0)
        cpu = {kk: cpu[kk] for kk in ("value", "unit", "cores", "kind", "sample")}

    if rank == 0:
        line = {
            "metric": "fused_moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong" if layer.ep else "weak", "vs_baseline": None,
            "dtype": dt, "data": "synthetic",
            "config": {"workload": f"{args.workload} H{h} I{i} E{e} top{k} M{m} per GPU, layer-layout weights",
                       "l2": "expert weights (GBs) exceed the 126 MB L2; no flush between steps",
                       "parallelism": ("single GPU" if world == 1 else
                                       f"expert parallel over {world} ranks, all-to-all dispatch/combine, global M {m * world}"
                                       if layer.ep else f"{world} independent replicas (no collective)")},
            "clocks": clocks.summary(), "e2e": e2e,
            "gpu_launches": len(kernel_names) * args.steps,
            "launches_per_step": {"kernels": len(kernel_names), "names": kernel_names},
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
