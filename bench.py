#!/usr/bin/env python
"""Benchmark of the operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the bandwidth-bound operator group of the headline configuration
over one batch of synthetic data: LayerNorm over the last dim of [8192, 4096] bf16
(fp32 statistics), GELU(tanh) on [8192, 4096] bf16 and the elementwise add of two
[8192, 4096] bf16 tensors.  The metric is algorithmic HBM bytes per second summed over all
ranks (weak scaling: every rank owns its own rows; no collective is on the data path).
The tensor-core operators of the same library (GEMM, FMHA) and the fp32 variants are timed
after the headline and reported under "workloads" in the same JSON line.

`--impl reference` times the reference's CPU arithmetic for the same step (the fp32 loop
nests of oracle/kcg_oracle.c on all host threads; the reference's own MLIR->LLVM CPU
lowering does not exist and MLIR is not installed, so there is nothing else to run).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, COLS = 8192, 4096
BUFFER_SETS = 4           # inputs rotate so that no read is served from the 126 MB L2
GRAPH_STEPS = 20          # steps captured per CUDA graph replay
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


CONFIG = {"workload": f"LayerNorm(last dim)+GELU(tanh)+add on [{ROWS},{COLS}] bf16 per GPU",
          "l2": f"inputs rotate over {BUFFER_SETS} buffer sets (1.8 GB) so reads miss the 126 MB L2",
          "launch": f"steps captured in a CUDA graph ({GRAPH_STEPS} steps per replay); each kernel is a programmatic dependent of the one before",
          "sharding": "rows per rank, no collective"}


def step_bytes(esize: int = 2) -> dict:
    n = ROWS * COLS
    return {
        "layernorm": n * 2 * esize + 2 * COLS * esize,
        "gelu": n * 2 * esize,
        "add": n * 3 * esize,
    }


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
            "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def ncu_traffic(kernel: str):
    """DRAM bytes per launch of `kernel` taken from the committed ncu summary, or None."""
    p = ROOT / "profiles" / "ncu_traffic.json"
    if p.exists():
        try:
            return json.loads(p.read_text()).get(kernel)
        except Exception:
            return None
    return None


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a timed region runs."""

    def __init__(self, index: int, interval: float = 0.004):
        self.index = index
        self.interval = interval
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _run(self):
        nv = self._nvml
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.interval)

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------ reference arm
def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as O

    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core it may run on
    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    rng = np.random.default_rng(0xC0DE)
    x = rng.standard_normal((ROWS, COLS), dtype=np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(COLS)).astype(np.float32)
    b = (0.1 * rng.standard_normal(COLS)).astype(np.float32)
    u = rng.standard_normal((ROWS, COLS), dtype=np.float32)
    a1 = rng.standard_normal((ROWS, COLS), dtype=np.float32)
    a2 = rng.standard_normal((ROWS, COLS), dtype=np.float32)
    nbytes = sum(step_bytes().values())

    def step():
        O.ref32.layernorm(x, g, b, 1, threads=threads)
        O.ref32.unary("Gelu", u, threads=threads)
        O.ref32.binary_same("Add", a1, a2, threads=threads)

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    val = nbytes / dt / 1e9
    sample = (f"full [{ROWS},{COLS}] step in fp32 (LayerNorm + GELU + add loop nests), {steps} steps, "
              "bytes counted as the bf16 workload's algorithmic bytes")
    print(json.dumps({
        "impl": "reference", "metric": "hbm_gbs_ln_gelu_add", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": CONFIG,
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_side_by_side(workloads: dict) -> None:
    """Put the CPU loop nests' throughput beside each GEMM / FMHA workload: a bounded sample of
    the same shape, in fp32, on every host core this process may run on."""
    import numpy as np
    from oracle import oracle as O
    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    rng = np.random.default_rng(0xC0DE)

    def note(key, flops, dtc, sample):
        if key in workloads:
            workloads[key]["cpu"] = {"value": flops / dtc / 1e12, "unit": "TFLOP/s", "cores": threads,
                                     "kind": "port", "sample": sample}

    if "gemm_f32_1024" in workloads:
        n = 1024
        A = rng.uniform(-1, 1, (n, n)).astype(np.float32); B = rng.uniform(-1, 1, (n, n)).astype(np.float32)
        t0 = time.perf_counter()
        O.ref32.matmul(A, B, threads=threads)
        note("gemm_f32_1024", 2 * n ** 3, time.perf_counter() - t0, "the full 1024^3 product, fp32 loop nest")
    if "gemm_bf16_8192" in workloads:
        n, rows = 8192, 32
        A = rng.standard_normal((n, n), dtype=np.float32); B = rng.standard_normal((n, n), dtype=np.float32)
        t0 = time.perf_counter()
        O.ref32.matmul(A, B, rows=(0, rows), threads=threads)
        dtc = time.perf_counter() - t0
        for key in ("gemm_bf16_8192", "gemm_fp8_8192"):
            note(key, 2 * rows * n * n, dtc, f"{rows} of the 8192 rows of C at N = K = 8192, fp32 loop nest")
        del A, B
    for causal in (False, True):
        key = f"fmha_bf16_s4096_{'causal' if causal else 'full'}"
        if key not in workloads:
            continue
        S, D = 4096, 128
        Q, K, V = (rng.standard_normal((1, 1, S, D), dtype=np.float32) for _ in range(3))
        t0 = time.perf_counter()
        O.ref32.attention(Q, K, V, D ** -0.5, causal, threads=threads)
        fl = 4 * S * S * D if not causal else 2 * S * (S + 1) * D
        note(key, fl, time.perf_counter() - t0,
             "one of the 256 (batch, head) slices at S = 4096, D = 128: the unfused fp32 chain "
             "BatchedMatmul -> Softmax -> BatchedMatmul")


# ------------------------------------------------------------------------------ our arm
def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the GEMM/FMHA/fp32 side measurements")
    ap.add_argument("--only", default="", help="comma list of extras to run (bw,fp32,bw2,gemm,sgemm,fmha,move,sweep,gather)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from kernelcodegen_b200 import _lib, host, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    _lib.load()
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dt = torch.bfloat16
    gen = torch.Generator(device="cuda").manual_seed(0xC0DE + rank)

    def rnd(shape, dtype=dt, mean=0.0, std=1.0):
        return (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * std + mean).to(dtype)

    sets = []
    for _ in range(BUFFER_SETS):
        sets.append({
            "x": rnd((ROWS, COLS)), "y": torch.empty((ROWS, COLS), dtype=dt, device="cuda"),
            "u": rnd((ROWS, COLS)), "v": torch.empty((ROWS, COLS), dtype=dt, device="cuda"),
            "a": rnd((ROWS, COLS)), "b": rnd((ROWS, COLS)), "c": torch.empty((ROWS, COLS), dtype=dt, device="cuda"),
        })
    gamma, beta = rnd((COLS,), mean=1.0, std=0.1), rnd((COLS,), std=0.1)

    def step(i: int):
        s = sets[i % BUFFER_SETS]
        ops.layernorm(s["x"], gamma, beta, 1, 1e-5, out=s["y"])
        ops.elementwise(s["u"], "Gelu", out=s["v"])
        ops.binary(s["a"], s["b"], "Add", out=s["c"])

    bytes_step = step_bytes(2)
    total_step_bytes = sum(bytes_step.values())

    # The steps are captured once into a CUDA graph (GRAPH_STEPS steps over rotating buffers)
    # and replayed, so that the ~10 us of host work per launch does not sit between 25 us kernels.
    cap_stream = torch.cuda.Stream()
    with torch.cuda.stream(cap_stream):
        for i in range(args.warmup):
            step(i)
    torch.cuda.synchronize()
    graph_steps = min(GRAPH_STEPS, args.steps)
    replays = (args.steps + graph_steps - 1) // graph_steps
    args.steps = replays * graph_steps
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=cap_stream):
        for i in range(graph_steps):
            step(i)
    ln_graph = torch.cuda.CUDAGraph()
    n_roof = 4 * BUFFER_SETS
    with torch.cuda.graph(ln_graph, stream=cap_stream):
        for i in range(n_roof):
            s = sets[i % BUFFER_SETS]
            # x, u, a and b of the 4 sets serve as 16 distinct 64 MB inputs, so none is L2-resident
            src = s[("x", "u", "a", "b")[(i // BUFFER_SETS) % 4]]
            ops.layernorm(src, gamma, beta, 1, 1e-5, out=s["y"])
    graph.replay()
    ln_graph.replay()
    sampler = ClockSampler(local_rank).start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = ms_total / args.steps
    value = world * total_step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- roofline of the dominant kernel (LayerNorm): n_roof launches on distinct inputs,
    # timed with CUDA events on the stream they run on
    peaks = measured_peaks()
    roof_reps = max(3, min(50, args.steps // n_roof))
    e0.record()
    for _ in range(roof_reps):
        ln_graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ln_ms = e0.elapsed_time(e1) / (roof_reps * n_roof)
    clocks = sampler.stop()
    ln_gbs = bytes_step["layernorm"] / (ln_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "ln_block_rows<bf16,8>", "achieved": ln_gbs, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": ln_gbs / peaks["hbm_gbs"], "traffic": ncu_traffic("ln_block_rows_bf16_8192x4096"),
                "algorithmic_bytes_per_launch": bytes_step["layernorm"], "avg_launch_ms": ln_ms,
                "launches_timed": roof_reps * n_roof, "peak_source": peaks["source"]}
    if _lib.device_status() != 0:
        raise SystemExit("a kernel reported a timed-out device-side wait")

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region
    hx = sets[0]["x"].cpu().pin_memory(); hu = sets[0]["u"].cpu().pin_memory()
    ha = sets[0]["a"].cpu().pin_memory(); hb = sets[0]["b"].cpu().pin_memory()
    hg, hbt = gamma.cpu().pin_memory(), beta.cpu().pin_memory()
    oy, ov, oc = (torch.empty((ROWS, COLS), dtype=dt, pin_memory=True) for _ in range(3))

    def e2e_step():
        host.layernorm(hx, hg, hbt, 1, 1e-5, out=oy)
        host.elementwise(hu, "Gelu", out=ov)
        host.binary(ha, hb, "Add", out=oc)

    e2e_steps = max(3, min(args.steps, 30))
    for _ in range(2):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    h2d = (hx.numel() + hu.numel() + ha.numel() + hb.numel() + hg.numel() + hbt.numel()) * 2
    d2h = 3 * ROWS * COLS * 2
    e2e = {"value": world * total_step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
           "steps": e2e_steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    host.clear_staging()
    del hx, hu, ha, hb, oy, ov, oc

    # ---- the other operators of the library, each timed on its BASELINE configuration
    pending_clock = []

    class Workloads(dict):
        """Each entry gets the SM clock sampled while its timed region ran (see time_op)."""

        def __setitem__(self, key, entry):
            if pending_clock and isinstance(entry, dict):
                c = pending_clock.pop()
                entry = dict(entry, sm_mhz=c["sm_mhz"], throttle_reasons=c["reasons"])
            super().__setitem__(key, entry)

    workloads = Workloads()
    only = set(filter(None, args.only.split(",")))

    def want(name):
        return not args.no_extras and (not only or name in only)

    def time_op(fn, iters, warm=3):
        """Average device time of `fn`: `iters` calls captured in a CUDA graph, replayed once timed.
        A short idle gap first lets the power-capped SM clock recover from the previous workload,
        so every entry is a burst figure from the same starting state."""
        torch.cuda.synchronize()
        time.sleep(0.25)
        with torch.cuda.stream(cap_stream):
            for _ in range(warm):
                fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=cap_stream):
            for _ in range(iters):
                fn()
        g.replay()
        barrier()
        smp = ClockSampler(local_rank, interval=0.001).start()
        e0.record()
        g.replay()
        e1.record()
        barrier()
        del pending_clock[:]
        pending_clock.append(smp.stop())
        return max_over_ranks(e0.elapsed_time(e1)) / iters

    for op_name in ("layernorm", "gelu", "add"):
        # per-op split of the headline step, from the same buffers
        def one(i=[0]):
            s = sets[i[0] % BUFFER_SETS]; i[0] += 1
            if op_name == "layernorm":
                ops.layernorm(s["x"], gamma, beta, 1, 1e-5, out=s["y"])
            elif op_name == "gelu":
                ops.elementwise(s["u"], "Gelu", out=s["v"])
            else:
                ops.binary(s["a"], s["b"], "Add", out=s["c"])
        ms = time_op(one, 40)
        gbs = world * bytes_step[op_name] / (ms * 1e-3) / 1e9
        workloads[f"{op_name}_bf16_{ROWS}x{COLS}"] = {"ms": ms, "value": gbs, "unit": "GB/s",
                                                     "frac_of_hbm_peak": gbs / world / peaks["hbm_gbs"]}
    if not args.no_extras:
        # the same three operators as one fused pass (x and the residual in, y out: 3 tensor passes, not 7)
        def fused(i=[0]):
            s = sets[i[0] % BUFFER_SETS]; i[0] += 1
            ops.layernorm_gelu_add(s["x"], gamma, beta, s["a"], 1e-5, out=s["y"])
        ms = time_op(fused, 40)
        fb = 3 * ROWS * COLS * 2 + 2 * COLS * 2
        workloads[f"layernorm_gelu_add_fused_bf16_{ROWS}x{COLS}"] = {
            "ms": ms, "value": world * fb / (ms * 1e-3) / 1e9, "unit": "GB/s",
            "frac_of_hbm_peak": fb / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "speedup_vs_three_kernels": (workloads[f"layernorm_bf16_{ROWS}x{COLS}"]["ms"] +
                                         workloads[f"gelu_bf16_{ROWS}x{COLS}"]["ms"] +
                                         workloads[f"add_bf16_{ROWS}x{COLS}"]["ms"]) / ms}
    del sets
    torch.cuda.empty_cache()

    if want("fp32"):
        xs = [rnd((ROWS, COLS), torch.float32) for _ in range(BUFFER_SETS)]
        ys = [torch.empty_like(xs[0]) for _ in range(2)]
        g32, b32 = rnd((COLS,), torch.float32, 1.0, 0.1), rnd((COLS,), torch.float32, 0.0, 0.1)
        fb = step_bytes(4)
        cnt = [0]

        def ln32():
            cnt[0] += 1
            ops.layernorm(xs[cnt[0] % BUFFER_SETS], g32, b32, 1, 1e-5, out=ys[cnt[0] % 2])

        def gelu32():
            cnt[0] += 1
            ops.elementwise(xs[cnt[0] % BUFFER_SETS], "Gelu", out=ys[cnt[0] % 2])

        def add32():
            cnt[0] += 1
            ops.binary(xs[cnt[0] % BUFFER_SETS], xs[(cnt[0] + 1) % BUFFER_SETS], "Add", out=ys[cnt[0] % 2])

        for name, fn, key in (("layernorm", ln32, "layernorm"), ("gelu", gelu32, "gelu"), ("add", add32, "add")):
            ms = time_op(fn, 40)
            gbs = world * fb[key] / (ms * 1e-3) / 1e9
            workloads[f"{name}_f32_{ROWS}x{COLS}"] = {"ms": ms, "value": gbs, "unit": "GB/s",
                                                     "frac_of_hbm_peak": gbs / world / peaks["hbm_gbs"]}
        del xs, ys
        torch.cuda.empty_cache()

    if want("gemm"):
        n = 8192
        A = rnd((n, n), std=n ** -0.5); B = rnd((n, n)); C = torch.empty((n, n), dtype=dt, device="cuda")
        ms = time_op(lambda: ops.matmul(A, B, out=C), 20)
        tf = world * 2 * n ** 3 / (ms * 1e-3) / 1e12
        workloads["gemm_bf16_8192"] = {"ms": ms, "value": tf, "unit": "TFLOP/s",
                                       "frac_of_measured_bf16_peak": tf / world / peaks["bf16_tflops"],
                                       "frac_of_nominal_2250": tf / world / 2250.0}
        A8 = A.to(torch.float8_e4m3fn); B8 = B.to(torch.float8_e4m3fn)
        one = torch.ones(1, device="cuda")
        ms = time_op(lambda: ops.matmul(A8, B8, out_dtype=dt, scale_a=one, scale_b=one, out=C), 20)
        tf = world * 2 * n ** 3 / (ms * 1e-3) / 1e12
        workloads["gemm_fp8_8192"] = {"ms": ms, "value": tf, "unit": "TFLOP/s", "frac_of_nominal_4500": tf / world / 4500.0}
        del A, B, C, A8, B8
        torch.cuda.empty_cache()

    if want("sgemm"):
        n = 1024
        A = (torch.rand((n, n), generator=gen, device="cuda") * 2 - 1); B = (torch.rand((n, n), generator=gen, device="cuda") * 2 - 1)
        C = torch.empty((n, n), device="cuda")
        ms = time_op(lambda: ops.matmul(A, B, out=C), 20)
        workloads["gemm_f32_1024"] = {"ms": ms, "value": world * 2 * n ** 3 / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                                      "path": "tensor cores: three tf32 products of hi/lo-split operands, K in chunks of 256"}
        _lib.load().kcg_gemm_set_fp32_mode(0)
        try:
            ms = time_op(lambda: ops.matmul(A, B, out=C), 20)
        finally:
            _lib.load().kcg_gemm_set_fp32_mode(-1)
        workloads["gemm_f32_1024_cuda_cores"] = {"ms": ms, "value": world * 2 * n ** 3 / (ms * 1e-3) / 1e12,
                                                 "unit": "TFLOP/s", "path": "FFMA kernel, reference accumulation order"}

    if want("fmha"):
        Bq, H, S, D = 8, 32, 4096, 128
        Q, K, V = rnd((Bq, H, S, D)), rnd((Bq, H, S, D)), rnd((Bq, H, S, D))
        Oo = torch.empty_like(Q)
        for causal in (False, True):
            ms = time_op(lambda: ops.fmha(Q, K, V, D ** -0.5, causal, out=Oo), 10)
            fl = 4 * Bq * H * S * S * D if not causal else 2 * Bq * H * S * (S + 1) * D
            tf = world * fl / (ms * 1e-3) / 1e12
            workloads[f"fmha_bf16_s4096_{'causal' if causal else 'full'}"] = {
                "ms": ms, "value": tf, "unit": "TFLOP/s",
                "frac_of_measured_bf16_peak": tf / world / peaks["bf16_tflops"],
                "frac_of_nominal_2250": tf / world / 2250.0}
        del Q, K, V, Oo
        torch.cuda.empty_cache()
    if want("bw2"):
        # the remaining bandwidth operators on the headline shape: softmax over the last dim (in
        # place, as the reference does it), a bias-style broadcast add, and a widening Cast
        xs2 = [rnd((ROWS, COLS)) for _ in range(4)]
        bias_v = rnd((COLS,))
        outs2 = [torch.empty((ROWS, COLS), dtype=dt, device="cuda") for _ in range(4)]
        wide = [torch.empty((ROWS, COLS), dtype=torch.float32, device="cuda") for _ in range(2)]
        esz = 2

        def sm(i=[0]):
            i[0] += 1
            ops.softmax(xs2[i[0] % 4])

        def badd(i=[0]):
            i[0] += 1
            ops.binary(xs2[i[0] % 4], bias_v, "Add", out=outs2[i[0] % 4])

        def cast(i=[0]):
            i[0] += 1
            ops.elementwise(xs2[i[0] % 4], "Cast", dtype=torch.float32, out=wide[i[0] % 2])

        for name, fn, nbytes in (("softmax_inplace", sm, 2 * ROWS * COLS * esz),
                                 ("broadcast_add_row", badd, 2 * ROWS * COLS * esz + COLS * esz),
                                 ("cast_bf16_to_f32", cast, ROWS * COLS * (esz + 4))):
            ms = time_op(fn, 40)
            gbs = world * nbytes / (ms * 1e-3) / 1e9
            workloads[f"{name}_bf16_{ROWS}x{COLS}"] = {"ms": ms, "value": gbs, "unit": "GB/s",
                                                       "frac_of_hbm_peak": gbs / world / peaks["hbm_gbs"]}
        del xs2, outs2, wide
        torch.cuda.empty_cache()
    if want("move"):
        # data-movement operators: embedding-style row gather and a batched transpose
        rows_t, width, n_idx = 200000, 4096, 131072
        table = rnd((rows_t, width))
        idx = torch.randint(0, rows_t, (n_idx,), generator=gen, device="cuda")
        out = torch.empty((n_idx, width), dtype=dt, device="cuda")
        ms = time_op(lambda: ops.gather(table, idx, 0, out=out), 20)
        gbs = world * 2 * out.numel() * 2 / (ms * 1e-3) / 1e9
        workloads["gather_rows_bf16_131072x4096"] = {"ms": ms, "value": gbs, "unit": "GB/s",
                                                     "frac_of_hbm_peak": gbs / world / peaks["hbm_gbs"]}
        del table, idx, out
        x = rnd((4, 8192, 8192)); y = torch.empty((4, 8192, 8192), dtype=dt, device="cuda")
        ms = time_op(lambda: ops.transpose(x, out=y), 20)
        gbs = world * 2 * x.numel() * 2 / (ms * 1e-3) / 1e9
        workloads["transpose_bf16_4x8192x8192"] = {"ms": ms, "value": gbs, "unit": "GB/s",
                                                   "frac_of_hbm_peak": gbs / world / peaks["hbm_gbs"]}
        del x, y
        torch.cuda.empty_cache()
    if want("sweep"):
        # the other sizes of the GEMM and FMHA configurations (per GPU; N ranks run N copies)
        Bq, H, D = 8, 32, 128
        for S in (1024, 2048):
            Q, K, V = rnd((Bq, H, S, D)), rnd((Bq, H, S, D)), rnd((Bq, H, S, D))
            Oo = torch.empty_like(Q)
            for causal in (False, True):
                ms = time_op(lambda: ops.fmha(Q, K, V, D ** -0.5, causal, out=Oo), 20)
                fl = 4 * Bq * H * S * S * D if not causal else 2 * Bq * H * S * (S + 1) * D
                tf = world * fl / (ms * 1e-3) / 1e12
                workloads[f"fmha_bf16_s{S}_{'causal' if causal else 'full'}"] = {
                    "ms": ms, "value": tf, "unit": "TFLOP/s", "frac_of_nominal_2250": tf / world / 2250.0}
            del Q, K, V, Oo
        torch.cuda.empty_cache()
        for n in (1024, 2048, 4096, 16384):
            for tdt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "f16")):
                A = rnd((n, n), tdt, std=n ** -0.5); B = rnd((n, n), tdt)
                C = torch.empty((n, n), dtype=tdt, device="cuda")
                ms = time_op(lambda: ops.matmul(A, B, out=C), 20 if n <= 4096 else 8)
                tf = world * 2 * n ** 3 / (ms * 1e-3) / 1e12
                workloads[f"gemm_{tag}_{n}"] = {"ms": ms, "value": tf, "unit": "TFLOP/s",
                                                "frac_of_nominal_2250": tf / world / 2250.0}
                if n <= 4096:
                    workloads[f"gemm_{tag}_{n}"]["note"] = "operands fit the 126 MB L2 (compute-bound shape)"
                del A, B, C
            A8 = rnd((n, n), torch.float32, std=n ** -0.5).to(torch.float8_e4m3fn)
            B8 = rnd((n, n), torch.float32).to(torch.float8_e4m3fn)
            C = torch.empty((n, n), dtype=dt, device="cuda")
            one = torch.ones(1, device="cuda")
            ms = time_op(lambda: ops.matmul(A8, B8, out_dtype=dt, scale_a=one, scale_b=one, out=C), 20 if n <= 4096 else 8)
            tf = world * 2 * n ** 3 / (ms * 1e-3) / 1e12
            workloads[f"gemm_fp8_{n}"] = {"ms": ms, "value": tf, "unit": "TFLOP/s", "frac_of_nominal_4500": tf / world / 4500.0}
            del A8, B8, C
            torch.cuda.empty_cache()
    if world > 1 and not args.no_extras:
        # the optional exchange: NCCL all-gather of a sharded output (here the 128 MiB bf16 C
        # block of the GEMM shard and the 64 MiB LayerNorm block), timed on the device
        for name, shape in (("allgather_gemm_c_block", (8192, 8192)), ("allgather_ln_block", (ROWS, COLS))):
            loc = torch.zeros(shape, dtype=dt, device="cuda")
            out = torch.empty((shape[0] * world, shape[1]), dtype=dt, device="cuda")
            for _ in range(3):
                dist.all_gather_into_tensor(out, loc)
            barrier()
            e0.record()
            for _ in range(5):
                dist.all_gather_into_tensor(out, loc)
            e1.record()
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1)) / 5
            recv = (world - 1) * loc.numel() * 2
            workloads[name] = {"ms": ms, "value": recv / (ms * 1e-3) / 1e9, "unit": "GB/s received per GPU"}
            del loc, out
        torch.cuda.empty_cache()
    if world > 1 and want("gather"):
        # replicated C from a row-sharded GEMM, two ways: the epilogue that stores every tile into
        # all ranks' buffers (peer stores over NVLink) against the plain kernel followed by an
        # NCCL all-gather.  Per rank M = N = K = 8192; ranks meet on the stream once per iteration.
        from kernelcodegen_b200 import shard
        n = 8192
        A = rnd((n, n), std=n ** -0.5); B = rnd((n, n))
        try:
            bufs = shard.GatherBuffers(world * n, n, dt)   # raises on every rank if peer mapping fails on any
        except RuntimeError as exc:
            bufs = None
            workloads["gemm_allgather_fused_epilogue"] = {"error": str(exc)[:300]}
    if world > 1 and want("gather") and bufs is not None:
        Cl = torch.empty((n, n), dtype=dt, device="cuda")
        Cg = torch.empty((world * n, n), dtype=dt, device="cuda")

        def fused_iter():
            shard.matmul_allgather(A, B, bufs, sync=False)
            shard.stream_barrier()

        def nccl_iter():
            ops.matmul(A, B, out=Cl)
            dist.all_gather_into_tensor(Cg, Cl)

        for name, fn in (("gemm_allgather_fused_epilogue", fused_iter), ("gemm_then_nccl_allgather", nccl_iter)):
            for _ in range(3):
                fn()
            barrier()
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1)) / 10
            workloads[name] = {"ms": ms, "value": world * 2 * n ** 3 / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                               "bytes_sent_per_gpu": (world - 1) * n * n * 2,
                               "link_gbs_per_gpu": (world - 1) * n * n * 2 / (ms * 1e-3) / 1e9}
        workloads["gemm_allgather_fused_epilogue"]["bit_identical_to_nccl_path"] = bool(torch.equal(bufs.local, Cg))
        del A, B, Cl, Cg
        bufs.close()
        torch.cuda.empty_cache()
        # the same comparison for attention: 8 batches x 32 heads per rank, S = 4096, D = 128, causal
        Bq, H, S, D = 8, 32, 4096, 128
        Q, K, V = rnd((Bq, H, S, D)), rnd((Bq, H, S, D)), rnd((Bq, H, S, D))
        fb = shard.GatherBuffers(world * Bq * H * S, D, dt)   # the mapping worked for the GEMM buffers above
        Ol = torch.empty_like(Q)
        Og = torch.empty((world * Bq, H, S, D), dtype=dt, device="cuda")

        def fused_attn():
            shard.fmha_allgather(Q, K, V, fb, world * Bq, D ** -0.5, True, sync=False)
            shard.stream_barrier()

        def nccl_attn():
            ops.fmha(Q, K, V, D ** -0.5, True, out=Ol)
            dist.all_gather_into_tensor(Og, Ol)

        fl = 2 * Bq * H * S * (S + 1) * D
        for name, fn in (("fmha_allgather_fused_epilogue", fused_attn), ("fmha_then_nccl_allgather", nccl_attn)):
            for _ in range(3):
                fn()
            barrier()
            e0.record()
            for _ in range(5):
                fn()
            e1.record()
            barrier()
            ms = max_over_ranks(e0.elapsed_time(e1)) / 5
            workloads[name] = {"ms": ms, "value": world * fl / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                               "bytes_sent_per_gpu": (world - 1) * Q.numel() * 2,
                               "link_gbs_per_gpu": (world - 1) * Q.numel() * 2 / (ms * 1e-3) / 1e9}
        workloads["fmha_allgather_fused_epilogue"]["bit_identical_to_nccl_path"] = bool(
            torch.equal(fb.local.view(world * Bq, H, S, D), Og))
        del Q, K, V, Ol, Og
        fb.close()
        torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_extras:
        cpu_side_by_side(workloads)
    if _lib.device_status() != 0:
        raise SystemExit("a kernel reported a timed-out device-side wait")

    # ---- CPU baseline beside it (rank 0, single GPU runs only): the fp32 loop nests, one core
    cpu_baseline = None
    if rank == 0 and world == 1:
        import numpy as np
        from oracle import oracle as O
        rng = np.random.default_rng(0xC0DE)
        x = rng.standard_normal((ROWS, COLS), dtype=np.float32)
        g = np.ones(COLS, np.float32); b = np.zeros(COLS, np.float32)
        t0 = time.perf_counter()
        O.ref32.layernorm(x, g, b, 1, threads=1)
        O.ref32.unary("Gelu", x, threads=1)
        O.ref32.binary_same("Add", x, x, threads=1)
        dtc = time.perf_counter() - t0
        cpu_baseline = {"value": total_step_bytes / dtc / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                        "sample": f"one full [{ROWS},{COLS}] step of the fp32 loop nests on one core ({dtc:.2f} s); "
                                  "bytes counted as the bf16 workload's algorithmic bytes"}

    if rank == 0:
        print(json.dumps({
            "metric": "hbm_gbs_ln_gelu_add", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": CONFIG,
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": 3 * args.steps,
            "clocks": clocks, "workloads": workloads,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
