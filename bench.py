#!/usr/bin/env python
"""Benchmark of the operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the bandwidth-bound operator group of the headline configuration
over one batch of synthetic data: LayerNorm over the last dim of [8192, 4096] bf16
(fp32 statistics), GELU(tanh) on [8192, 4096] bf16 and the elementwise add of two
[8192, 4096] bf16 tensors.  The metric is algorithmic HBM bytes per second summed over all
ranks (weak scaling: every rank owns its own rows; no collective is on the data path).

The tensor-core operators of the same library are timed after the headline.  Their results are
reported twice in the one JSON line: in full under "workloads", and inside "roofline" —
"roofline.tensor" (bf16 / FP8 GEMM 8192^3 and attention S = 4096, each with median and best over
at least 50 launches, the SM clock seen, the DRAM traffic of the matching profile and the CPU
loop nests beside it), "roofline.sweep" (the other GEMM / attention sizes next to cuBLAS on the
same GPU) and "roofline.sharded" (the fixed-size 8-GPU workloads split over the ranks of this run,
compute only and with the gather of the outputs).

`--impl reference` times the reference's CPU arithmetic for the same step (the fp32 loop
nests of oracle/kcg_oracle.c on all host threads; the reference's own MLIR->LLVM CPU
lowering does not exist and MLIR is not installed, so there is nothing else to run).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, COLS = 8192, 4096
BUFFER_SETS = 4           # inputs rotate so that no read is served from the 126 MB L2
GRAPH_STEPS = 20          # steps captured per CUDA graph replay
HEADLINE_REPLAYS = 10     # timed replays of the captured steps; the median replay is reported
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
NOMINAL_BF16_TFLOPS = 2250.0
NOMINAL_FP8_TFLOPS = 4500.0


CONFIG = {"workload": f"LayerNorm(last dim)+GELU(tanh)+add on [{ROWS},{COLS}] bf16 per GPU",
          "l2": f"inputs rotate over {BUFFER_SETS} buffer sets (1.8 GB) so reads miss the 126 MB L2",
          "launch": f"steps captured in a CUDA graph ({GRAPH_STEPS} steps per replay, {HEADLINE_REPLAYS} timed replays, "
                    "median replay reported); each kernel is a programmatic dependent of the one before",
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


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


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


def bind_to_gpu_numa_node(local_rank: int) -> dict:
    """Restrict this process to the CPUs of the NUMA node its GPU hangs off, so that pinned host
    buffers allocated afterwards (first touch) and the copy threads sit next to the GPU's PCIe
    root.  Reads sysfs only; nothing about the GPU or the driver is changed.  Returns what was done."""
    info = {"numa_node": None, "cpus": None}
    try:
        import pynvml
        pynvml.nvmlInit()
        index = local_rank
        visible = os.environ.get("CUDA_VISIBLE_DEVICES", "")
        if visible and all(v.strip().isdigit() for v in visible.split(",")):
            index = int(visible.split(",")[local_rank])
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        dev = Path("/sys/bus/pci/devices") / bus.lower()[-12:]
        if not dev.exists():
            dev = Path("/sys/bus/pci/devices") / ("0000:" + bus.lower().split(":", 1)[1])
        node = int((dev / "numa_node").read_text().strip())
        info["numa_node"] = node
        cpulist = (dev / "local_cpulist").read_text().strip()
        cpus = set()
        for part in cpulist.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        allowed = cpus & set(os.sched_getaffinity(0))
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["cpus"] = len(allowed)
    except Exception as exc:   # noqa: BLE001 - affinity is an optimisation, never a requirement
        info["note"] = str(exc)[:120]
    return info


# ------------------------------------------------------------------------------ reference arm
def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as O

    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core it may run on
    threads = host_threads()
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

    # bounded: a step of the loop nests takes ~50 ms on 16 cores, so the caps only matter for huge K / W
    warmup = max(1, min(args.warmup, 50))
    steps = max(1, min(args.steps, 200))
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    val = nbytes / dt / 1e9
    sample = (f"full [{ROWS},{COLS}] step in fp32 (LayerNorm + GELU + add loop nests), {steps} steps after {warmup} "
              "warm-up steps, bytes counted as the bf16 workload's algorithmic bytes")
    print(json.dumps({
        "impl": "reference", "metric": "hbm_gbs_ln_gelu_add", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
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
    threads = host_threads()
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
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the GEMM/FMHA/fp32 side measurements")
    ap.add_argument("--only", default="",
                    help="comma list of extras to run (bw,fp32,bw2,gemm,sgemm,fmha,move,sweep,gather,sharded)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    args.warmup = max(args.warmup, 3)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # before torch allocates anything pinned: sit on the CPUs next to this rank's GPU (undone after
    # the end-to-end section, so that the CPU legs may use every core again)
    affinity_before = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None
    numa = bind_to_gpu_numa_node(local_rank)

    import torch
    import torch.distributed as dist
    from kernelcodegen_b200 import _lib, host, ops

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

    def rnd_big(shape, dtype=dt, std=1.0):
        """N(0, std) in `dtype` without a full-size fp32 temporary (tensors of several GiB)."""
        out = torch.empty(shape, dtype=dtype, device="cuda")
        flat = out.view(-1)
        piece = 1 << 27
        for s in range(0, flat.numel(), piece):
            e = min(flat.numel(), s + piece)
            flat[s:e] = (torch.randn(e - s, generator=gen, device="cuda", dtype=torch.float32) * std).to(dtype)
        return out

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

    # The K steps are captured once into a CUDA graph (over rotating buffers) so that the ~10 us of
    # host work per launch does not sit between 25 us kernels.  The graph is then replayed
    # HEADLINE_REPLAYS times, each replay between its own pair of events; the reported time per
    # step is the median replay divided by K (the mean and the best are reported beside it).
    cap_stream = torch.cuda.Stream()
    with torch.cuda.stream(cap_stream):
        for i in range(args.warmup):
            step(i)
    torch.cuda.synchronize()
    graph_steps = max(1, args.steps)
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
    replays = HEADLINE_REPLAYS
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
    barrier()
    evs[0].record()
    for r in range(replays):
        graph.replay()
        evs[r + 1].record()
    barrier()
    replay_ms = [evs[r].elapsed_time(evs[r + 1]) for r in range(replays)]
    ms_median = max_over_ranks(statistics.median(replay_ms)) / graph_steps
    ms_mean = max_over_ranks(sum(replay_ms) / replays) / graph_steps
    ms_best = max_over_ranks(min(replay_ms)) / graph_steps
    ms_per_step = ms_median
    value = world * total_step_bytes / (ms_per_step * 1e-3) / 1e9
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # ---- roofline of the dominant kernel (LayerNorm): n_roof launches on distinct inputs per
    # replay, each replay timed with CUDA events on the stream it runs on
    peaks = measured_peaks()
    roof_reps = 8
    revs = [torch.cuda.Event(enable_timing=True) for _ in range(roof_reps + 1)]
    revs[0].record()
    for r in range(roof_reps):
        ln_graph.replay()
        revs[r + 1].record()
    torch.cuda.synchronize()
    rms = [revs[r].elapsed_time(revs[r + 1]) / n_roof for r in range(roof_reps)]
    ln_ms = sum(rms) / roof_reps
    clocks = sampler.stop()
    ln_gbs = bytes_step["layernorm"] / (ln_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "ln_rows<bf16> (LayerNorm row kernel)", "achieved": ln_gbs, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": ln_gbs / peaks["hbm_gbs"], "traffic": ncu_traffic("ln_block_rows_bf16_8192x4096"),
                "algorithmic_bytes_per_launch": bytes_step["layernorm"], "avg_launch_ms": ln_ms,
                "median_launch_ms": statistics.median(rms), "best_launch_ms": min(rms),
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
           "steps": e2e_steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           # what limits it: the PCIe copies of one rank (both directions overlap on two copy streams)
           "h2d_gbs_per_rank": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (e2e_ms * 1e-3) / 1e9,
           "host_numa": numa}
    host.clear_staging()
    del hx, hu, ha, hb, oy, ov, oc
    if affinity_before is not None:
        os.sched_setaffinity(0, affinity_before)

    # ---- the other operators of the library, each timed on its own configuration
    workloads = {}
    only = set(filter(None, args.only.split(",")))

    def want(name):
        return not args.no_extras and (not only or name in only)

    def time_op(fn, iters, replays=1, warm=10, idle=0.25):
        """Device time of one call of `fn`: `iters` calls captured in a CUDA graph that is replayed
        `replays` times, each replay between its own pair of events on the launching stream.
        Returns a dict with the median, best and mean time per call over the replays
        (iters x replays launches) and the SM clock sampled meanwhile.  A short idle gap first lets
        the power-capped SM clock recover from the previous workload, so every entry starts from
        the same state; with many replays the later ones run at the sustained clock."""
        torch.cuda.synchronize()
        time.sleep(idle)
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
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(replays + 1)]
        smp = ClockSampler(local_rank, interval=0.001).start()
        ev[0].record()
        for r in range(replays):
            g.replay()
            ev[r + 1].record()
        barrier()
        clk = smp.stop()
        per = [ev[r].elapsed_time(ev[r + 1]) / iters for r in range(replays)]
        return {"ms": max_over_ranks(statistics.median(per)), "best_ms": max_over_ranks(min(per)),
                "mean_ms": max_over_ranks(sum(per) / len(per)), "launches": iters * replays,
                "sm_mhz": clk["sm_mhz"], "throttle_reasons": clk["reasons"]}

    def entry(t, work, unit, **extra):
        """Workload record from a time_op() result: value from the median time, best beside it."""
        scale = 1e12 if unit == "TFLOP/s" else 1e9
        e = {"ms": t["ms"], "best_ms": t["best_ms"], "launches": t["launches"],
             "value": world * work / (t["ms"] * 1e-3) / scale, "best": world * work / (t["best_ms"] * 1e-3) / scale,
             "unit": unit, "sm_mhz": t["sm_mhz"], "throttle_reasons": t["throttle_reasons"]}
        e.update(extra)
        return e

    def cublas_tflops(A, B, C, iters, replays):
        """torch.matmul (cuBLAS) on the same operands, same timing: the library figure beside ours."""
        t = time_op(lambda: torch.matmul(A, B, out=C), iters, replays)
        return t

    def cublaslt_fp8_tflops(A8, B8, one, C, iters, replays, flops):
        """cuBLASLt's FP8 GEMM (torch._scaled_mm) on the same values: the library wants B column-major,
        so it gets the transpose of a row-major [N, K] copy.  None when this torch build has no such call."""
        try:
            Bt = B8.t().contiguous()
            fn = lambda: torch._scaled_mm(A8, Bt.t(), scale_a=one, scale_b=one, out_dtype=C.dtype, out=C)
            fn()
            t = time_op(fn, iters, replays)
            return flops / (t["ms"] * 1e-3) / 1e12
        except Exception:   # noqa: BLE001 - the comparison is optional
            return None

    def sdpa_tflops(Q, K, V, causal, iters, replays, flops):
        """torch's fused attention (whichever library backend it picks for these tensors) on the same
        operands, same timing: the library figure beside ours.  None when it cannot run."""
        try:
            F = torch.nn.functional
            fn = lambda: F.scaled_dot_product_attention(Q, K, V, is_causal=causal)
            fn()
            t = time_op(fn, iters, replays)
            return flops / (t["ms"] * 1e-3) / 1e12
        except Exception:   # noqa: BLE001 - the comparison is optional
            return None

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
        t = time_op(one, 40, 3)
        e = entry(t, bytes_step[op_name], "GB/s")
        e["frac_of_hbm_peak"] = e["value"] / world / peaks["hbm_gbs"]
        workloads[f"{op_name}_bf16_{ROWS}x{COLS}"] = e
    if not args.no_extras:
        # the same three operators as one fused pass (x and the residual in, y out: 3 tensor passes, not 7)
        def fused(i=[0]):
            s = sets[i[0] % BUFFER_SETS]; i[0] += 1
            ops.layernorm_gelu_add(s["x"], gamma, beta, s["a"], 1e-5, out=s["y"])
        t = time_op(fused, 40, 3)
        fb = 3 * ROWS * COLS * 2 + 2 * COLS * 2
        e = entry(t, fb, "GB/s")
        e["frac_of_hbm_peak"] = e["value"] / world / peaks["hbm_gbs"]
        e["speedup_vs_three_kernels"] = (workloads[f"layernorm_bf16_{ROWS}x{COLS}"]["ms"] +
                                         workloads[f"gelu_bf16_{ROWS}x{COLS}"]["ms"] +
                                         workloads[f"add_bf16_{ROWS}x{COLS}"]["ms"]) / t["ms"]
        workloads[f"layernorm_gelu_add_fused_bf16_{ROWS}x{COLS}"] = e
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
            t = time_op(fn, 40, 3)
            e = entry(t, fb[key], "GB/s")
            e["frac_of_hbm_peak"] = e["value"] / world / peaks["hbm_gbs"]
            workloads[f"{name}_f32_{ROWS}x{COLS}"] = e
        del xs, ys
        torch.cuda.empty_cache()

    tensor = {}   # the tensor-core targets, kept inside "roofline"

    def tensor_entry(key, kernel, e, flops, nominal, traffic_key, cublas=None):
        per_gpu = e["value"] / world
        r = {"kernel": kernel, "flops_per_launch": flops, "launches": e["launches"], "median_ms": e["ms"],
             "best_ms": e["best_ms"], "achieved": per_gpu, "best": e["best"] / world, "unit": "TFLOP/s per GPU",
             "peak": peaks["bf16_tflops"] * (nominal / NOMINAL_BF16_TFLOPS), "peak_source": peaks["source"] +
             (" bf16 cuBLAS burst" if nominal == NOMINAL_BF16_TFLOPS else " bf16 cuBLAS burst x 2 (no FP8 peak was measured)"),
             "frac": per_gpu / (peaks["bf16_tflops"] * (nominal / NOMINAL_BF16_TFLOPS)),
             "frac_of_sustained": per_gpu / (peaks["bf16_tflops_sustained"] * (nominal / NOMINAL_BF16_TFLOPS)),
             "frac_of_nominal": per_gpu / nominal, "nominal_peak": nominal,
             "sm_mhz": e["sm_mhz"], "throttle_reasons": e["throttle_reasons"], "traffic": ncu_traffic(traffic_key)}
        if cublas is not None:
            r["cublas_tflops"] = cublas
        tensor[key] = r

    if want("gemm"):
        n = 8192
        A = rnd((n, n), std=n ** -0.5); B = rnd((n, n)); C = torch.empty((n, n), dtype=dt, device="cuda")
        fl = 2 * n ** 3
        e = entry(time_op(lambda: ops.matmul(A, B, out=C), 10, 6), fl, "TFLOP/s")
        tc = cublas_tflops(A, B, C, 10, 6)
        e["cublas_tflops"] = fl / (tc["ms"] * 1e-3) / 1e12
        e["frac_of_measured_bf16_peak"] = e["value"] / world / peaks["bf16_tflops"]
        e["frac_of_nominal_2250"] = e["value"] / world / NOMINAL_BF16_TFLOPS
        workloads["gemm_bf16_8192"] = e
        tensor_entry("gemm_bf16_8192", "gemm_tcgen05_pair_kernel<f16 kind, bf16>", e, fl, NOMINAL_BF16_TFLOPS,
                     "gemm_tcgen05_pair_bf16_8192", e["cublas_tflops"])
        A8 = A.to(torch.float8_e4m3fn); B8 = B.to(torch.float8_e4m3fn)
        one = torch.ones(1, device="cuda")
        e = entry(time_op(lambda: ops.matmul(A8, B8, out_dtype=dt, scale_a=one, scale_b=one, out=C), 10, 6), fl, "TFLOP/s")
        e["frac_of_nominal_4500"] = e["value"] / world / NOMINAL_FP8_TFLOPS
        e["cublas_tflops"] = cublaslt_fp8_tflops(A8, B8, one, C, 10, 6, fl)
        workloads["gemm_fp8_8192"] = e
        tensor_entry("gemm_fp8_8192", "gemm_tcgen05_pair_kernel<f8f6f4 kind, e4m3 -> bf16>", e, fl, NOMINAL_FP8_TFLOPS,
                     "gemm_tcgen05_pair_fp8_8192", e["cublas_tflops"])
        del A, B, C, A8, B8
        torch.cuda.empty_cache()

    if want("sgemm"):
        n = 1024
        A = (torch.rand((n, n), generator=gen, device="cuda") * 2 - 1); B = (torch.rand((n, n), generator=gen, device="cuda") * 2 - 1)
        C = torch.empty((n, n), device="cuda")
        e = entry(time_op(lambda: ops.matmul(A, B, out=C), 20, 3), 2 * n ** 3, "TFLOP/s")
        e["path"] = "tensor cores: three tf32 products of hi/lo-split operands, K in chunks of 256"
        workloads["gemm_f32_1024"] = e
        _lib.load().kcg_gemm_set_fp32_mode(0)
        try:
            e = entry(time_op(lambda: ops.matmul(A, B, out=C), 20, 3), 2 * n ** 3, "TFLOP/s")
        finally:
            _lib.load().kcg_gemm_set_fp32_mode(-1)
        e["path"] = "FFMA kernel, reference accumulation order"
        workloads["gemm_f32_1024_cuda_cores"] = e

    if want("fmha"):
        Bq, H, S, D = 8, 32, 4096, 128
        Q, K, V = rnd((Bq, H, S, D)), rnd((Bq, H, S, D)), rnd((Bq, H, S, D))
        Oo = torch.empty_like(Q)
        for causal in (False, True):
            fl = 4 * Bq * H * S * S * D if not causal else 2 * Bq * H * S * (S + 1) * D
            e = entry(time_op(lambda: ops.fmha(Q, K, V, D ** -0.5, causal, out=Oo), 10, 5), fl, "TFLOP/s")
            e["frac_of_measured_bf16_peak"] = e["value"] / world / peaks["bf16_tflops"]
            e["frac_of_nominal_2250"] = e["value"] / world / NOMINAL_BF16_TFLOPS
            key = f"fmha_bf16_s4096_{'causal' if causal else 'full'}"
            e["torch_sdpa_tflops"] = sdpa_tflops(Q, K, V, causal, 10, 5, fl)
            workloads[key] = e
            tensor_entry(key, "fmha_fwd_kernel2p<bf16, D=128> (persistent two-tile kernel)", e, fl, NOMINAL_BF16_TFLOPS,
                         "fmha_fwd_bf16_b8_h32_s4096_d128" + ("_causal" if causal else ""))
            if e["torch_sdpa_tflops"] is not None:
                tensor[key]["torch_sdpa_tflops"] = e["torch_sdpa_tflops"]
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
            e = entry(time_op(fn, 40, 3), nbytes, "GB/s")
            e["frac_of_hbm_peak"] = e["value"] / world / peaks["hbm_gbs"]
            workloads[f"{name}_bf16_{ROWS}x{COLS}"] = e
        del xs2, outs2, wide
        torch.cuda.empty_cache()
    if want("move"):
        # data-movement operators: embedding-style row gather and a batched transpose
        rows_t, width, n_idx = 200000, 4096, 131072
        table = rnd((rows_t, width))
        idx = torch.randint(0, rows_t, (n_idx,), generator=gen, device="cuda")
        out = torch.empty((n_idx, width), dtype=dt, device="cuda")
        e = entry(time_op(lambda: ops.gather(table, idx, 0, out=out), 20, 3), 2 * out.numel() * 2, "GB/s")
        e["frac_of_hbm_peak"] = e["value"] / world / peaks["hbm_gbs"]
        workloads["gather_rows_bf16_131072x4096"] = e
        del table, idx, out
        x = rnd((4, 8192, 8192)); y = torch.empty((4, 8192, 8192), dtype=dt, device="cuda")
        e = entry(time_op(lambda: ops.transpose(x, out=y), 20, 3), 2 * x.numel() * 2, "GB/s")
        e["frac_of_hbm_peak"] = e["value"] / world / peaks["hbm_gbs"]
        workloads["transpose_bf16_4x8192x8192"] = e
        del x, y
        torch.cuda.empty_cache()
    sweep = {}    # compact copy kept inside "roofline": name -> [median, best, library median] TFLOP/s per GPU
    if want("sweep"):
        # the other sizes of the GEMM and FMHA configurations (per GPU; N ranks run N copies)
        Bq, H, D = 8, 32, 128
        for S in (1024, 2048):
            Q, K, V = rnd((Bq, H, S, D)), rnd((Bq, H, S, D)), rnd((Bq, H, S, D))
            Oo = torch.empty_like(Q)
            for causal in (False, True):
                fl = 4 * Bq * H * S * S * D if not causal else 2 * Bq * H * S * (S + 1) * D
                e = entry(time_op(lambda: ops.fmha(Q, K, V, D ** -0.5, causal, out=Oo), 20, 3), fl, "TFLOP/s")
                e["frac_of_nominal_2250"] = e["value"] / world / NOMINAL_BF16_TFLOPS
                key = f"fmha_bf16_s{S}_{'causal' if causal else 'full'}"
                lib = sdpa_tflops(Q, K, V, causal, 20, 3, fl)
                e["torch_sdpa_tflops"] = lib
                workloads[key] = e
                sweep[key] = [round(e["value"] / world, 1), round(e["best"] / world, 1), None if lib is None else round(lib, 1)]
            del Q, K, V, Oo
        torch.cuda.empty_cache()
        for n in (1024, 2048, 4096, 16384):
            iters, reps = (20, 3) if n <= 4096 else (5, 10)
            for tdt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "f16")):
                A = rnd((n, n), tdt, std=n ** -0.5); B = rnd((n, n), tdt)
                C = torch.empty((n, n), dtype=tdt, device="cuda")
                fl = 2 * n ** 3
                e = entry(time_op(lambda: ops.matmul(A, B, out=C), iters, reps), fl, "TFLOP/s")
                tc = cublas_tflops(A, B, C, iters, reps)
                e["cublas_tflops"] = fl / (tc["ms"] * 1e-3) / 1e12
                e["frac_of_cublas"] = e["value"] / world / e["cublas_tflops"]
                e["frac_of_nominal_2250"] = e["value"] / world / NOMINAL_BF16_TFLOPS
                if n <= 4096:
                    e["note"] = "operands fit the 126 MB L2 (compute-bound shape)"
                workloads[f"gemm_{tag}_{n}"] = e
                sweep[f"gemm_{tag}_{n}"] = [round(e["value"] / world, 1), round(e["best"] / world, 1),
                                            round(e["cublas_tflops"], 1)]
                del A, B, C
            A8 = rnd((n, n), torch.float32, std=n ** -0.5).to(torch.float8_e4m3fn)
            B8 = rnd((n, n), torch.float32).to(torch.float8_e4m3fn)
            C = torch.empty((n, n), dtype=dt, device="cuda")
            one = torch.ones(1, device="cuda")
            e = entry(time_op(lambda: ops.matmul(A8, B8, out_dtype=dt, scale_a=one, scale_b=one, out=C), iters, reps),
                      2 * n ** 3, "TFLOP/s")
            e["frac_of_nominal_4500"] = e["value"] / world / NOMINAL_FP8_TFLOPS
            e["cublas_tflops"] = cublaslt_fp8_tflops(A8, B8, one, C, iters, reps, 2 * n ** 3)
            workloads[f"gemm_fp8_{n}"] = e
            sweep[f"gemm_fp8_{n}"] = [round(e["value"] / world, 1), round(e["best"] / world, 1),
                                      None if e["cublas_tflops"] is None else round(e["cublas_tflops"], 1)]
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

    def timed_loop(fn, iters, warm=3):
        """Eager launches between two events, max over ranks (collectives cannot sit in one graph
        with IPC-mapped stores on every NCCL version, and these steps take a millisecond or more)."""
        for _ in range(warm):
            fn()
        barrier()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / iters

    def multicast_buffers(rows, cols):
        """Symmetric-memory gather buffers bound to an NVLink multicast object, or None (every rank
        gets the same answer: the outcome is agreed on before anyone uses the buffers)."""
        from kernelcodegen_b200 import shard
        mb, good = None, 1
        try:
            mb = shard.MulticastBuffers(rows, cols, dt)
            good = 1 if mb.mc_ptr else 0
        except Exception:   # noqa: BLE001 - no symmetric memory on this host: the peer-store path remains
            good = 0
        flag = torch.tensor([good], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            if mb is not None:
                mb.close()
            return None
        return mb

    bufs = None
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
            ms = timed_loop(fn, 10)
            workloads[name] = {"ms": ms, "value": world * 2 * n ** 3 / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                               "bytes_sent_per_gpu": (world - 1) * n * n * 2,
                               "link_gbs_per_gpu": (world - 1) * n * n * 2 / (ms * 1e-3) / 1e9}
        workloads["gemm_allgather_fused_epilogue"]["bit_identical_to_nccl_path"] = bool(torch.equal(bufs.local, Cg))
        mb = multicast_buffers(world * n, n)
        if mb is not None:
            def mc_iter():
                shard.matmul_allgather(A, B, mb, sync=False)
                shard.stream_barrier()
            ms = timed_loop(mc_iter, 10)
            workloads["gemm_allgather_multicast_epilogue"] = {
                "ms": ms, "value": world * 2 * n ** 3 / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "bytes_sent_per_gpu": n * n * 2, "bit_identical_to_nccl_path": bool(torch.equal(mb.local, Cg))}
            mb.close()
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
            ms = timed_loop(fn, 5)
            workloads[name] = {"ms": ms, "value": world * fl / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                               "bytes_sent_per_gpu": (world - 1) * Q.numel() * 2,
                               "link_gbs_per_gpu": (world - 1) * Q.numel() * 2 / (ms * 1e-3) / 1e9}
        workloads["fmha_allgather_fused_epilogue"]["bit_identical_to_nccl_path"] = bool(
            torch.equal(fb.local.view(world * Bq, H, S, D), Og))
        mb = multicast_buffers(world * Bq * H * S, D)
        if mb is not None:
            def mc_attn():
                shard.fmha_allgather(Q, K, V, mb, world * Bq, D ** -0.5, True, sync=False)
                shard.stream_barrier()
            ms = timed_loop(mc_attn, 5)
            workloads["fmha_allgather_multicast_epilogue"] = {
                "ms": ms, "value": world * fl / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "bytes_sent_per_gpu": Q.numel() * 2,
                "bit_identical_to_nccl_path": bool(torch.equal(mb.local.view(world * Bq, H, S, D), Og))}
            mb.close()
        del Q, K, V, Ol, Og
        fb.close()
        torch.cuda.empty_cache()

    # ---- the fixed-size sharded workloads (strong scaling): the whole problem is split over the
    # ranks of this run; "compute" is every rank's kernel on its shard, "gather" adds the exchange
    # that leaves the full output on every rank (fused into the epilogue where the kernel has one,
    # NCCL all-gather otherwise).  Times are the max over ranks; values count the whole problem.
    sharded = {}
    if want("sharded"):
        from kernelcodegen_b200 import shard
        # GEMM M = 65536, N = K = 8192, bf16: rows of A / C split, B replicated
        Mt, n = 65536, 8192
        b0, cnt = _lib.shard_range(Mt, world, rank, shard.GEMM_ROW_GRANULE)
        A = rnd_big((cnt, n), std=n ** -0.5); B = rnd((n, n))
        Cl = torch.empty((cnt, n), dtype=dt, device="cuda")
        fl = 2 * Mt * n * n
        ms = timed_loop(lambda: ops.matmul(A, B, out=Cl), 5)
        rec = {"shape": f"M={Mt} N=K={n} bf16, {cnt} rows per rank", "compute_ms": ms,
               "compute_tflops": fl / (ms * 1e-3) / 1e12}
        if world > 1:
            gb = None
            try:
                gb = shard.GatherBuffers(Mt, n, dt)
            except RuntimeError as exc:
                rec["gather_error"] = str(exc)[:200]
            if gb is not None:
                def fused_g():
                    shard.matmul_allgather(A, B, gb, sync=False)
                    shard.stream_barrier()
                ms = timed_loop(fused_g, 5)
                rec["gather_fused_ms"] = ms
                rec["gather_fused_tflops"] = fl / (ms * 1e-3) / 1e12
                Cg = torch.empty((Mt, n), dtype=dt, device="cuda")

                def nccl_g():
                    ops.matmul(A, B, out=Cl)
                    dist.all_gather_into_tensor(Cg, Cl)
                ms = timed_loop(nccl_g, 5)
                rec["gather_nccl_ms"] = ms
                rec["gather_fused_bit_identical_to_nccl"] = bool(torch.equal(gb.local, Cg))
                gb.close()
                mb = multicast_buffers(Mt, n)
                if mb is not None:
                    def mc_g():
                        shard.matmul_allgather(A, B, mb, sync=False)
                        shard.stream_barrier()
                    ms = timed_loop(mc_g, 5)
                    rec["gather_multicast_ms"] = ms
                    rec["gather_multicast_tflops"] = fl / (ms * 1e-3) / 1e12
                    rec["gather_multicast_bit_identical_to_nccl"] = bool(torch.equal(mb.local, Cg))
                    mb.close()
                del Cg
        sharded["gemm_bf16_m65536"] = rec
        del A, B, Cl
        torch.cuda.empty_cache()
        # attention B = 64, H = 32, S = 4096, D = 128, causal: whole batches split
        Bt, H, S, D = 64, 32, 4096, 128
        b0, cnt = _lib.shard_range(Bt, world, rank, 1)
        Q, K, V = rnd_big((cnt, H, S, D)), rnd_big((cnt, H, S, D)), rnd_big((cnt, H, S, D))
        Ol = torch.empty_like(Q)
        fl = 2 * Bt * H * S * (S + 1) * D
        ms = timed_loop(lambda: ops.fmha(Q, K, V, D ** -0.5, True, out=Ol), 3)
        rec = {"shape": f"B={Bt} H={H} S={S} D={D} causal bf16, {cnt} batches per rank", "compute_ms": ms,
               "compute_tflops": fl / (ms * 1e-3) / 1e12}
        if world > 1:
            gb = None
            try:
                gb = shard.GatherBuffers(Bt * H * S, D, dt)
            except RuntimeError as exc:
                rec["gather_error"] = str(exc)[:200]
            if gb is not None:
                def fused_a():
                    shard.fmha_allgather(Q, K, V, gb, Bt, D ** -0.5, True, sync=False)
                    shard.stream_barrier()
                ms = timed_loop(fused_a, 3)
                rec["gather_fused_ms"] = ms
                rec["gather_fused_tflops"] = fl / (ms * 1e-3) / 1e12
                Og = torch.empty((Bt, H, S, D), dtype=dt, device="cuda")

                def nccl_a():
                    ops.fmha(Q, K, V, D ** -0.5, True, out=Ol)
                    dist.all_gather_into_tensor(Og, Ol)
                ms = timed_loop(nccl_a, 3)
                rec["gather_nccl_ms"] = ms
                rec["gather_fused_bit_identical_to_nccl"] = bool(torch.equal(gb.local.view(Bt, H, S, D), Og))
                gb.close()
                mb = multicast_buffers(Bt * H * S, D)
                if mb is not None:
                    def mc_a():
                        shard.fmha_allgather(Q, K, V, mb, Bt, D ** -0.5, True, sync=False)
                        shard.stream_barrier()
                    ms = timed_loop(mc_a, 3)
                    rec["gather_multicast_ms"] = ms
                    rec["gather_multicast_tflops"] = fl / (ms * 1e-3) / 1e12
                    rec["gather_multicast_bit_identical_to_nccl"] = bool(torch.equal(mb.local.view(Bt, H, S, D), Og))
                    mb.close()
                del Og
        sharded["fmha_bf16_b64_s4096_causal"] = rec
        del Q, K, V, Ol
        torch.cuda.empty_cache()
        # LayerNorm over [262144, 8192] bf16: rows split
        Rt, Ct = 262144, 8192
        b0, cnt = _lib.shard_range(Rt, world, rank, 1)
        x = rnd_big((cnt, Ct)); y = torch.empty_like(x)
        g2, b2 = rnd((Ct,), mean=1.0, std=0.1), rnd((Ct,), std=0.1)
        nb = Rt * Ct * 2 * 2 + 2 * Ct * 2
        ms = timed_loop(lambda: ops.layernorm(x, g2, b2, 1, 1e-5, out=y), 5)
        rec = {"shape": f"[{Rt},{Ct}] bf16, {cnt} rows per rank", "compute_ms": ms, "compute_gbs": nb / (ms * 1e-3) / 1e9,
               "frac_of_hbm_peak_per_gpu": nb / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        if world > 1:
            yg = torch.empty((Rt, Ct), dtype=dt, device="cuda")

            def nccl_l():
                ops.layernorm(x, g2, b2, 1, 1e-5, out=y)
                dist.all_gather_into_tensor(yg, y)
            ms = timed_loop(nccl_l, 3)
            rec["gather_nccl_ms"] = ms
            mb = multicast_buffers(Rt, Ct)
            if mb is not None:
                def mc_l():
                    shard.layernorm_allgather(x, g2, b2, mb, 1e-5, sync=False)
                    shard.stream_barrier()
                ms = timed_loop(mc_l, 3)
                rec["gather_multicast_ms"] = ms
                rec["gather_multicast_bit_identical_to_nccl"] = bool(torch.equal(mb.local, yg))
                mb.close()
            del yg
        sharded["layernorm_bf16_262144x8192"] = rec
        del x, y
        torch.cuda.empty_cache()
        workloads["sharded"] = sharded

    if rank == 0 and world == 1 and not args.no_extras:
        cpu_side_by_side(workloads)
        for key, r in tensor.items():
            if "cpu" in workloads.get(key, {}):
                r["cpu"] = workloads[key]["cpu"]
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

    if tensor:
        roofline["tensor"] = tensor
    if sweep:
        roofline["sweep"] = {"columns": ["median TFLOP/s", "best TFLOP/s", "library median TFLOP/s (cuBLAS / cuBLASLt for GEMM, torch SDPA for attention)"], **sweep}
    if sharded:
        roofline["sharded"] = sharded
    if rank == 0:
        # a compact copy of the tensor-core figures goes last so that it is what a truncated log keeps
        summary = {k: [round(v["achieved"], 1), round(v["frac"], 3)] for k, v in tensor.items()}
        summary.update({k: v[0] for k, v in sweep.items()})
        print(json.dumps({
            "metric": "hbm_gbs_ln_gelu_add", "value": value, "unit": "GB/s", "n_gpus": world, "steps": graph_steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": CONFIG,
            "timing": {"replays": replays, "ms_per_step_median": ms_median, "ms_per_step_mean": ms_mean,
                       "ms_per_step_best": ms_best},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": 3 * graph_steps * replays,
            "clocks": clocks, "workloads": workloads, "summary_tflops": summary,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
