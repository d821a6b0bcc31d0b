"""Seeded inputs and comparison helpers shared by the parity tests."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as O

# Tolerances (relative Frobenius error against the float64 oracle).
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 1e-2, "fp8": 3e-2}

SEED0 = 0xC0DE


def gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(SEED0 + seed)
    return g


def randn(shape, dtype, seed, mean=0.0, std=1.0):
    """Host tensor drawn in fp32 then rounded to the storage dtype."""
    t = torch.randn(shape, generator=gen(seed), dtype=torch.float32) * std + mean
    return t.to(dtype)


def uniform(shape, dtype, seed, lo=-1.0, hi=1.0):
    t = torch.rand(shape, generator=gen(seed), dtype=torch.float32) * (hi - lo) + lo
    return t.to(dtype)


def f64(t: torch.Tensor) -> np.ndarray:
    """The values a kernel sees, promoted to float64."""
    return t.detach().to("cpu").to(torch.float64).numpy()


def rel_fro(got: torch.Tensor, want: np.ndarray) -> float:
    return O.rel_fro(f64(got), want)


def sync_ok():
    """Synchronise and assert that no kernel reported a timed-out wait."""
    from kernelcodegen_b200 import _lib
    torch.cuda.synchronize()
    st = _lib.device_status()
    assert st == 0, f"device-side status {st}"
