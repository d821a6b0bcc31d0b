"""Operator calls on HOST tensors: the end-to-end form of ``ops``.

Each call copies its inputs from (ideally pinned) host memory to cached device staging
buffers, runs the same C-ABI kernel as ``ops`` on the current stream, and copies the result
back into a pinned host tensor.  Copies and the kernel are queued on one stream; the
caller synchronises when it needs the result.  This is what a caller that keeps its data
on the host — as every user of the reference does before handing buffers to the generated
kernels — pays per call.
"""
from __future__ import annotations

import torch

from . import ops

_stage: dict = {}


def _dev(tag: str, like: torch.Tensor, dtype=None) -> torch.Tensor:
    key = (tag, tuple(like.shape), dtype or like.dtype, torch.cuda.current_device())
    t = _stage.get(key)
    if t is None:
        t = torch.empty(like.shape, dtype=dtype or like.dtype, device="cuda")
        _stage[key] = t
    return t


def _up(tag: str, h: torch.Tensor) -> torch.Tensor:
    d = _dev(tag, h)
    d.copy_(h, non_blocking=True)
    return d


def _down(d: torch.Tensor, out: torch.Tensor | None) -> torch.Tensor:
    if out is None:
        out = torch.empty(d.shape, dtype=d.dtype, pin_memory=True)
    out.copy_(d, non_blocking=True)
    return out


def clear_staging() -> None:
    _stage.clear()


def layernorm(x, scale, bias, axis, eps=1e-5, out=None):
    y = ops.layernorm(_up("ln_x", x), _up("ln_g", scale), _up("ln_b", bias), axis, eps, out=_dev("ln_y", x))
    return _down(y, out)


def elementwise(x, operation, out=None):
    y = ops.elementwise(_up("ew_x", x), operation, out=_dev("ew_y", x))
    return _down(y, out)


def binary(a, b, operation, out=None):
    da, db = _up("bin_a", a), _up("bin_b", b)
    shape = ops._broadcast_shape(a.shape, b.shape)
    c = ops.binary(da, db, operation, out=_dev("bin_c", torch.empty(shape, dtype=a.dtype, device="meta")))
    return _down(c, out)


def matmul(A, B, out=None):
    C = ops.matmul(_up("mm_a", A), _up("mm_b", B))
    return _down(C, out)


def fmha(Q, K, V, softmax_scale=1.0, causal=False, out=None):
    O = ops.fmha(_up("fa_q", Q), _up("fa_k", K), _up("fa_v", V), softmax_scale, causal)
    return _down(O, out)
