"""Multi-GPU sharding of the operators: one process per GPU, no collective on the compute path.

The reference is a single-GPU code generator; sharding exists only here.  Every operator
of the library has independent units — GEMM rows of A / C (B replicated), attention
(batch, head) slices, LayerNorm and elementwise rows — so each rank runs the ordinary
single-GPU kernel on a contiguous block of units (``shard_range``) and results are
bit-identical to the single-GPU run.  The only exchange is the optional all-gather of the
outputs when the caller wants a replicated result; it goes through ``torch.distributed``
(NCCL over NVLink on GPUs, gloo in the CPU tests).

``compute`` arguments exist so that the partition / gather logic can be exercised on CPU
ranks with a stand-in for the CUDA kernel; the default is always the real kernel.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _lib

GEMM_ROW_GRANULE = 128   # CTA tile height of the tensor-core GEMM: keeps shards tile-aligned


def world_and_rank(group=None) -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def shard_range(total: int, granule: int = 1, group=None, world: Optional[int] = None,
                rank: Optional[int] = None) -> tuple[int, int]:
    """(begin, count) of the units this rank owns (C ABI: kcg_shard_range)."""
    if world is None or rank is None:
        world, rank = world_and_rank(group)
    return _lib.shard_range(total, world, rank, granule)


def shard_rows(full: torch.Tensor, granule: int = 1, group=None) -> torch.Tensor:
    """This rank's contiguous block of dim 0 of a replicated tensor (a view)."""
    b, c = shard_range(full.shape[0], granule, group)
    return full[b:b + c]


def all_gather_rows(local: torch.Tensor, total_rows: int, granule: int = 1, group=None) -> torch.Tensor:
    """Replicated [total_rows, ...] tensor assembled from every rank's block of dim 0.

    Blocks may differ in size (the split is by granules), so ranks exchange blocks padded to
    the largest one and drop the padding afterwards.
    """
    world, rank = world_and_rank(group)
    if world == 1:
        return local
    ranges = [_lib.shard_range(total_rows, world, r, granule) for r in range(world)]
    biggest = max(c for _, c in ranges)
    tail = tuple(local.shape[1:])
    if all(c == biggest for _, c in ranges):
        out = torch.empty((total_rows,) + tail, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((biggest,) + tail, dtype=local.dtype, device=local.device)
    padded[:local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:c] for p, (_, c) in zip(parts, ranges)], dim=0)


def _ops():
    from . import ops
    return ops


def matmul(A_local: torch.Tensor, B: torch.Tensor, total_rows: Optional[int] = None, gather: bool = False,
           group=None, compute: Optional[Callable] = None, **kw) -> torch.Tensor:
    """C = A B with A (and C) split along M and B replicated; A_local is this rank's row block."""
    fn = compute or _ops().matmul
    C_local = fn(A_local, B, **kw)
    if not gather:
        return C_local
    if total_rows is None:
        raise ValueError("gather=True needs total_rows (the M of the full problem)")
    return all_gather_rows(C_local, total_rows, GEMM_ROW_GRANULE, group)


def layernorm(x_local: torch.Tensor, scale, bias, axis: int, eps: float = 1e-5, total_rows: Optional[int] = None,
              gather: bool = False, group=None, compute: Optional[Callable] = None) -> torch.Tensor:
    """LayerNorm with the leading (non-normalised) dim split over ranks; axis must be >= 1."""
    ax = axis if axis >= 0 else axis + x_local.dim()
    if ax < 1:
        raise ValueError("sharded LayerNorm splits dim 0, so the normalised dims must start at axis >= 1")
    fn = compute or _ops().layernorm
    y_local = fn(x_local, scale, bias, axis, eps)
    if not gather:
        return y_local
    if total_rows is None:
        raise ValueError("gather=True needs total_rows")
    return all_gather_rows(y_local, total_rows, 1, group)


def elementwise(x_local: torch.Tensor, operation: str, total_rows: Optional[int] = None, gather: bool = False,
                group=None, compute: Optional[Callable] = None) -> torch.Tensor:
    fn = compute or _ops().elementwise
    y_local = fn(x_local, operation)
    if not gather:
        return y_local
    if total_rows is None:
        raise ValueError("gather=True needs total_rows")
    return all_gather_rows(y_local, total_rows, 1, group)


def fmha(Q_local, K_local, V_local, softmax_scale: float = 1.0, causal: bool = False,
         total_slices: Optional[int] = None, gather: bool = False, group=None,
         compute: Optional[Callable] = None) -> torch.Tensor:
    """Attention with the (batch*head) slices split over ranks.

    Operands are [slices, 1, S, D] (or [batch_block, H, S, D] when whole batches are split);
    dim 0 is the sharded one.
    """
    fn = compute or _ops().fmha
    O_local = fn(Q_local, K_local, V_local, softmax_scale, causal)
    if not gather:
        return O_local
    if total_slices is None:
        raise ValueError("gather=True needs total_slices")
    return all_gather_rows(O_local, total_slices, 1, group)
