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


# ---- gather fused into the GEMM epilogue: tiles stored straight into every rank's buffer -----

class _CudaArray:
    """Minimal __cuda_array_interface__ carrier so torch can view memory this library allocated."""

    def __init__(self, ptr: int, shape, typestr: str, owner):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}
        self._owner = owner


_TYPESTR = {torch.bfloat16: None, torch.float16: "<f2", torch.float32: "<f4"}


class GatherBuffers:
    """One [total_rows, cols] matrix per rank, each mapped into every process of the group.

    ``local`` is this rank's matrix as a torch tensor; ``ptrs[r]`` is the address of rank r's
    matrix as seen from this process (rank's own allocation, or a CUDA-IPC mapping of a peer's).
    Collective: every rank of the group must construct it (handles are exchanged with
    all_gather_object) and ``close()`` it.
    """

    def __init__(self, total_rows: int, cols: int, dtype: torch.dtype, group=None):
        import ctypes
        self.world, self.rank = world_and_rank(group)
        self.group = group
        self.total_rows, self.cols, self.dtype = int(total_rows), int(cols), dtype
        esize = torch.empty((), dtype=dtype).element_size()
        self.nbytes = self.total_rows * self.cols * esize
        lib = _lib.load()
        self._own = None
        self._opened = []
        self.ptrs = [None] * self.world
        # Every step that can fail on one rank is followed by an exchange of its outcome, so that
        # all ranks raise together instead of leaving the others inside a collective.
        err = None
        handle = None
        p = ctypes.c_void_p()
        try:
            _lib.check(lib.kcg_peer_alloc(self.nbytes, ctypes.byref(p)), "kcg_peer_alloc")
            self._own = p.value
            self.ptrs[self.rank] = self._own
            if self.world > 1:
                h = ctypes.create_string_buffer(64)
                _lib.check(lib.kcg_peer_export(self._own, h), "kcg_peer_export")
                handle = bytes(h.raw)
        except Exception as e:   # noqa: BLE001 - reported to every rank below
            err = f"rank {self.rank}: {e}"
        if self.world > 1:
            got = [None] * self.world
            dist.all_gather_object(got, (handle, err), group=group)
            errs = [e for _, e in got if e]
            if not errs:
                for r, (hb, _) in enumerate(got):
                    if r == self.rank:
                        continue
                    q = ctypes.c_void_p()
                    rc = lib.kcg_peer_open(ctypes.create_string_buffer(hb, 64), ctypes.byref(q))
                    if rc != 0:
                        err = f"rank {self.rank}: kcg_peer_open of rank {r}'s buffer: status {rc} ({lib.kcg_last_error().decode()})"
                        break
                    self.ptrs[r] = q.value
                    self._opened.append(q.value)
                got2 = [None] * self.world
                dist.all_gather_object(got2, err, group=group)
                errs = [e for e in got2 if e]
            if errs:
                self.local = None
                self.close()
                raise RuntimeError("GatherBuffers: " + "; ".join(errs))
        elif err:
            raise RuntimeError("GatherBuffers: " + err)
        # torch view of the local matrix (bf16 has no array-interface code: view 16-bit words)
        ts = _TYPESTR[dtype] or "<i2"
        t = torch.as_tensor(_CudaArray(self._own, (self.total_rows, self.cols), ts, self), device="cuda")
        self.local = t.view(dtype) if t.dtype != dtype else t

    def close(self) -> None:
        """Unmap the peers' matrices, then (after every rank has done so) free the local one."""
        lib = _lib.load()
        for q in self._opened:
            lib.kcg_peer_close(q)
        self._opened = []
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        if self._own:
            self.local = None
            lib.kcg_peer_free(self._own)
            self._own = None


class MulticastBuffers:
    """One [total_rows, cols] matrix per rank in symmetric memory that is also bound to an NVLink
    multicast object, so that one store to ``mc_ptr + offset`` lands in every rank's matrix.

    The allocation, the exchange of handles and the multicast binding are torch's
    (``torch.distributed._symmetric_memory``): plumbing.  ``local`` is this rank's matrix, ``ptrs[r]``
    rank r's matrix as seen from this process (usable for plain peer stores), ``mc_ptr`` the
    multicast address of the matrix (0 when the fabric or the driver offers no multicast: the gather
    epilogues then fall back to one peer store per rank).  Collective: every rank constructs it and
    calls ``close()``; no rank may exit while its memory is still bound, so ``close()`` ends with a
    barrier and drops the mapping on every rank before any of them moves on.
    """

    def __init__(self, total_rows: int, cols: int, dtype: torch.dtype, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.world, self.rank = world_and_rank(group)
        self.group = group
        self.total_rows, self.cols, self.dtype = int(total_rows), int(cols), dtype
        dev = torch.device("cuda", torch.cuda.current_device())
        self.local = symm_mem.empty((self.total_rows, self.cols), dtype=dtype, device=dev)
        pg = group if group is not None else dist.group.WORLD
        self._handle = symm_mem.rendezvous(self.local, pg)
        off = int(getattr(self._handle, "offset", 0))
        self.ptrs = [int(p) + off for p in self._handle.buffer_ptrs]
        mc = int(self._handle.multicast_ptr or 0)
        self.mc_ptr = mc + off if mc else 0

    def close(self) -> None:
        torch.cuda.synchronize()
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)
        self._handle = None
        self.local = None
        self.mc_ptr = 0
        if self.world > 1 and dist.is_initialized():
            dist.barrier(group=self.group)


_barrier_word = {}


def stream_barrier(group=None) -> None:
    """All ranks meet on the current CUDA stream (a one-element all-reduce): work queued after it
    starts only when every rank's earlier work on its stream has finished.  The host does not wait."""
    dev = torch.cuda.current_device()
    w = _barrier_word.get(dev)
    if w is None:
        w = _barrier_word[dev] = torch.zeros(1, device="cuda")
    dist.all_reduce(w, group=group)


def matmul_allgather(A_local: torch.Tensor, B: torch.Tensor, bufs: GatherBuffers, trans_b: bool = False,
                     scale_a=None, scale_b=None, bias=None, activation=None, sync: bool = True) -> torch.Tensor:
    """Replicated C = A B with A split along M: each rank's GEMM epilogue writes its row block
    into every rank's buffer (peer stores over NVLink), so no separate all-gather runs.

    With ``sync`` the ranks meet on the stream before the launch (nobody still reads the buffers)
    and after it (every block has landed); pass False to place those barriers yourself.
    Returns ``bufs.local``.
    """
    import ctypes
    from . import ops
    if not (A_local.is_cuda and B.is_cuda and A_local.is_contiguous() and B.is_contiguous()):
        raise ValueError("operands must be contiguous CUDA tensors")
    if A_local.dim() != 2 or B.dim() != 2:
        raise ValueError("Matmul takes rank-2 operands")
    if A_local.dtype != B.dtype:
        raise TypeError(f"operands must share a dtype (got {A_local.dtype} and {B.dtype})")
    M, K = A_local.shape
    N = B.shape[0] if trans_b else B.shape[1]
    if (B.shape[1] if trans_b else B.shape[0]) != K:
        raise ValueError("Can't apply Matmul Operation due to imcompatible K-dim.")
    if N != bufs.cols:
        raise ValueError("buffer width does not match N")
    begin, count = _lib.shard_range(bufs.total_rows, bufs.world, bufs.rank, GEMM_ROW_GRANULE)
    if count != M:
        raise ValueError(f"this rank owns {count} rows of the gathered matrix, A_local has {M}")
    act = {None: 0, "": 0, "Relu": 1, "Gelu": 2}[activation]
    stream = torch.cuda.current_stream().cuda_stream
    if sync and bufs.world > 1:
        stream_barrier(bufs.group)
    sa = scale_a.data_ptr() if scale_a is not None else None
    sb = scale_b.data_ptr() if scale_b is not None else None
    bp = bias.data_ptr() if bias is not None else None
    if getattr(bufs, "mc_ptr", 0):
        # one multimem.st per tile segment; NVSwitch delivers it to every rank's matrix
        _lib.check(_lib.load().kcg_gemm_allgather_multicast(
            ops._dt(A_local), ops._DT[bufs.dtype], M, N, K, 0, int(trans_b), A_local.data_ptr(), A_local.stride(0),
            B.data_ptr(), B.stride(0), bufs.ptrs[bufs.rank], bufs.mc_ptr, begin, bufs.cols, sa, sb, bp, act, stream),
            "kcg_gemm_allgather_multicast")
    else:
        arr = (ctypes.c_void_p * bufs.world)(*bufs.ptrs)
        _lib.check(_lib.load().kcg_gemm_allgather(
            ops._dt(A_local), ops._DT[bufs.dtype], M, N, K, 0, int(trans_b), A_local.data_ptr(), A_local.stride(0),
            B.data_ptr(), B.stride(0), arr, bufs.world, bufs.rank, begin, bufs.cols, sa, sb, bp, act, stream),
            "kcg_gemm_allgather")
    if sync and bufs.world > 1:
        stream_barrier(bufs.group)
    return bufs.local


def fmha_allgather(Q_local: torch.Tensor, K_local: torch.Tensor, V_local: torch.Tensor, bufs: GatherBuffers,
                   total_batches: int, softmax_scale: float = 1.0, causal: bool = False, sync: bool = True) -> torch.Tensor:
    """Replicated attention output with whole batches split over ranks: each rank's epilogue writes
    its [B_local, H, S, D] block into every rank's buffer.  ``bufs`` must hold total_batches*H*S
    rows of D columns; returns the local buffer viewed as [total_batches, H, S, D]."""
    import ctypes
    from . import ops
    ops.check_attention_operands(Q_local, K_local, V_local)
    Bl, H, Sq, D = Q_local.shape
    Skv = K_local.shape[2]
    if bufs.dtype != Q_local.dtype:
        raise TypeError(f"buffer dtype {bufs.dtype} does not match the operands' {Q_local.dtype}")
    if bufs.cols != D or bufs.total_rows != total_batches * H * Sq:
        raise ValueError("buffer shape does not match [total_batches*H*S, D]")
    begin, count = _lib.shard_range(total_batches, bufs.world, bufs.rank, 1)
    if count != Bl:
        raise ValueError(f"this rank owns {count} batches, the operands hold {Bl}")
    for t in (Q_local, K_local, V_local):
        if not t.is_cuda or t.dim() != 4 or t.stride(-1) != 1:
            raise ValueError("fmha takes [B,H,S,D] CUDA tensors with a contiguous head dimension")
    st = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    ost = (ctypes.c_int64 * 3)(H * Sq * D, Sq * D, D)
    if sync and bufs.world > 1:
        stream_barrier(bufs.group)
    if getattr(bufs, "mc_ptr", 0):
        _lib.check(_lib.load().kcg_fmha_fwd_allgather_multicast(
            ops._dt(Q_local), Bl, H, Sq, Skv, D, float(softmax_scale), int(causal), Q_local.data_ptr(), st(Q_local),
            K_local.data_ptr(), st(K_local), V_local.data_ptr(), st(V_local), bufs.ptrs[bufs.rank], bufs.mc_ptr, begin, ost,
            torch.cuda.current_stream().cuda_stream), "kcg_fmha_fwd_allgather_multicast")
    else:
        arr = (ctypes.c_void_p * bufs.world)(*bufs.ptrs)
        _lib.check(_lib.load().kcg_fmha_fwd_allgather(
            ops._dt(Q_local), Bl, H, Sq, Skv, D, float(softmax_scale), int(causal), Q_local.data_ptr(), st(Q_local),
            K_local.data_ptr(), st(K_local), V_local.data_ptr(), st(V_local), arr, bufs.world, bufs.rank, begin, ost,
            torch.cuda.current_stream().cuda_stream), "kcg_fmha_fwd_allgather")
    if sync and bufs.world > 1:
        stream_barrier(bufs.group)
    return bufs.local.view(total_batches, H, Sq, D)


def layernorm_allgather(x_local: torch.Tensor, scale: torch.Tensor, bias: torch.Tensor, bufs: "MulticastBuffers",
                        eps: float = 1e-5, sync: bool = True) -> torch.Tensor:
    """Replicated LayerNorm (over the last dim) of a row-sharded [total_rows, cols] tensor: each rank
    normalises its rows and stores every row once, to the multicast mapping of ``bufs``, so NVSwitch
    places it in every rank's matrix.  Needs buffers with a multicast address (``bufs.mc_ptr``);
    returns ``bufs.local``."""
    from . import ops
    if not getattr(bufs, "mc_ptr", 0):
        raise ValueError("layernorm_allgather needs MulticastBuffers with a multicast mapping")
    if x_local.dim() != 2 or x_local.shape[1] != bufs.cols or x_local.dtype != bufs.dtype:
        raise ValueError("x_local must be [rows, cols] of the buffers' dtype and width")
    if not (x_local.is_cuda and x_local.is_contiguous()):
        raise ValueError("operands must be contiguous CUDA tensors")
    for t in (scale, bias):
        if tuple(t.shape) != (bufs.cols,) or t.dtype != x_local.dtype or not t.is_cuda:
            raise ValueError("scale and bias hold one value per column, in the input's dtype, on the device")
    begin, count = _lib.shard_range(bufs.total_rows, bufs.world, bufs.rank, 1)
    if count != x_local.shape[0]:
        raise ValueError(f"this rank owns {count} rows of the gathered tensor, x_local has {x_local.shape[0]}")
    if sync and bufs.world > 1:
        stream_barrier(bufs.group)
    _lib.check(_lib.load().kcg_layernorm_allgather_multicast(
        ops._dt(x_local), count, bufs.cols, x_local.data_ptr(), scale.data_ptr(), bias.data_ptr(), float(eps),
        bufs.mc_ptr, begin, torch.cuda.current_stream().cuda_stream), "kcg_layernorm_allgather_multicast")
    if sync and bufs.world > 1:
        stream_barrier(bufs.group)
    return bufs.local
