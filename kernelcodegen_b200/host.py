"""Operator calls on HOST tensors: the end-to-end form of ``ops``.

Each call copies its inputs from (ideally pinned) host memory to cached device staging
buffers, runs the same C-ABI kernel as ``ops`` on the current stream, and copies the result
back into a pinned host tensor.  Large row-wise operators (LayerNorm, elementwise, same-shape
binary) are cut into row chunks whose upload, kernel and download overlap on three streams;
everything else is queued on the current stream.  Either way the caller synchronises the
current stream when it needs the result.  This is what a caller that keeps its data
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
    """Drop the cached device staging tensors.  They were allocated on the current stream but are
    also read and written by the two copy streams, so those streams (and the current one) are
    drained first: the caching allocator may then hand the memory to anyone."""
    if torch.cuda.is_available():
        for up, down in _copy_streams.values():
            up.synchronize()
            down.synchronize()
        torch.cuda.current_stream().synchronize()
    _stage.clear()
    _last_reader.clear()


# ---- row-chunked pipeline: upload of chunk i+1, kernel on chunk i and download of chunk i-1 overlap

PIPELINE_MIN_BYTES = 8 << 20   # tensors below this go through in one piece
PIPELINE_CHUNKS = 8

_copy_streams: dict = {}


def _streams():
    dev = torch.cuda.current_device()
    st = _copy_streams.get(dev)
    if st is None:
        st = _copy_streams[dev] = (torch.cuda.Stream(), torch.cuda.Stream())
    return st


def _row_chunks(rows: int, nbytes: int):
    """[(begin, end)] over dim 0, or None when the tensor is too small to be worth splitting."""
    if nbytes < PIPELINE_MIN_BYTES or rows < 2 * PIPELINE_CHUNKS:
        return None
    step = -(-rows // PIPELINE_CHUNKS)
    return [(b, min(rows, b + step)) for b in range(0, rows, step)]


def _pipelined(chunks, uploads, run, d_out: torch.Tensor, h_out: torch.Tensor) -> None:
    """uploads: [(host tensor, device staging tensor)] sliced along dim 0 per chunk; run(b, e)
    launches the kernel for rows [b, e) on the current stream; d_out[b:e] -> h_out[b:e] follows.
    PCIe is full duplex, so with the copies on their own streams the step costs about the longer
    of its upload and its download instead of their sum.  On return the current stream has waited
    for the last download: synchronising it is enough to read h_out."""
    cur = torch.cuda.current_stream()
    up, down = _streams()
    # An upload may overwrite a staging buffer only after the last kernel that read it (an earlier
    # call of the same operator); uploads of one operator may overlap the downloads of another.
    for _, d in uploads:
        ev = _last_reader.get(d.data_ptr())
        if ev is not None:
            up.wait_event(ev)
    last = ev_k = None
    for (b, e) in chunks:
        with torch.cuda.stream(up):
            for h, d in uploads:
                d[b:e].copy_(h[b:e], non_blocking=True)
            ev_up = torch.cuda.Event()
            ev_up.record(up)
        cur.wait_event(ev_up)
        run(b, e)
        ev_k = torch.cuda.Event()
        ev_k.record(cur)
        with torch.cuda.stream(down):
            down.wait_event(ev_k)
            h_out[b:e].copy_(d_out[b:e], non_blocking=True)
            last = torch.cuda.Event()
            last.record(down)
    for _, d in uploads:
        _last_reader[d.data_ptr()] = ev_k
    cur.wait_event(last)


_last_reader: dict = {}


def layernorm(x, scale, bias, axis, eps=1e-5, out=None):
    ax = axis if axis >= 0 else axis + x.dim()
    chunks = _row_chunks(x.shape[0], x.numel() * x.element_size()) if ax >= 1 else None
    if chunks is None:
        y = ops.layernorm(_up("ln_x", x), _up("ln_g", scale), _up("ln_b", bias), axis, eps, out=_dev("ln_y", x))
        return _down(y, out)
    dx, dy = _dev("ln_x", x), _dev("ln_y", x)
    dg, db = _up("ln_g", scale), _up("ln_b", bias)
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
    _pipelined(chunks, [(x, dx)], lambda b, e: ops.layernorm(dx[b:e], dg, db, axis, eps, out=dy[b:e]), dy, out)
    return out


def elementwise(x, operation, out=None):
    chunks = _row_chunks(x.shape[0], x.numel() * x.element_size()) if x.dim() >= 1 else None
    if chunks is None:
        y = ops.elementwise(_up("ew_x", x), operation, out=_dev("ew_y", x))
        return _down(y, out)
    dx, dy = _dev("ew_x", x), _dev("ew_y", x)
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
    _pipelined(chunks, [(x, dx)], lambda b, e: ops.elementwise(dx[b:e], operation, out=dy[b:e]), dy, out)
    return out


def binary(a, b, operation, out=None):
    if tuple(a.shape) == tuple(b.shape) and a.dim() >= 1:
        chunks = _row_chunks(a.shape[0], a.numel() * a.element_size())
        if chunks is not None:
            da, db, dc = _dev("bin_a", a), _dev("bin_b", b), _dev("bin_c", a)
            if out is None:
                out = torch.empty(a.shape, dtype=a.dtype, pin_memory=True)
            _pipelined(chunks, [(a, da), (b, db)], lambda s, e: ops.binary(da[s:e], db[s:e], operation, out=dc[s:e]), dc, out)
            return out
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
