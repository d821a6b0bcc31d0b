"""Operator calls on torch CUDA tensors, one per reference Frontend operator.

Names and argument meaning follow the reference's operator builders
(include/Frontend/Operators.h:75-133): ``matmul`` (Matmul), ``batched_matmul``
(BatchedMatmul with Layout flags), ``softmax``, ``layernorm`` (axis, eps), ``elementwise``
("Tanh" | "Sqrt" | "Log" | "Relu" | "Cast" | "Gelu"), ``relu``, ``binary`` ("Add" | "Mul" |
"Div" | "Sub" | "Pow" | "Equal" | "Greater"), ``gather``, ``transpose`` and ``fmha`` for the
fused BatchedMatmul -> Softmax -> BatchedMatmul chain.  torch only supplies device memory and
the current stream; every computation is a call through the C ABI into the sm_100a
kernels, and there is no fallback path.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from ._lib import KcgError, check  # noqa: F401  (re-exported)

_DT = {
    torch.float32: _lib.F32,
    torch.float16: _lib.F16,
    torch.bfloat16: _lib.BF16,
    torch.int32: _lib.I32,
}
if hasattr(torch, "float8_e4m3fn"):
    _DT[torch.float8_e4m3fn] = _lib.F8E4M3

DTYPE_NAMES = {
    "float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16, "int32": torch.int32,
    "float8_e4m3": getattr(torch, "float8_e4m3fn", None),
}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"dtype {t.dtype} has no kernel") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if not t.is_cuda:
            raise ValueError("operands must be CUDA tensors (there is no CPU path)")
        if not t.is_contiguous():
            raise ValueError("operands must be contiguous")


def _check_out(out, shape, dtype, like, what: str) -> None:
    """An ``out=`` tensor is written through its raw pointer with the strides of a dense tensor,
    so anything else (wrong shape or dtype, a view with gaps, another device) must stop here."""
    if out is None:
        return
    if tuple(out.shape) != tuple(shape):
        raise ValueError(f"{what}: out has shape {tuple(out.shape)}, the result has {tuple(shape)}")
    if out.dtype != dtype:
        raise ValueError(f"{what}: out has dtype {out.dtype}, the result has {dtype}")
    if out.device != like.device:
        raise ValueError(f"{what}: out is on {out.device}, the operands are on {like.device}")
    if not out.is_contiguous():
        raise ValueError(f"{what}: out must be contiguous")


def _same_dtype(what: str, *ts) -> None:
    for t in ts[1:]:
        if t.dtype != ts[0].dtype:
            raise TypeError(f"{what}: operands must share a dtype (got {ts[0].dtype} and {t.dtype})")


def _i64arr(v):
    return (ctypes.c_int64 * len(v))(*[int(x) for x in v])


def _broadcast_shape(sa, sb):
    """Trailing-aligned broadcast of two shapes (the rule of Binary::build, Operators.cc:797-821)."""
    out = []
    for i in range(1, max(len(sa), len(sb)) + 1):
        da = sa[-i] if i <= len(sa) else 1
        db = sb[-i] if i <= len(sb) else 1
        if da != db and da != 1 and db != 1:
            raise ValueError("dim not equal")
        out.append(db if da == 1 else da)
    return tuple(reversed(out))


def layernorm(x, scale, bias, axis: int, eps: float = 1e-5, inplace: bool = False, out=None):
    """LayerNorm over dims [axis..] (reference: LayerNorm::build, Operators.h:125-128)."""
    _same_dtype("layernorm", x, scale, bias)
    _check_out(out, x.shape, x.dtype, x, "layernorm")
    _need_cuda(x, scale, bias)
    nd = x.dim()
    if axis >= nd or axis <= -nd:
        raise ValueError("axis is out of bounds for array of dimension.")
    if axis < 0:
        axis += nd
    norm_shape = tuple(x.shape[axis:])
    cols = math.prod(norm_shape)
    rows = x.numel() // cols if cols else 0
    if tuple(scale.shape) != norm_shape or tuple(bias.shape) != norm_shape:
        # trailing-aligned broadcast with 1-dims (Operators.cc:1102-1123)
        scale = scale.expand(norm_shape).contiguous()
        bias = bias.expand(norm_shape).contiguous()
    y = x if inplace else (out if out is not None else torch.empty_like(x))
    check(_lib.load().kcg_layernorm(_dt(x), rows, cols, x.data_ptr(), scale.data_ptr(), bias.data_ptr(),
                                    float(eps), y.data_ptr(), _stream()), "kcg_layernorm")
    return y


def layernorm_with_stats(x, scale, bias, axis: int, eps: float = 1e-5, out=None):
    """(Y, mean, invStdDev): LayerNorm over dims [axis..] that also returns the fp32 row mean and
    1/sqrt(var + eps), shaped like x with the normalised dims removed — the result tuple the
    reference's design notes plan (doc/pass.md:789-791).  ``scale`` / ``bias`` may be None."""
    _same_dtype("layernorm_with_stats", x, *[t for t in (scale, bias) if t is not None])
    _check_out(out, x.shape, x.dtype, x, "layernorm_with_stats")
    _need_cuda(x, *[t for t in (scale, bias) if t is not None])
    nd = x.dim()
    if axis >= nd or axis <= -nd:
        raise ValueError("axis is out of bounds for array of dimension.")
    if axis < 0:
        axis += nd
    norm_shape = tuple(x.shape[axis:])
    cols = math.prod(norm_shape)
    rows = x.numel() // cols if cols else 0
    if scale is not None and tuple(scale.shape) != norm_shape:
        scale = scale.expand(norm_shape).contiguous()
    if bias is not None and tuple(bias.shape) != norm_shape:
        bias = bias.expand(norm_shape).contiguous()
    y = out if out is not None else torch.empty_like(x)
    mean = torch.empty(tuple(x.shape[:axis]), dtype=torch.float32, device=x.device)
    inv_std = torch.empty_like(mean)
    check(_lib.load().kcg_layernorm_stats(_dt(x), rows, cols, x.data_ptr(),
                                          scale.data_ptr() if scale is not None else None,
                                          bias.data_ptr() if bias is not None else None,
                                          float(eps), y.data_ptr(), mean.data_ptr(), inv_std.data_ptr(), _stream()),
          "kcg_layernorm_stats")
    return y, mean, inv_std


def layernorm_gelu_add(x, scale, bias, residual, eps: float = 1e-5, out=None):
    """Gelu(LayerNorm(x over the last dim)) + residual in one kernel; bit-identical to the chain
    layernorm -> elementwise("Gelu") -> binary("Add")."""
    if tuple(residual.shape) != tuple(x.shape) or residual.dtype != x.dtype:
        raise ValueError("residual must match x in shape and dtype")
    _same_dtype("layernorm_gelu_add", x, scale, bias)
    _check_out(out, x.shape, x.dtype, x, "layernorm_gelu_add")
    _need_cuda(x, scale, bias, residual)
    cols = x.shape[-1]
    if tuple(scale.shape) != (cols,) or tuple(bias.shape) != (cols,):
        raise ValueError("scale and bias must have the length of the last dim")
    rows = x.numel() // cols if cols else 0
    y = out if out is not None else torch.empty_like(x)
    check(_lib.load().kcg_layernorm_gelu_add(_dt(x), rows, cols, x.data_ptr(), scale.data_ptr(), bias.data_ptr(),
                                             float(eps), residual.data_ptr(), y.data_ptr(), _stream()),
          "kcg_layernorm_gelu_add")
    return y


def elementwise(x, operation: str, dtype=None, inplace: bool = False, out=None):
    """Unary map (reference: ElementWise::build, Operators.h:114-123)."""
    if operation not in _lib.UNARY_OPS:
        raise KeyError(operation)
    out_dtype = x.dtype if dtype is None else (DTYPE_NAMES[dtype] if isinstance(dtype, str) else dtype)
    _check_out(None if inplace else out, x.shape, out_dtype, x, "elementwise")
    _need_cuda(x)
    if inplace:
        y = x
    else:
        y = out if out is not None else torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(_lib.load().kcg_eltwise(_lib.UNARY_OPS[operation], _dt(x), _dt(y), x.numel(), x.data_ptr(),
                                  y.data_ptr(), _stream()), "kcg_eltwise")
    return y


def relu(x, inplace: bool = False):
    """Reference: Relu::build (Operators.h:83-85)."""
    return elementwise(x, "Relu", inplace=inplace)


def binary(a, b, operation: str, inplace: bool = False, out=None):
    """Broadcasting binary map (reference: Binary::build, Operators.h:101-112)."""
    if operation not in _lib.BINARY_OPS:
        raise KeyError(operation)
    if a.dtype != b.dtype:
        raise TypeError("binary: operands must share a dtype")
    oshape = _broadcast_shape(a.shape, b.shape)
    _check_out(None if inplace else out, oshape, a.dtype, a, "binary")
    _need_cuda(a, b)
    if inplace:
        if tuple(a.shape) != tuple(oshape):
            raise ValueError("inplace needs the left operand to have the output shape")
        c = a
    else:
        c = out if out is not None else torch.empty(oshape, dtype=a.dtype, device=a.device)
    check(_lib.load().kcg_binary(_lib.BINARY_OPS[operation], _dt(a), a.dim(), _i64arr(a.shape), b.dim(),
                                 _i64arr(b.shape), a.data_ptr(), b.data_ptr(), c.data_ptr(), _stream()),
          "kcg_binary")
    return c


def softmax(x, axis: int = -1, scale: float = 1.0, causal: bool = False, inplace: bool = True):
    """Softmax over the last dim, in place like the reference (Softmax::build, Operators.h:93-95)."""
    _need_cuda(x)
    if axis not in (-1, x.dim() - 1):
        raise ValueError("At present, only support reduction on the last dim.")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    q_len = x.shape[-2] if x.dim() >= 2 else 1
    y = x if inplace else torch.empty_like(x)
    check(_lib.load().kcg_softmax(_dt(x), rows, cols, float(scale), int(causal), q_len, x.data_ptr(),
                                  y.data_ptr(), _stream()), "kcg_softmax")
    return y


def _scale_ptr(s):
    if s is None:
        return None
    if not (s.is_cuda and s.dtype == torch.float32 and s.numel() == 1):
        raise ValueError("per-tensor scales are one float32 on the device")
    return s.data_ptr()


_ACT = {None: 0, "": 0, "Relu": 1, "Gelu": 2}


def batched_matmul(A, B, trans_a: bool = False, trans_b: bool = False, out_dtype=None, scale_a=None,
                   scale_b=None, out=None, bias=None, activation=None):
    """C = op(A) op(B) over leading batch dims (reference: BatchedMatmul::build with
    Layout::rowMajor / Layout::colMajor, Operators.h:87-89; trans_x=True is colMajor)."""
    if A.dim() < 2 or A.dim() != B.dim():
        raise ValueError("BatchedMatmul: A, B dim not matched.")
    # the kernel reads both operands with A's element size: a narrower B would be read past its end
    _same_dtype("BatchedMatmul", A, B)
    m, k1 = (A.shape[-1], A.shape[-2]) if trans_a else (A.shape[-2], A.shape[-1])
    n, k2 = (B.shape[-2], B.shape[-1]) if trans_b else (B.shape[-1], B.shape[-2])
    if k1 != k2:
        raise ValueError("Can't apply BatchedMatmul Operation due to imcompatible K-dim.")
    if tuple(A.shape[:-2]) != tuple(B.shape[:-2]):
        raise ValueError("BatchedMatmul: batch dims differ")
    batch = math.prod(A.shape[:-2])
    if out_dtype is None:
        if out is not None:
            out_dtype = out.dtype
        else:
            out_dtype = torch.bfloat16 if A.dtype == getattr(torch, "float8_e4m3fn", None) else A.dtype
    _check_out(out, tuple(A.shape[:-2]) + (m, n), out_dtype, A, "BatchedMatmul")
    _need_cuda(A, B)
    C = out if out is not None else torch.empty(tuple(A.shape[:-2]) + (m, n), dtype=out_dtype, device=A.device)
    if bias is not None and (not bias.is_cuda or bias.dtype != C.dtype or bias.numel() != n):
        raise ValueError("bias holds N values of the output dtype on the device")
    check(_lib.load().kcg_gemm_fused(_dt(A), _DT[C.dtype], m, n, k1, batch, int(trans_a), int(trans_b),
                                     A.data_ptr(), A.shape[-1], A.shape[-1] * A.shape[-2],
                                     B.data_ptr(), B.shape[-1], B.shape[-1] * B.shape[-2],
                                     C.data_ptr(), n, m * n, _scale_ptr(scale_a), _scale_ptr(scale_b),
                                     None if bias is None else bias.data_ptr(), _ACT[activation], _stream()),
          "kcg_gemm")
    return C


def matmul(A, B, out_dtype=None, scale_a=None, scale_b=None, out=None, bias=None, activation=None):
    """C[M,N] = A[M,K] B[K,N], both row-major (reference: Matmul::build, Operators.h:79-81)."""
    if A.dim() != 2 or B.dim() != 2:
        raise ValueError("Matmul takes rank-2 operands")
    if A.shape[1] != B.shape[0]:
        raise ValueError("Can't apply Matmul Operation due to imcompatible K-dim.")
    return batched_matmul(A, B, False, False, out_dtype, scale_a, scale_b, out, bias, activation)


_ESIZE_DT = {1: _lib.BOOL, 2: _lib.I16, 4: _lib.I32, 8: _lib.I64}


def _move_dt(t: torch.Tensor) -> int:
    """dtype code for kernels that move elements without interpreting them."""
    return _DT.get(t.dtype, _ESIZE_DT[t.element_size()])


def gather(x, indices, axis: int = 0, out=None):
    """out = take(x, indices, axis) (reference: Gather::build, Operators.cc:1253-1352): the dim
    ``axis`` of x is replaced by the shape of ``indices`` — or dropped when ``indices`` has
    shape [1], as the reference does."""
    if indices.dtype not in (torch.int32, torch.int64):
        raise TypeError("gather: indices must be int32 or int64")
    if axis >= x.dim() or axis < 0:
        raise ValueError("Can't apply Gather Operation due to axis is greater than shape of input.")
    outer = math.prod(x.shape[:axis])
    inner = math.prod(x.shape[axis + 1:])
    idx_shape = () if tuple(indices.shape) == (1,) else tuple(indices.shape)
    shape = tuple(x.shape[:axis]) + idx_shape + tuple(x.shape[axis + 1:])
    _check_out(out, shape, x.dtype, x, "gather")
    _need_cuda(x, indices)
    if out is None:
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    check(_lib.load().kcg_gather(_move_dt(x), _lib.I32 if indices.dtype == torch.int32 else _lib.I64, outer,
                                 x.shape[axis], inner, indices.numel(), x.data_ptr(), indices.data_ptr(),
                                 out.data_ptr(), _stream()), "kcg_gather")
    return out


def transpose(x, out=None):
    """Swap the two innermost dims (reference: Transpose::build is declared with a single operand
    and an empty body, Operators.h:97-99)."""
    if x.dim() < 2:
        raise ValueError("Transpose takes an operand of rank 2 or more")
    r, c = x.shape[-2], x.shape[-1]
    batch = math.prod(x.shape[:-2])
    _check_out(out, tuple(x.shape[:-2]) + (c, r), x.dtype, x, "transpose")
    _need_cuda(x)
    if out is None:
        out = torch.empty(tuple(x.shape[:-2]) + (c, r), dtype=x.dtype, device=x.device)
    check(_lib.load().kcg_transpose(_move_dt(x), batch, r, c, x.data_ptr(), out.data_ptr(), _stream()),
          "kcg_transpose")
    return out


def check_attention_operands(Q, K, V) -> None:
    """Q [B,H,Sq,D], K and V [B,H,Skv,D] of one dtype, head dimension contiguous.  The kernel builds
    the K and V tensor maps from K's shape, so a shorter V (or a narrower dtype) would be read
    past its end: anything that does not match stops here."""
    for t in (Q, K, V):
        if t.dim() != 4 or t.stride(-1) != 1:
            raise ValueError("fmha takes [B,H,S,D] tensors with a contiguous head dimension")
    if K.dtype != Q.dtype or V.dtype != Q.dtype:
        raise TypeError(f"fmha: Q, K and V must share a dtype (got {Q.dtype}, {K.dtype}, {V.dtype})")
    B, H, _, D = Q.shape
    for name, t in (("K", K), ("V", V)):
        if t.shape[0] != B or t.shape[1] != H or t.shape[3] != D:
            raise ValueError(f"fmha: {name} has shape {tuple(t.shape)}; batch, heads and head dimension must match "
                             f"Q's {tuple(Q.shape)}")
    if K.shape[2] != V.shape[2]:
        raise ValueError(f"fmha: K has {K.shape[2]} keys, V has {V.shape[2]}")


def fmha(Q, K, V, softmax_scale: float = 1.0, causal: bool = False, out_layout: str = "bhsd", out=None):
    """Fused attention forward on [B,H,S,D] tensors: softmax(scale * Q K^T [+ causal mask]) V,
    the chain BatchedMatmul(NT) -> Softmax -> BatchedMatmul(NN) the reference fuses
    (test/test.cc:128-130).  ``out_layout`` "bshd" returns O as [B,S,H,D]."""
    check_attention_operands(Q, K, V)
    B, H, Sq, D = Q.shape
    Skv = K.shape[2]
    if out is not None:
        # out may be a strided view (e.g. a [B,S,H,D] buffer seen as [B,H,S,D]); its strides are passed on
        if tuple(out.shape) != (B, H, Sq, D) or out.dtype != Q.dtype or out.device != Q.device or out.stride(-1) != 1:
            raise ValueError(f"fmha: out must be a [B,H,Sq,D] = {(B, H, Sq, D)} {Q.dtype} tensor on {Q.device} with a "
                             "contiguous head dimension")
    for t in (Q, K, V):
        if not t.is_cuda:
            raise ValueError("operands must be CUDA tensors (there is no CPU path)")
    if out is None:
        if out_layout == "bhsd":
            out = torch.empty((B, H, Sq, D), dtype=Q.dtype, device=Q.device)
        elif out_layout == "bshd":
            out = torch.empty((B, Sq, H, D), dtype=Q.dtype, device=Q.device).permute(0, 2, 1, 3)
        else:
            raise ValueError(out_layout)
    st = lambda t: _i64arr([t.stride(0), t.stride(1), t.stride(2)])
    check(_lib.load().kcg_fmha_fwd(_dt(Q), B, H, Sq, Skv, D, float(softmax_scale), int(causal),
                                   Q.data_ptr(), st(Q), K.data_ptr(), st(K), V.data_ptr(), st(V),
                                   out.data_ptr(), st(out), _stream()), "kcg_fmha_fwd")
    return out
