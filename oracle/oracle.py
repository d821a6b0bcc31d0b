"""CPU oracle: the checker for the CUDA kernels.  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU legs may import this module; the
shipped library never does.

PARITY UNPINNED: the reference ships no golden vectors and cannot be built here (it needs
LLVM/MLIR 15), so these functions are pinned by the operator definitions they restate
(cited below, paths relative to the reference repository), not by reference outputs.

Two layers:

* ``ref32`` — the reference-faithful fp32 loop nests of ``kcg_oracle.c`` (same loop order,
  same fp32 accumulation as the affine nests in src/Frontend/Operators.cc).  Used as the
  timed CPU baseline and as a cross-check.
* module-level ``*_f64`` functions — the graded oracle: the same operator definitions
  evaluated in float64 with numpy on the inputs exactly as the kernel sees them (after
  rounding to the storage dtype).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libkcg_oracle.so"

UNARY_OPS = {"Tanh": 0, "Sqrt": 1, "Log": 2, "Relu": 3, "Cast": 4, "Gelu": 5}
BINARY_OPS = {"Add": 0, "Mul": 1, "Div": 2, "Sub": 3, "Pow": 4, "Equal": 5, "Greater": 6}


def build(force: bool = False) -> Path:
    """Compile kcg_oracle.c with gcc (a second or two)."""
    src = _HERE / "kcg_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        r = subprocess.run(["make", "-C", str(_HERE), "-B", "libkcg_oracle.so"], capture_output=True, text=True)
        if r.returncode != 0:
            # No OpenMP runtime on this host: build the sequential nests only.
            subprocess.run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-o", str(_LIB_PATH),
                            str(src), "-lm"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def _c():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        i64, f32p, i64p, ci = ctypes.c_int64, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int64), ctypes.c_int
        _lib.oracle_max_threads.restype = ci
        _lib.oracle_matmul_f32.argtypes = [f32p, f32p, f32p, i64, i64, i64, i64, i64, ci]
        _lib.oracle_batched_matmul_f32.argtypes = [f32p, f32p, f32p, i64, i64, i64, i64, ci, ci, i64, i64, ci]
        _lib.oracle_softmax_f32.argtypes = [f32p, i64, i64, ctypes.c_float, ci, i64, ci]
        _lib.oracle_layernorm_f32.argtypes = [f32p, f32p, f32p, f32p, i64, i64, ctypes.c_float, ci]
        _lib.oracle_unary_f32.argtypes = [ci, f32p, f32p, i64, ci]
        _lib.oracle_binary_f32.argtypes = [ci, ci, i64p, ci, i64p, f32p, f32p, f32p]
        _lib.oracle_binary_f32.restype = i64
        _lib.oracle_binary_same_f32.argtypes = [ci, f32p, f32p, f32p, i64, ci]
        _lib.oracle_attention_f32.argtypes = [f32p, f32p, f32p, f32p, i64, i64, i64, i64, i64, ctypes.c_float, ci,
                                              i64p, i64p, i64p, i64p, i64, i64, ci]
    return _lib


def _p(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _i64(v):
    arr = (ctypes.c_int64 * len(v))(*[int(t) for t in v])
    return arr


def max_threads() -> int:
    return int(_c().oracle_max_threads())


class ref32:
    """Reference-faithful fp32 loop nests (C)."""

    @staticmethod
    def matmul(A, B, rows=None, threads=1):
        """src/Frontend/Operators.cc:186-213.  `rows` = (begin, end) restricts the C rows computed."""
        A = np.ascontiguousarray(A, np.float32); B = np.ascontiguousarray(B, np.float32)
        M, K = A.shape; K2, N = B.shape
        assert K == K2
        C = np.zeros((M, N), np.float32)
        r0, r1 = rows if rows is not None else (0, M)
        _c().oracle_matmul_f32(_p(A), _p(B), _p(C), M, N, K, r0, r1, threads)
        return C

    @staticmethod
    def batched_matmul(A, B, trans_a=False, trans_b=False, batches=None, threads=1):
        """src/Frontend/Operators.cc:390-452; leading dims are batch."""
        A = np.ascontiguousarray(A, np.float32); B = np.ascontiguousarray(B, np.float32)
        m, k = (A.shape[-1], A.shape[-2]) if trans_a else (A.shape[-2], A.shape[-1])
        n = B.shape[-2] if trans_b else B.shape[-1]
        batch = int(np.prod(A.shape[:-2], dtype=np.int64))
        C = np.zeros(A.shape[:-2] + (m, n), np.float32)
        b0, b1 = batches if batches is not None else (0, batch)
        _c().oracle_batched_matmul_f32(_p(A), _p(B), _p(C), batch, m, n, k, int(trans_a), int(trans_b), b0, b1, threads)
        return C

    @staticmethod
    def softmax(x, scale=1.0, causal=False, q_len=None, threads=1):
        """src/Frontend/Operators.cc:540-570 (no max subtraction); returns a new array."""
        y = np.array(x, np.float32, order="C", copy=True)
        cols = y.shape[-1]
        rows = y.size // cols
        _c().oracle_softmax_f32(_p(y), rows, cols, scale, int(causal), q_len or (y.shape[-2] if y.ndim > 1 else 1), threads)
        return y

    @staticmethod
    def layernorm(x, gamma, beta, axis, eps=1e-5, threads=1):
        """src/Frontend/Operators.cc:1179-1243; gamma/beta cover the normalised dims."""
        x = np.ascontiguousarray(x, np.float32)
        axis = axis + x.ndim if axis < 0 else axis
        cols = int(np.prod(x.shape[axis:], dtype=np.int64))
        rows = x.size // cols
        g = np.ascontiguousarray(np.broadcast_to(gamma, x.shape[axis:]), np.float32).reshape(-1)
        b = np.ascontiguousarray(np.broadcast_to(beta, x.shape[axis:]), np.float32).reshape(-1)
        y = np.empty_like(x)
        _c().oracle_layernorm_f32(_p(x), _p(g), _p(b), _p(y), rows, cols, eps, threads)
        return y

    @staticmethod
    def unary(op, x, threads=1):
        """src/Frontend/Operators.cc:960-995."""
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        _c().oracle_unary_f32(UNARY_OPS[op], _p(x), _p(y), x.size, threads)
        return y

    @staticmethod
    def binary(op, a, b):
        """src/Frontend/Operators.cc:772-889 (broadcast rule and indexing)."""
        a = np.ascontiguousarray(a, np.float32); b = np.ascontiguousarray(b, np.float32)
        sa, sb = _i64(a.shape), _i64(b.shape)
        total = _c().oracle_binary_f32(BINARY_OPS[op], a.ndim, sa, b.ndim, sb, _p(a), _p(b), None)
        if total < 0:
            raise ValueError("dim not equal")
        out_shape = np.broadcast_shapes(a.shape, b.shape)
        c = np.empty(out_shape, np.float32)
        assert c.size == total
        _c().oracle_binary_f32(BINARY_OPS[op], a.ndim, sa, b.ndim, sb, _p(a), _p(b), _p(c))
        return c

    @staticmethod
    def binary_same(op, a, b, threads=1):
        """Equal-shape case of the binary nest, optionally multi-threaded (CPU baseline)."""
        a = np.ascontiguousarray(a, np.float32); b = np.ascontiguousarray(b, np.float32)
        assert a.shape == b.shape
        c = np.empty_like(a)
        _c().oracle_binary_same_f32(BINARY_OPS[op], _p(a), _p(b), _p(c), a.size, threads)
        return c

    @staticmethod
    def attention(Q, K, V, scale=1.0, causal=False, slices=None, threads=1):
        """test/test.cc:128-130 chain on [B,H,S,D] arrays; `slices` = (begin, end) over B*H."""
        Q = np.ascontiguousarray(Q, np.float32); K = np.ascontiguousarray(K, np.float32); V = np.ascontiguousarray(V, np.float32)
        B, H, Sq, D = Q.shape
        Skv = K.shape[2]
        O = np.zeros((B, H, Sq, D), np.float32)
        st = lambda S: _i64([H * S * D, S * D, D])
        s0, s1 = slices if slices is not None else (0, B * H)
        _c().oracle_attention_f32(_p(Q), _p(K), _p(V), _p(O), B, H, Sq, Skv, D, scale, int(causal),
                                  st(Sq), st(Skv), st(Skv), st(Sq), s0, s1, threads)
        return O


# ---------------------------------------------------------------------------- fp64 oracle
def matmul_f64(A, B, trans_a=False, trans_b=False):
    """C = op(A) op(B) in float64 (Operators.cc:186-213 / :390-452); leading dims are batch."""
    A = np.asarray(A, np.float64); B = np.asarray(B, np.float64)
    if trans_a: A = np.swapaxes(A, -1, -2)
    if trans_b: B = np.swapaxes(B, -1, -2)
    return np.matmul(A, B)


def softmax_f64(x, scale=1.0, causal=False):
    """exp(s*x)/sum(exp(s*x)) over the last dim (Operators.cc:540-570), max-subtracted form;
    causal masks j > i + (cols - q_len) within the trailing [q_len, cols] matrix."""
    x = np.asarray(x, np.float64) * scale
    if causal:
        q, c = x.shape[-2], x.shape[-1]
        mask = np.arange(c)[None, :] > (np.arange(q)[:, None] + (c - q))
        x = np.where(mask, -np.inf, x)
    m = np.max(x, axis=-1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    e = np.exp(x - m)
    s = np.sum(e, axis=-1, keepdims=True)
    return np.divide(e, s, out=np.zeros_like(e), where=s > 0)


def layernorm_f64(x, gamma, beta, axis, eps=1e-5):
    """Operators.cc:1179-1243: biased variance over dims [axis..]; y = gamma*(d/sqrt(var+eps))+beta."""
    x = np.asarray(x, np.float64)
    axis = axis + x.ndim if axis < 0 else axis
    ax = tuple(range(axis, x.ndim))
    mean = x.mean(axis=ax, keepdims=True)
    d = x - mean
    var = (d * d).mean(axis=ax, keepdims=True)
    return np.asarray(gamma, np.float64) * (d / np.sqrt(var + np.float64(np.float32(eps)))) + np.asarray(beta, np.float64)


def layernorm_stats_f64(x, axis, eps=1e-5):
    """(mean, invStdDev) of the same statistics layernorm_f64 uses, with the normalised dims
    removed (the extra results the reference's notes plan, doc/pass.md:789-791)."""
    x = np.asarray(x, np.float64)
    axis = axis + x.ndim if axis < 0 else axis
    ax = tuple(range(axis, x.ndim))
    mean = x.mean(axis=ax)
    d = x - x.mean(axis=ax, keepdims=True)
    var = (d * d).mean(axis=ax)
    return mean, 1.0 / np.sqrt(var + np.float64(np.float32(eps)))


def gather_shape(in_shape, idx_shape, axis):
    """Operators.cc:1286-1293: the axis is erased, then the index dims are inserted there unless
    the indices are a single [1] vector."""
    shape = list(in_shape)
    del shape[axis]
    if tuple(idx_shape) != (1,):
        shape[axis:axis] = list(idx_shape)
    return tuple(shape)


def gather_nest(x, indices, axis):
    """The reference's loop nest, literally (Operators.cc:1320-1340): one iteration per output
    element; the output's index dims select indices[...], which replaces them in the input index.
    Pure-Python loops: small cases only."""
    x = np.asarray(x); indices = np.asarray(indices)
    single = tuple(indices.shape) == (1,)
    out = np.empty(gather_shape(x.shape, indices.shape, axis), x.dtype)
    for ivs in np.ndindex(*out.shape):
        if single:
            k = int(indices[0])
            src = list(ivs)
        else:
            k = int(indices[tuple(ivs[axis:axis + indices.ndim])])
            src = list(ivs[:axis]) + list(ivs[axis + indices.ndim:])
        src.insert(axis, k)
        out[ivs] = x[tuple(src)]
    return out


def gather_take(x, indices, axis):
    """numpy formulation of the same operator, for sizes the loop nest cannot do in seconds."""
    x = np.asarray(x); indices = np.asarray(indices)
    out = np.take(x, indices, axis=axis)
    return out.reshape(gather_shape(x.shape, indices.shape, axis))


def transpose_last2(x):
    """out[..., j, i] = in[..., i, j] (Transpose has a declaration only, Operators.h:97-99)."""
    return np.ascontiguousarray(np.swapaxes(np.asarray(x), -1, -2))


def unary_f64(op, x):
    """Operators.cc:960-995; Gelu uses the reference's literal fp32 constants."""
    x = np.asarray(x, np.float64)
    if op == "Tanh": return np.tanh(x)
    if op == "Sqrt": return np.sqrt(x)
    if op == "Log": return np.log(x)
    if op == "Relu": return np.maximum(0.0, x)
    if op == "Cast": return x.copy()
    if op == "Gelu":
        c0 = np.float64(np.float32(0.797884)); c1 = np.float64(np.float32(0.044715))
        return 0.5 * x * (1.0 + np.tanh(c0 * (x + c1 * x * x * x)))
    raise KeyError(op)


def binary_f64(op, a, b):
    """Operators.cc:581-607 with numpy broadcasting (same rule as :797-821)."""
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    if op == "Add": return a + b
    if op == "Mul": return a * b
    if op == "Div": return a / b
    if op == "Sub": return a - b
    if op == "Pow": return np.power(a, b)
    if op == "Equal": return (a == b).astype(np.float64)
    if op == "Greater": return (a > b).astype(np.float64)
    raise KeyError(op)


def attention_f64(Q, K, V, scale=1.0, causal=False):
    """softmax(scale * Q K^T) V per (batch, head) on [B,H,S,D] arrays (test/test.cc:128-130)."""
    Q = np.asarray(Q, np.float64); K = np.asarray(K, np.float64); V = np.asarray(V, np.float64)
    S = np.matmul(Q, np.swapaxes(K, -1, -2))
    P = softmax_f64(S, scale=scale, causal=causal)
    return np.matmul(P, V)


def rel_fro(got, want) -> float:
    """Relative Frobenius error ||got - want|| / ||want|| in float64."""
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    denom = np.linalg.norm(want.ravel())
    num = np.linalg.norm((got - want).ravel())
    return float(num / denom) if denom > 0 else float(num)


# ---------------------------------------------------------------------------- storage rounding
def round_bf16(x):
    """float32 -> bfloat16 (round to nearest even) -> float32, in numpy."""
    x = np.ascontiguousarray(x, np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out)


def round_f16(x):
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def quantize_e4m3(x):
    """Round-to-nearest-even, saturating conversion to FP8 E4M3 (bias 7, max 448, no inf).

    Returns (bits uint8, values float32) so that a kernel and the oracle can be fed the
    very same 8-bit inputs.
    """
    x = np.asarray(x, np.float64)
    sign = np.signbit(x)
    a = np.minimum(np.abs(x), 448.0)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6.0)
    quantum = np.exp2(e - 3.0)
    q = np.rint(a / quantum) * quantum          # rint = round half to even
    q = np.minimum(q, 448.0)
    # encode
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(q > 0, q, 1.0)))
    normal = q >= 2.0 ** -6
    exp_field = np.where(normal, e2 + 7, 0).astype(np.int64)
    mant = np.where(normal, np.rint((q / np.exp2(e2) - 1.0) * 8.0), np.rint(q / 2.0 ** -9)).astype(np.int64)
    bits = (sign.astype(np.int64) << 7) | (exp_field << 3) | mant
    vals = np.where(sign, -q, q).astype(np.float32)
    return bits.astype(np.uint8), vals


def decode_e4m3(bits):
    bits = np.asarray(bits, np.uint8).astype(np.int64)
    sign = np.where(bits & 0x80, -1.0, 1.0)
    ef = (bits >> 3) & 0xF
    m = bits & 7
    v = np.where(ef == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2(ef - 7.0))
    return (sign * v).astype(np.float32)
