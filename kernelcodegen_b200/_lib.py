"""ctypes binding of lib/libkcg_kernels.so (the C ABI declared in include/kcg_kernels.h).

There is no fallback: if the shared library has not been built, importing the operators
raises, so a missing CUDA build can never be mistaken for a working one.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "lib" / "libkcg_kernels.so"

# enum kcg_dtype
F32, F16, BF16, F8E4M3, I32, F64, I64, I16, BOOL = range(9)
# enum kcg_status
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_CUDA, ERR_TIMEOUT, ERR_NO_DEVICE = range(7)

UNARY_OPS = {"Tanh": 0, "Sqrt": 1, "Log": 2, "Relu": 3, "Cast": 4, "Gelu": 5}
BINARY_OPS = {"Add": 0, "Mul": 1, "Div": 2, "Sub": 3, "Pow": 4, "Equal": 5, "Greater": 6}

# Every symbol include/kcg_kernels.h declares, with its ctypes signature.
_i64 = ctypes.c_int64
_ci = ctypes.c_int
_vp = ctypes.c_void_p
_fp = ctypes.c_float
_i64p = ctypes.POINTER(ctypes.c_int64)
SIGNATURES = {
    "kcg_status_string": ([_ci], ctypes.c_char_p),
    "kcg_last_error": ([], ctypes.c_char_p),
    "kcg_version": ([], _ci),
    "kcg_device_status": ([], _ci),
    "kcg_dtype_size": ([_ci], ctypes.c_size_t),
    "kcg_layernorm": ([_ci, _i64, _i64, _vp, _vp, _vp, _fp, _vp, _vp], _ci),
    "kcg_layernorm_gelu_add": ([_ci, _i64, _i64, _vp, _vp, _vp, _fp, _vp, _vp, _vp], _ci),
    "kcg_layernorm_split_static": ([_ci, _i64, _i64, _vp, _vp, _vp, _fp, _vp, _vp], _ci),
    "kcg_layernorm_stats": ([_ci, _i64, _i64, _vp, _vp, _vp, _fp, _vp, _vp, _vp, _vp], _ci),
    "kcg_layernorm_set_warp_row_limit": ([_ci], None),
    "kcg_layernorm_set_block_shape": ([_ci, _ci], None),
    "kcg_eltwise": ([_ci, _ci, _ci, _i64, _vp, _vp, _vp], _ci),
    "kcg_binary": ([_ci, _ci, _ci, _i64p, _ci, _i64p, _vp, _vp, _vp, _vp], _ci),
    "kcg_softmax": ([_ci, _i64, _i64, _fp, _ci, _i64, _vp, _vp, _vp], _ci),
    "kcg_gemm": ([_ci, _ci, _i64, _i64, _i64, _i64, _ci, _ci, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64,
                  _vp, _vp, _vp], _ci),
    "kcg_gemm_fused": ([_ci, _ci, _i64, _i64, _i64, _i64, _ci, _ci, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _i64, _i64,
                        _vp, _vp, _vp, _ci, _vp], _ci),
    "kcg_gemm_set_pair_mode": ([_ci], None),
    "kcg_gemm_set_fp32_mode": ([_ci], None),
    "kcg_gemm_allgather": ([_ci, _ci, _i64, _i64, _i64, _ci, _ci, _vp, _i64, _vp, _i64, ctypes.POINTER(_vp), _ci, _ci,
                            _i64, _i64, _vp, _vp, _vp, _ci, _vp], _ci),
    "kcg_gemm_allgather_multicast": ([_ci, _ci, _i64, _i64, _i64, _ci, _ci, _vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64,
                                      _vp, _vp, _vp, _ci, _vp], _ci),
    "kcg_fmha_fwd_allgather_multicast": ([_ci, _i64, _i64, _i64, _i64, _i64, _fp, _ci, _vp, _i64p, _vp, _i64p, _vp, _i64p,
                                          _vp, _vp, _i64, _i64p, _vp], _ci),
    "kcg_layernorm_allgather_multicast": ([_ci, _i64, _i64, _vp, _vp, _vp, _fp, _vp, _i64, _vp], _ci),
    "kcg_peer_alloc": ([ctypes.c_size_t, ctypes.POINTER(_vp)], _ci),
    "kcg_peer_free": ([_vp], _ci),
    "kcg_peer_export": ([_vp, ctypes.c_char_p], _ci),
    "kcg_peer_open": ([ctypes.c_char_p, ctypes.POINTER(_vp)], _ci),
    "kcg_peer_close": ([_vp], _ci),
    "kcg_fmha_fwd": ([_ci, _i64, _i64, _i64, _i64, _i64, _fp, _ci, _vp, _i64p, _vp, _i64p, _vp, _i64p, _vp, _i64p,
                      _vp], _ci),
    "kcg_fmha_fwd_allgather": ([_ci, _i64, _i64, _i64, _i64, _i64, _fp, _ci, _vp, _i64p, _vp, _i64p, _vp, _i64p,
                                ctypes.POINTER(_vp), _ci, _ci, _i64, _i64p, _vp], _ci),
    "kcg_fmha_set_p_in_tmem": ([_ci], None),
    "kcg_gather": ([_ci, _ci, _i64, _i64, _i64, _i64, _vp, _vp, _vp, _vp], _ci),
    "kcg_transpose": ([_ci, _i64, _i64, _i64, _vp, _vp, _vp], _ci),
    "kcg_device_count": ([ctypes.POINTER(_ci)], _ci),
    "kcg_device_memset": ([_vp, _ci, ctypes.c_size_t, _vp], _ci),
    "kcg_timer_begin": ([_vp, ctypes.POINTER(_vp)], _ci),
    "kcg_timer_end": ([_vp, _vp, ctypes.POINTER(_fp)], _ci),
    "kcg_selftest_bounded_wait": ([ctypes.c_uint64, _vp, _vp], _ci),
    "kcg_shard_range": ([_i64, _ci, _ci, _i64, _i64p, _i64p], _ci),
    "kcg_shard_allgather": ([_vp, _i64, _i64, _i64, _ci, _ci, _vp, _vp], _ci),
    "kcg_nccl_unique_id": ([ctypes.c_char_p], _ci),
    "kcg_nccl_comm_create": ([_ci, _ci, ctypes.c_char_p, ctypes.POINTER(_vp)], _ci),
    "kcg_nccl_comm_destroy": ([_vp], _ci),
}

_lib = None


class KcgError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str):
        super().__init__(f"{where}: status {status} ({detail})")
        self.status = status


def load() -> ctypes.CDLL:
    """Load the kernel library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m kernelcodegen_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means header and library disagree
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
    return _lib


def check(status: int, where: str) -> None:
    if status != OK:
        lib = load()
        detail = lib.kcg_last_error().decode() or lib.kcg_status_string(status).decode()
        raise KcgError(status, where, detail)


def device_status() -> int:
    """Status word written by kernels whose bounded waits gave up (read after a sync)."""
    return int(load().kcg_device_status())


def shard_range(total: int, world: int, rank: int, granule: int = 1) -> tuple[int, int]:
    b, c = ctypes.c_int64(), ctypes.c_int64()
    check(load().kcg_shard_range(total, world, rank, granule, ctypes.byref(b), ctypes.byref(c)), "kcg_shard_range")
    return int(b.value), int(c.value)
