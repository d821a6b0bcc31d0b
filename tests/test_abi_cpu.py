"""The C-ABI library loads without a GPU and exports every symbol the header declares;
argument errors that need no device are reported, not crashed on."""
import ctypes
import re
from pathlib import Path

import pytest

from kernelcodegen_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "kcg_kernels.h").read_text()
    return sorted(set(re.findall(r"KCG_API\s+[\w\s\*]+?\b(kcg_\w+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = declared_symbols()
    assert "kcg_gemm" in names and "kcg_fmha_fwd" in names and "kcg_layernorm" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/kcg_kernels.h but not exported"
    # and the ctypes table covers the whole header
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_status_strings(lib):
    assert lib.kcg_status_string(0) == b"ok"
    assert b"timed out" in lib.kcg_status_string(_lib.ERR_TIMEOUT)
    assert lib.kcg_version() >= 100
    assert [lib.kcg_dtype_size(d) for d in (_lib.F32, _lib.F16, _lib.BF16, _lib.F8E4M3, _lib.I32)] == [4, 2, 2, 1, 4]


def test_argument_errors_without_device(lib):
    assert lib.kcg_layernorm(_lib.F32, -1, 4, None, None, None, 1e-5, None, None) == _lib.ERR_INVALID_ARG
    assert lib.kcg_layernorm(_lib.F32, 4, 4, None, None, None, 1e-5, None, None) == _lib.ERR_INVALID_ARG
    assert b"null" in lib.kcg_last_error()
    assert lib.kcg_layernorm(_lib.F32, 0, 4, None, None, None, 1e-5, None, None) == _lib.OK  # empty input
    assert lib.kcg_eltwise(99, _lib.F32, _lib.F32, 4, 8, 8, None) == _lib.ERR_INVALID_ARG
    assert lib.kcg_eltwise(_lib.UNARY_OPS["Gelu"], _lib.F32, _lib.BF16, 4, 8, 8, None) == _lib.ERR_INVALID_ARG
    assert lib.kcg_eltwise(_lib.UNARY_OPS["Gelu"], _lib.F32, _lib.F32, 0, None, None, None) == _lib.OK
    sa = (ctypes.c_int64 * 2)(4, 5)
    sb = (ctypes.c_int64 * 2)(4, 3)
    assert lib.kcg_binary(0, _lib.F32, 2, sa, 2, sb, 8, 8, 8, None) == _lib.ERR_INVALID_ARG
    assert b"dim not equal" in lib.kcg_last_error()
    assert lib.kcg_gemm(_lib.BF16, _lib.BF16, 8, 8, 0, 1, 0, 0, 8, 8, 0, 8, 8, 0, 8, 8, 0, None, None, None) == _lib.ERR_INVALID_ARG
    assert lib.kcg_gemm(_lib.BF16, _lib.BF16, 8, 8, 8, 1, 0, 0, 8, 4, 0, 8, 8, 0, 8, 8, 0, None, None, None) == _lib.ERR_INVALID_ARG
    assert lib.kcg_gemm(_lib.BF16, _lib.BF16, 0, 8, 8, 1, 0, 0, None, 8, 0, None, 8, 0, None, 8, 0, None, None, None) == _lib.OK


@pytest.mark.parametrize("total,world,granule", [(65536, 8, 128), (100, 8, 1), (1000, 3, 128), (5, 8, 1), (0, 4, 1)])
def test_shard_range_partitions(total, world, granule):
    pos = 0
    for r in range(world):
        b, c = _lib.shard_range(total, world, r, granule)
        assert b == pos and c >= 0
        if r < world - 1 and c:
            assert c % granule == 0 or b + c == total
        pos += c
    assert pos == total


def test_shard_range_rejects_bad_rank(lib):
    b, c = ctypes.c_int64(), ctypes.c_int64()
    assert lib.kcg_shard_range(10, 4, 4, 1, ctypes.byref(b), ctypes.byref(c)) == _lib.ERR_INVALID_ARG


def test_shard_allgather_argument_errors_without_device(lib):
    # refused before NCCL is even looked for
    assert lib.kcg_shard_allgather(None, 8, 4, 1, 2, 0, None, None) == _lib.ERR_INVALID_ARG
    assert b"null" in lib.kcg_last_error()
    assert lib.kcg_shard_allgather(None, 8, 4, 0, 2, 0, None, None) == _lib.ERR_INVALID_ARG
    assert lib.kcg_shard_allgather(None, 8, 4, 1, 2, 2, None, None) == _lib.ERR_INVALID_ARG
    assert lib.kcg_shard_allgather(None, 0, 4, 1, 2, 0, None, None) == _lib.OK
    assert lib.kcg_nccl_comm_create(0, 0, None, None) == _lib.ERR_INVALID_ARG
    assert lib.kcg_nccl_comm_destroy(None) == _lib.OK
