"""kcg_layernorm_split_static: the LayerNorm entry point for callers that cannot let a
library call allocate device memory (everything is in their own pool, or they sit in a
latency-critical loop where cudaMalloc's implicit synchronisation is not acceptable).  Its
scratch is a fixed array inside the library, so the checks here are: same result as
kcg_layernorm on consecutive calls that reuse that array with different shapes, and a clear
refusal beyond the array's size.  Collected last on purpose (file name), and it must pass
both alone in a fresh process and after every other test."""
import pytest
import torch

from tests.helpers import randn, f64, rel_fro, sync_ok
from oracle import oracle as O

pytestmark = pytest.mark.gpu

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _static_ln(x, g, b, eps=1e-5):
    from kernelcodegen_b200 import _lib
    lib = _lib.load()
    rows, cols = x.shape[0], x[0].numel()
    y = torch.empty_like(x)
    rc = lib.kcg_layernorm_split_static(_DT[x.dtype], rows, cols, x.data_ptr(), g.data_ptr(), b.data_ptr(), eps,
                                        y.data_ptr(), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "kcg_layernorm_split_static")
    return y


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_matches_allocating_entry_point_twice_in_a_row(dtype):
    from kernelcodegen_b200 import ops
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    # two calls back to back with different shapes: the second finds the first one's
    # statistics still in the shared array and must not be affected by them
    for seed, shape in ((900, (3, 40000)), (910, (2, 96, 1000))):
        x = randn(shape, dtype, seed, mean=3.0).cuda()
        g = randn(shape[1:], dtype, seed + 1, mean=1.0, std=0.1).cuda()
        b = randn(shape[1:], dtype, seed + 2, std=0.1).cuda()
        got = _static_ln(x, g, b)
        want = ops.layernorm(x, g, b, 1)
        sync_ok()
        assert rel_fro(got, f64(want)) <= tol
        assert rel_fro(got, O.layernorm_f64(f64(x), f64(g), f64(b), 1)) <= tol
    # and the same input again gives the same bits
    again = _static_ln(x, g, b)
    sync_ok()
    assert torch.equal(again, got)


def test_device_memory_in_use_does_not_change():
    """After the first call on the device (which only looks up the array's address), further calls
    must leave the amount of free device memory exactly as it was: the outputs are allocated here,
    before the measurement, and the entry point itself must not allocate or free anything."""
    from kernelcodegen_b200 import _lib
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    shapes = [(3, 40000), (200, 9000), (1, 100000)]
    bufs = []
    for i, (rows, cols) in enumerate(shapes):
        x = randn((rows, cols), torch.float32, 930 + i).cuda()
        g = randn((cols,), torch.float32, 940 + i, mean=1.0, std=0.1).cuda()
        b = randn((cols,), torch.float32, 950 + i, std=0.1).cuda()
        bufs.append((rows, cols, x, g, b, torch.empty_like(x)))
    rows, cols, x, g, b, y = bufs[0]
    _lib.check(lib.kcg_layernorm_split_static(0, rows, cols, x.data_ptr(), g.data_ptr(), b.data_ptr(), 1e-5,
                                              y.data_ptr(), stream), "first call")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        for rows, cols, x, g, b, y in bufs:
            _lib.check(lib.kcg_layernorm_split_static(0, rows, cols, x.data_ptr(), g.data_ptr(), b.data_ptr(), 1e-5,
                                                      y.data_ptr(), stream), "kcg_layernorm_split_static")
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    sync_ok()
    for rows, cols, x, g, b, y in bufs:
        assert rel_fro(y, O.layernorm_f64(f64(x), f64(g), f64(b), 1)) <= 1e-5


def test_rejects_sizes_beyond_the_builtin_scratch():
    from kernelcodegen_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(8, device="cuda")
    # 40000 rows of one chunk each: more (row, chunk) pairs than the 32768 the array holds
    rc = lib.kcg_layernorm_split_static(0, 40000, 16, x.data_ptr(), x.data_ptr(), x.data_ptr(), 1e-5, x.data_ptr(), None)
    assert rc == _lib.ERR_UNSUPPORTED
    assert b"exceeds the built-in scratch" in lib.kcg_last_error()
    # empty input is a no-op, null pointers are refused
    assert lib.kcg_layernorm_split_static(0, 0, 16, None, None, None, 1e-5, None, None) == _lib.OK
    assert lib.kcg_layernorm_split_static(0, 4, 16, None, None, None, 1e-5, None, None) == _lib.ERR_INVALID_ARG
