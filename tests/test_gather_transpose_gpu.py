"""Gather, Transpose and LayerNorm-with-statistics through the C ABI: bit-exact data movement
against the oracle's loop nest / numpy formulation; statistics against float64."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import TOL, randn, f64, rel_fro, sync_ok

pytestmark = pytest.mark.gpu


def ops():
    from kernelcodegen_b200 import ops as _ops
    return _ops


def ints(shape, hi, seed, dtype=torch.int64):
    g = torch.Generator(device="cpu").manual_seed(0xC0DE + seed)
    return torch.randint(0, hi, shape, generator=g, dtype=dtype)


GATHER_CASES = [
    # input shape, index shape, axis
    ((16, 8), (5,), 0),            # rows of 8 floats: 16-byte vector path
    ((16, 8), (5,), 1),            # along the last axis: scalar path
    ((4, 9, 6), (3, 2), 1),        # index tensor of rank 2 in the middle
    ((4, 9, 6), (1,), 1),          # single index: the axis is dropped
    ((7, 5, 3), (4,), 2),
    ((3, 1000, 64), (2000,), 1),   # more indices than the axis is long
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("shape,idx_shape,axis", GATHER_CASES)
def test_gather_matches_loop_nest(shape, idx_shape, axis, idx_dtype, dtype):
    x = (randn(shape, torch.float32, 700) * 100).to(dtype)
    idx = ints(idx_shape, shape[axis], 701, idx_dtype)
    out = ops().gather(x.cuda(), idx.cuda(), axis)
    sync_ok()
    xn = x.view(torch.int16).numpy() if dtype == torch.bfloat16 else x.numpy()
    on = out.cpu().view(torch.int16).numpy() if dtype == torch.bfloat16 else out.cpu().numpy()
    want = O.gather_take(xn, idx.numpy(), axis)
    assert on.shape == want.shape == O.gather_shape(shape, idx_shape, axis)
    assert np.array_equal(on, want)
    if np.prod(want.shape) <= 4096:
        assert np.array_equal(on, O.gather_nest(xn, idx.numpy(), axis))


def test_gather_embedding_rows_large():
    # an embedding lookup: 50000 x 1024 bf16 table, 65536 tokens
    table = randn((50000, 1024), torch.bfloat16, 710).cuda()
    idx = ints((65536,), 50000, 711).cuda()
    out = ops().gather(table, idx, 0)
    sync_ok()
    assert torch.equal(out, table[idx])   # a copy: bit-exact
    # gather of gather composes like index composition
    idx2 = ints((1000,), 65536, 712).cuda()
    assert torch.equal(ops().gather(out, idx2, 0), ops().gather(table, idx[idx2], 0))


def test_gather_negative_and_out_of_range_indices():
    from kernelcodegen_b200 import _lib
    x = randn((10, 4), torch.float32, 720).cuda()
    out = ops().gather(x, torch.tensor([-1, 0, -10], device="cuda"), 0)
    sync_ok()
    assert torch.equal(out, x[[9, 0, 0]])
    # an index past the end is not dereferenced: zero slice and a reported status
    out = ops().gather(x, torch.tensor([3, 10], device="cuda"), 0)
    torch.cuda.synchronize()
    assert _lib.device_status() == 1   # KCG_ERR_INVALID_ARG; reading the status clears it
    assert _lib.device_status() == 0
    assert torch.equal(out[0], x[3]) and bool((out[1] == 0).all())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64, torch.uint8])
@pytest.mark.parametrize("shape", [(1, 1), (32, 32), (64, 64), (33, 65), (3, 100, 7), (2, 2, 129, 255), (1024, 4096),
                                   (3, 128, 256), (192, 128), (2, 64, 384)])
def test_transpose_bit_exact(shape, dtype):
    g = torch.Generator(device="cpu").manual_seed(730)
    if dtype.is_floating_point:
        x = torch.randn(shape, generator=g).to(dtype)
    else:
        x = torch.randint(0, 200, shape, generator=g).to(dtype)
    out = ops().transpose(x.cuda())
    sync_ok()
    assert out.shape == tuple(shape[:-2]) + (shape[-1], shape[-2])
    assert torch.equal(out.cpu(), x.transpose(-1, -2).contiguous())
    # an involution
    assert torch.equal(ops().transpose(out).cpu(), x)


def test_transpose_feeds_gemm_layouts():
    # A B computed from B^T stored transposed must equal the NN product bit for bit
    A = randn((256, 512), torch.bfloat16, 740).cuda()
    B = randn((512, 384), torch.bfloat16, 741).cuda()
    Bt = ops().transpose(B)
    assert torch.equal(ops().batched_matmul(A, Bt, False, True), ops().matmul(A, B))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,axis", [((64, 256), 1), ((37, 1000), 1), ((8192 // 64, 4096), 1), ((4, 6, 10, 16), 2),
                                        ((3, 40000), 1), ((5, 70001), 1)])
def test_layernorm_with_stats(shape, axis, dtype):
    x = randn(shape, dtype, 750, mean=0.5)
    norm = shape[axis:]
    g = randn(norm, dtype, 751, mean=1.0, std=0.1)
    b = randn(norm, dtype, 752, std=0.1)
    y, mean, rstd = ops().layernorm_with_stats(x.cuda(), g.cuda(), b.cuda(), axis, 1e-5)
    sync_ok()
    # Y is the plain LayerNorm's Y, bit for bit
    assert torch.equal(y, ops().layernorm(x.cuda(), g.cuda(), b.cuda(), axis, 1e-5))
    m64, r64 = O.layernorm_stats_f64(f64(x), axis, 1e-5)
    assert mean.shape == tuple(shape[:axis]) and mean.dtype == torch.float32
    assert rel_fro(mean, m64) <= 1e-5 and rel_fro(rstd, r64) <= 1e-5
    # optional scale / bias
    y0, mean0, rstd0 = ops().layernorm_with_stats(x.cuda(), None, None, axis, 1e-5)
    sync_ok()
    assert torch.equal(mean0, mean) and torch.equal(rstd0, rstd)
    ones = torch.ones(norm, dtype=dtype); zeros = torch.zeros(norm, dtype=dtype)
    assert rel_fro(y0, O.layernorm_f64(f64(x), f64(ones), f64(zeros), axis, 1e-5)) <= TOL[dtype]
    y1, _, _ = ops().layernorm_with_stats(x.cuda(), g.cuda(), None, axis, 1e-5)
    sync_ok()
    assert rel_fro(y1, O.layernorm_f64(f64(x), f64(g), f64(zeros), axis, 1e-5)) <= TOL[dtype]
