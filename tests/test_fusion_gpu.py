"""Fused kernels against the chains they replace.  The criterion is bit-equality with the
separate operators (the fused kernels round to the storage dtype exactly where the chain would
store); the comparison with the float64 oracle is held to the operators' own tolerance
(relative Frobenius 1e-5 for fp32, 1e-2 for 16-bit storage)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import TOL, randn, f64, rel_fro, sync_ok

pytestmark = pytest.mark.gpu


def ops():
    from kernelcodegen_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(64, 4096), (33, 8192), (257, 256), (7, 1000), (5, 1001), (3, 40000), (2, 6, 128)])
def test_layernorm_gelu_add_equals_chain(shape, dtype):
    cols = shape[-1]
    x = randn(shape, dtype, 700).cuda()
    r = randn(shape, dtype, 701).cuda()
    g = randn((cols,), dtype, 702, mean=1.0, std=0.1).cuda()
    b = randn((cols,), dtype, 703, std=0.1).cuda()
    fused = ops().layernorm_gelu_add(x, g, b, r)
    chain = ops().binary(ops().elementwise(ops().layernorm(x, g, b, -1), "Gelu"), r, "Add")
    sync_ok()
    assert torch.equal(fused, chain)
    want = O.binary_f64("Add", O.unary_f64("Gelu", O.layernorm_f64(f64(x), f64(g), f64(b), -1)), f64(r))
    assert rel_fro(fused, want) <= TOL[dtype]


def test_layernorm_gelu_add_in_place():
    x = randn((128, 2048), torch.bfloat16, 710).cuda()
    r = randn((128, 2048), torch.bfloat16, 711).cuda()
    g = randn((2048,), torch.bfloat16, 712, mean=1.0, std=0.1).cuda()
    b = randn((2048,), torch.bfloat16, 713, std=0.1).cuda()
    want = ops().layernorm_gelu_add(x, g, b, r)
    got = ops().layernorm_gelu_add(x, g, b, r, out=x)
    sync_ok()
    assert got.data_ptr() == x.data_ptr() and torch.equal(got, want)


def test_layernorm_gelu_add_in_place_on_the_residual():
    """y may be the residual's own storage where the one-pass kernel runs; rows that fall back to
    three in-place launches (1001 columns: not a whole number of 16-byte vectors) would read the
    residual after it has been overwritten, so that combination is refused, not computed wrongly."""
    from kernelcodegen_b200 import _lib
    for cols, fused_ok in ((2048, True), (1001, False)):
        x = randn((16, cols), torch.bfloat16, 715).cuda()
        r = randn((16, cols), torch.bfloat16, 716).cuda()
        g = randn((cols,), torch.bfloat16, 717, mean=1.0, std=0.1).cuda()
        b = randn((cols,), torch.bfloat16, 718, std=0.1).cuda()
        want = ops().layernorm_gelu_add(x, g, b, r)
        sync_ok()
        if fused_ok:
            got = ops().layernorm_gelu_add(x, g, b, r, out=r)
            sync_ok()
            assert torch.equal(got, want)
        else:
            keep = r.clone()
            with pytest.raises(_lib.KcgError) as e:
                ops().layernorm_gelu_add(x, g, b, r, out=r)
            assert e.value.status == _lib.ERR_UNSUPPORTED
            sync_ok()
            assert torch.equal(r, keep)   # refused before anything was launched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("act", [None, "Relu", "Gelu"])
@pytest.mark.parametrize("with_bias", [False, True])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (520, 264, 136)])
def test_gemm_fused_epilogue_equals_chain(m, n, k, with_bias, act, dtype):
    # (128,..) runs on single CTAs, (520,..) on CTA pairs; fp32 runs on the CUDA-core kernel
    A = randn((m, k), dtype, 720, std=k ** -0.5).cuda()
    B = randn((k, n), dtype, 721).cuda()
    bias = randn((n,), dtype, 722).cuda() if with_bias else None
    fused = ops().matmul(A, B, bias=bias, activation=act)
    chain = ops().matmul(A, B)
    if with_bias:
        chain = ops().binary(chain, bias, "Add")
    if act:
        chain = ops().elementwise(chain, act)
    sync_ok()
    assert torch.equal(fused, chain)
    want = O.matmul_f64(f64(A), f64(B))
    if with_bias:
        want = want + f64(bias)
    if act:
        want = O.unary_f64(act, want)
    assert rel_fro(fused, want) <= TOL[dtype]


def test_gemm_fused_rejects_bad_activation():
    from kernelcodegen_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    rc = lib.kcg_gemm_fused(_lib.BF16, _lib.BF16, 64, 64, 64, 1, 0, 0, x.data_ptr(), 64, 0, x.data_ptr(), 64, 0,
                            x.data_ptr(), 64, 0, None, None, None, 7, None)
    assert rc == _lib.ERR_INVALID_ARG
