"""GEMM parity through the C ABI: float32 on the CUDA cores (1e-5), bf16 / fp16 (1e-2) and
FP8 e4m3 (3e-2) on tcgen05, all four operand layouts, batches, ragged sizes."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import TOL, randn, uniform, f64, rel_fro, sync_ok

pytestmark = pytest.mark.gpu


def ops():
    from kernelcodegen_b200 import ops as _ops
    return _ops


def test_fp32_config_1024_cubed():
    # the fp32 reference workload: A, B uniform[-1,1], row-major, 1024^3
    A = uniform((1024, 1024), torch.float32, 500)
    B = uniform((1024, 1024), torch.float32, 501)
    C = ops().matmul(A.cuda(), B.cuda())
    sync_ok()
    assert rel_fro(C, O.matmul_f64(f64(A), f64(B))) <= 1e-5
    # and against the reference-faithful fp32 nest on a row slice
    part = O.ref32.matmul(A.numpy(), B.numpy(), rows=(100, 132), threads=0)
    assert O.rel_fro(C.cpu().numpy()[100:132], part[100:132]) <= 1e-5


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (130, 70, 33), (257, 129, 100), (64, 300, 7)])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_fp32_layouts_ragged(m, n, k, ta, tb):
    A = randn((2, 3) + ((k, m) if ta else (m, k)), torch.float32, 510)
    B = randn((2, 3) + ((n, k) if tb else (k, n)), torch.float32, 511)
    C = ops().batched_matmul(A.cuda(), B.cuda(), ta, tb)
    sync_ok()
    assert rel_fro(C, O.matmul_f64(f64(A), f64(B), ta, tb)) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, True), (True, False)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (384, 256, 1024)])
def test_tc_layouts_tile_multiples(m, n, k, ta, tb, dtype):
    A = randn((k, m) if ta else (m, k), dtype, 520, std=1.0 / np.sqrt(k))
    B = randn((n, k) if tb else (k, n), dtype, 521)
    C = ops().batched_matmul(A.cuda(), B.cuda(), ta, tb)
    sync_ok()
    assert C.dtype == dtype
    assert rel_fro(C, O.matmul_f64(f64(A), f64(B), ta, tb)) <= TOL[dtype]


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, True), (True, False)])
@pytest.mark.parametrize("m,n,k", [(8, 8, 8), (200, 136, 72), (136, 264, 520), (1000, 1000, 1000)])
def test_tc_ragged(m, n, k, ta, tb):
    dtype = torch.bfloat16
    A = randn((k, m) if ta else (m, k), dtype, 530, std=1.0 / np.sqrt(k))
    B = randn((n, k) if tb else (k, n), dtype, 531)
    C = ops().batched_matmul(A.cuda(), B.cuda(), ta, tb)
    sync_ok()
    assert rel_fro(C, O.matmul_f64(f64(A), f64(B), ta, tb)) <= 1e-2


def test_tc_many_tiles_and_f32_out():
    # more tiles than SMs, so every CTA loops and both accumulator buffers are reused
    dtype = torch.bfloat16
    A = randn((2048, 512), dtype, 540, std=1.0 / np.sqrt(512))
    B = randn((512, 4096), dtype, 541)
    C = ops().matmul(A.cuda(), B.cuda(), out_dtype=torch.float32)
    sync_ok()
    assert C.dtype == torch.float32
    assert rel_fro(C, O.matmul_f64(f64(A), f64(B))) <= 1e-5  # fp32 output of exact bf16 products


def test_tc_batched_reference_shape():
    # test/test.cc:41-43: BatchedMatmul [b,2048,64] x [b,2048,64]^T (NT); batch scaled down
    A = randn((6, 2048, 64), torch.bfloat16, 550)
    B = randn((6, 2048, 64), torch.bfloat16, 551)
    C = ops().batched_matmul(A.cuda(), B.cuda(), False, True)
    sync_ok()
    assert C.shape == (6, 2048, 2048)
    assert rel_fro(C, O.matmul_f64(f64(A), f64(B), False, True)) <= 1e-2


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, True), (True, False)])
def test_fp8_per_tensor_scales(ta, tb):
    m, n, k = 256, 384, 512
    a32 = randn((k, m) if ta else (m, k), torch.float32, 560, std=1.0 / np.sqrt(k))
    b32 = randn((n, k) if tb else (k, n), torch.float32, 561)
    sa = float(a32.abs().max()) / 448.0
    sb = float(b32.abs().max()) / 448.0
    abits, avals = O.quantize_e4m3(a32.numpy() / sa)
    bbits, bvals = O.quantize_e4m3(b32.numpy() / sb)
    A8 = torch.from_numpy(abits).cuda().view(torch.float8_e4m3fn)
    B8 = torch.from_numpy(bbits).cuda().view(torch.float8_e4m3fn)
    C = ops().batched_matmul(A8, B8, ta, tb, out_dtype=torch.bfloat16,
                             scale_a=torch.tensor([sa], device="cuda"), scale_b=torch.tensor([sb], device="cuda"))
    sync_ok()
    # oracle on the very same 8-bit inputs
    want = O.matmul_f64(avals, bvals, ta, tb) * (np.float64(np.float32(sa)) * np.float64(np.float32(sb)))
    assert rel_fro(C, want) <= 1e-2
    assert rel_fro(C, want) <= 3e-2  # the FP8 tolerance proper (the line above is tighter)
    # sanity only: quantisation itself keeps the product within a few percent
    assert rel_fro(C, O.matmul_f64(a32.numpy(), b32.numpy(), ta, tb)) <= 6e-2


def test_bitwise_repeatable():
    A = randn((512, 1024), torch.bfloat16, 570).cuda()
    B = randn((1024, 768), torch.bfloat16, 571).cuda()
    c1 = ops().matmul(A, B)
    c2 = ops().matmul(A, B)
    sync_ok()
    assert torch.equal(c1, c2)


def test_alignment_is_reported():
    from kernelcodegen_b200 import _lib
    A = randn((64, 36), torch.bfloat16, 580).cuda()   # lda*2 = 72 bytes: not a multiple of 16
    B = randn((36, 64), torch.bfloat16, 581).cuda()
    with pytest.raises(_lib.KcgError) as e:
        ops().matmul(A, B)
    assert e.value.status == _lib.ERR_ALIGNMENT


@pytest.mark.parametrize("m,n,k", [(512, 640, 256), (1024, 1024, 1024), (392, 264, 520)])
def test_tile_shapes_give_identical_bits(m, n, k):
    # 128x256, CTA-pair 256x256, 128x128 and 128x64 tiles accumulate every output over k in the same order
    from kernelcodegen_b200 import _lib
    A = randn((m, k), torch.bfloat16, 580, std=1.0 / np.sqrt(k)).cuda()
    B = randn((k, n), torch.bfloat16, 581).cuda()
    Bt = B.t().contiguous()
    outs = []
    try:
        for mode in (0, 1, 2, 3, -1):
            _lib.load().kcg_gemm_set_pair_mode(mode)
            outs.append(ops().matmul(A, B))
            outs.append(ops().batched_matmul(A, Bt, False, True))
            outs.append(ops().batched_matmul(A.t().contiguous(), Bt, True, True))
            sync_ok()
    finally:
        _lib.load().kcg_gemm_set_pair_mode(-1)
    assert rel_fro(outs[0], O.matmul_f64(f64(A), f64(B))) <= 1e-2
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (130, 70, 33), (257, 129, 100), (1000, 520, 1001)])
def test_fp32_on_tensor_cores_split_operands(m, n, k, ta, tb):
    # three tf32 products of hi/lo-split operands: fp32-grade accuracy from the tensor cores
    from kernelcodegen_b200 import _lib
    A = randn((2,) + ((k, m) if ta else (m, k)), torch.float32, 590)
    B = randn((2,) + ((n, k) if tb else (k, n)), torch.float32, 591)
    try:
        _lib.load().kcg_gemm_set_fp32_mode(1)
        C = ops().batched_matmul(A.cuda(), B.cuda(), ta, tb)
        sync_ok()
        _lib.load().kcg_gemm_set_fp32_mode(0)
        C0 = ops().batched_matmul(A.cuda(), B.cuda(), ta, tb)
        sync_ok()
    finally:
        _lib.load().kcg_gemm_set_fp32_mode(-1)
    want = O.matmul_f64(f64(A), f64(B), ta, tb)
    assert rel_fro(C, want) <= 1e-5
    assert rel_fro(C0, want) <= 1e-5
    assert rel_fro(C, want) <= 4e-6      # in practice an order of magnitude inside the tolerance


def test_fp32_tensor_path_special_values_and_epilogue():
    from kernelcodegen_b200 import _lib
    A = randn((256, 256), torch.float32, 592)
    B = randn((256, 256), torch.float32, 593)
    A[3, 5] = float("inf"); A[7, :] = 0.0; B[:, 9] = 1e-30
    bias = randn((256,), torch.float32, 594).cuda()
    try:
        _lib.load().kcg_gemm_set_fp32_mode(1)
        C = ops().matmul(A.cuda(), B.cuda(), bias=bias, activation="Relu")
        sync_ok()
    finally:
        _lib.load().kcg_gemm_set_fp32_mode(-1)
    ref = torch.relu(A.double() @ B.double() + bias.cpu().double())
    row_ok = torch.ones(256, dtype=torch.bool); row_ok[3] = False
    assert rel_fro(C[row_ok], ref[row_ok].numpy()) <= 1e-5
    assert bool(torch.isinf(C[3]).logical_or(torch.isnan(C[3])).logical_or(C[3] == 0).all())   # the infinite row stays non-finite or is clamped by Relu
    assert bool((C[7].cpu() == torch.relu(bias.cpu())).all())
