"""GEMM whose epilogue writes its block into several gathered matrices (kcg_gemm_allgather).
On one GPU the "peers" are further buffers of the same device: the kernel and its staged
128-byte stores are the ones a multi-GPU run uses, only the addresses differ."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import randn, f64, rel_fro, sync_ok

pytestmark = pytest.mark.gpu


def call(A, B, bufs, rank, row_offset, trans_b=False, out_dtype=None, bias=None, act=0, scale_a=None, scale_b=None):
    from kernelcodegen_b200 import _lib, ops
    M, K = A.shape
    N = B.shape[0] if trans_b else B.shape[1]
    arr = (ctypes.c_void_p * len(bufs))(*[b.data_ptr() for b in bufs])
    rc = _lib.load().kcg_gemm_allgather(
        ops._dt(A), ops._DT[out_dtype or A.dtype], M, N, K, 0, int(trans_b), A.data_ptr(), A.stride(0), B.data_ptr(),
        B.stride(0), arr, len(bufs), rank, row_offset, bufs[0].shape[1],
        scale_a.data_ptr() if scale_a is not None else None, scale_b.data_ptr() if scale_b is not None else None,
        bias.data_ptr() if bias is not None else None, act, torch.cuda.current_stream().cuda_stream)
    return rc


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k,world", [(256, 256, 64, 2), (512, 768, 256, 3), (1000, 520, 136, 4), (2048, 4096, 512, 8)])
def test_every_destination_gets_the_block(m, n, k, world, dtype):
    from kernelcodegen_b200 import ops
    A = randn((m, k), dtype, 800, std=1.0 / np.sqrt(k)).cuda()
    B = randn((k, n), dtype, 801).cuda()
    total = m * world
    for rank in (0, world - 1):
        bufs = [torch.full((total, n), 7.0, dtype=dtype, device="cuda") for _ in range(world)]
        assert call(A, B, bufs, rank, rank * m) == 0
        sync_ok()
        want = ops.matmul(A, B)     # the plain kernel: the gathered block must hold the same bits
        assert rel_fro(want, O.matmul_f64(f64(A), f64(B))) <= 1e-2
        for b in bufs:
            assert torch.equal(b[rank * m:(rank + 1) * m], want)
            # nothing outside this rank's rows is touched
            assert bool((b[:rank * m] == 7.0).all()) and bool((b[(rank + 1) * m:] == 7.0).all())


def test_emulated_ranks_assemble_the_full_product():
    # four "ranks" run one after the other on this GPU, each writing its block everywhere
    from kernelcodegen_b200 import ops
    world, m, n, k = 4, 384, 512, 256
    A = randn((world * m, k), torch.bfloat16, 810, std=1.0 / np.sqrt(k)).cuda()
    B = randn((n, k), torch.bfloat16, 811).cuda()      # transposed-B layout
    bufs = [torch.zeros((world * m, n), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    for r in range(world):
        assert call(A[r * m:(r + 1) * m], B, bufs, r, r * m, trans_b=True) == 0
    sync_ok()
    full = ops.batched_matmul(A, B, False, True)
    for b in bufs:
        assert torch.equal(b, full)


def test_fp8_bias_activation_and_wide_ldc():
    from kernelcodegen_b200 import ops
    m, n, k = 512, 256, 256
    a32 = randn((m, k), torch.float32, 820, std=1.0 / np.sqrt(k)); b32 = randn((k, n), torch.float32, 821)
    A8 = a32.cuda().to(torch.float8_e4m3fn); B8 = b32.cuda().to(torch.float8_e4m3fn)
    sa = torch.tensor([0.5], device="cuda"); sb = torch.tensor([2.0], device="cuda")
    bias = randn((n,), torch.bfloat16, 822).cuda()
    bufs = [torch.zeros((2 * m, n + 64), dtype=torch.bfloat16, device="cuda") for _ in range(2)]   # ldc > N
    assert call(A8, B8, bufs, 1, m, out_dtype=torch.bfloat16, bias=bias, act=2, scale_a=sa, scale_b=sb) == 0
    sync_ok()
    want = ops.matmul(A8, B8, out_dtype=torch.bfloat16, scale_a=sa, scale_b=sb, bias=bias, activation="Gelu")
    for b in bufs:
        assert torch.equal(b[m:, :n], want)
        assert bool((b[:, n:] == 0).all()) and bool((b[:m] == 0).all())


def test_rejections():
    from kernelcodegen_b200 import _lib
    A = randn((128, 64), torch.bfloat16, 830).cuda(); B = randn((64, 256), torch.bfloat16, 831).cuda()
    bufs = [torch.zeros((256, 256), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    assert call(A, B, bufs, 0, 0) == _lib.ERR_UNSUPPORTED          # M must exceed 128 with peers
    assert call(A, B, bufs, 2, 0) == _lib.ERR_INVALID_ARG          # rank outside the world
    A32 = randn((256, 64), torch.float32, 832).cuda(); B32 = randn((64, 256), torch.float32, 833).cuda()
    b32 = [torch.zeros((512, 256), device="cuda") for _ in range(2)]
    assert call(A32, B32, b32, 0, 0) == _lib.ERR_UNSUPPORTED       # fp32 inputs have no tensor-core path
    torch.cuda.synchronize()


def test_gather_buffers_single_process():
    from kernelcodegen_b200 import shard, ops
    bufs = shard.GatherBuffers(512, 256, torch.bfloat16)
    try:
        assert bufs.world == 1 and bufs.local.shape == (512, 256) and bufs.local.dtype == torch.bfloat16
        A = randn((512, 128), torch.bfloat16, 840).cuda(); B = randn((128, 256), torch.bfloat16, 841).cuda()
        out = shard.matmul_allgather(A, B, bufs)
        sync_ok()
        assert out.data_ptr() == bufs.ptrs[0]
        assert torch.equal(out, ops.matmul(A, B))
    finally:
        bufs.close()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("Bl,H,S,D,world", [(1, 2, 256, 128, 2), (2, 3, 200, 128, 3), (1, 2, 384, 64, 4), (1, 1, 1024, 128, 8)])
def test_fmha_every_destination_gets_the_slices(Bl, H, S, D, world, causal):
    # attention whose epilogue writes its batches into several gathered tensors (here all local)
    from kernelcodegen_b200 import _lib, ops
    Q, K, V = (randn((Bl, H, S, D), torch.bfloat16, 850 + i).cuda() for i in range(3))
    want = ops.fmha(Q, K, V, D ** -0.5, causal)
    sync_ok()
    i64 = ctypes.c_int64
    st = (i64 * 3)(H * S * D, S * D, D)
    for rank in (0, world - 1):
        bufs = [torch.full((world * Bl, H, S, D), 3.0, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
        rc = _lib.load().kcg_fmha_fwd_allgather(2, Bl, H, S, S, D, D ** -0.5, int(causal), Q.data_ptr(), st, K.data_ptr(), st,
                                                V.data_ptr(), st, arr, world, rank, rank * Bl, st,
                                                torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        sync_ok()
        for b in bufs:
            assert torch.equal(b[rank * Bl:(rank + 1) * Bl], want)     # same kernel, same bits
            assert bool((b[:rank * Bl] == 3.0).all()) and bool((b[(rank + 1) * Bl:] == 3.0).all())
