"""Sharded operators on real GPUs (NCCL): each rank runs the ordinary kernel on its block;
the all-gathered result must equal the single-GPU result bit for bit (same kernel, same
tile order).  Needs at least two GPUs; skipped otherwise."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    import torch.distributed as dist
    from kernelcodegen_b200 import ops, shard, _lib
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g = torch.Generator(device="cuda").manual_seed(99)  # same stream of numbers on every rank
        A = (torch.randn(1024 + 128, 512, generator=g, device="cuda") * 512 ** -0.5).bfloat16()
        B = torch.randn(512, 768, generator=g, device="cuda").bfloat16()
        full = ops.matmul(A, B)
        b0, c0 = shard.shard_range(A.shape[0], shard.GEMM_ROW_GRANULE)
        C = shard.matmul(A[b0:b0 + c0].contiguous(), B, total_rows=A.shape[0], gather=True)
        ok = torch.equal(C, full)
        x = torch.randn(4096, 2048, generator=g, device="cuda").bfloat16()
        gm = torch.randn(2048, generator=g, device="cuda").bfloat16()
        y = shard.layernorm(shard.shard_rows(x).contiguous(), gm, gm, 1, 1e-5, total_rows=4096, gather=True)
        ok = ok and torch.equal(y, ops.layernorm(x, gm, gm, 1, 1e-5))
        Q, K, V = (torch.randn(6, 2, 256, 128, generator=g, device="cuda").bfloat16() for _ in range(3))
        Oo = shard.fmha(shard.shard_rows(Q).contiguous(), shard.shard_rows(K).contiguous(),
                        shard.shard_rows(V).contiguous(), 128 ** -0.5, True, total_slices=6, gather=True)
        ok = ok and torch.equal(Oo, ops.fmha(Q, K, V, 128 ** -0.5, True))
        # the gather done by the GEMM epilogue itself: peer stores into every rank's buffer
        bufs = shard.GatherBuffers(A.shape[0], B.shape[1], torch.bfloat16)
        try:
            for _ in range(3):    # repeated use of the same buffers, barriers placed by the call
                bufs.local.zero_()
                out = shard.matmul_allgather(A[b0:b0 + c0].contiguous(), B, bufs)
            torch.cuda.synchronize()
            ok = ok and torch.equal(out, full)
        finally:
            bufs.close()
        # attention with the gather in its epilogue: 6 batches over the ranks
        fb = shard.GatherBuffers(6 * 2 * 256, 128, torch.bfloat16)
        try:
            out = shard.fmha_allgather(shard.shard_rows(Q).contiguous(), shard.shard_rows(K).contiguous(),
                                       shard.shard_rows(V).contiguous(), fb, 6, 128 ** -0.5, True)
            torch.cuda.synchronize()
            ok = ok and torch.equal(out, ops.fmha(Q, K, V, 128 ** -0.5, True))
        finally:
            fb.close()
        torch.cuda.synchronize()
        ok = ok and _lib.device_status() == 0
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_gpu_shard_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
        assert p.exitcode == 0
    assert dict(results) == {0: True, 1: True}
