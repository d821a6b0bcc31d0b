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
        # the same two gathers with the replication done by NVSwitch (multimem.st to a multicast
        # mapping; torch's symmetric memory does the binding).  Where the fabric offers no multicast
        # mc_ptr is 0 and the calls take the peer-store path over the same buffers.
        mb = None
        try:
            mb = shard.MulticastBuffers(A.shape[0], B.shape[1], torch.bfloat16)
        except Exception as exc:   # noqa: BLE001 - symmetric memory may be unavailable on a host
            print(f"rank {rank}: symmetric memory unavailable: {exc}", flush=True)
        if mb is not None:
            try:
                for _ in range(2):
                    mb.local.zero_()
                    out = shard.matmul_allgather(A[b0:b0 + c0].contiguous(), B, mb)
                torch.cuda.synchronize()
                ok = ok and torch.equal(out, full)
                print(f"rank {rank}: multicast gather used: {bool(mb.mc_ptr)}", flush=True)
            finally:
                mb.close()
            ml = shard.MulticastBuffers(4096, 2048, torch.bfloat16)
            try:
                if ml.mc_ptr:
                    yl = shard.layernorm_allgather(shard.shard_rows(x).contiguous(), gm, gm, ml, 1e-5)
                    torch.cuda.synchronize()
                    ok = ok and torch.equal(yl, ops.layernorm(x, gm, gm, 1, 1e-5))
            finally:
                ml.close()
            mf = shard.MulticastBuffers(6 * 2 * 256, 128, torch.bfloat16)
            try:
                out = shard.fmha_allgather(shard.shard_rows(Q).contiguous(), shard.shard_rows(K).contiguous(),
                                           shard.shard_rows(V).contiguous(), mf, 6, 128 ** -0.5, True)
                torch.cuda.synchronize()
                ok = ok and torch.equal(out, ops.fmha(Q, K, V, 128 ** -0.5, True))
            finally:
                mf.close()
        # the C entry a host program without Python uses: an NCCL communicator made through the
        # library's own wrappers (the id travels by other means, here torch's object broadcast),
        # then the in-place gather of a row-sharded buffer, with even and with ragged blocks
        import ctypes
        lib = _lib.load()
        uid = ctypes.create_string_buffer(128)
        if rank == 0:
            _lib.check(lib.kcg_nccl_unique_id(uid), "kcg_nccl_unique_id")
        box = [bytes(uid.raw)]
        dist.broadcast_object_list(box, src=0)
        comm = ctypes.c_void_p()
        _lib.check(lib.kcg_nccl_comm_create(world, rank, ctypes.create_string_buffer(box[0], 128), ctypes.byref(comm)),
                   "kcg_nccl_comm_create")
        stream = torch.cuda.current_stream().cuda_stream
        for total, granule in ((4096, 1), (1000, 128)):
            want = torch.arange(total * 64, device="cuda", dtype=torch.float32).view(total, 64)
            buf = torch.full_like(want, -1.0)
            b1, c1 = _lib.shard_range(total, world, rank, granule)
            buf[b1:b1 + c1] = want[b1:b1 + c1]
            _lib.check(lib.kcg_shard_allgather(buf.data_ptr(), total, 64 * 4, granule, world, rank, comm, stream),
                       "kcg_shard_allgather")
            torch.cuda.synchronize()
            ok = ok and torch.equal(buf, want)
        # a communicator of another size is refused
        ok = ok and lib.kcg_shard_allgather(buf.data_ptr(), 16, 4, 1, world + 1, rank, comm, stream) == _lib.ERR_INVALID_ARG
        _lib.check(lib.kcg_nccl_comm_destroy(comm), "kcg_nccl_comm_destroy")
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
