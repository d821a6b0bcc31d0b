"""The multi-rank path on CPU: two gloo ranks partition a problem, run a stand-in for the
kernel (the CPU oracle; the CUDA kernels have no CPU form) on their block, and all-gather;
the result must equal the unsharded computation bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernelcodegen_b200 import _lib, shard
from oracle import oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_matmul(A, B):
    return torch.from_numpy(O.ref32.matmul(A.numpy(), B.numpy()))


def _oracle_layernorm(x, g, b, axis, eps):
    return torch.from_numpy(O.ref32.layernorm(x.numpy(), g.numpy(), b.numpy(), axis, eps))


def _oracle_gelu(x, op):
    return torch.from_numpy(O.ref32.unary(op, x.numpy()))


def _oracle_fmha(Q, K, V, scale, causal):
    return torch.from_numpy(O.ref32.attention(Q.numpy(), K.numpy(), V.numpy(), scale, causal))


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1234)       # same data on every rank
        # GEMM: M = 300 is not a multiple of the 128-row granule -> uneven shards (256 + 44)
        A = torch.randn(300, 64, generator=g); B = torch.randn(64, 48, generator=g)
        b0, c0 = shard.shard_range(300, shard.GEMM_ROW_GRANULE)
        C = shard.matmul(A[b0:b0 + c0], B, total_rows=300, gather=True, compute=_oracle_matmul)
        ok = torch.equal(C, _oracle_matmul(A, B)) and (b0, c0) == ((0, 256) if rank == 0 else (256, 44))
        # LayerNorm: even shards -> all_gather_into_tensor path
        x = torch.randn(64, 96, generator=g); gm = torch.randn(96, generator=g); bt = torch.randn(96, generator=g)
        y = shard.layernorm(shard.shard_rows(x), gm, bt, 1, 1e-5, total_rows=64, gather=True, compute=_oracle_layernorm)
        ok = ok and torch.equal(y, _oracle_layernorm(x, gm, bt, 1, 1e-5))
        # without gather each rank keeps only its rows
        y_local = shard.layernorm(shard.shard_rows(x), gm, bt, 1, 1e-5, compute=_oracle_layernorm)
        ok = ok and y_local.shape[0] == 32
        # elementwise, odd row count
        u = torch.randn(7, 33, generator=g)
        v = shard.elementwise(shard.shard_rows(u), "Gelu", total_rows=7, gather=True, compute=_oracle_gelu)
        ok = ok and torch.equal(v, _oracle_gelu(u, "Gelu"))
        # attention over (batch*head) slices
        Q = torch.randn(6, 1, 16, 8, generator=g); K = torch.randn(6, 1, 16, 8, generator=g); V = torch.randn(6, 1, 16, 8, generator=g)
        Oo = shard.fmha(shard.shard_rows(Q), shard.shard_rows(K), shard.shard_rows(V), 0.3, True, total_slices=6,
                        gather=True, compute=_oracle_fmha)
        ok = ok and torch.equal(Oo, _oracle_fmha(Q, K, V, 0.3, True))
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather():
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert dict(results) == {0: True, 1: True}


def test_single_process_is_identity():
    x = torch.arange(12.0).reshape(6, 2)
    assert shard.shard_range(6) == (0, 6)
    assert torch.equal(shard.shard_rows(x), x)
    assert shard.all_gather_rows(x, 6) is x
    with pytest.raises(ValueError):
        shard.layernorm(x, x, x, 0, compute=lambda *a: a[0])


def test_weak_scaling_ranges_cover_bench_shapes():
    # config 5: M = 65536 rows over 8 GPUs -> 8192 rows each, tile aligned
    for r in range(8):
        assert _lib.shard_range(65536, 8, r, 128) == (r * 8192, 8192)
    # B*H = 64*32 slices over 8 GPUs
    assert [_lib.shard_range(2048, 8, r, 1)[1] for r in range(8)] == [256] * 8
