"""Kernels launched as programmatic dependents of their predecessor must still see its results:
chains with read-after-write and write-after-read hazards between consecutive launches, run
eagerly and as a CUDA graph, against the same chain computed by torch / in float64."""
import numpy as np
import pytest
import torch

from helpers import f64, randn, rel_fro

pytestmark = pytest.mark.gpu


def _ops():
    from kernelcodegen_b200 import _lib, ops
    return _lib, ops


def _bandwidth_chain(ops, a, b, g, beta, steps):
    # every launch reads what the one before wrote, and overwrites what the one before read
    for _ in range(steps):
        ops.binary(a, b, "Add", out=a)            # a <- a + b           (in place)
        ops.elementwise(a, "Relu", out=b)          # b <- relu(a)         (overwrites the last launch's input)
        ops.layernorm(b, g, beta, 1, 1e-5, out=a)  # a <- LN(b)
    return a, b


def _torch_chain(a, b, g, beta, steps):
    for _ in range(steps):
        a = (a.float() + b.float()).to(a.dtype)
        b = torch.relu(a)
        a = torch.nn.functional.layer_norm(b.float(), (b.shape[1],), g.float(), beta.float(), 1e-5).to(a.dtype)
    return a, b


@pytest.mark.parametrize("rows,cols", [(2048, 4096), (333, 1024)])
def test_bandwidth_chain_eager_and_graph(rows, cols):
    L, ops = _ops()
    dt = torch.bfloat16
    a0, b0 = randn((rows, cols), dt, 1).cuda(), randn((rows, cols), dt, 2).cuda()
    g, beta = randn((cols,), dt, 3, mean=1.0, std=0.1).cuda(), randn((cols,), dt, 4, std=0.1).cuda()
    want_a, want_b = _torch_chain(a0.clone(), b0.clone(), g, beta, 6)

    a, b = _bandwidth_chain(ops, a0.clone(), b0.clone(), g, beta, 6)
    torch.cuda.synchronize()
    # six rounds of 16-bit rounding separate the two chains; a launch that ran early would have
    # read whole rows of stale data, which is an error of order one
    assert rel_fro(b, f64(want_b)) < 2e-2
    assert rel_fro(a, f64(want_a)) < 2e-2

    # the same chain captured in a graph (the programmatic edges survive capture) and replayed
    ga, gb = a0.clone(), b0.clone()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        _bandwidth_chain(ops, ga.clone(), gb.clone(), g, beta, 1)   # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        _bandwidth_chain(ops, ga, gb, g, beta, 6)
    ga.copy_(a0); gb.copy_(b0)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(ga, a) and torch.equal(gb, b)   # eager and replayed chains agree bit for bit
    assert L.device_status() == 0


def test_gemm_chain_small_tiles():
    # few tiles per launch: the next GEMM's CTAs are resident on idle SMs while this one still runs
    L, ops = _ops()
    dt = torch.bfloat16
    n = 512
    x = randn((n, n), dt, 5, std=1.0).cuda()
    w = (randn((n, n), torch.float32, 6, std=1.0) / np.sqrt(n)).to(dt).cuda()
    cur = x.clone()
    ref = f64(x)
    wf = f64(w)
    outs = [torch.empty((n, n), dtype=dt, device="cuda") for _ in range(2)]
    for i in range(8):
        nxt = outs[i % 2]
        ops.matmul(cur, w, out=nxt)               # reads the previous launch's output, overwrites its input
        ref = f64(torch.from_numpy(ref @ wf).to(dt))   # round to bf16 after every product, as the kernel does
        cur = nxt
    torch.cuda.synchronize()
    assert rel_fro(cur, ref) < 1e-2
    assert L.device_status() == 0


def test_mixed_chain_with_library_kernels():
    # an ordinary (torch) kernel between two overlapped launches is a full dependency on both sides
    L, ops = _ops()
    dt = torch.bfloat16
    a, b = randn((1024, 2048), dt, 7).cuda(), randn((1024, 2048), dt, 8).cuda()
    want = a.clone()
    for _ in range(5):
        ops.binary(a, b, "Add", out=a)
        a.mul_(0.5)                                # torch kernel, launched the ordinary way
        ops.elementwise(a, "Relu", out=a)
        want = torch.relu(((want.float() + b.float()).to(dt).float() * 0.5).to(dt))
    torch.cuda.synchronize()
    assert torch.equal(a, want)
    assert L.device_status() == 0
