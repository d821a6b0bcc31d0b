"""The host-tensor API (pinned buffers in, pinned buffers out): results must be the bits the
device API produces, whether a call goes through in one piece or as overlapped row chunks, and
back-to-back calls that reuse the staging buffers must not see each other's data."""
import pytest
import torch

from tests.helpers import randn, sync_ok

pytestmark = pytest.mark.gpu


def mods():
    from kernelcodegen_b200 import host, ops
    return host, ops


@pytest.mark.parametrize("shape", [(64, 512), (4096, 2048), (1000, 4104)])   # below / above the chunking threshold, ragged
def test_host_ops_match_device_ops(shape):
    host, ops = mods()
    x = randn(shape, torch.bfloat16, 1000).pin_memory()
    r = randn(shape, torch.bfloat16, 1001).pin_memory()
    g = randn(shape[-1:], torch.bfloat16, 1002, mean=1.0, std=0.1).pin_memory()
    b = randn(shape[-1:], torch.bfloat16, 1003, std=0.1).pin_memory()
    y = host.layernorm(x, g, b, 1, 1e-5)
    v = host.elementwise(x, "Gelu")
    c = host.binary(x, r, "Add")
    sync_ok()
    assert y.is_pinned() and not y.is_cuda
    assert torch.equal(y, ops.layernorm(x.cuda(), g.cuda(), b.cuda(), 1, 1e-5).cpu())
    assert torch.equal(v, ops.elementwise(x.cuda(), "Gelu").cpu())
    assert torch.equal(c, ops.binary(x.cuda(), r.cuda(), "Add").cpu())
    host.clear_staging()


def test_back_to_back_calls_reuse_staging_safely():
    host, ops = mods()
    shape = (4096, 2048)
    xs = [randn(shape, torch.bfloat16, 1010 + i).pin_memory() for i in range(4)]
    outs = [torch.empty(shape, dtype=torch.bfloat16).pin_memory() for _ in range(4)]
    for i in range(4):          # queued without synchronising in between
        host.elementwise(xs[i], "Relu", out=outs[i])
    torch.cuda.current_stream().synchronize()   # the documented contract: the current stream is enough
    for i in range(4):
        assert torch.equal(outs[i], torch.relu(xs[i]))
    host.clear_staging()
