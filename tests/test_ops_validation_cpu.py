"""The Python operator wrappers hand raw pointers to the C ABI, so every mismatch between the
operands and what the kernel will read or write has to be refused on the host, before any
launch.  These cases run on CPU tensors: each must raise for its own reason (not merely because
the tensors are not on a GPU)."""
import pytest
import torch

from kernelcodegen_b200 import ops


def t(*shape, dtype=torch.bfloat16):
    return torch.zeros(shape, dtype=dtype)


def test_matmul_mixed_dtypes_refused():
    with pytest.raises(TypeError, match="share a dtype"):
        ops.matmul(t(64, 32, dtype=torch.float32), t(32, 16, dtype=torch.bfloat16))
    with pytest.raises(TypeError, match="share a dtype"):
        ops.batched_matmul(t(2, 64, 32), t(2, 16, 32, dtype=torch.float16), trans_b=True)


def test_matmul_out_checked():
    A, B = t(64, 32), t(32, 16)
    with pytest.raises(ValueError, match="out has shape"):
        ops.matmul(A, B, out=t(64, 8))
    with pytest.raises(ValueError, match="out has dtype"):
        ops.matmul(A, B, out_dtype=torch.bfloat16, out=t(64, 16, dtype=torch.float32))
    with pytest.raises(ValueError, match="contiguous"):
        ops.matmul(A, B, out=t(16, 64).t())


def test_fmha_operands_checked():
    Q = t(2, 4, 128, 64)
    with pytest.raises(ValueError, match="keys"):
        ops.fmha(Q, t(2, 4, 256, 64), t(2, 4, 128, 64))
    with pytest.raises(TypeError, match="share a dtype"):
        ops.fmha(Q, t(2, 4, 128, 64, dtype=torch.float16), t(2, 4, 128, 64))
    with pytest.raises(ValueError, match="must match"):
        ops.fmha(Q, t(2, 2, 128, 64), t(2, 2, 128, 64))
    with pytest.raises(ValueError, match="must match"):
        ops.fmha(Q, t(2, 4, 128, 128), t(2, 4, 128, 128))
    with pytest.raises(ValueError, match="out must be"):
        ops.fmha(Q, t(2, 4, 128, 64), t(2, 4, 128, 64), out=t(2, 4, 64, 64))
    with pytest.raises(ValueError, match="contiguous head"):
        ops.fmha(Q.transpose(2, 3), t(2, 4, 128, 64), t(2, 4, 128, 64))


@pytest.mark.parametrize("call", [
    lambda: ops.layernorm(t(8, 64), t(64), t(64), 1, out=t(8, 32)),
    lambda: ops.layernorm_gelu_add(t(8, 64), t(64), t(64), t(8, 64), out=t(4, 64)),
    lambda: ops.elementwise(t(8, 64), "Gelu", out=t(8, 65)),
    lambda: ops.binary(t(8, 64), t(64), "Add", out=t(64)),
    lambda: ops.gather(t(8, 64), torch.zeros(3, dtype=torch.int64), 0, out=t(4, 64)),
    lambda: ops.transpose(t(8, 64), out=t(8, 64)),
])
def test_out_shape_checked(call):
    with pytest.raises(ValueError, match="out has shape"):
        call()


def test_out_dtype_and_layout_checked():
    with pytest.raises(ValueError, match="out has dtype"):
        ops.elementwise(t(8, 64), "Relu", out=t(8, 64, dtype=torch.float32))
    with pytest.raises(ValueError, match="contiguous"):
        ops.layernorm(t(8, 64), t(64), t(64), 1, out=t(64, 8).t())
    with pytest.raises(TypeError, match="share a dtype"):
        ops.layernorm(t(8, 64), t(64, dtype=torch.float32), t(64), 1)


def test_cpu_tensors_still_refused():
    with pytest.raises(ValueError, match="CUDA tensors"):
        ops.matmul(t(64, 32), t(32, 16))


class _FakeBuffers:
    """Stands in for shard.MulticastBuffers: only the fields the argument checks read."""
    def __init__(self, total_rows, cols, dtype, mc_ptr, world=2, rank=0):
        self.total_rows, self.cols, self.dtype, self.mc_ptr = total_rows, cols, dtype, mc_ptr
        self.world, self.rank, self.group, self.local = world, rank, None, None


def test_layernorm_allgather_arguments_checked():
    # every mismatch that would make the kernel write outside the gathered tensor raises before any launch
    from kernelcodegen_b200 import shard
    x = torch.zeros(8, 64, dtype=torch.bfloat16)
    g = torch.ones(64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="multicast"):
        shard.layernorm_allgather(x, g, g, _FakeBuffers(16, 64, torch.bfloat16, 0))
    with pytest.raises(ValueError, match="width"):
        shard.layernorm_allgather(x, g, g, _FakeBuffers(16, 128, torch.bfloat16, 1 << 20))
    with pytest.raises(ValueError, match="dtype"):
        shard.layernorm_allgather(x.float(), g, g, _FakeBuffers(16, 64, torch.bfloat16, 1 << 20))
    with pytest.raises(ValueError, match="CUDA"):
        shard.layernorm_allgather(x, g, g, _FakeBuffers(16, 64, torch.bfloat16, 1 << 20))
