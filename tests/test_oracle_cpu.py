"""The oracle against independent formulas (torch float64 on CPU) and against itself
(reference-faithful fp32 nests vs the float64 layer).  No GPU needed."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import randn, uniform, f64


def test_matmul_layers_agree():
    A = uniform((96, 80), torch.float32, 1).numpy()
    B = uniform((80, 72), torch.float32, 2).numpy()
    want = O.matmul_f64(A, B)
    assert O.rel_fro(O.ref32.matmul(A, B), want) < 1e-6
    assert O.rel_fro(torch.from_numpy(A).double() @ torch.from_numpy(B).double(), want) < 1e-14
    # a row slice computes only those rows
    part = O.ref32.matmul(A, B, rows=(8, 24))
    assert np.array_equal(part[8:24], O.ref32.matmul(A, B)[8:24]) and not part[:8].any()


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_batched_matmul_layouts(ta, tb):
    m, n, k = 24, 40, 16
    A = randn((3, 2) + ((k, m) if ta else (m, k)), torch.float32, 3).numpy()
    B = randn((3, 2) + ((n, k) if tb else (k, n)), torch.float32, 4).numpy()
    want = O.matmul_f64(A, B, ta, tb)
    assert want.shape == (3, 2, m, n)
    assert O.rel_fro(O.ref32.batched_matmul(A, B, ta, tb), want) < 1e-6


def test_softmax_matches_torch():
    x = randn((2, 3, 17, 33), torch.float32, 5)
    want = torch.softmax(x.double() * 0.25, dim=-1).numpy()
    assert O.rel_fro(O.softmax_f64(x.numpy(), scale=0.25), want) < 1e-14
    assert O.rel_fro(O.ref32.softmax(x.numpy(), scale=0.25), want) < 1e-6
    # causal: row i of the trailing [q, c] matrix keeps columns j <= i + (c - q)
    q, c = 17, 33
    mask = torch.ones(q, c, dtype=torch.bool).tril(diagonal=c - q)
    wantc = torch.softmax((x.double() * 0.25).masked_fill(~mask, float("-inf")), dim=-1).numpy()
    assert O.rel_fro(O.softmax_f64(x.numpy(), scale=0.25, causal=True), wantc) < 1e-14
    assert O.rel_fro(O.ref32.softmax(x.numpy(), scale=0.25, causal=True), wantc) < 1e-6


@pytest.mark.parametrize("shape,axis,pshape", [((6, 40), 1, (40,)), ((2, 12, 20), 1, (12, 20)), ((2, 12, 20), -1, (20,)),
                                              ((2, 12, 20), 1, (12, 1))])
def test_layernorm_matches_torch(shape, axis, pshape):
    x = randn(shape, torch.float32, 6)
    g = randn(pshape, torch.float32, 7, mean=1.0, std=0.1)
    b = randn(pshape, torch.float32, 8, std=0.1)
    ax = axis if axis >= 0 else axis + len(shape)
    norm_shape = shape[ax:]
    want = torch.nn.functional.layer_norm(x.double(), norm_shape, g.double().expand(norm_shape),
                                          b.double().expand(norm_shape), eps=float(np.float32(1e-5))).numpy()
    assert O.rel_fro(O.layernorm_f64(x.numpy(), g.numpy(), b.numpy(), axis), want) < 1e-13
    assert O.rel_fro(O.ref32.layernorm(x.numpy(), g.numpy(), b.numpy(), axis), want) < 1e-6


def test_unary_ops():
    x = randn((7, 130), torch.float32, 9)
    xp = x.abs() + 0.1
    assert O.rel_fro(O.unary_f64("Tanh", x.numpy()), torch.tanh(x.double()).numpy()) < 1e-14
    assert O.rel_fro(O.unary_f64("Sqrt", xp.numpy()), torch.sqrt(xp.double()).numpy()) < 1e-14
    assert O.rel_fro(O.unary_f64("Log", xp.numpy()), torch.log(xp.double()).numpy()) < 1e-14
    assert O.rel_fro(O.unary_f64("Relu", x.numpy()), torch.relu(x.double()).numpy()) == 0
    # the reference's Gelu constants are truncated (0.797884 for sqrt(2/pi)); torch's tanh
    # GELU uses the exact ones, so the two agree only to ~1e-6.
    tg = torch.nn.functional.gelu(x.double(), approximate="tanh").numpy()
    assert O.rel_fro(O.unary_f64("Gelu", x.numpy()), tg) < 5e-6
    for op, arg in [("Tanh", x), ("Sqrt", xp), ("Log", xp), ("Relu", x), ("Gelu", x), ("Cast", x)]:
        assert O.rel_fro(O.ref32.unary(op, arg.numpy()), O.unary_f64(op, arg.numpy())) < 1e-6


@pytest.mark.parametrize("sa,sb", [((16, 1, 1, 32), (1, 12, 32)), ((4, 5, 6), (4, 5, 6)), ((4, 5, 6), (6,)),
                                   ((4, 5, 6), (5, 1)), ((1,), (3, 4)), ((3, 1, 5), (1, 4, 1))])
def test_binary_broadcast(sa, sb):
    a = randn(sa, torch.float32, 10).numpy()
    b = randn(sb, torch.float32, 11).numpy() + 3.0
    for op in ["Add", "Mul", "Div", "Sub", "Equal", "Greater"]:
        want = O.binary_f64(op, a, b)
        got = O.ref32.binary(op, a, b)
        assert got.shape == want.shape
        assert O.rel_fro(got, want) < 1e-6
    want = O.binary_f64("Pow", np.abs(a) + 0.5, b)
    assert O.rel_fro(O.ref32.binary("Pow", np.abs(a) + 0.5, b), want) < 1e-6


def test_binary_rejects_mismatch():
    with pytest.raises(ValueError):
        O.ref32.binary("Add", np.zeros((4, 5), np.float32), np.zeros((4, 3), np.float32))


def test_attention_matches_torch():
    Q = randn((2, 3, 24, 16), torch.float32, 12)
    K = randn((2, 3, 40, 16), torch.float32, 13)
    V = randn((2, 3, 40, 16), torch.float32, 14)
    for causal in (False, True):
        want = torch.nn.functional.scaled_dot_product_attention(
            Q.double(), K.double(), V.double(), scale=0.25,
            attn_mask=torch.ones(24, 40, dtype=torch.bool).tril(diagonal=16) if causal else None).numpy()
        assert O.rel_fro(O.attention_f64(Q.numpy(), K.numpy(), V.numpy(), 0.25, causal), want) < 1e-13
        assert O.rel_fro(O.ref32.attention(Q.numpy(), K.numpy(), V.numpy(), 0.25, causal), want) < 1e-6
    # a (batch, head) slice range computes only those slices
    part = O.ref32.attention(Q.numpy(), K.numpy(), V.numpy(), 0.25, False, slices=(1, 3))
    full = O.ref32.attention(Q.numpy(), K.numpy(), V.numpy(), 0.25, False)
    assert np.array_equal(part.reshape(6, 24, 16)[1:3], full.reshape(6, 24, 16)[1:3])
    assert not part.reshape(6, 24, 16)[0].any()


def test_storage_rounding_matches_torch():
    x = torch.randn(50000, generator=torch.Generator().manual_seed(3)) * 5
    assert np.array_equal(O.round_bf16(x.numpy()), x.bfloat16().float().numpy())
    assert np.array_equal(O.round_f16(x.numpy()), x.half().float().numpy())
    bits, vals = O.quantize_e4m3(x.numpy() * 40)  # exercises saturation at +-448
    t8 = (x * 40).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert np.array_equal(bits, t8.view(torch.uint8).numpy())
    assert np.array_equal(vals, t8.float().numpy())
    assert np.array_equal(O.decode_e4m3(np.arange(256, dtype=np.uint8))[:127],
                          torch.arange(127, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy())
    assert vals.max() == 448.0 and vals.min() == -448.0


def test_threads_do_not_change_results():
    A = uniform((64, 64), torch.float32, 20).numpy()
    B = uniform((64, 64), torch.float32, 21).numpy()
    assert np.array_equal(O.ref32.matmul(A, B, threads=1), O.ref32.matmul(A, B, threads=4))
    x = randn((32, 100), torch.float32, 22).numpy()
    g = np.ones(100, np.float32); b = np.zeros(100, np.float32)
    assert np.array_equal(O.ref32.layernorm(x, g, b, 1, threads=1), O.ref32.layernorm(x, g, b, 1, threads=4))


def test_gather_loop_nest_against_numpy_take():
    rng = np.random.default_rng(77)
    for shape, idx_shape, axis in [((5, 4), (3,), 0), ((5, 4), (3,), 1), ((3, 6, 2), (2, 2), 1), ((3, 6, 2), (1,), 1),
                                   ((2, 3, 4), (5,), 2)]:
        x = rng.standard_normal(shape).astype(np.float32)
        idx = rng.integers(0, shape[axis], idx_shape)
        a, b = O.gather_nest(x, idx, axis), O.gather_take(x, idx, axis)
        assert a.shape == b.shape == O.gather_shape(shape, idx_shape, axis)
        assert np.array_equal(a, b)
    # the reference's shape rule: a [1] index vector drops the axis, any other shape replaces it
    assert O.gather_shape((4, 9, 6), (1,), 1) == (4, 6)
    assert O.gather_shape((4, 9, 6), (3, 2), 1) == (4, 3, 2, 6)
    assert O.gather_shape((4, 9, 6), (1, 1), 1) == (4, 1, 1, 6)


def test_layernorm_stats_consistent_with_layernorm():
    rng = np.random.default_rng(78)
    x = rng.standard_normal((6, 5, 40)) * 3 + 1
    g = rng.standard_normal((5, 40)); b = rng.standard_normal((5, 40))
    mean, rstd = O.layernorm_stats_f64(x, 1, 1e-5)
    assert mean.shape == rstd.shape == (6,)
    y = g * ((x - mean[:, None, None]) * rstd[:, None, None]) + b
    assert O.rel_fro(y, O.layernorm_f64(x, g, b, 1, 1e-5)) < 1e-14
    assert np.array_equal(O.transpose_last2(np.arange(6).reshape(1, 2, 3)), np.array([[[0, 3], [1, 4], [2, 5]]]))
