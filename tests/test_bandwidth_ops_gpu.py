"""Parity of the HBM-bound kernels (LayerNorm, unary, binary, softmax) with the float64
oracle, through the C ABI.  Tolerances are relative Frobenius errors: 1e-5 for float32
storage, 1e-2 for bfloat16 / float16 storage."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import TOL, randn, uniform, f64, rel_fro, sync_ok

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16]


def ops():
    from kernelcodegen_b200 import ops as _ops
    return _ops


# --------------------------------------------------------------------------- LayerNorm
LN_SHAPES = [
    ((64, 4096), 1),       # block-per-row path (the benchmark's row width)
    ((33, 8192), 1),
    ((257, 256), 1),       # warp-per-row path
    ((100, 64), -1),
    ((7, 1000), 1),        # cols % 8 == 0 but not a power of two
    ((5, 1001), 1),        # ragged: not vectorisable -> split-row path
    ((3, 40000), 1),       # longer than one block holds -> split-row path, 5 chunks
    ((2, 96, 96), 1),      # the reference test's shape class: [2,768,768] axis 1, scaled down
    ((4, 6, 128), -1),
    ((1, 8), 1),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,axis", LN_SHAPES)
def test_layernorm(shape, axis, dtype):
    ax = axis if axis >= 0 else axis + len(shape)
    pshape = shape[ax:]
    x = randn(shape, dtype, 100)
    g = randn(pshape, dtype, 101, mean=1.0, std=0.1)
    b = randn(pshape, dtype, 102, std=0.1)
    y = ops().layernorm(x.cuda(), g.cuda(), b.cuda(), axis)
    sync_ok()
    want = O.layernorm_f64(f64(x), f64(g), f64(b), axis)
    assert y.shape == x.shape and y.dtype == dtype
    assert rel_fro(y, want) <= TOL[dtype]


def test_layernorm_reference_test_shape():
    # test/test.cc:28-30: [2,768,768] float32, axis 1, scale/bias [768,768]
    x = randn((2, 768, 768), torch.float32, 110)
    g = randn((768, 768), torch.float32, 111, mean=1.0, std=0.1)
    b = randn((768, 768), torch.float32, 112, std=0.1)
    y = ops().layernorm(x.cuda(), g.cuda(), b.cuda(), 1)
    sync_ok()
    assert rel_fro(y, O.layernorm_f64(f64(x), f64(g), f64(b), 1)) <= 1e-5


def test_layernorm_inplace_and_offset_mean():
    x = randn((129, 2048), torch.float32, 120, mean=50.0, std=0.5)  # large mean: two-pass variance matters
    g = randn((2048,), torch.float32, 121, mean=1.0, std=0.1)
    b = randn((2048,), torch.float32, 122)
    xd = x.cuda()
    y = ops().layernorm(xd, g.cuda(), b.cuda(), 1, inplace=True)
    sync_ok()
    assert y.data_ptr() == xd.data_ptr()
    assert rel_fro(y, O.layernorm_f64(f64(x), f64(g), f64(b), 1)) <= 1e-5


def test_layernorm_broadcast_scale():
    x = randn((4, 12, 64), torch.float32, 130)
    g = randn((12, 1), torch.float32, 131)
    b = randn((64,), torch.float32, 132)
    y = ops().layernorm(x.cuda(), g.cuda(), b.cuda(), 1)
    sync_ok()
    assert rel_fro(y, O.layernorm_f64(f64(x), f64(g), f64(b), 1)) <= 1e-5


def test_layernorm_matches_fp32_nest():
    # the reference-faithful fp32 nest and the kernel see the same fp32 inputs
    x = randn((16, 4096), torch.float32, 140)
    g = randn((4096,), torch.float32, 141, mean=1.0, std=0.1)
    b = randn((4096,), torch.float32, 142, std=0.1)
    y = ops().layernorm(x.cuda(), g.cuda(), b.cuda(), 1)
    sync_ok()
    assert O.rel_fro(y.cpu().numpy(), O.ref32.layernorm(x.numpy(), g.numpy(), b.numpy(), 1)) <= 1e-5


def test_layernorm_empty_and_bad_axis():
    x = torch.empty((0, 16), device="cuda")
    g = torch.ones(16, device="cuda")
    assert ops().layernorm(x, g, g, 1).shape == (0, 16)
    with pytest.raises(ValueError):
        ops().layernorm(torch.ones(4, 4, device="cuda"), g, g, 2)


# --------------------------------------------------------------------------- unary
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", ["Tanh", "Sqrt", "Log", "Relu", "Gelu"])
@pytest.mark.parametrize("n", [1, 7, 4096, 1000003])
def test_unary(op, n, dtype):
    x = randn((n,), dtype, 200, std=2.0)
    if op in ("Sqrt", "Log"):
        x = (x.float().abs() + 0.05).to(dtype)
    y = ops().elementwise(x.cuda(), op)
    sync_ok()
    assert rel_fro(y, O.unary_f64(op, f64(x))) <= TOL[dtype]


def test_unary_gelu_bench_shape_slice():
    x = randn((512, 4096), torch.bfloat16, 210)
    y = ops().elementwise(x.cuda(), "Gelu")
    sync_ok()
    assert rel_fro(y, O.unary_f64("Gelu", f64(x))) <= 1e-2
    # bf16 result should be the correctly rounded value almost everywhere
    want = torch.from_numpy(O.unary_f64("Gelu", f64(x))).to(torch.bfloat16)
    assert (y.cpu() == want).float().mean() > 0.98


def test_unary_unaligned_and_inplace():
    base = randn((4099,), torch.float32, 220).cuda()
    x = base[1:]  # 4-byte aligned only
    y = ops().elementwise(x.contiguous(), "Relu")
    z = torch.empty(4100, device="cuda")[1:4099]
    from kernelcodegen_b200 import _lib
    _lib.check(_lib.load().kcg_eltwise(_lib.UNARY_OPS["Relu"], _lib.F32, _lib.F32, x.numel(), x.data_ptr(),
                                       z.data_ptr(), None), "kcg_eltwise")
    sync_ok()
    want = O.unary_f64("Relu", f64(x))
    assert rel_fro(y, want) == 0 and rel_fro(z, want) == 0
    r = ops().relu(base, inplace=True)
    sync_ok()
    assert r.data_ptr() == base.data_ptr() and float(base.min()) >= 0


@pytest.mark.parametrize("src,dst", [(torch.float32, torch.int32), (torch.float32, torch.bfloat16),
                                     (torch.bfloat16, torch.float32), (torch.float16, torch.float32),
                                     (torch.int32, torch.float32), (torch.float32, torch.float16)])
def test_cast(src, dst):
    # test/test.cc:20-24 casts a [2,768,768] float32 tensor to int32
    if src == torch.int32:
        x = torch.randint(-1000, 1000, (2, 96, 97), generator=torch.Generator().manual_seed(5), dtype=torch.int32)
    else:
        x = randn((2, 96, 97), src, 230, std=20.0)
    y = ops().elementwise(x.cuda(), "Cast", dtype=dst)
    sync_ok()
    assert y.dtype == dst
    assert torch.equal(y.cpu(), x.to(dst))


# --------------------------------------------------------------------------- binary
BIN_SHAPES = [((16, 1, 1, 256), (1, 128, 256)),   # test/test.cc:32-34
              ((64, 4096), (64, 4096)), ((64, 4096), (4096,)), ((33, 7, 5), (7, 1)),
              ((1,), (9, 130)), ((3, 1, 5), (1, 4, 1)), ((10, 1003), (10, 1003)), ((2, 3, 4, 5, 6), (4, 1, 6))]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sa,sb", BIN_SHAPES)
def test_binary_add_mul_sub_div(sa, sb, dtype):
    a = randn(sa, dtype, 300)
    b = (randn(sb, dtype, 301).float().abs() + 0.5).to(dtype)
    for op in ["Add", "Mul", "Sub", "Div"]:
        c = ops().binary(a.cuda(), b.cuda(), op)
        sync_ok()
        want = O.binary_f64(op, f64(a), f64(b))
        assert tuple(c.shape) == want.shape
        assert rel_fro(c, want) <= TOL[dtype], op


def test_binary_compare_and_pow():
    a = randn((40, 130), torch.float32, 310)
    b = a.clone()
    b[::2] += 1.0
    for op in ["Equal", "Greater"]:
        c = ops().binary(a.cuda(), b.cuda(), op)
        sync_ok()
        assert np.array_equal(c.cpu().numpy().astype(np.float64), O.binary_f64(op, f64(a), f64(b)))
    base = (a.abs() + 0.5)
    e = randn((130,), torch.float32, 311)
    c = ops().binary(base.cuda(), e.cuda(), "Pow")
    sync_ok()
    assert rel_fro(c, O.binary_f64("Pow", f64(base), f64(e))) <= 1e-5


def test_binary_matches_fp32_nest_bitwise():
    a = randn((16, 1, 1, 64), torch.float32, 320)
    b = randn((1, 12, 64), torch.float32, 321)
    c = ops().binary(a.cuda(), b.cuda(), "Add")
    sync_ok()
    assert np.array_equal(c.cpu().numpy(), O.ref32.binary("Add", a.numpy(), b.numpy()))


def test_binary_rejects_mismatch_and_inplace():
    with pytest.raises(ValueError):
        ops().binary(torch.ones(4, 5, device="cuda"), torch.ones(4, 3, device="cuda"), "Add")
    a = randn((8, 256), torch.float32, 330).cuda()
    b = randn((256,), torch.float32, 331).cuda()
    want = O.binary_f64("Add", f64(a), f64(b))
    c = ops().binary(a, b, "Add", inplace=True)
    sync_ok()
    assert c.data_ptr() == a.data_ptr() and rel_fro(a, want) <= 1e-6


# --------------------------------------------------------------------------- softmax
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(2, 3, 64, 64), (5, 1000), (1, 2, 17, 333), (16, 4096), (2, 2, 128, 512), (3, 16384),
                                   (2, 3, 40, 2056), (2, 40000)])
@pytest.mark.parametrize("causal", [False, True])
def test_softmax(shape, dtype, causal):
    if causal and len(shape) < 3:
        pytest.skip("causal needs a trailing [q, kv] matrix")
    x = randn(shape, dtype, 400)
    xd = x.cuda()
    y = ops().softmax(xd, -1, scale=0.5, causal=causal)
    sync_ok()
    assert y.data_ptr() == xd.data_ptr()  # in place, like the reference op
    assert rel_fro(y, O.softmax_f64(f64(x), 0.5, causal)) <= TOL[dtype]


def test_softmax_negative_scale_and_out_of_place():
    x = randn((33, 2048), torch.float32, 410)
    y = ops().softmax(x.cuda(), -1, scale=-1.5, inplace=False)
    sync_ok()
    assert rel_fro(y, O.softmax_f64(f64(x), -1.5, False)) <= 1e-5
    assert float((y.sum(-1) - 1).abs().max()) <= 1e-5
