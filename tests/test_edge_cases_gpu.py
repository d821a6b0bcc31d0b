"""Empty inputs are accepted (nothing is launched) and malformed calls return a status with a
message instead of faulting: every entry point of the C ABI, called directly."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def lib():
    from kernelcodegen_b200 import _lib
    return _lib


def test_empty_inputs_return_ok():
    L = lib()
    l = L.load()
    ops = __import__("kernelcodegen_b200.ops", fromlist=["ops"])
    e = torch.empty((0, 64), dtype=torch.bfloat16, device="cuda")
    g = torch.ones(64, dtype=torch.bfloat16, device="cuda")
    assert ops.layernorm(e, g, g, 1).shape == (0, 64)
    assert ops.elementwise(e, "Gelu").shape == (0, 64)
    assert ops.binary(e, e, "Add").shape == (0, 64)
    assert ops.binary(e, g, "Mul").shape == (0, 64)
    assert ops.softmax(e).shape == (0, 64)
    assert ops.transpose(e).shape == (64, 0)
    idx = torch.empty((0,), dtype=torch.int64, device="cuda")
    assert ops.gather(torch.ones((5, 8), device="cuda"), idx, 0).shape == (0, 8)
    A0 = torch.empty((0, 64), dtype=torch.bfloat16, device="cuda")
    B = torch.ones((64, 128), dtype=torch.bfloat16, device="cuda")
    assert ops.matmul(A0, B).shape == (0, 128)
    assert ops.matmul(torch.ones((128, 64), dtype=torch.bfloat16, device="cuda"),
                      torch.empty((64, 0), dtype=torch.bfloat16, device="cuda")).shape == (128, 0)
    q0 = torch.empty((0, 2, 128, 128), dtype=torch.bfloat16, device="cuda")
    assert ops.fmha(q0, q0, q0).shape == (0, 2, 128, 128)
    torch.cuda.synchronize()
    assert L.device_status() == 0


def test_malformed_calls_report_a_status():
    L = lib()
    l = L.load()
    x = torch.ones((4, 64), dtype=torch.bfloat16, device="cuda")
    p = x.data_ptr()
    st = (ctypes.c_int64 * 3)(64, 64, 64)
    sh = (ctypes.c_int64 * 2)(4, 64)
    cases = [
        (l.kcg_layernorm(L.BF16, 4, 64, None, p, p, 1e-5, p, None), L.ERR_INVALID_ARG),
        (l.kcg_layernorm(L.BF16, -1, 64, p, p, p, 1e-5, p, None), L.ERR_INVALID_ARG),
        (l.kcg_layernorm(L.I32, 4, 64, p, p, p, 1e-5, p, None), L.ERR_UNSUPPORTED),
        (l.kcg_layernorm_stats(L.BF16, 4, 64, p, None, None, 1e-5, p, None, None, None), L.ERR_INVALID_ARG),
        (l.kcg_eltwise(99, L.BF16, L.BF16, 8, p, p, None), L.ERR_INVALID_ARG),
        (l.kcg_eltwise(L.UNARY_OPS["Gelu"], L.BF16, L.F32, 8, p, p, None), L.ERR_INVALID_ARG),
        (l.kcg_binary(L.BINARY_OPS["Add"], L.BF16, 2, sh, 2, (ctypes.c_int64 * 2)(3, 64), p, p, p, None), L.ERR_INVALID_ARG),
        (l.kcg_softmax(L.BF16, 4, 64, 1.0, 0, 4, None, p, None), L.ERR_INVALID_ARG),
        (l.kcg_gemm(L.BF16, L.BF16, 4, 64, 0, 1, 0, 0, p, 64, 0, p, 64, 0, p, 64, 0, None, None, None), L.ERR_INVALID_ARG),
        (l.kcg_gemm(L.BF16, L.BF16, 4, 64, 64, 1, 0, 0, p, 8, 0, p, 64, 0, p, 64, 0, None, None, None), L.ERR_INVALID_ARG),
        (l.kcg_gemm(L.BF16, L.BF16, 4, 64, 64, 1, 0, 0, p + 2, 64, 0, p, 64, 0, p, 64, 0, None, None, None), L.ERR_ALIGNMENT),
        (l.kcg_gemm(L.I32, L.I32, 4, 64, 64, 1, 0, 0, p, 64, 0, p, 64, 0, p, 64, 0, None, None, None), L.ERR_UNSUPPORTED),
        (l.kcg_fmha_fwd(L.BF16, 1, 1, 4, 4, 96, 1.0, 0, p, st, p, st, p, st, p, st, None), L.ERR_UNSUPPORTED),
        (l.kcg_fmha_fwd(L.F32, 1, 1, 4, 4, 64, 1.0, 0, p, st, p, st, p, st, p, st, None), L.ERR_UNSUPPORTED),
        (l.kcg_gather(L.BF16, L.F32, 1, 4, 64, 2, p, p, p, None), L.ERR_UNSUPPORTED),
        (l.kcg_transpose(L.BF16, 1, 4, 64, p, p, None), L.ERR_INVALID_ARG),
        (l.kcg_peer_alloc(0, None), L.ERR_INVALID_ARG),
    ]
    for i, (got, want) in enumerate(cases):
        assert got == want, f"case {i}: status {got}, expected {want}: {l.kcg_last_error().decode()}"
        assert l.kcg_last_error()      # a message was recorded
    assert l.kcg_status_string(L.ERR_TIMEOUT) == b"device-side wait timed out"
    torch.cuda.synchronize()
    assert L.device_status() == 0


def test_device_utilities():
    L = lib()
    l = L.load()
    n = ctypes.c_int(-1)
    assert l.kcg_device_count(ctypes.byref(n)) == 0 and n.value >= 1
    p = ctypes.c_void_p()
    assert l.kcg_peer_alloc(1 << 20, ctypes.byref(p)) == 0 and p.value
    t = ctypes.c_void_p()
    assert l.kcg_timer_begin(None, ctypes.byref(t)) == 0
    assert l.kcg_device_memset(p, 0x5a, 1 << 20, None) == 0
    ms = ctypes.c_float(-1.0)
    assert l.kcg_timer_end(None, t, ctypes.byref(ms)) == 0 and ms.value >= 0.0
    h = ctypes.create_string_buffer(64)
    assert l.kcg_peer_export(p, h) == 0 and any(h.raw)
    assert l.kcg_peer_free(p) == 0


def test_bounded_wait_gives_up_and_context_survives():
    # a barrier nobody signals: the wait must run out of its budget, report a status and return
    L = lib()
    l = L.load()
    waited = torch.zeros(1, dtype=torch.int64, device="cuda")
    assert l.kcg_selftest_bounded_wait(2_000_000, waited.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert L.device_status() == L.ERR_TIMEOUT
    assert L.device_status() == 0                      # reading clears it
    assert 2_000_000 <= int(waited.item()) < 50_000_000   # gave up after the budget, well before 50 ms
    # the context is intact: an ordinary kernel runs and is correct afterwards
    from kernelcodegen_b200 import ops
    x = torch.randn(64, 256, device="cuda").bfloat16()
    assert torch.equal(ops.elementwise(x, "Relu"), torch.relu(x))
    assert l.kcg_selftest_bounded_wait(0, waited.data_ptr(), None) == L.ERR_INVALID_ARG


_SCRATCH_SCRIPT = r"""
import sys, torch
sys.path.insert(0, sys.argv[1])
from kernelcodegen_b200 import _lib, ops
lib = _lib.load()
dt = torch.bfloat16
def ln(x, g, b, y):
    return lib.kcg_layernorm(_lib.BF16, x.shape[0], x.shape[1], x.data_ptr(), g.data_ptr(), b.data_ptr(), 1e-5,
                             y.data_ptr(), torch.cuda.current_stream().cuda_stream)
# rows of 1001 elements are not a whole number of 16-byte vectors: the split-row kernels run and
# keep per-chunk statistics in the library's scratch buffer (1 MiB is the smallest it allocates)
xs = torch.randn(64, 1001, device="cuda").to(dt); gs = torch.ones(1001, device="cuda", dtype=dt); bs = torch.zeros_like(gs)
ys = torch.empty_like(xs)
assert ln(xs, gs, bs, ys) == 0                       # first call: allocates the buffer
want_small = ys.clone()
side = torch.cuda.Stream()
g1 = torch.cuda.CUDAGraph()
with torch.cuda.graph(g1, stream=side):
    assert ln(xs, gs, bs, ys) == 0                   # fits the buffer: may be captured
# 65535 rows of three chunks need more than 1 MiB of statistics
xb = torch.randn(65535, 16387, device="cuda", dtype=dt); gb = torch.ones(16387, device="cuda", dtype=dt); bb = torch.zeros_like(gb)
yb = torch.empty_like(xb)
g2 = torch.cuda.CUDAGraph()
with torch.cuda.graph(g2, stream=side):
    rc = ln(xb, gb, bb, yb)                          # would have to grow inside the capture: refused
    msg = lib.kcg_last_error().decode()
    assert ln(xs, gs, bs, ys) == 0                   # the capture itself is still valid
assert rc == _lib.ERR_UNSUPPORTED and "captured" in msg, (rc, msg)
assert ln(xb, gb, bb, yb) == 0                       # outside a capture the buffer grows
torch.cuda.synchronize()
ref = torch.nn.functional.layer_norm(xb[:64].float(), (16387,), gb.float(), bb.float(), 1e-5)
assert (yb[:64].float() - ref).norm() / ref.norm() < 1e-2
# the graph captured before the growth still names the old buffer, which must still exist
ys.zero_()
g1.replay(); g2.replay()
torch.cuda.synchronize()
assert torch.equal(ys, want_small)
assert _lib.device_status() == 0
print("scratch rules ok")
"""


def test_scratch_buffer_is_never_freed_and_never_grows_inside_a_capture():
    """Run in a fresh process so that the library's scratch buffer starts unallocated."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, "-c", _SCRATCH_SCRIPT, str(root)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "scratch rules ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
