"""Fused attention forward against the float64 oracle (softmax(scale * Q K^T [+mask]) V per
batch and head), through the C ABI.  Tolerance: relative Frobenius error 1e-2 (16-bit
tensor-core path)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.helpers import randn, f64, rel_fro, sync_ok

pytestmark = pytest.mark.gpu


def ops():
    from kernelcodegen_b200 import ops as _ops
    return _ops


CASES = [
    # B, H, Sq, Skv, D
    (1, 1, 128, 128, 128),
    (2, 3, 256, 256, 128),
    (1, 2, 384, 384, 64),
    (2, 2, 200, 200, 128),    # ragged: partial query tile and partial key block
    (1, 2, 128, 520, 128),    # more keys than queries
    (1, 1, 1, 300, 128),      # a single query (decode-like)
    (1, 2, 1024, 1024, 128),  # 8 key blocks: both score buffers and both ring stages wrap
    (2, 2, 700, 900, 128),    # six query tiles (the second group of four half empty), ragged keys
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,Sq,Skv,D", CASES)
def test_fmha_matches_oracle(B, H, Sq, Skv, D, causal, dtype):
    Q = randn((B, H, Sq, D), dtype, 600)
    K = randn((B, H, Skv, D), dtype, 601)
    V = randn((B, H, Skv, D), dtype, 602)
    scale = 1.0 / np.sqrt(D)
    out = ops().fmha(Q.cuda(), K.cuda(), V.cuda(), scale, causal)
    sync_ok()
    want = O.attention_f64(f64(Q), f64(K), f64(V), scale, causal)
    assert out.shape == (B, H, Sq, D)
    assert rel_fro(out, want) <= 1e-2


@pytest.fixture
def variant(request):
    """Selects the attention kernel for the calling thread and restores the default afterwards."""
    from kernelcodegen_b200 import _lib
    lib = _lib.load()
    lib.kcg_fmha_set_p_in_tmem(request.param)
    yield request.param
    lib.kcg_fmha_set_p_in_tmem(-1)


# Every kernel the library ships is held to the same parity bar, not only the one the default
# picks for a shape: 0 / 1 = one query tile per CTA with P through shared / tensor memory (also
# for long sequences), 2 = two query tiles per CTA (also for a single, partly empty tile pair),
# 3 = a CTA pair on four query tiles (also when most of the four are empty), 4 = a CTA pair with one
# tile per CTA whose warpgroups take alternate key blocks (D = 64 runs variant 2 for both), 5 = the
# two-tile kernel as a persistent grid.
@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4, 5], indirect=True)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,Sq,Skv,D", CASES)
def test_fmha_every_variant_matches_oracle(B, H, Sq, Skv, D, causal, dtype, variant):
    Q = randn((B, H, Sq, D), dtype, 600)
    K = randn((B, H, Skv, D), dtype, 601)
    V = randn((B, H, Skv, D), dtype, 602)
    scale = 1.0 / np.sqrt(D)
    out = ops().fmha(Q.cuda(), K.cuda(), V.cuda(), scale, causal)
    again = ops().fmha(Q.cuda(), K.cuda(), V.cuda(), scale, causal)
    sync_ok()
    assert rel_fro(out, O.attention_f64(f64(Q), f64(K), f64(V), scale, causal)) <= 1e-2
    assert torch.equal(out, again)


def test_fmha_reference_semantics_no_scale_no_mask():
    # the reference chain has no scale and no mask (test/test.cc:128-130); D=64 as in its demo
    Q = randn((2, 4, 256, 64), torch.bfloat16, 610, std=0.3)
    K = randn((2, 4, 256, 64), torch.bfloat16, 611, std=0.3)
    V = randn((2, 4, 256, 64), torch.bfloat16, 612)
    out = ops().fmha(Q.cuda(), K.cuda(), V.cuda(), 1.0, False)
    sync_ok()
    assert rel_fro(out, O.attention_f64(f64(Q), f64(K), f64(V), 1.0, False)) <= 1e-2
    # and the reference-faithful fp32 three-call chain agrees with both
    chain = O.ref32.attention(Q.float().numpy(), K.float().numpy(), V.float().numpy(), 1.0, False, threads=0)
    assert O.rel_fro(out.float().cpu().numpy(), chain) <= 1e-2


def test_fmha_bshd_output_and_strided_inputs():
    B, H, S, D = 2, 4, 256, 128
    # inputs stored [B,S,H,D] and viewed as [B,H,S,D]; output requested as [B,S,H,D]
    Q = randn((B, S, H, D), torch.bfloat16, 620)
    K = randn((B, S, H, D), torch.bfloat16, 621)
    V = randn((B, S, H, D), torch.bfloat16, 622)
    Qv, Kv, Vv = (t.cuda().permute(0, 2, 1, 3) for t in (Q, K, V))
    out = ops().fmha(Qv, Kv, Vv, 1.0 / np.sqrt(D), True, out_layout="bshd")
    sync_ok()
    assert out.shape == (B, H, S, D) and out.stride() == (S * H * D, D, H * D, 1)
    want = O.attention_f64(f64(Q.permute(0, 2, 1, 3)), f64(K.permute(0, 2, 1, 3)), f64(V.permute(0, 2, 1, 3)),
                           1.0 / np.sqrt(D), True)
    assert rel_fro(out, want) <= 1e-2


def test_fmha_large_scores_need_rescale():
    # growing score magnitude along the keys forces the running max to move in later blocks
    B, H, S, D = 1, 2, 512, 128
    Q = randn((B, H, S, D), torch.bfloat16, 630)
    K = randn((B, H, S, D), torch.bfloat16, 631)
    ramp = torch.linspace(0.2, 3.0, S).view(1, 1, S, 1)
    K = (K.float() * ramp).to(torch.bfloat16)
    V = randn((B, H, S, D), torch.bfloat16, 632)
    out = ops().fmha(Q.cuda(), K.cuda(), V.cuda(), 0.5, False)
    sync_ok()
    assert rel_fro(out, O.attention_f64(f64(Q), f64(K), f64(V), 0.5, False)) <= 1e-2


def test_fmha_config_shape_sampled():
    # the attention benchmark configuration at S=1024: B=8, H=32, D=128; oracle on a sample of (batch, head) slices
    B, H, S, D = 8, 32, 1024, 128
    g = torch.Generator(device="cuda").manual_seed(640)
    Q, K, V = (torch.randn((B, H, S, D), generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16) for _ in range(3))
    for causal in (False, True):
        out = ops().fmha(Q, K, V, 1.0 / np.sqrt(D), causal)
        sync_ok()
        for (b, h) in [(0, 0), (3, 17), (7, 31)]:
            want = O.attention_f64(f64(Q[b:b + 1, h:h + 1]), f64(K[b:b + 1, h:h + 1]), f64(V[b:b + 1, h:h + 1]),
                                   1.0 / np.sqrt(D), causal)
            assert rel_fro(out[b:b + 1, h:h + 1], want) <= 1e-2


def test_fmha_bitwise_repeatable():
    Q = randn((2, 2, 512, 128), torch.bfloat16, 650).cuda()
    K = randn((2, 2, 512, 128), torch.bfloat16, 651).cuda()
    V = randn((2, 2, 512, 128), torch.bfloat16, 652).cuda()
    a = ops().fmha(Q, K, V, 0.1, True)
    b = ops().fmha(Q, K, V, 0.1, True)
    sync_ok()
    assert torch.equal(a, b)


def test_fmha_rejects_unsupported():
    from kernelcodegen_b200 import _lib
    Q = torch.zeros((1, 1, 128, 96), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.KcgError) as e:
        ops().fmha(Q, Q, Q)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    Q32 = torch.zeros((1, 1, 128, 128), dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.KcgError):
        ops().fmha(Q32, Q32, Q32)


# The persistent kernel with more work items than SMs, so that every CTA walks over several items:
# ragged last tile pair (one tile and an empty one), Sq != Skv, both masks, both head dimensions.
@pytest.mark.parametrize("variant", [5], indirect=True)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("B,H,Sq,Skv,D", [(2, 26, 640, 896, 128), (2, 38, 512, 512, 64), (3, 25, 300, 260, 128)])
def test_fmha_persistent_many_items(B, H, Sq, Skv, D, causal, variant):
    dtype = torch.bfloat16
    Q = randn((B, H, Sq, D), dtype, 610)
    K = randn((B, H, Skv, D), dtype, 611)
    V = randn((B, H, Skv, D), dtype, 612)
    scale = 1.0 / np.sqrt(D)
    out = ops().fmha(Q.cuda(), K.cuda(), V.cuda(), scale, causal)
    again = ops().fmha(Q.cuda(), K.cuda(), V.cuda(), scale, causal)
    sync_ok()
    want = O.attention_f64(f64(Q), f64(K), f64(V), scale, causal)
    assert rel_fro(out, want) <= 1e-2
    assert torch.equal(out, again)
