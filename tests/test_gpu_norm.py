"""Parity of the CUDA RMSNorm kernels (forward, fused forward+quantise, backward) with the
CPU oracle.

Tolerances.  The row variance is a float32 reduction whose order differs between any two
implementations, so `rnorm` may differ from the oracle's in the last bits; the tests
therefore (a) bound |rnorm - oracle| by 2 ulp and (b) demand BIT-EXACT outputs against the
oracle evaluated with the kernel's own rnorm.  The backward's two row/column sums are
float32 reductions too: dx may differ by one bf16 ulp on a small fraction of elements
(bound: 1 ulp + 2^-14 RMS for cancelled values, < 1 % of elements), dgamma by 2^-7 relative (one bf16 ulp) of its RMS.
"""
import numpy as np
import pytest
import torch

from oracle import fp8_oracle as fo
from oracle import norm_oracle as no
from tests.gpu_util import BF16, f8_bytes, from_torch_bf16, normal_bf16, to_torch_bf16

pytestmark = pytest.mark.gpu


def _ulp_diff_f32(a, b):
    return np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))


def _inputs(shape, seed, eps):
    rng = np.random.default_rng(seed)
    x = normal_bf16(rng, shape, outlier_p=1e-3)
    gamma = (1.0 + 0.1 * rng.standard_normal(shape[-1])).astype(BF16)   # never uniform: hides index bugs
    return x, gamma


@pytest.mark.parametrize("shape", [(5, 128), (3, 20, 256), (33, 768), (100, 1024), (64, 2048), (17, 4096), (9, 8192)])
@pytest.mark.parametrize("pure", [False, True])
def test_forward_bit_exact_given_rnorm(shape, pure):
    from train_gpt_b200 import ops
    eps = 1e-6
    x, gamma = _inputs(shape, 11, eps)
    y, rn = ops.rmsnorm_fwd(to_torch_bf16(x), to_torch_bf16(gamma), eps, pure=pure, want_rnorm=True)
    rn = rn.cpu().numpy()[..., None]
    assert _ulp_diff_f32(rn, no.rnorm_of(x, eps)).max() <= 2
    ref = (no.rms_norm_pure if pure else no.rms_norm)(x, gamma, eps, rnorm=rn)
    assert np.array_equal(from_torch_bf16(y).view(np.uint16), ref.view(np.uint16))


def test_pure_norm_matches_reference_vectors(golden):
    from train_gpt_b200 import kernels
    x = np.asarray(golden["norm_x"]).view(BF16)
    gamma = np.asarray(golden["norm_gamma"]).view(BF16)
    y = kernels._rms_norm_pure(to_torch_bf16(x), to_torch_bf16(gamma), float(golden["norm_eps"]))
    got = from_torch_bf16(y).view(np.uint16)
    # the fixture's rnorm comes from a float64 variance; allow the rare last-bit rnorm flip
    assert (got != golden["norm_pure_y"]).mean() < 2e-3
    d = np.abs(got.view(BF16).astype(np.float32) - np.asarray(golden["norm_pure_y"]).view(BF16).astype(np.float32))
    assert (d <= 2.0 ** -7 * np.abs(got.view(BF16).astype(np.float32)) + 1e-30).all()


@pytest.mark.parametrize("shape", [(5, 128), (3, 20, 256), (100, 1024), (64, 2048), (9, 8192), (7, 384)])
@pytest.mark.parametrize("pure", [False, True])
def test_fused_norm_quant_bit_exact_given_rnorm(shape, pure):
    from train_gpt_b200 import ops
    eps = 1e-6
    x, gamma = _inputs(shape, 13, eps)
    q, s, y, rn = ops.rmsnorm_quant_fwd(to_torch_bf16(x), to_torch_bf16(gamma), eps, pure=pure, want_y=True, want_rnorm=True)
    rn = rn.cpu().numpy()[..., None]
    assert _ulp_diff_f32(rn, no.rnorm_of(x, eps)).max() <= 2
    q_ref, s_ref, y_ref = no.rmsnorm_quant(x, gamma, eps, rnorm=rn, pure=pure)
    assert np.array_equal(from_torch_bf16(y).view(np.uint16), y_ref.view(np.uint16))
    assert np.array_equal(f8_bytes(q), q_ref.view(np.uint8))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    # against the oracle's own rnorm: byte match rate (reported, loosely bounded)
    q_own, s_own, _ = no.rmsnorm_quant(x, gamma, eps, pure=pure)
    assert (f8_bytes(q) != q_own.view(np.uint8)).mean() < 5e-3
    # without the optional outputs the bytes are the same
    q2, s2, y2, rn2 = ops.rmsnorm_quant_fwd(to_torch_bf16(x), to_torch_bf16(gamma), eps, pure=pure)
    assert y2 is None and rn2 is None and torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s2, s)


def test_fused_equals_norm_then_quantise_kernels():
    """The fused kernel against the two-kernel composition on a config-1-sized input."""
    from train_gpt_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(32768, 2048, device="cuda", generator=g)
    x = torch.where(torch.rand(x.shape, device="cuda", generator=g) < 1e-3, x * 50, x).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(2048, device="cuda", generator=g)).to(torch.bfloat16)
    q, s, _, _ = ops.rmsnorm_quant_fwd(x, gamma, 1e-6)
    y = ops.rmsnorm_fwd(x, gamma, 1e-6)
    q2, s2 = ops.quantize_rowwise(y)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)


@pytest.mark.parametrize("shape", [(5, 128), (3, 20, 256), (33, 768), (700, 1024), (40, 1280), (50, 1792), (3000, 2048),
                                   (17, 4096), (9, 8192)])
def test_backward(shape):
    from train_gpt_b200 import ops
    eps = 1e-5
    x, gamma = _inputs(shape, 17, eps)
    gy = normal_bf16(np.random.default_rng(3), shape)
    dx, dgamma = ops.rmsnorm_bwd(to_torch_bf16(x), to_torch_bf16(gamma), to_torch_bf16(gy), eps)
    dx_ref, dgamma_ref = no.rms_norm_bwd(x, gamma, gy, eps)
    a, b = from_torch_bf16(dx).astype(np.float32), dx_ref.astype(np.float32)
    # one bf16 ulp, plus the float32 cancellation error of gs - normed*dot on near-zero results
    tol = np.abs(b) * 2.0 ** -7 + np.sqrt(np.mean(b * b)) * 2.0 ** -14
    assert (np.abs(a - b) <= tol).all() and (a != b).mean() < 1e-2
    dg, dg_ref = from_torch_bf16(dgamma).astype(np.float32), dgamma_ref.astype(np.float32)
    assert np.abs(dg - dg_ref).max() <= 2.0 ** -7 * np.sqrt(np.mean(dg_ref ** 2)) + 2.0 ** -7 * np.abs(dg_ref).max()


@pytest.mark.parametrize("shape", [(5, 128), (3, 20, 256), (33, 768), (700, 1024), (40, 1280), (300, 2048)])
@pytest.mark.parametrize("pure", [False, True])
def test_residual_add_folded_into_the_norm(shape, pure):
    """tg_add_rmsnorm_quant_fwd: the sum equals the elementwise bf16 add bit for bit, and every other output
    equals tg_rmsnorm_quant_fwd of that sum bit for bit; without a quantised consumer only y is produced."""
    from train_gpt_b200 import ops
    eps = 1e-5
    x, gamma = _inputs(shape, 23, eps)
    res = normal_bf16(np.random.default_rng(5), shape, std=0.3)
    xt, rt, gt = to_torch_bf16(x), to_torch_bf16(res), to_torch_bf16(gamma)
    s, q, sc, y = ops.add_rmsnorm_quant_fwd(xt, rt, gt, eps, pure=pure)
    s_ref = xt + rt
    assert torch.equal(s.view(torch.int16), s_ref.view(torch.int16))
    q2, sc2, y2, _ = ops.rmsnorm_quant_fwd(s_ref, gt, eps, pure=pure, want_y=True)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(sc, sc2)
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    s3, q3, sc3, y3 = ops.add_rmsnorm_quant_fwd(xt, rt, gt, eps, pure=pure, want_q=False)
    assert q3 is None and sc3 is None and torch.equal(y3.view(torch.int16), y2.view(torch.int16))
    assert torch.equal(s3.view(torch.int16), s_ref.view(torch.int16))
    with pytest.raises(ValueError):
        ops.add_rmsnorm_quant_fwd(xt, rt, gt, eps, want_q=False, want_y=False)


def test_residual_add_rejects_wide_rows():
    from train_gpt_b200 import ops
    x = torch.zeros((4, 4096), dtype=torch.bfloat16, device="cuda")
    g = torch.ones((4096,), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.add_rmsnorm_quant_fwd(x, x, g, 1e-5)
    with pytest.raises(ValueError):
        ops.rmsnorm_bwd(x, g, x, 1e-5, addend=x)


@pytest.mark.parametrize("shape", [(5, 128), (3, 20, 256), (33, 768), (700, 1024), (40, 1280), (3000, 2048)])
def test_backward_with_the_skip_gradient_added(shape):
    """tg_rmsnorm_bwd_add: dgamma bit-equal to tg_rmsnorm_bwd; dx = bf16(addend + the unrounded input gradient),
    i.e. within half a bf16 ulp (of the sum) plus the plain kernel's own tolerance of addend + oracle dx."""
    from train_gpt_b200 import ops
    eps = 1e-5
    x, gamma = _inputs(shape, 17, eps)
    gy = normal_bf16(np.random.default_rng(3), shape)
    ad = normal_bf16(np.random.default_rng(4), shape, std=0.5)
    xt, gt, gyt, adt = to_torch_bf16(x), to_torch_bf16(gamma), to_torch_bf16(gy), to_torch_bf16(ad)
    dx_plain, dgamma_plain = ops.rmsnorm_bwd(xt, gt, gyt, eps)
    dx, dgamma = ops.rmsnorm_bwd(xt, gt, gyt, eps, addend=adt)
    assert torch.equal(dgamma.view(torch.int16), dgamma_plain.view(torch.int16))
    dx_ref, _ = no.rms_norm_bwd(x, gamma, gy, eps)
    want = ad.astype(np.float32) + dx_ref.astype(np.float32)
    got = from_torch_bf16(dx).astype(np.float32)
    b = dx_ref.astype(np.float32)
    tol = np.abs(want) * 2.0 ** -8 + np.abs(b) * 2.0 ** -7 + np.sqrt(np.mean(b * b)) * 2.0 ** -14
    assert (np.abs(got - want) <= tol).all()
    # and against the two-launch composition on the device: the same value up to the extra rounding of dx
    two = from_torch_bf16(adt + dx_plain).astype(np.float32)
    assert (np.abs(got - two) <= np.abs(two) * 2.0 ** -7 + np.abs(b) * 2.0 ** -8 + 1e-30).all()


def test_backward_matches_reference_vectors_and_autograd(golden):
    from train_gpt_b200 import kernels
    x = to_torch_bf16(np.asarray(golden["norm_x"]).view(BF16)).requires_grad_(True)
    gamma = to_torch_bf16(np.asarray(golden["norm_gamma"]).view(BF16)).requires_grad_(True)
    gy = to_torch_bf16(np.asarray(golden["norm_gy"]).view(BF16))
    y = kernels.rms_norm(x, gamma, float(golden["norm_eps"]))
    y.backward(gy)
    dx = from_torch_bf16(x.grad).astype(np.float32)
    ref = np.asarray(golden["norm_dx"]).view(BF16).astype(np.float32)
    assert (np.abs(dx - ref) <= np.abs(ref) * 2.0 ** -7 + 1e-30).all() and (dx != ref).mean() < 1e-2
    dg = from_torch_bf16(gamma.grad).astype(np.float32)
    dg_ref = np.asarray(golden["norm_dgamma"]).view(BF16).astype(np.float32)
    assert np.abs(dg - dg_ref).max() <= 2.0 ** -6 * np.abs(dg_ref).max()
    assert x.grad.dtype == torch.bfloat16 and gamma.grad.shape == (256,)
