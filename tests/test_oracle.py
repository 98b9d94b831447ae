"""The CPU oracle against the reference's own vectors (tests/golden/) and known answers."""
import ml_dtypes
import numpy as np
import pytest

from oracle import fp8_oracle as fo
from oracle import norm_oracle as no

BF16 = ml_dtypes.bfloat16
F8 = ml_dtypes.float8_e4m3fn


def bf(u16):
    return np.asarray(u16).view(BF16)


def test_quantiser_matches_reference_vectors(golden):
    x = bf(golden["q_act_in"]).astype(np.float32)
    q, s = fo.quantize_to_fp8(x, 128)
    assert np.array_equal(q.view(np.uint8), golden["q_act_bytes"])
    assert np.array_equal(s.view(np.uint32), golden["q_act_scales"].view(np.uint32))
    # the edge tiles planted by the generator
    assert s[3, 1] == np.float32(1e-30) and not q.view(np.uint8)[3, 128:256].any()
    assert s[4, 0] == np.float32(1e-30)
    assert q.view(np.uint8)[6, 7] == 0x80


def test_weight_quantiser_is_colwise_of_b(golden):
    b = bf(golden["q_w_in"]).astype(np.float32)
    q, s = fo.quantize_colwise(b, 128)            # (K,N), (K/128,N)
    assert np.array_equal(q.view(np.uint8).T, golden["q_wt_bytes"])
    assert np.array_equal(s.T.view(np.uint32), np.ascontiguousarray(golden["q_wt_scales"]).view(np.uint32))
    qt, st = fo.quantize_to_fp8(b.T, 128)
    assert np.array_equal(qt.view(np.uint8), golden["q_wt_bytes"])


def test_ones_known_answer(golden):
    # debug_fp8.py:105-109: amax 1 -> scale 1/448, every byte 0x7E (=448), product exactly 128
    q, s = fo.quantize_to_fp8(np.ones((4, 128), np.float32))
    assert np.array_equal(q.view(np.uint8), golden["q_ones_bytes"]) and (q.view(np.uint8) == 0x7E).all()
    assert np.array_equal(s, golden["q_ones_scales"]) and (s == np.float32(1) / np.float32(448)).all()
    y = fo.block_scaled_matmul(np.ones((4, 128), BF16), np.ones((128, 4), BF16))
    assert (y.astype(np.float32) == 128.0).all()


def test_e4m3_rounding_table():
    v = np.array([448.00003, 464.0, 465.0, 2.0 ** -10, 2.0 ** -9, -0.0, np.nan], np.float32).astype(F8).view(np.uint8)
    assert list(v[:6]) == [0x7E, 0x7E, 0x7F, 0x00, 0x01, 0x80] and (v[6] & 0x7F) == 0x7F


def test_ste_backward_matches_reference_vectors(golden):
    a, g, b = bf(golden["ste_a"]), bf(golden["ste_g"]), bf(golden["q_w_in"])
    da, db = fo.backward_bf16_ste(a, b, g)
    assert np.array_equal(da.view(np.uint16), golden["ste_da"])
    assert np.array_equal(db.view(np.uint16), golden["ste_db"])


def test_pure_norm_matches_reference_vectors(golden):
    x, gamma = bf(golden["norm_x"]), bf(golden["norm_gamma"])
    y = no.rms_norm_pure(x, gamma, float(golden["norm_eps"]))
    assert np.array_equal(y.view(np.uint16), golden["norm_pure_y"])
    # the single-rounding (Pallas-kernel) form agrees with it to bf16 rounding
    y2 = no.rms_norm(x, gamma, float(golden["norm_eps"])).astype(np.float32)
    assert np.max(np.abs(y2 - y.astype(np.float32)) / (np.abs(y2) + 1e-3)) < 2.0 ** -6


def test_norm_backward_matches_reference_vectors(golden):
    x, gamma, gy = bf(golden["norm_x"]), bf(golden["norm_gamma"]), bf(golden["norm_gy"])
    dx, dgamma = no.rms_norm_bwd(x, gamma, gy, float(golden["norm_eps"]))
    assert np.array_equal(dx.view(np.uint16), golden["norm_dx"])
    assert np.array_equal(dgamma.view(np.uint16), golden["norm_dgamma"])


def test_shape_errors_follow_reference():
    with pytest.raises(ValueError, match="contracted-dim mismatch"):
        fo.block_scaled_matmul(np.zeros((2, 128), BF16), np.zeros((256, 4), BF16))
    with pytest.raises(ValueError, match="not divisible by block_k"):
        fo.block_scaled_matmul(np.zeros((2, 192), BF16), np.zeros((192, 4), BF16))


def test_nan_and_inf_propagate_like_jnp_max():
    x = np.ones((1, 256), np.float32)
    x[0, 5] = np.nan
    x[0, 130] = np.inf
    q, s = fo.quantize_to_fp8(x)
    assert np.isnan(s[0, 0]) and np.isinf(s[0, 1])
    b = q.view(np.uint8)
    assert ((b[0, :128] & 0x7F) == 0x7F).all()          # whole tile NaN
    assert (b[0, 130] & 0x7F) == 0x7F and not b[0, 131]  # inf/inf NaN, finite/inf 0


def test_block2d_and_fp8_backward_are_close_to_ste():
    rng = np.random.default_rng(1)
    a = rng.standard_normal((200, 256)).astype(BF16)     # ragged token count for wgrad
    b = (rng.standard_normal((256, 384)) * 0.02).astype(BF16)
    g = rng.standard_normal((200, 384)).astype(BF16)
    da_ref, db_ref = fo.backward_bf16_ste(a, b, g)
    for tile in [(128, 1), (128, 128)]:
        da, db = fo.backward_fp8(a, b, g, weight_tile=tile)
        assert fo.rel_frobenius(da, da_ref) < 0.06 and fo.rel_frobenius(db, db_ref) < 0.06
        y = fo.block_scaled_matmul(a, b, weight_tile=tile)
        y_ref = a.astype(np.float64) @ b.astype(np.float64)
        assert fo.rel_frobenius(y, y_ref) < 0.05


def test_rmsnorm_quant_composition():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((5, 7, 256)).astype(BF16)
    gamma = (1 + 0.1 * rng.standard_normal(256)).astype(BF16)
    q, s, y = no.rmsnorm_quant(x, gamma, 1e-6)
    q2, s2 = fo.quantize_to_fp8(no.rms_norm(x, gamma, 1e-6).astype(np.float32))
    assert np.array_equal(q.view(np.uint8), q2.view(np.uint8)) and np.array_equal(s, s2)
    assert q.shape == x.shape and s.shape == (5, 7, 2)


def test_loss_oracle_matches_the_reference_fixture(golden):
    """losses.py:8-12 executed from the reference's source on capped logits."""
    from oracle import loss_oracle as lo
    z = golden["ce_logits"].view(fo.BF16)
    loss, nll, lse = lo.cross_entropy(z, golden["ce_targets"])
    assert abs(float(loss) - float(golden["ce_loss"])) <= 2e-6 * abs(float(golden["ce_loss"]))
    assert nll.shape == (z.shape[0],) and np.all(nll > 0)


def test_softcap_restatement_properties():
    """model.py:97 op by op in bf16: odd, bounded by the cap, identity-like near zero."""
    from oracle import loss_oracle as lo
    bits = np.arange(0, 0x7F80, dtype=np.uint16)                     # every finite non-negative bf16
    x = bits.view(fo.BF16)
    z, t = lo.softcap(x, 15.0)
    zn, _ = lo.softcap((-x.astype(np.float32)).astype(fo.BF16), 15.0)
    assert np.array_equal(z.view(np.uint16) ^ 0x8000, zn.view(np.uint16))
    zf = z.astype(np.float32)
    assert zf.max() == 15.0 and np.all(np.diff(zf) >= 0)
    small = (x.astype(np.float32) < 0.05) & (x.astype(np.float32) > 1e-30)     # subnormals lose bits in x / cap
    assert np.allclose(zf[small], x.astype(np.float32)[small], rtol=2 ** -7, atol=0)


def test_loss_gradient_restatement_against_finite_differences():
    from oracle import loss_oracle as lo
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((6, 64)) * 4).astype(fo.BF16)
    tg = rng.integers(0, 64, size=6)
    g = lo.softcap_cross_entropy_grad(x, tg, 15.0)
    assert np.allclose(g.sum(axis=1) * 0, 0) and g.shape == x.shape
    # the analytic gradient of the SMOOTH function (no bf16 rounding) agrees to rounding level
    xs = x.astype(np.float64)
    z = 15.0 * np.tanh(xs / 15.0)
    p = np.exp(z - z.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
    p[np.arange(6), tg] -= 1
    smooth = p * (1 - np.tanh(xs / 15.0) ** 2) / 6
    assert np.allclose(g, smooth, rtol=0.05, atol=2e-3)


def test_activation_oracle_known_answers_and_derivatives():
    """model.py:72 (`jax.nn.relu(h) ** 2`) worked by hand, its cotangent, and the GELU restatement
    against central differences of its own float64 forward."""
    from oracle import act_oracle as ao
    h = np.array([-3.0, -0.0, 0.0, 0.5, 1.5, 3.0, 255.0], np.float32).astype(fo.BF16)
    assert np.array_equal(ao.relu2(h).astype(np.float32), [0, 0, 0, 0.25, 2.25, 9, 65024.0])   # 255^2 = 65025 -> bf16
    g = np.array([1, 1, 1, -2, 0.5, 3, 1], np.float32).astype(fo.BF16)
    assert np.array_equal(ao.relu2_bwd(h, g).astype(np.float32), [0, 0, 0, -2, 1.5, 18, 510])
    x = np.linspace(-6, 6, 97).astype(np.float32).astype(fo.BF16)
    y = ao.gelu(x).astype(np.float32)
    xf = x.astype(np.float64)
    assert abs(y[48]) == 0 and np.all(y[xf > 5] == x.astype(np.float32)[xf > 5]) and np.all(np.abs(y[xf < -5.5]) < 1e-6)
    from scipy.special import erf
    f = lambda t: t * 0.5 * (1 + erf(t / np.sqrt(2)))
    num = (f(xf + 1e-6) - f(xf - 1e-6)) / 2e-6
    d = ao.gelu_bwd(x, np.ones_like(x)).astype(np.float64)
    assert np.allclose(d, num, rtol=2 ** -7, atol=2 ** -9)
    for name in ao.ACTS:
        assert ao.apply(name, x, x).dtype == fo.BF16
