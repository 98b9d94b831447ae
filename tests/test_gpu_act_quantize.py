"""The activation folded into the row+column quantiser (tg_act_quantize_rowcol) against the CPU
oracle: squared ReLU (model.py:72) and its cotangent bit-exact; GELU within one bf16 ulp of the
float64 value on a small fraction of elements, and equal to the unfused GPU composition."""
import numpy as np
import pytest
import torch

from oracle import act_oracle as ao
from oracle import fp8_oracle as fo
from tests.gpu_util import BF16, f8_bytes, normal_bf16, to_torch_bf16

pytestmark = pytest.mark.gpu


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def _inputs(shape, seed):
    rng = np.random.default_rng(seed)
    x = normal_bf16(rng, shape, outlier_p=0.002).astype(np.float32)
    if shape[0] > 4 and shape[1] >= 256:
        x[1, 0:128] = -np.abs(x[1, 0:128])     # relu2: an all-zero tile -> scale 1e-30, bytes 0
        x[2, 128:256] = 0.0
        x[3, 5] = -0.0
    g = normal_bf16(rng, shape, std=0.05)
    return x.astype(BF16), g


def _check_exact(out, y_bf16):
    """Kernel outputs against the oracle's quantisers applied to the oracle's bf16 activation."""
    q_row, s_row, q_col, s_col = out
    y = np.asarray(y_bf16).astype(np.float32)
    qr, sr = fo.quantize_to_fp8(y)
    qc, sc = fo.quantize_colwise(y)
    assert np.array_equal(f8_bytes(q_row), qr.view(np.uint8))
    assert np.array_equal(_bits(s_row.cpu().numpy()), _bits(sr))
    assert np.array_equal(f8_bytes(q_col), qc.view(np.uint8))
    assert np.array_equal(_bits(s_col.cpu().numpy()), _bits(sc))


@pytest.mark.parametrize("shape", [(1, 128), (7, 384), (300, 1024), (1000, 512)])
@pytest.mark.parametrize("act", ["relu2", "relu2_bwd"])
def test_relu2_bit_exact(shape, act):
    from train_gpt_b200 import ops
    x, g = _inputs(shape, seed=shape[0] * 7 + shape[1])
    gate = to_torch_bf16(g) if act.endswith("_bwd") else None
    out = ops.act_quantize_rowcol(to_torch_bf16(x), act, gate)
    _check_exact(out, ao.apply(act, x, g))


def test_relu2_known_answers():
    """Worked by hand: relu(h)**2 of (-3, 0, 1.5, 3) = (0, 0, 2.25, 9); 9/448 is the tile's scale."""
    from train_gpt_b200 import ops
    x = np.zeros((1, 128), np.float32)
    x[0, :4] = [-3.0, 0.0, 1.5, 3.0]
    q_row, s_row, _, _ = ops.act_quantize_rowcol(to_torch_bf16(x), "relu2")
    s = np.float32(9.0) / np.float32(448.0)
    assert s_row.cpu().numpy()[0, 0] == s
    deq = q_row.float().cpu().numpy()[0, :4] * s
    assert deq[0] == 0 and deq[1] == 0 and abs(deq[2] - 2.25) <= 2.25 / 16 and deq[3] == np.float32(448.0) * s


@pytest.mark.parametrize("act", ["gelu", "gelu_bwd"])
def test_gelu_matches_unfused_composition_and_float64(act):
    """(a) Same bytes and scales as torch's elementwise kernel followed by tg_quantize_rowcol -- the
    composition the fused kernel replaces.  (b) Against the float64 oracle: the dequantised row form
    within the quantisation step of the tile (a bf16 ulp flip moves a value by at most one e4m3 step),
    scales equal to 2 float32 ulps on all but a few tiles, >= 99 % of the bytes equal."""
    from train_gpt_b200 import ops
    shape = (515, 1024)
    x, g = _inputs(shape, seed=11)
    xt, gt = to_torch_bf16(x), to_torch_bf16(g)
    out = ops.act_quantize_rowcol(xt, act, gt if act.endswith("_bwd") else None)
    xg = xt.clone().requires_grad_(True)
    y_t = torch.nn.functional.gelu(xg)
    if act == "gelu_bwd":
        (y_t,) = torch.autograd.grad(y_t, xg, gt)
    ref = ops.quantize_rowcol(y_t.detach().contiguous())
    for got, want in zip(out, ref):
        a, b = got.contiguous().view(torch.uint8), want.contiguous().view(torch.uint8)
        assert (a == b).float().mean().item() >= 0.999, "differs from torch gelu + tg_quantize_rowcol"
    y = ao.apply(act, x, g).astype(np.float32)
    qr, sr = fo.quantize_to_fp8(y)
    assert (f8_bytes(out[0]) == qr.view(np.uint8)).mean() >= 0.99
    s_got = out[1].cpu().numpy()
    assert np.mean(np.abs(s_got - sr) <= 2 * np.spacing(sr)) >= 0.99
    deq = out[0].float().cpu().numpy().reshape(shape[0], -1, 128) * s_got[..., None]
    step = np.maximum(np.abs(y).reshape(shape[0], -1, 128) / 8, s_got[..., None] * 2.0 ** -9)   # e4m3: 3 mantissa bits
    assert np.all(np.abs(deq - y.reshape(shape[0], -1, 128)) <= step + 1e-30)


def test_rejects_bad_arguments():
    from train_gpt_b200 import ops
    x = torch.zeros((4, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.act_quantize_rowcol(x, "swish")
    with pytest.raises(ValueError):
        ops.act_quantize_rowcol(x, "gelu_bwd")                      # no gate
    with pytest.raises(ValueError):
        ops.act_quantize_rowcol(torch.zeros((4, 100), dtype=torch.bfloat16, device="cuda"), "relu2")


def test_gelu_every_finite_bf16_argument():
    """All 65280 finite bf16 values, 128 consecutive bit patterns (one binade) per row: the bytes and
    scales of torch's elementwise GELU followed by tg_quantize_rowcol.  The kernel's erf is its own
    (one ex2 and a polynomial, not libdevice's erff); both put it into the float32 form
    x/2 (1 + erf), whose result has no correct digits left once 1 + erf cancels -- below x = -4 a
    rounding error of erf is a relative error of 2^-9 and more in the result.  So: row-tile scales and
    bytes as before, column scales equal for the three row groups above -4, and for the last group
    (x from -4 down) equal for the columns whose largest element has digits, within a factor of 2.5
    for the rest.
    (A range split with a shared-memory table for the erf, bit-identical on this test, measured SLOWER
    than evaluating the function per element -- 1.5 against 2.0 TB/s: random 2-byte table reads
    conflict in the banks -- and was dropped.)"""
    from train_gpt_b200 import ops
    bits = np.concatenate([np.arange(0, 0x7F80), np.arange(0x8000, 0xFF80)]).astype(np.uint16)
    x = to_torch_bf16(bits.view(BF16).reshape(510, 128))
    out = ops.act_quantize_rowcol(x, "gelu")
    ref = ops.quantize_rowcol(torch.nn.functional.gelu(x).contiguous())
    assert torch.equal(out[1], ref[1]), "row-tile scales"
    assert (out[0].view(torch.uint8) == ref[0].view(torch.uint8)).float().mean().item() >= 0.9995
    assert float(x[383, 127]) > -4.0 and float(x[384, 0]) == -4.0            # the fourth group of 128 rows starts at -4
    assert (out[3][:3] == ref[3][:3]).float().mean().item() >= 0.995
    assert (out[3][3] == ref[3][3]).float().mean().item() >= 0.9
    ratio = out[3][3] / ref[3][3]
    assert float(ratio.min()) > 0.4 and float(ratio.max()) < 2.5
