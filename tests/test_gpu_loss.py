"""Capped-logit cross-entropy kernels (tg_softcap_ce_fwd / _bwd) against the CPU oracle.

Tolerances: per-token nll and lse within 2e-6 relative + 2e-6 absolute of the float64 oracle
(the kernel sums exp() in float32); the bf16 tanh values bit-exact except where float32 tanhf
and float64 tanh round differently (bounded below at 99.9 % equal, never more than one bf16
ulp apart); gradients within rtol 2e-2 / atol 1e-2 * RMS, the bar stated for gradients.
"""
import numpy as np
import pytest
import torch

from oracle import fp8_oracle as fo
from oracle import loss_oracle as lo
from tests.gpu_util import from_torch_bf16, to_torch_bf16

pytestmark = pytest.mark.gpu


def _case(rows, vocab, seed, spread=6.0):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((rows, vocab)) * spread).astype(fo.BF16)
    t = rng.integers(0, vocab, size=rows).astype(np.int32)
    return x, t


@pytest.mark.parametrize("rows,vocab,spread", [(7, 512, 6.0), (33, 50304, 3.0), (4, 2056, 40.0),
                                               (5, 50257, 3.0), (3, 12, 2.0), (2, 2049, 6.0)])   # 50257: train-gpt config.py:8
def test_forward_matches_oracle(rows, vocab, spread):
    from train_gpt_b200 import ops
    x, t = _case(rows, vocab, rows + vocab, spread)
    nll, lse, th = ops.softcap_ce_fwd(to_torch_bf16(x), torch.from_numpy(t).cuda(), 15.0)
    z_ref, t_ref = lo.softcap(x, 15.0)
    _, nll_ref, lse_ref = lo.cross_entropy(z_ref, t)
    assert th.shape == (rows, vocab)
    th_bits = from_torch_bf16(th).view(np.uint16).astype(np.int32)
    ref_bits = t_ref.view(np.uint16).astype(np.int32)
    assert np.abs(th_bits - ref_bits).max() <= 1
    assert (th_bits == ref_bits).mean() > 0.999
    assert np.allclose(lse.cpu().numpy(), lse_ref, rtol=2e-6, atol=2e-6)
    assert np.allclose(nll.cpu().numpy(), nll_ref, rtol=2e-5, atol=2e-5)


def test_every_finite_bf16_logit():
    """All 65280 finite bf16 values as logits of one long row: the capped values the kernel
    implies (through lse) and its tanh output follow the oracle over the whole input domain."""
    from train_gpt_b200 import ops
    bits = np.concatenate([np.arange(0, 0x7F80), np.arange(0x8000, 0xFF80)]).astype(np.uint16)
    x = bits.view(fo.BF16).reshape(1, -1)                      # 65280 = 8 * 8160 columns
    t = np.array([12345], dtype=np.int32)
    nll, lse, th = ops.softcap_ce_fwd(to_torch_bf16(x), torch.from_numpy(t).cuda(), 15.0)
    z_ref, t_ref = lo.softcap(x, 15.0)
    _, nll_ref, lse_ref = lo.cross_entropy(z_ref, t)
    d = np.abs(from_torch_bf16(th).view(np.uint16).astype(np.int32) - t_ref.view(np.uint16).astype(np.int32))
    assert d.max() <= 1 and (d == 0).mean() > 0.999
    assert np.allclose(lse.cpu().numpy(), lse_ref, rtol=2e-6) and np.allclose(nll.cpu().numpy(), nll_ref, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("rows,vocab", [(9, 512), (16, 50304), (6, 50257), (5, 12)])
def test_backward_matches_oracle(rows, vocab):
    from train_gpt_b200 import ops
    x, t = _case(rows, vocab, 3 * rows + vocab, 4.0)
    tt = torch.from_numpy(t).cuda()
    _, lse, th = ops.softcap_ce_fwd(to_torch_bf16(x), tt, 15.0)
    gs = torch.tensor([0.75], dtype=torch.float32, device="cuda")
    d = ops.softcap_ce_bwd(th, tt, lse, gs, 15.0)
    th2 = torch.full((rows, th.stride(0)), 7.0, dtype=torch.bfloat16, device="cuda")      # same row pitch, marked padding
    th2[:, :vocab].copy_(th)
    d_inplace = ops.softcap_ce_bwd(th2[:, :vocab], tt, lse, gs, 15.0, in_place=True)
    assert torch.equal(d, d_inplace) and d.shape == (rows, vocab)
    assert bool((th2[:, vocab:] == 7.0).all())                  # nothing is stored past the vocabulary
    ref = lo.softcap_cross_entropy_grad(x, t, 15.0, gscale=0.75)
    got = from_torch_bf16(d).astype(np.float64)
    rms = np.sqrt((ref ** 2).mean())
    assert np.all(np.abs(got - ref) <= 2e-2 * np.abs(ref) + 1e-2 * rms)
    # the target column carries the -1: check it separately, it dominates the row
    assert np.allclose(got[np.arange(rows), t], ref[np.arange(rows), t], rtol=1e-2)


def test_autograd_function_matches_torch_ops():
    """losses.capped_cross_entropy against the op-by-op torch composition of model.py:97 +
    losses.py:9-12 on the same GPU."""
    from train_gpt_b200 import losses
    torch.manual_seed(0)
    logits = (torch.randn(4, 24, 512, device="cuda") * 5).to(torch.bfloat16)
    tg = torch.randint(0, 512, (4, 24), device="cuda")
    a = logits.clone().requires_grad_(True)
    b = logits.clone().requires_grad_(True)
    la = losses.capped_cross_entropy(a, tg, 15.0)
    capped = 15.0 * torch.tanh(b / 15.0)
    lb = torch.nn.functional.cross_entropy(capped.float().view(-1, 512), tg.view(-1))
    (la * 2.0).backward()
    (lb * 2.0).backward()
    assert abs(float(la) - float(lb)) < 2e-5 * abs(float(lb))
    ga, gb = a.grad.float(), b.grad.float()
    rms = gb.pow(2).mean().sqrt()
    assert bool(((ga - gb).abs() <= 2e-2 * gb.abs() + 1e-2 * rms).all())


def test_rejects_bad_arguments():
    from train_gpt_b200 import ops
    with pytest.raises(TypeError):
        ops.softcap_ce_fwd(torch.zeros((2, 16), dtype=torch.bfloat16, device="cuda"),
                           torch.zeros(2, dtype=torch.int64, device="cuda"), 15.0)
    with pytest.raises(ValueError):
        ops.softcap_ce_fwd(torch.zeros((2, 16), dtype=torch.bfloat16, device="cuda"),
                           torch.zeros(2, dtype=torch.int32, device="cuda"), 0.0)          # cap must be positive


def test_reference_default_vocabulary_through_autograd():
    """vocab 50257 (train-gpt config.py:8, not a multiple of 8) through losses.capped_cross_entropy."""
    from train_gpt_b200 import losses
    torch.manual_seed(1)
    logits = (torch.randn(2, 8, 50257, device="cuda") * 4).to(torch.bfloat16)
    tg = torch.randint(0, 50257, (2, 8), device="cuda")
    a = logits.clone().requires_grad_(True)
    b = logits.clone().requires_grad_(True)
    la = losses.capped_cross_entropy(a, tg, 15.0)
    lb = torch.nn.functional.cross_entropy((15.0 * torch.tanh(b / 15.0)).float().view(-1, 50257), tg.view(-1))
    la.backward()
    lb.backward()
    assert abs(float(la) - float(lb)) < 2e-5 * abs(float(lb))
    ga, gb = a.grad.float(), b.grad.float()
    assert ga.shape == gb.shape
    rms = gb.pow(2).mean().sqrt()
    assert bool(((ga - gb).abs() <= 2e-2 * gb.abs() + 1e-2 * rms).all())
