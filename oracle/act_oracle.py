"""CPU oracle for the MLP activation that the fused activation + quantise kernel folds into its load.

TEST INFRASTRUCTURE ONLY -- imported by `tests/` and `__graft_entry__.smoke()`, never by the
shipped package.

Pin status:
* `relu2` and its cotangent restate train-gpt's `model.py:72` (`jax.nn.relu(h) ** 2` on a bf16
  tensor) and the derivative autodiff gives it, `g * 2 * relu(h)`.  Both are exact arithmetic
  followed by ONE rounding to bf16: the product of two bf16 numbers is exact in float32, so every
  evaluation order the reference's compiler may choose gives these bits.  The reference stores no
  outputs of that line and cannot be executed here (no JAX); the known answers in
  `tests/test_oracle.py` are worked by hand.
* `gelu` is NOT in the reference (its MLP is the squared ReLU); the benchmark's training
  configuration names it.  The oracle evaluates the erf form in float64 and rounds once to bf16;
  a float32 implementation may differ by one bf16 ulp on a small fraction of the elements, and the
  tests state that tolerance.  PARITY UNPINNED for gelu.
"""
from __future__ import annotations

import numpy as np
from scipy.special import erf

from .fp8_oracle import BF16, to_bf16

ACTS = ("relu2", "gelu", "relu2_bwd", "gelu_bwd")


def _f32(x):
    return np.asarray(x).astype(BF16).astype(np.float32)


def relu2(x):
    """model.py:72 -- `jax.nn.relu(h) ** 2`, bf16 in, bf16 out."""
    r = np.maximum(_f32(x), np.float32(0))
    return (r * r).astype(BF16)


def relu2_bwd(x, gate):
    """Cotangent of model.py:72 for upstream gradient `gate`: gate * 2 * relu(x), one rounding."""
    r2 = np.float32(2) * np.maximum(_f32(x), np.float32(0))          # exact
    return (_f32(gate).astype(np.float64) * r2.astype(np.float64)).astype(np.float32).astype(BF16)


def gelu(x):
    """x/2 (1 + erf(x / sqrt 2)) in float64, rounded once to bf16."""
    x64 = _f32(x).astype(np.float64)
    return (x64 * 0.5 * (1.0 + erf(x64 / np.sqrt(2.0)))).astype(np.float32).astype(BF16)


def gelu_bwd(x, gate):
    """gate * (Phi(x) + x phi(x)) in float64, rounded once to bf16."""
    x64 = _f32(x).astype(np.float64)
    cdf = 0.5 * (1.0 + erf(x64 / np.sqrt(2.0)))
    pdf = np.exp(-0.5 * x64 * x64) / np.sqrt(2.0 * np.pi)
    return (_f32(gate).astype(np.float64) * (cdf + x64 * pdf)).astype(np.float32).astype(BF16)


def apply(act: str, x, gate=None):
    """The bf16 tensor the fused kernel quantises for activation name `act`."""
    if act == "relu2":
        return relu2(x)
    if act == "gelu":
        return gelu(x)
    if act == "relu2_bwd":
        return relu2_bwd(x, gate)
    if act == "gelu_bwd":
        return gelu_bwd(x, gate)
    raise ValueError(f"unknown activation {act!r}")
