"""CPU oracle for train-gpt's capped-logit cross-entropy (`model.py:97` + `losses.py:8-12`).

TEST INFRASTRUCTURE ONLY -- imported by `tests/` and `__graft_entry__.smoke()`, never by the
shipped package.

Pin status: the loss composition (`losses.py:9-12`: float32 cast, log_softmax, gather, mean)
is PINNED against a fixture produced by running the reference's own `cross_entropy_loss`
source with NumPy standing in for `jax.numpy` and a stub for `model.forward`
(`tests/golden/make_golden.py`).  The cap itself is one line (`model.py:97`), restated here
with op-by-op bfloat16 semantics: each of the divide, tanh and multiply rounds to bf16, and the
Python-float cap is weakly typed, i.e. becomes bf16.  XLA may keep excess precision inside a
fusion, so this is one of the results the reference can produce; PARITY UNPINNED for that line.
The gradient is the analytic derivative of this forward, (softmax - onehot) * (1 - tanh^2) / rows,
in float64; JAX's autodiff rounds intermediate cotangents to bf16, which stays inside the
gradient tolerance the tests state.
"""
from __future__ import annotations

import numpy as np

from .fp8_oracle import BF16


def softcap(logits, cap: float):
    """model.py:97 -- `cap * tanh(logits / cap)` on bf16 logits, every op rounding to bf16.

    Returns (z, t): the capped logits and the bf16 tanh values."""
    x = np.asarray(logits).astype(BF16).astype(np.float32)
    c = np.float32(BF16(cap))
    a = (x / c).astype(BF16).astype(np.float32)
    t = np.tanh(a.astype(np.float64)).astype(np.float32).astype(BF16)
    z = (c * t.astype(np.float32)).astype(BF16)
    return z, t


def cross_entropy(z, targets):
    """losses.py:9-12 on capped logits z (rows, vocab): returns (mean loss f32, nll f32 (rows,), lse f32 (rows,))."""
    z64 = np.asarray(z).astype(np.float32).astype(np.float64)
    m = z64.max(axis=-1, keepdims=True)
    lse = (m + np.log(np.exp(z64 - m).sum(axis=-1, keepdims=True)))[:, 0]
    zt = np.take_along_axis(z64, np.asarray(targets)[:, None].astype(np.int64), axis=-1)[:, 0]
    nll = (lse - zt).astype(np.float32)
    return np.float32(nll.astype(np.float64).mean()), nll, lse.astype(np.float32)


def softcap_cross_entropy(logits, targets, cap: float):
    z, _ = softcap(logits, cap)
    return cross_entropy(z, targets)


def softcap_cross_entropy_grad(logits, targets, cap: float, gscale: float = 1.0):
    """d(mean nll)/d(logits) in float64, shape of logits."""
    z, t = softcap(logits, cap)
    z64 = z.astype(np.float32).astype(np.float64)
    t64 = t.astype(np.float32).astype(np.float64)
    m = z64.max(axis=-1, keepdims=True)
    p = np.exp(z64 - m)
    p /= p.sum(axis=-1, keepdims=True)
    rows = z64.shape[0]
    p[np.arange(rows), np.asarray(targets).astype(np.int64)] -= 1.0
    return p * (1.0 - t64 * t64) * (gscale / rows)
