"""CPU oracle for the optimiser half of train-gpt's train step (train.py:114-123,132-134):
optax.global_norm, optax.clip_by_global_norm and optax.adamw on bf16 parameters.

TEST INFRASTRUCTURE ONLY -- imported by `tests/`, never by the shipped package.

PARITY UNPINNED: optax (0.2.x per the reference's lock file) is a third-party dependency absent
from the reference tree, and the reference stores no optimiser outputs.  This restates optax's
published update rules -- scale_by_adam with moments in the parameter dtype, bias correction by
1 - b^t, add_decayed_weights, scale by -lr, clip factor min(1, max_norm / norm) -- with float32
arithmetic between bf16 stores.
"""
from __future__ import annotations

import numpy as np

from .fp8_oracle import BF16


def _r(x):
    return np.asarray(x, dtype=np.float32).astype(BF16).astype(np.float32)


def global_norm(grads) -> np.float32:
    """optax.global_norm: sqrt of the sum of squares over every leaf (float64 sum here)."""
    return np.float32(np.sqrt(sum(float((np.asarray(g).astype(np.float64) ** 2).sum()) for g in grads)))


def clip_factor(norm, max_norm: float) -> np.float32:
    """optax.clip_by_global_norm: gradients are multiplied by max_norm / norm when norm > max_norm."""
    n = np.float32(norm)
    return np.float32(1.0) if n < np.float32(max_norm) else np.float32(max_norm) / n


def adamw_step(p, g, m, v, t: int, lr: float, b1=0.9, b2=0.999, eps=1e-8, weight_decay=0.0, gscale=1.0):
    """One step; p, g, m, v bf16 arrays; returns (p, m, v) as bf16 arrays."""
    f = np.float32
    p32, g32, m32, v32 = (np.asarray(a).astype(np.float32) for a in (p, g, m, v))
    gc = _r(g32 * f(gscale))
    m_new = _r(f(b1) * m32 + (f(1.0) - f(b1)) * gc)
    v_new = _r(f(b2) * v32 + (f(1.0) - f(b2)) * gc * gc)
    inv_bc1 = f(1.0) / (f(1.0) - f(b1) ** f(t))
    inv_bc2 = f(1.0) / (f(1.0) - f(b2) ** f(t))
    u = (m_new * inv_bc1) / (np.sqrt(v_new * inv_bc2) + f(eps)) + f(weight_decay) * p32
    p_new = _r(p32 - f(lr) * u)
    return p_new.astype(BF16), m_new.astype(BF16), v_new.astype(BF16)
