"""CPU oracle for train-gpt's RMSNorm (`kernels.py`) and its fusion with the FP8
quantiser (`fp8.py:39-47`).

TEST INFRASTRUCTURE ONLY -- imported by `tests/`, `__graft_entry__.smoke()` and
the CPU-baseline legs of `bench.py`, never by the shipped package.

Pin status: the pure-JAX norm (`kernels.py:30-33`) and the backward formulae
(`kernels.py:104-118`) are PINNED against fixtures produced by running the
reference's own source with NumPy standing in for `jax.numpy`
(`tests/golden/make_golden.py`).  The Pallas kernel body (`kernels.py:44-53`)
cannot be executed without JAX/Mosaic; its restatement here is checked only
against the pure norm within bf16 rounding.  Row variance is a reduction whose
order XLA does not specify, so this oracle fixes it as the float64 sum rounded to
float32; a CUDA kernel's f32 tree sum may differ from it in the last bit, which is
why `rmsnorm_quant` accepts an externally supplied `rnorm`.
"""
from __future__ import annotations

import numpy as np

from .fp8_oracle import BF16, DEFAULT_BLOCK_K, quantize_to_fp8


def row_variance(x) -> np.ndarray:
    """`mean(f32(x)**2, -1)` (kernels.py:31,66,108) -> float32, shape (..., 1)."""
    x64 = np.asarray(x).astype(np.float64)
    return np.mean(x64 * x64, axis=-1, keepdims=True).astype(np.float32)


def rsqrt_f32(v: np.ndarray) -> np.ndarray:
    """Correctly rounded float32 reciprocal square root (via float64)."""
    return (1.0 / np.sqrt(np.asarray(v, dtype=np.float32).astype(np.float64))).astype(np.float32)


def rnorm_of(x, eps: float) -> np.ndarray:
    """`rsqrt(var + eps)` with the f32 add of kernels.py:32,50,109."""
    var = row_variance(x)
    return rsqrt_f32(var + np.float32(eps))


def rms_norm_pure(x, scale, eps: float, rnorm=None) -> np.ndarray:
    """kernels.py:30-33 in op-by-op semantics: rsqrt rounded to bf16, then two bf16
    multiplies (each rounds once)."""
    x = np.asarray(x).astype(BF16)
    scale = np.asarray(scale).astype(BF16)
    if rnorm is None:
        rnorm = rnorm_of(x, eps)
    r_bf = rnorm.astype(BF16)                                          # kernels.py:32 `.astype(x.dtype)`
    x_n = (x.astype(np.float32) * r_bf.astype(np.float32)).astype(BF16)
    return (x_n.astype(np.float32) * scale.astype(np.float32)).astype(BF16)   # kernels.py:33


def rms_norm(x, scale, eps: float, rnorm=None) -> np.ndarray:
    """kernels.py:44-53: `bf16(f32(x) * rnorm * f32(scale))`, products left to right in
    float32, ONE rounding to bf16."""
    x = np.asarray(x).astype(BF16)
    scale = np.asarray(scale).astype(BF16)
    if rnorm is None:
        rnorm = rnorm_of(x, eps)
    y = (x.astype(np.float32) * rnorm.astype(np.float32)) * scale.astype(np.float32)
    return y.astype(BF16)


def rms_norm_bwd(x, scale, g, eps: float, rnorm=None):
    """kernels.py:104-118: recompute-based backward.  Returns (dx bf16, dscale bf16)."""
    x = np.asarray(x).astype(BF16)
    scale = np.asarray(scale).astype(BF16)
    g = np.asarray(g).astype(BF16)
    x32 = x.astype(np.float32)                                         # :107
    if rnorm is None:
        rnorm = rnorm_of(x, eps)                                       # :108-109
    normed = x32 * rnorm                                               # :110
    g32 = g.astype(np.float32)                                         # :111
    gs = g32 * scale.astype(np.float32)                                # :112
    dot = np.mean((gs * normed).astype(np.float64), axis=-1, keepdims=True).astype(np.float32)  # :113
    grad_x = (rnorm * (gs - normed * dot)).astype(BF16)                # :114
    D = x.shape[-1]
    grad_scale = np.sum((g32 * normed).astype(np.float64).reshape(-1, D), axis=0).astype(np.float32).astype(BF16)  # :115-117
    return grad_x, grad_scale


def rmsnorm_quant(x, scale, eps: float, block_k: int = DEFAULT_BLOCK_K, rnorm=None, pure: bool = False):
    """The composition the reference runs between a norm and the GEMM that consumes
    it: `rms_norm(...)` returns bf16 (model.py:76), `fp8.py:66` upcasts that bf16 to
    f32 and `fp8.py:39-47` quantises it.  Returns (q e4m3, scales f32, y bf16)."""
    fn = rms_norm_pure if pure else rms_norm
    y = fn(x, scale, eps, rnorm=rnorm)
    D = y.shape[-1]
    q, s = quantize_to_fp8(y.reshape(-1, D).astype(np.float32), block_k)
    return q.reshape(y.shape), s.reshape(*y.shape[:-1], D // block_k), y
