"""The two seams through which train-gpt reaches the hot path: the norm dispatch of
`model._norm` (model.py:11-16) and the `mm` / `norm` callables of the benchmark's
`build_loss` (bench_fp8_norm.py:81-86, :130-138)."""
from __future__ import annotations

from .fp8 import block_scaled_matmul
from .kernels import _rms_norm_pure, rms_norm


def _norm(x, w, cfg):
    """model.py:11-16: `cfg.use_pallas_norm` picks the fused kernel or the pure form."""
    fn = rms_norm if cfg.use_pallas_norm else _rms_norm_pure
    return fn(x, w, cfg.rms_eps)


def mm_fp8(a, b):
    """bench_fp8_norm.py:131."""
    return block_scaled_matmul(a, b)


def mm_bf16(a, b):
    """bench_fp8_norm.py:130."""
    return a @ b
