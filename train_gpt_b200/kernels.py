"""RMSNorm: the call surface of train-gpt's `kernels.py` on B200 kernels.

`rms_norm(x, scale, eps)` is the fused single-rounding norm (kernels.py:44-53 with the
variance pass of :66 folded in) with the recompute backward of kernels.py:104-118;
`_rms_norm_pure(x, scale, eps)` is the three-rounding form (kernels.py:30-33).  Both are
positional-only in the reference's order; `eps` is static (not differentiated).
`rms_norm_quant` is the fused norm + 1x128 e4m3 quantise the FP8 linear layers consume.
"""
from __future__ import annotations

import torch

from . import ops


class _RmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, eps, pure):
        ctx.save_for_backward(x, scale)                             # kernels.py:101-102
        ctx.eps = eps
        return ops.rmsnorm_fwd(x, scale, eps, pure=pure)

    @staticmethod
    def backward(ctx, g):
        x, scale = ctx.saved_tensors
        dx, dscale = ops.rmsnorm_bwd(x, scale, g.to(torch.bfloat16), ctx.eps)   # kernels.py:104-118
        return dx, dscale, None, None


def rms_norm(x: torch.Tensor, scale: torch.Tensor, eps: float) -> torch.Tensor:
    return _RmsNorm.apply(x, scale, float(eps), False)


def _rms_norm_pure(x: torch.Tensor, scale: torch.Tensor, eps: float) -> torch.Tensor:
    return _RmsNorm.apply(x, scale, float(eps), True)


class NormedQuantized:
    """Output of `rms_norm_quant`: the norm's bf16 result in quantised form (q, scales),
    usable as `a_quantized=` of `fp8.block_scaled_matmul` by every GEMM that consumes the
    same normed activation, plus the bf16 tensor itself when it was asked for."""

    def __init__(self, q, scales, y):
        self.q, self.scales, self.y = q, scales, y

    def as_pair(self):
        return self.q, self.scales


def rms_norm_quant(x, scale, eps: float, pure: bool = False, want_y: bool = False) -> NormedQuantized:
    """model.py:76-77 `_norm(...)` followed by the quantiser of fp8.py:66, one kernel.
    Forward only (no autograd); training code pairs it with `rms_norm`'s backward."""
    q, s, y, _ = ops.rmsnorm_quant_fwd(x, scale, float(eps), pure=pure, want_y=want_y)
    return NormedQuantized(q, s, y)
