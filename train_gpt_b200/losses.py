"""train-gpt's `losses.py` on the CUDA path: the capped-logit cross-entropy as one fused
forward pass and one backward pass over the logits.

The reference computes `cross_entropy_loss(params, input_ids, target_ids, cfg)` as
`forward(...)` (which ends with `cap * tanh(logits / cap)`, model.py:97), a float32 cast,
`log_softmax`, a gather and a mean (losses.py:8-12).  Here the part after the unembedding
GEMM is `capped_cross_entropy(logits, target_ids, cap)`: it takes the GEMM's raw bf16 output,
so the capped logits and their float32 copy are never written to memory.
"""
from __future__ import annotations

import torch

from . import ops


class _SoftcapCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, cap):
        shape = logits.shape
        l2 = logits.reshape(-1, shape[-1])
        t = targets.reshape(-1).to(torch.int32)
        nll, lse, th = ops.softcap_ce_fwd(l2, t, cap, want_tanh=True)
        ctx.save_for_backward(th, t, lse)
        ctx.cap, ctx.shape = cap, shape
        return nll.mean()                                                      # losses.py:12

    @staticmethod
    def backward(ctx, g):
        th, t, lse = ctx.saved_tensors
        # the tanh buffer is this function's own: the gradient replaces it in place
        d = ops.softcap_ce_bwd(th, t, lse, g.to(torch.float32), ctx.cap, in_place=True)
        return d.reshape(ctx.shape), None, None


def capped_cross_entropy(logits: torch.Tensor, target_ids: torch.Tensor, cap: float) -> torch.Tensor:
    """Mean over tokens of -log_softmax(cap * tanh(logits / cap))[target] (model.py:97, losses.py:8-12).

    logits: (..., vocab) bf16, the unembedding GEMM's output BEFORE the cap; target_ids: (...)
    integer.  Any vocabulary size (the reference's default 50257 is not a multiple of 8).
    Differentiable with respect to logits."""
    if logits.shape[:-1] != target_ids.shape:
        raise ValueError(f"logits {tuple(logits.shape)} and target_ids {tuple(target_ids.shape)} do not match")
    return _SoftcapCE.apply(logits, target_ids, float(cap))
