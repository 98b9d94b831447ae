"""The optimiser of train-gpt's train step on the CUDA path: `make_optimizer(lr, weight_decay,
clip_norm)` (train.py:114-123) = optax.chain(clip_by_global_norm, adamw), for bf16 parameters
whose gradients live in flat buckets (`dp.GradBuckets`).

Global norm: one sum-of-squares kernel per bucket, their float32 results added on the device.
Update: one kernel per parameter tensor that applies the clip factor to the gradient as it
reads it, so the clipped gradient is never written.  Step count and clip factor stay on the
device, which lets the whole step be replayed from a CUDA graph.
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import ops


class ClippedAdamW:
    def __init__(self, params: Sequence[torch.nn.Parameter], lr: float, weight_decay: float = 1e-4, clip_norm: float = 1.0,
                 b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8):
        self.params = [p for p in params if p.requires_grad]
        self.lr, self.wd, self.clip, self.b1, self.b2, self.eps = lr, weight_decay, clip_norm, b1, b2, eps
        dev = self.params[0].device
        self.m = [torch.zeros_like(p) for p in self.params]           # optax: moments in the parameter dtype
        self.v = [torch.zeros_like(p) for p in self.params]
        self.step_t = torch.zeros((), dtype=torch.int32, device=dev)
        self._scratch = None
        self._sq = None

    def state_tensors(self):
        return self.m + self.v + [self.step_t]

    def global_norm(self, flat_grads: Sequence[torch.Tensor]) -> torch.Tensor:
        """optax.global_norm (train.py:132) over the flat gradient buckets."""
        flats = [f for f in flat_grads if f.numel()]
        if self._sq is None:
            dev = flats[0].device
            self._sq = torch.empty((len(flats),), dtype=torch.float32, device=dev)
            self._scratch = torch.empty((ops._lib.load().tg_sumsq_scratch_bytes(),), dtype=torch.uint8, device=dev)
        for i, f in enumerate(flats):
            ops.sumsq(f, out=self._sq[i:i + 1], scratch=self._scratch)
        return self._sq.sum().sqrt()

    def step(self, gnorm: torch.Tensor) -> None:
        """Clip by `gnorm` (optax.clip_by_global_norm: factor clip/norm when norm > clip) and update."""
        scale = torch.where(gnorm < self.clip, torch.ones_like(gnorm), self.clip / gnorm).to(torch.float32)
        self.step_t += 1
        for p, m, v in zip(self.params, self.m, self.v):
            if p.grad is None:
                continue
            ops.adamw_step(p.data, p.grad, m, v, self.step_t, self.lr, self.b1, self.b2, self.eps, self.wd, gscale=scale)
