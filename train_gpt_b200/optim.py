"""The optimiser of train-gpt's train step on the CUDA path: `make_optimizer(lr, weight_decay,
clip_norm)` (train.py:114-123) = optax.chain(clip_by_global_norm, adamw), for bf16 parameters
whose gradients live in flat buckets (`dp.GradBuckets`).

Global norm: one sum-of-squares kernel per bucket, their float32 results added on the device.
Update: one kernel per parameter tensor -- or, when the parameters of a bucket live in one flat
tensor laid out like the bucket's gradients (`flat=`; optax's adamw has the same hyper-parameters
for every leaf, so the update is one elementwise map over the concatenation), one kernel per
bucket -- that applies the clip factor to the gradient as it reads it, so the clipped gradient is
never written.  Step count and clip factor stay on the device, which lets the whole step be
replayed from a CUDA graph.
"""
from __future__ import annotations

from typing import Sequence

import torch

from . import ops


class ClippedAdamW:
    def __init__(self, params: Sequence[torch.nn.Parameter], lr: float, weight_decay: float = 1e-4, clip_norm: float = 1.0,
                 b1: float = 0.9, b2: float = 0.999, eps: float = 1e-8, flat=None):
        """flat: optional list of (flat parameters, flat gradients, the parameters that are views of the
        former, views) with views(t) = the per-parameter views of a flat tensor t in that layout --
        `dp.GradBuckets.flatten_parameters` / `.views` make them; they must cover `params`."""
        self.params = [p for p in params if p.requires_grad]
        self.lr, self.wd, self.clip, self.b1, self.b2, self.eps = lr, weight_decay, clip_norm, b1, b2, eps
        dev = self.params[0].device
        self._flat = None
        if flat is not None:
            groups = [(fp, fg, list(ps), views) for fp, fg, ps, views in flat if fp.numel()]
            covered = {id(p) for _, _, ps, _ in groups for p in ps}
            if covered != {id(p) for p in self.params}:
                raise ValueError("the flat groups must hold exactly the optimised parameters")
            self._flat, by_id = [], {}
            for fp, fg, ps, views in groups:
                if fp.shape != fg.shape or sum(p.numel() for p in ps) != fp.numel():
                    raise ValueError("flat parameters, flat gradients and their views must have the same length")
                fm, fv = torch.zeros_like(fp), torch.zeros_like(fp)
                self._flat.append((fp, fg, fm, fv))
                for p, m, v in zip(ps, views(fm), views(fv)):
                    by_id[id(p)] = (m, v)
            self.m = [by_id[id(p)][0] for p in self.params]           # per-parameter views of the flat moments
            self.v = [by_id[id(p)][1] for p in self.params]
        else:
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
        if self._flat is not None:
            for fp, fg, fm, fv in self._flat:
                ops.adamw_step(fp, fg, fm, fv, self.step_t, self.lr, self.b1, self.b2, self.eps, self.wd, gscale=scale)
            return
        for p, m, v in zip(self.params, self.m, self.v):
            if p.grad is None:
                continue
            ops.adamw_step(p.data, p.grad, m, v, self.step_t, self.lr, self.b1, self.b2, self.eps, self.wd, gscale=scale)
