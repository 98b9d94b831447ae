"""Data-parallel gradient exchange for the training step: the one collective the hot path
has.  train-gpt itself is single-device (train.py:1); the exchange belongs between
`value_and_grad` (train.py:129) and `global_norm` (train.py:132).

Gradients of one bucket (one decoder layer, or the embedding / head group) live in ONE flat
buffer; every parameter's `.grad` is a view into it.  When the last gradient of a bucket has
been accumulated during backward, the bucket's all-reduce is launched asynchronously, so the
exchange of layer l overlaps the backward of layers l-1 .. 0.  NCCL (NVLink/NVSwitch) on GPUs,
gloo on CPU -- the class only uses `torch.distributed`.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.distributed as dist


class GradBuckets:
    """Flat gradient buckets with overlap of all-reduce and backward.

    buckets: list of lists of parameters, in the order their gradients become ready LAST to
    FIRST does not matter -- each bucket fires when its own parameters are all done.
    """

    def __init__(self, buckets: Sequence[Sequence[torch.nn.Parameter]], world_size: int, average: bool = True,
                 group=None):
        self.world_size = world_size
        self.average = average
        self.group = group
        self.flat: List[torch.Tensor] = []
        self._pending: List[int] = []
        self._sizes: List[int] = []
        self._handles = []
        self._hooks = []
        self._nccl = world_size > 1 and dist.is_initialized() and dist.get_backend(group) == "nccl"
        self.params: List[List[torch.nn.Parameter]] = []
        for bi, params in enumerate(buckets):
            params = [p for p in params if p.requires_grad]
            self.params.append(params)
            if not params:
                self.flat.append(torch.empty(0))
                self._sizes.append(0)
                self._pending.append(0)
                continue
            dtype, device = params[0].dtype, params[0].device
            n = sum(p.numel() for p in params)
            flat = torch.zeros(n, dtype=dtype, device=device)
            off = 0
            for p in params:
                if p.dtype != dtype:
                    raise TypeError("all parameters of a bucket must share a dtype")
                p.grad = flat[off:off + p.numel()].view_as(p)
                off += p.numel()
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(bi)))
            self.flat.append(flat)
            self._sizes.append(len(params))
            self._pending.append(len(params))

    def _make_hook(self, bi: int):
        def hook(_param):
            self._pending[bi] -= 1
            if self._pending[bi] == 0:
                self._launch(bi)
        return hook

    def _launch(self, bi: int):
        if self.world_size > 1:
            # NCCL averages inside the collective; gloo (the CPU tests) has no AVG: sum, then scale in finish()
            op = dist.ReduceOp.AVG if (self.average and self._nccl) else dist.ReduceOp.SUM
            self._handles.append(dist.all_reduce(self.flat[bi], op=op, group=self.group, async_op=True))

    def finish(self):
        """Wait for every bucket's exchange, turn sums into means, re-arm for the next step."""
        for bi, left in enumerate(self._pending):
            if left != 0 and self._sizes[bi] != 0:
                # a parameter that got no gradient this step: exchange what there is
                self._launch(bi)
        for h in self._handles:
            h.wait()
        self._handles.clear()
        if self.world_size > 1 and self.average and not self._nccl:
            for f in self.flat:
                if f.numel():
                    f.mul_(1.0 / self.world_size)
        self._pending = list(self._sizes)

    def flatten_parameters(self) -> List[torch.Tensor]:
        """Move every bucket's parameters into one flat tensor per bucket, laid out like its gradients
        (each parameter becomes a view of its slice; values are kept), and return those tensors.  An
        elementwise optimiser whose hyper-parameters are the same for every tensor can then update a
        bucket with one launch over (flat parameters, flat gradients) instead of one per tensor."""
        out = []
        for params, fg in zip(self.params, self.flat):
            if not params:
                out.append(torch.empty(0))
                continue
            fp = torch.empty_like(fg)
            off = 0
            with torch.no_grad():
                for p in params:
                    dst = fp[off:off + p.numel()].view_as(p)
                    dst.copy_(p.data)
                    p.data = dst
                    off += p.numel()
            out.append(fp)
        return out

    def zero(self):
        for f in self.flat:
            if f.numel():
                f.zero_()

    def global_norm(self) -> torch.Tensor:
        """optax.global_norm (train.py:132) over all buckets, in float32."""
        sq = [f.float().pow(2).sum() for f in self.flat if f.numel()]
        return torch.stack(sq).sum().sqrt()

    def bytes(self) -> int:
        return sum(f.numel() * f.element_size() for f in self.flat)
