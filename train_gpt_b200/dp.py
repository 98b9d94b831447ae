"""Data-parallel gradient exchange for the training step: the one collective the hot path
has.  train-gpt itself is single-device (train.py:1); the exchange belongs between
`value_and_grad` (train.py:129) and `global_norm` (train.py:132).

Gradients of one bucket (one decoder layer, or the embedding / head group) live in ONE flat
buffer; every parameter's `.grad` is a view into it.  When the last gradient of a bucket has
been accumulated during backward, the bucket's all-reduce is launched asynchronously, so the
exchange of layer l overlaps the backward of layers l-1 .. 0 (at once, or -- `defer=True` -- at
points of the backward pass the caller picks with `flush()`).  NCCL (NVLink/NVSwitch) on GPUs,
gloo on CPU -- the class only uses `torch.distributed`.

Two options serve the CUDA step (train_gpt_b200.step): the buckets can hand out gradient slots
(`enable_direct`, `GradSlot`) that a weight-gradient GEMM writes into, and they can lay a bucket's
parameters out like its gradients (`flatten_parameters`) for an optimiser that updates a bucket
with one launch.
"""
from __future__ import annotations

from typing import List, Sequence

import torch
import torch.distributed as dist


class GradSlot:
    """Where the op that computes a parameter's gradient may write it, instead of handing autograd a
    tensor that is then added into the (zeroed) bucket: `take()` gives the destination -- the parameter's
    slice of its bucket, or, for parameters laid out side by side, the one matrix that holds all their
    gradients as column slices -- and `ready()` says that the gradients of `params` are now in place (what
    autograd's post-accumulate hook says for the others).  The op then returns None as that gradient.
    A slot serves one write per step: a parameter used twice has to go through autograd's accumulation."""

    def __init__(self, owner: "GradBuckets", bi: int, params, out: torch.Tensor):
        self.owner, self.bi, self.params, self.out, self.used = owner, bi, tuple(params), out, False

    def take(self) -> torch.Tensor:
        if self.used:
            raise RuntimeError("a parameter with a direct gradient slot produced two gradients in one step")
        self.used = True
        return self.out

    def ready(self) -> None:
        for _ in self.params:
            self.owner._one_done(self.bi)


class GradBuckets:
    """Flat gradient buckets with overlap of all-reduce and backward.

    buckets: list of lists of parameters, in the order their gradients become ready LAST to
    FIRST does not matter -- each bucket fires when its own parameters are all done.  An entry of
    a bucket may be a tuple of 2-D parameters with the same number of rows: these are laid out SIDE
    BY SIDE, as column slices of one (rows, total columns) matrix, so that one GEMM can produce all
    their gradients (their `.grad` views are then not contiguous).
    """

    def __init__(self, buckets: Sequence[Sequence], world_size: int, average: bool = True,
                 group=None, defer: bool = False):
        """defer: a finished bucket's all-reduce is not launched at once but at the next `flush()` (or at
        `finish()`): the caller picks points of the backward pass where the collective's kernel shares the GPU
        gracefully (see `flush`)."""
        self.defer = defer
        self._deferred: List[int] = []
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
        self._layout: List[list] = []        # per bucket: (offset, rows, cols, (params...)) per entry; rows == 0: one contiguous parameter
        self._where = {}                     # id(parameter) -> (bucket, entry)
        self._slots: List[GradSlot] = []
        for bi, entries in enumerate(buckets):
            layout, params, off = [], [], 0
            for e in entries:
                grp = tuple(p for p in (e if isinstance(e, (tuple, list)) else (e,)) if p.requires_grad)
                if not grp:
                    continue
                if len(grp) > 1:
                    rows = grp[0].shape[0]
                    if any(p.dim() != 2 or p.shape[0] != rows for p in grp):
                        raise ValueError("parameters laid out side by side must be 2-D with the same number of rows")
                    layout.append((off, rows, sum(p.shape[1] for p in grp), grp))
                else:
                    layout.append((off, 0, grp[0].numel(), grp))
                for p in grp:
                    self._where[id(p)] = (bi, len(layout) - 1)
                params.extend(grp)
                off += sum(p.numel() for p in grp)
            self.params.append(params)
            self._layout.append(layout)
            if not params:
                self.flat.append(torch.empty(0))
                self._sizes.append(0)
                self._pending.append(0)
                continue
            dtype, device = params[0].dtype, params[0].device
            if any(p.dtype != dtype for p in params):
                raise TypeError("all parameters of a bucket must share a dtype")
            flat = torch.zeros(off, dtype=dtype, device=device)
            for p, view in zip(params, self.views(bi, flat)):
                p.grad = view
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(bi)))
            self.flat.append(flat)
            self._sizes.append(len(params))
            self._pending.append(len(params))
        self._zero_ranges = [[(0, f.numel())] if f.numel() else [] for f in self.flat]

    def views(self, bi: int, flat: torch.Tensor) -> List[torch.Tensor]:
        """Per-parameter views of `flat` (a tensor as long as bucket `bi`) in the bucket's layout, in the
        order of `self.params[bi]`."""
        out = []
        for off, rows, cols, grp in self._layout[bi]:
            if rows == 0:
                out.append(flat[off:off + cols].view_as(grp[0]))
                continue
            region, c = flat[off:off + rows * cols].view(rows, cols), 0
            for p in grp:
                out.append(region[:, c:c + p.shape[1]])
                c += p.shape[1]
        return out

    def enable_direct(self, params) -> None:
        """Give these parameters a `grad_slot` (GradSlot): their gradients will be written into the bucket
        by the op that computes them, once per step, so their part of the bucket is not zeroed before the
        backward pass and no add into it is launched.  Parameters laid out side by side share one slot
        (all of them must be named); only ops that look for `grad_slot` honour it, so name a parameter here
        only if every use of it goes through one."""
        want = {id(p) for p in params}
        for bi, layout in enumerate(self._layout):
            for off, rows, cols, grp in layout:
                hit = [id(p) in want for p in grp]
                if not any(hit):
                    continue
                if not all(hit):
                    raise ValueError("parameters laid out side by side take a direct gradient slot together or not at all")
                n = cols if rows == 0 else rows * cols
                if (off * self.flat[bi].element_size()) % 16 or grp[0].dim() != 2:
                    continue                 # a GEMM cannot write here (16-byte alignment; matrices only): stays with autograd
                out = self.flat[bi][off:off + n]
                out = out.view_as(grp[0]) if rows == 0 else out.view(rows, cols)
                slot = GradSlot(self, bi, grp, out)
                self._slots.append(slot)
                for p in grp:
                    p.grad_slot = slot
                # what is left to zero in this bucket
                left = []
                for a, b in self._zero_ranges[bi]:
                    if off >= b or off + n <= a:
                        left.append((a, b))
                        continue
                    if a < off:
                        left.append((a, off))
                    if off + n < b:
                        left.append((off + n, b))
                self._zero_ranges[bi] = left

    def _one_done(self, bi: int) -> None:
        self._pending[bi] -= 1
        if self._pending[bi] == 0:
            self._launch(bi)

    def _make_hook(self, bi: int):
        def hook(_param):
            self._one_done(bi)
        return hook

    def _launch(self, bi: int):
        if self.defer and self.world_size > 1:
            self._deferred.append(bi)
            return
        self._exchange(bi)

    def flush(self):
        """Launch the all-reduce of every bucket that has finished since the last call.  An all-reduce kernel
        needs a few SMs.  Launched while a persistent GEMM holds all of them it waits for that GEMM to end, takes
        its SMs, and the NEXT persistent GEMM then runs short of those SMs until the collective is done: the
        blocks assigned to them start late and the whole GEMM waits for them.  Launched just before a kernel of
        many short blocks (attention backward), it gets its SMs as blocks retire and gives them back before the
        next GEMM."""
        pending, self._deferred = self._deferred, []
        for bi in pending:
            self._exchange(bi)

    def _exchange(self, bi: int):
        if self.world_size > 1:
            # NCCL averages inside the collective; gloo (the CPU tests) has no AVG: sum, then scale in finish()
            op = dist.ReduceOp.AVG if (self.average and self._nccl) else dist.ReduceOp.SUM
            self._handles.append(dist.all_reduce(self.flat[bi], op=op, group=self.group, async_op=True))

    def finish(self):
        """Wait for every bucket's exchange, turn sums into means, re-arm for the next step."""
        self.flush()
        for bi, left in enumerate(self._pending):
            if left != 0 and self._sizes[bi] != 0:
                # a parameter that got no gradient this step: exchange what there is
                self._exchange(bi)
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
        (each parameter becomes a view of its slice -- a column slice, not contiguous, for parameters laid
        out side by side, which also get `side_by_side = (the whole matrix, the parameters in it)`; values
        are kept), and return those tensors.  An
        elementwise optimiser whose hyper-parameters are the same for every tensor can then update a
        bucket with one launch over (flat parameters, flat gradients) instead of one per tensor."""
        out = []
        for bi, (params, fg) in enumerate(zip(self.params, self.flat)):
            if not params:
                out.append(torch.empty(0))
                continue
            fp = torch.empty_like(fg)
            with torch.no_grad():
                for p, dst in zip(params, self.views(bi, fp)):
                    dst.copy_(p.data)
                    p.data = dst
            # parameters laid out side by side can be read as the one matrix they are column slices of
            for off, rows, cols, grp in self._layout[bi]:
                if rows:
                    whole = fp[off:off + rows * cols].view(rows, cols)
                    for q in grp:
                        q.side_by_side = (whole, grp)
            out.append(fp)
        return out

    def zero(self):
        for f, ranges in zip(self.flat, self._zero_ranges):
            for a, b in ranges:
                f[a:b].zero_()
        for slot in self._slots:
            slot.used = False

    def global_norm(self) -> torch.Tensor:
        """optax.global_norm (train.py:132) over all buckets, in float32."""
        sq = [f.float().pow(2).sum() for f in self.flat if f.numel()]
        return torch.stack(sq).sum().sqrt()

    def bytes(self) -> int:
        return sum(f.numel() * f.element_size() for f in self.flat)
