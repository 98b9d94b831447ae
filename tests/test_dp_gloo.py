"""Host logic of the data-parallel step on CPU: two gloo ranks, bucketed all-reduce
overlapping backward, against one process holding both ranks' batches.

The model here runs on torch ops only (mm "bf16", norm "torch_reference") -- the CUDA kernels
have no CPU path, and what is under test is the gradient exchange, not the kernels.
"""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cfg():
    from train_gpt_b200.step import SMALL, StepConfig
    return StepConfig(**SMALL, mm="bf16", norm="torch_reference", loss="torch", optimizer="torch", activation="relu2")


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from train_gpt_b200.step import Trainer, synthetic_batch
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    cfg = _cfg()
    tr = Trainer(cfg, "cpu", world_size=world, seed=0)
    ids, tgt = synthetic_batch(cfg, 2, "cpu", seed=100 + rank, learnable=True)
    launched = []
    orig = tr.buckets._launch
    tr.buckets._launch = lambda bi: (launched.append(bi), orig(bi))[1]
    exchanged, pending_at_exchange = [], []
    orig_x = tr.buckets._exchange
    tr.buckets._exchange = lambda bi: (exchanged.append(bi), pending_at_exchange.append(len(launched)), orig_x(bi))[2]
    assert tr.buckets.defer and tr.model.exchange is tr.buckets      # more than one rank: the exchange is deferred
    loss, gnorm = tr.step(ids, tgt)
    torch.save({"loss": loss, "gnorm": gnorm, "grads": [f.clone() for f in tr.buckets.flat],
                "params": [p.detach().clone() for p in tr.model.parameters()], "launched": launched,
                "exchanged": exchanged, "pending_at_exchange": pending_at_exchange},
               os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_exchange_matches_full_batch(tmp_path):
    from train_gpt_b200.step import Trainer, synthetic_batch
    world, port = 2, _free_port()
    mp.start_processes(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    r0, r1 = (torch.load(tmp_path / f"rank{r}.pt") for r in range(2))

    # every bucket fired exactly once, in backward order (head group first, embeddings last)
    n_buckets = 2 + _cfg().n_layers
    assert r0["launched"] == list(range(n_buckets)) and r1["launched"] == r0["launched"]
    # ... and was exchanged once, in the same order, at a flush point (the attention backward of a later layer) or
    # at the end of the backward pass: never before it had finished
    assert r0["exchanged"] == r0["launched"] and r1["exchanged"] == r0["launched"]
    assert all(n > bi for bi, n in zip(r0["exchanged"], r0["pending_at_exchange"]))
    # both ranks hold the same reduced gradients, norm and updated parameters
    for a, b in zip(r0["grads"], r1["grads"]):
        assert torch.equal(a, b)
    assert torch.equal(r0["gnorm"], r1["gnorm"])
    for a, b in zip(r0["params"], r1["params"]):
        assert torch.equal(a, b)

    # one process, both batches: its gradient is the mean of the two ranks' gradients
    cfg = _cfg()
    tr = Trainer(cfg, "cpu", world_size=1, seed=0)
    b0 = synthetic_batch(cfg, 2, "cpu", seed=100, learnable=True)
    b1 = synthetic_batch(cfg, 2, "cpu", seed=101, learnable=True)
    ids, tgt = torch.cat([b0[0], b1[0]]), torch.cat([b0[1], b1[1]])
    tr.buckets.zero()
    loss = tr.model.loss(ids, tgt)
    loss.backward()
    tr.buckets.finish()
    assert abs(float(loss) - 0.5 * (float(r0["loss"]) + float(r1["loss"]))) < 5e-3
    for full, dp in zip(tr.buckets.flat, r0["grads"]):
        # r0's stored gradients are post-clip; compare direction and scale before the clip factor
        scale = min(1.0, cfg.clip_norm / (float(r0["gnorm"]) + 1e-6))
        ref = full.float() * scale
        err = (dp.float() - ref).norm() / (ref.norm() + 1e-12)
        assert float(err) < 3e-2, float(err)          # bf16 gradients, different summation order
    assert abs(float(tr.buckets.global_norm()) - float(r0["gnorm"])) / float(r0["gnorm"]) < 2e-2


def test_single_rank_step_runs_and_lowers_the_loss():
    from train_gpt_b200.step import Trainer, synthetic_batch
    cfg = _cfg()
    tr = Trainer(cfg, "cpu", world_size=1, seed=0)
    ids, tgt = synthetic_batch(cfg, 4, "cpu", seed=7, learnable=True)
    first, _ = tr.step(ids, tgt)
    assert abs(float(first) - torch.log(torch.tensor(float(cfg.vocab_size)))) < 0.3     # test_overfit.py:33-35
    for _ in range(30):
        last, _ = tr.step(ids, tgt)
    assert float(last) < float(first) - 0.5


def test_flatten_parameters_keeps_values_and_aliases_the_flat_tensors():
    from train_gpt_b200.dp import GradBuckets
    torch.manual_seed(0)
    a = [torch.nn.Parameter(torch.randn(3, 5)), torch.nn.Parameter(torch.randn(7))]
    b = [torch.nn.Parameter(torch.randn(2, 2))]
    frozen = torch.nn.Parameter(torch.randn(4), requires_grad=False)
    before = [p.detach().clone() for p in a + b]
    gb = GradBuckets([a + [frozen], b, []], world_size=1)
    flats = gb.flatten_parameters()
    assert [f.numel() for f in flats] == [22, 4, 0]
    for p, q in zip(a + b, before):
        assert torch.equal(p.detach(), q)
    assert torch.equal(flats[0], torch.cat([before[0].reshape(-1), before[1]]))
    with torch.no_grad():
        flats[0].add_(1.0)                       # an update of the flat tensor is an update of the parameters
    assert torch.equal(a[0].detach(), before[0] + 1.0) and torch.equal(a[1].detach(), before[1] + 1.0)
    assert gb.params[0] == a and gb.params[1] == b     # frozen parameters take no part
    # gradients still land in the bucket's flat gradient tensor
    (a[0].sum() + 2.0 * a[1].sum()).backward()
    assert torch.equal(gb.flat[0], torch.cat([torch.ones(15), 2.0 * torch.ones(7)]))


def test_side_by_side_entries_and_direct_gradient_slots():
    """A tuple entry of a bucket is laid out as column slices of one matrix; a direct slot hands out that
    matrix (or a lone parameter's slice), its part of the bucket is not zeroed, and `ready()` counts like
    autograd's hook."""
    from train_gpt_b200.dp import GradBuckets
    torch.manual_seed(1)
    g = torch.nn.Parameter(torch.randn(8))
    wq, wk, wv = (torch.nn.Parameter(torch.randn(4, n)) for n in (8, 8, 16))
    wo = torch.nn.Parameter(torch.randn(8, 4))
    before = [p.detach().clone() for p in (g, wq, wk, wv, wo)]
    gb = GradBuckets([[g, (wq, wk, wv), wo]], world_size=1)
    launched = []
    gb._launch = lambda bi: launched.append(bi)
    assert gb.flat[0].numel() == 8 + 4 * 32 + 32
    region = gb.flat[0][8:8 + 128].view(4, 32)
    assert wk.grad.data_ptr() == region[:, 8:16].data_ptr() and wk.grad.stride() == (32, 1)
    flats = gb.flatten_parameters()
    for p, q in zip((g, wq, wk, wv, wo), before):
        assert torch.equal(p.detach(), q)
    whole, members = wq.side_by_side
    assert torch.equal(whole, torch.cat(before[1:4], dim=1)) and members == (wq, wk, wv)
    assert whole.data_ptr() == flats[0][8:].data_ptr()
    try:
        gb.enable_direct([wq, wk])
        assert False, "a partial group must be refused"
    except ValueError:
        pass
    gb.enable_direct([wq, wk, wv, wo])
    assert wq.grad_slot is wk.grad_slot is wv.grad_slot and wo.grad_slot is not wq.grad_slot
    assert gb._zero_ranges[0] == [(0, 8)]
    gb.flat[0].fill_(7.0)
    gb.zero()
    assert float(gb.flat[0][:8].abs().sum()) == 0.0 and float(gb.flat[0][8:].min()) == 7.0
    out = wq.grad_slot.take()
    assert out.shape == (4, 32) and out.data_ptr() == region.data_ptr()
    try:
        wq.grad_slot.take()
        assert False, "a slot serves one write per step"
    except RuntimeError:
        pass
    out.copy_(torch.arange(128.0).view(4, 32))
    wq.grad_slot.ready()
    assert torch.equal(wv.grad, torch.arange(128.0).view(4, 32)[:, 16:]) and not launched
    wo.grad_slot.take().fill_(1.0)
    wo.grad_slot.ready()
    assert not launched
    (3.0 * g).sum().backward()                     # the last gradient of the bucket comes through autograd
    assert launched == [0] and torch.equal(g.grad, torch.full((8,), 3.0))
    gb.finish()
    gb.zero()
    assert wq.grad_slot.take() is not None         # re-armed


def test_deferred_exchange_waits_for_flush():
    """defer=True: a finished bucket is exchanged at the next flush() (or at finish()), in the order the buckets
    finished; without it, at once."""
    from train_gpt_b200.dp import GradBuckets
    a, b = torch.nn.Parameter(torch.randn(4)), torch.nn.Parameter(torch.randn(3))
    for defer in (False, True):
        gb = GradBuckets([[a], [b]], world_size=2, average=False, defer=defer)
        sent = []
        gb._exchange = lambda bi: sent.append(bi)
        gb.zero()
        (2.0 * b).sum().backward()
        assert sent == ([] if defer else [1])
        gb.flush()
        assert sent == [1]
        a.sum().backward()
        assert sent == ([1] if defer else [1, 0])
        gb.finish()
        assert sent == [1, 0]
        for h in gb._hooks:
            h.remove()
        a.grad = b.grad = None
