"""tg_sumsq_bf16 / tg_adamw_bf16 against the CPU oracle (optax's update rules restated).

Tolerances: sum of squares within 2e-6 relative of the float64 sum; parameters and moments equal
to the oracle's bf16 values except where float32 `powf`/`sqrtf`/division on the device and NumPy
round an intermediate differently: at most one bf16 ulp apart (one ulp of the OLD value where the
update nearly cancels it), at least 99.5 % identical.
"""
import numpy as np
import pytest
import torch

from oracle import fp8_oracle as fo
from oracle import optim_oracle as oo
from tests.gpu_util import from_torch_bf16, to_torch_bf16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [5, 4096, 1_000_003])
def test_sumsq(n):
    from train_gpt_b200 import ops
    x = np.random.default_rng(n).standard_normal(n).astype(fo.BF16)
    got = float(ops.sumsq(to_torch_bf16(x)).item())
    ref = float((x.astype(np.float64) ** 2).sum())
    assert abs(got - ref) <= 2e-6 * ref


def _ulp_gap(a, b):
    return np.abs(a.view(np.uint16).astype(np.int32) - b.view(np.uint16).astype(np.int32))


@pytest.mark.parametrize("n,t,gscale", [(8, 1, None), (1003, 1, 0.37), (65536, 7, 1.0), (4099, 250, 0.02)])
def test_adamw_step_matches_oracle(n, t, gscale):
    from train_gpt_b200 import ops
    rng = np.random.default_rng(n + t)
    p = (rng.standard_normal(n) * 0.02).astype(fo.BF16)
    g = (rng.standard_normal(n) * 1e-3).astype(fo.BF16)
    m = (rng.standard_normal(n) * 1e-4).astype(fo.BF16) if t > 1 else np.zeros(n, fo.BF16)
    v = (rng.random(n) * 1e-7).astype(fo.BF16) if t > 1 else np.zeros(n, fo.BF16)
    tp, tg_, tm, tv = (to_torch_bf16(a).clone() for a in (p, g, m, v))
    step = torch.tensor(t, dtype=torch.int32, device="cuda")
    gs = None if gscale is None else torch.tensor([gscale], dtype=torch.float32, device="cuda")
    ops.adamw_step(tp, tg_, tm, tv, step, lr=3e-4, weight_decay=0.1, gscale=gs)
    rp, rm, rv = oo.adamw_step(p, g, m, v, t, lr=3e-4, weight_decay=0.1, gscale=1.0 if gscale is None else gscale)
    for got, ref, old, name in ((tp, rp, p, "p"), (tm, rm, m, "m"), (tv, rv, v, "v")):
        got = from_torch_bf16(got)
        gap = _ulp_gap(got, ref)
        # where the update nearly cancels the old value the result is tiny and one of ITS ulps means
        # nothing: there the bound is one ulp of the old value
        diff = np.abs(got.astype(np.float32) - ref.astype(np.float32))
        ok = (gap <= 1) | (diff <= 2.0 ** -8 * np.abs(old.astype(np.float32)))
        assert ok.all(), (name, gap.max())
        assert (gap == 0).mean() >= 0.995, (name, (gap == 0).mean())


def test_clipped_adamw_follows_oracle_over_steps():
    """optim.ClippedAdamW on two tensors for five steps: global norm, clip factor, update."""
    from train_gpt_b200 import optim
    rng = np.random.default_rng(0)
    shapes = [(64, 48), (1000,)]
    ps = [(rng.standard_normal(s) * 0.05).astype(fo.BF16) for s in shapes]
    params = [torch.nn.Parameter(to_torch_bf16(p).clone()) for p in ps]
    opt = optim.ClippedAdamW(params, lr=1e-2, weight_decay=0.1, clip_norm=1.0)
    ms = [np.zeros(s, fo.BF16) for s in shapes]
    vs = [np.zeros(s, fo.BF16) for s in shapes]
    for t in range(1, 6):
        gs = [(rng.standard_normal(s) * (3.0 if t % 2 else 0.01)).astype(fo.BF16) for s in shapes]   # clipped and unclipped steps
        for p, g in zip(params, gs):
            p.grad = to_torch_bf16(g).clone()
        gn = opt.global_norm([p.grad.reshape(-1) for p in params])
        opt.step(gn)
        ref_gn = oo.global_norm(gs)
        assert abs(float(gn) - float(ref_gn)) <= 1e-5 * float(ref_gn)
        f = oo.clip_factor(float(gn), 1.0)
        for i in range(len(ps)):
            ps[i], ms[i], vs[i] = oo.adamw_step(ps[i], gs[i], ms[i], vs[i], t, lr=1e-2, weight_decay=0.1, gscale=f)
    for p, ref in zip(params, ps):
        got = from_torch_bf16(p.data).astype(np.float32)
        gap = _ulp_gap(from_torch_bf16(p.data), ref)
        assert (gap == 0).mean() > 0.98                         # five steps of compounding last-bit differences
        assert np.abs(got - ref.astype(np.float32)).max() <= 2.0 ** -6 * np.abs(ref.astype(np.float32)).max()
