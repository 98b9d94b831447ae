"""CPU timing leg: the oracle's FP8 linear layer (forward + FP8 dgrad + FP8 wgrad) arranged
for speed rather than for exactness -- NumPy/ml_dtypes quantisers (fp8.py:39-47) and, per
GEMM, one dequantise + float32 `torch.matmul` on all host threads instead of the oracle's
per-block float64 products.  TEST/BENCH INFRASTRUCTURE ONLY: imported by `bench.py` for the
`cpu_baseline` object and the `--impl reference` arm, never by the package.

The reference's own CPU path cannot be timed: it is JAX, JAX is not installable here, and
its `jax.nn.scaled_matmul` has no CPU lowering (check_fp8_hlo.py:3).  This port is what
stands in for it ("kind": "port").
"""
from __future__ import annotations

import time

import numpy as np
import torch

from . import fp8_oracle as fo


def _deq(q, s_full) -> torch.Tensor:
    return torch.from_numpy(q.astype(np.float32) * s_full)


def linear_fwd_bwd(x, w, g, weight_tile=(128, 128)):
    """One FP8 linear layer, forward + dgrad + wgrad, on the host.  x (M,K), w (K,N),
    g (M,N) as ml_dtypes bf16 arrays.  Returns (y, dx, dw) float32 torch tensors."""
    x32, w32, g32 = (np.asarray(t).astype(np.float32) for t in (x, w, g))
    M, K = x32.shape
    N = w32.shape[1]
    # forward
    xq, xs = fo.quantize_to_fp8(x32)
    if tuple(weight_tile) == (128, 128):
        wq, ws = fo.quantize_block2d(w32)
        ws_full = np.repeat(np.repeat(ws, 128, axis=0)[:K], 128, axis=1)
        wq_d, ws_d = wq, ws_full
    else:
        wq, ws = fo.quantize_colwise(w32)
        ws_full = np.repeat(ws, 128, axis=0)[:K]
        wq_d, s_d = fo.quantize_to_fp8(w32)
        ws_d = np.repeat(s_d, 128, axis=1)
    y = _deq(xq, np.repeat(xs, 128, axis=1)) @ _deq(wq, ws_full)
    # dgrad
    gq, gs = fo.quantize_to_fp8(g32)
    dx = _deq(gq, np.repeat(gs, 128, axis=1)) @ _deq(wq_d, ws_d).T
    # wgrad
    xqc, xsc = fo.quantize_colwise(x32)
    gqc, gsc = fo.quantize_colwise(g32)
    dw = _deq(xqc, np.repeat(xsc, 128, axis=0)[:M]).T @ _deq(gqc, np.repeat(gsc, 128, axis=0)[:M])
    return y, dx, dw


def time_linear_set(shapes, m_sample: int, seed: int = 0, repeats: int = 1):
    """Time `linear_fwd_bwd` over (K, N) `shapes` on `m_sample` tokens.  Returns
    (seconds per pass over the set, flops per pass)."""
    rng = np.random.default_rng(seed)
    data = []
    flops = 0.0
    for K, N in shapes:
        x = rng.standard_normal((m_sample, K)).astype(np.float32).astype(fo.BF16)
        w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32).astype(fo.BF16)
        g = rng.standard_normal((m_sample, N)).astype(np.float32).astype(fo.BF16)
        data.append((x, w, g))
        flops += 6.0 * m_sample * K * N
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        for x, w, g in data:
            linear_fwd_bwd(x, w, g)
        best = min(best, time.perf_counter() - t0)
    return best, flops
