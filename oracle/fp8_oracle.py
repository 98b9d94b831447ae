"""CPU oracle for the per-block-scaled FP8 matmul of train-gpt (`fp8.py`).

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; only
`tests/`, `__graft_entry__.smoke()` and the `cpu_baseline` / `--impl reference`
legs of `bench.py` do, and there only as the checker or as the timed CPU
baseline.

Every function restates, in NumPy + ml_dtypes, the arithmetic visible in the
reference at the cited lines.  The reference is JAX; JAX cannot be installed
where this runs, so the reference itself is never imported here.

Pin status
----------
* quantiser (`quantize_to_fp8`): PINNED.  `tests/golden/make_golden.py` executed
  the reference's own `fp8._quantize_to_fp8` source with NumPy + ml_dtypes
  standing in for `jax.numpy` (ml_dtypes is the library JAX itself uses for the
  float8 cast) and stored bytes + scales; `tests/test_oracle.py` checks this
  restatement against those fixtures, and against the reference's only
  closed-form known answer (ones(4,128) @ ones(128,4) -> 128, every byte 0x7E,
  `debug_fp8.py:105-109`).
* block-scaled contraction (`scaled_matmul`): PARITY UNPINNED.  The arithmetic
  lives in `jax.nn.scaled_matmul` (jax 0.10.0, pinned in `uv.lock`), whose source
  is not part of the reference tree and which has no CPU lowering
  (`check_fp8_hlo.py:3`); the reference holds no stored outputs for it.  This file
  restates the documented block-scaled-dot semantics
  `out[m,n] = sum_kb a_s[m,kb] * b_s[n,kb] * sum_{k in kb} a_q[m,k] * b_q[n,k]`
  with the inner sums exact (float64) and the outer sum in float64.
* straight-through backward (`backward_bf16_ste`): restates `fp8.py:85-98`
  (plain bf16 matmuls, f32 accumulate); pinned only by construction.
"""
from __future__ import annotations

import ml_dtypes
import numpy as np

E4M3_MAX = 448.0          # fp8.py:26
DEFAULT_BLOCK_K = 128     # fp8.py:27

F8 = ml_dtypes.float8_e4m3fn
BF16 = ml_dtypes.bfloat16


def to_bf16(x) -> np.ndarray:
    """Round an array to bfloat16 (RNE), as `.astype(jnp.bfloat16)` does."""
    return np.asarray(x).astype(BF16)


def _scale_from_amax(amax: np.ndarray) -> np.ndarray:
    # fp8.py:44 -- `jnp.maximum(amax / E4M3_MAX, 1e-30)` in float32; np.maximum
    # propagates NaN the same way jnp.maximum does.
    return np.maximum(amax.astype(np.float32) / np.float32(E4M3_MAX), np.float32(1e-30))


def quantize_to_fp8(x_f32: np.ndarray, block_k: int = DEFAULT_BLOCK_K):
    """fp8.py:39-47.  Tiles of `block_k` along the last axis.

    Returns (q, scales): q has x's shape, dtype float8_e4m3fn; scales has shape
    (..., K // block_k), float32.
    """
    x_f32 = np.asarray(x_f32, dtype=np.float32)
    *leading, K = x_f32.shape
    n_tiles = K // block_k
    tiled = x_f32.reshape(*leading, n_tiles, block_k)            # fp8.py:42
    amax = np.max(np.abs(tiled), axis=-1)                         # fp8.py:43
    scales = _scale_from_amax(amax)                               # fp8.py:44
    with np.errstate(invalid="ignore", divide="ignore"):
        quant = tiled / scales[..., None]                         # fp8.py:45
    q = quant.astype(F8).reshape(*leading, K)                     # fp8.py:46
    return q, scales


def quantize_colwise(x_f32: np.ndarray, block: int = DEFAULT_BLOCK_K):
    """Tiles of `block` rows x 1 column of a 2-D array (scale per column per row block).

    This is the granularity the reference gives the weight: it quantises `b.T`
    (N, K) with 1x128 tiles along K (fp8.py:68), i.e. 128x1 tiles of b (K, N).
    `quantize_colwise(b)` == `quantize_to_fp8(b.T)` transposed back: q (K, N),
    scales (ceil(K/128), N).  A ragged last row block takes its amax over the rows
    that exist.
    """
    x_f32 = np.asarray(x_f32, dtype=np.float32)
    R, C = x_f32.shape
    nb = -(-R // block)
    q = np.empty((R, C), dtype=F8)
    scales = np.empty((nb, C), dtype=np.float32)
    for i in range(nb):
        blk = x_f32[i * block:(i + 1) * block]
        amax = np.max(np.abs(blk), axis=0)
        s = _scale_from_amax(amax)
        scales[i] = s
        with np.errstate(invalid="ignore", divide="ignore"):
            q[i * block:(i + 1) * block] = (blk / s[None, :]).astype(F8)
    return q, scales


def quantize_block2d(x_f32: np.ndarray, block: int = DEFAULT_BLOCK_K):
    """Tiles of `block` x `block` (one scale per tile): the weight granularity the
    benchmark configurations name.  Same scale rule as fp8.py:43-46.  Rows may be
    ragged; columns must be a multiple of `block`."""
    x_f32 = np.asarray(x_f32, dtype=np.float32)
    R, C = x_f32.shape
    if C % block:
        raise ValueError(f"C={C} not divisible by block={block}")
    nb = -(-R // block)
    q = np.empty((R, C), dtype=F8)
    scales = np.empty((nb, C // block), dtype=np.float32)
    for i in range(nb):
        blk = x_f32[i * block:(i + 1) * block].reshape(-1, C // block, block)
        amax = np.max(np.abs(blk), axis=(0, 2))
        s = _scale_from_amax(amax)
        scales[i] = s
        with np.errstate(invalid="ignore", divide="ignore"):
            q[i * block:(i + 1) * block] = (blk / s[None, :, None]).astype(F8).reshape(-1, C)
    return q, scales


def scaled_matmul(a_q, b_q_t, a_s, b_s, block_k: int = DEFAULT_BLOCK_K) -> np.ndarray:
    """Semantics of the call at fp8.py:70-76 (batch dim dropped).

    a_q (M, K) e4m3, b_q_t (N, K) e4m3, a_s (M, K/bk) f32, b_s (N, K/bk) f32 ->
    (M, N) float32.  Inner sums are exact in float64 (an e4m3 product has 8
    significant bits; 128 of them span < 53 bits).
    """
    a_q = np.asarray(a_q)
    b_q_t = np.asarray(b_q_t)
    M, K = a_q.shape
    N = b_q_t.shape[0]
    out = np.zeros((M, N), dtype=np.float64)
    for kb in range(K // block_k):
        sl = slice(kb * block_k, (kb + 1) * block_k)
        # operands are widened one block at a time: the sampled full-size checks pass (N, K)
        # arrays of 10^8 elements, whose float64 copy would not fit comfortably in host memory
        part = a_q[:, sl].astype(np.float64) @ b_q_t[:, sl].astype(np.float64).T
        out += part * (a_s[:, kb].astype(np.float64)[:, None] * b_s[:, kb].astype(np.float64)[None, :])
    return out.astype(np.float32)


def _check_shapes(a, b, block_k):
    K = a.shape[-1]
    K_b = b.shape[0]
    if K != K_b:                                                   # fp8.py:53-54
        raise ValueError(f"contracted-dim mismatch: a K={K}, b K={K_b}")
    if K % block_k != 0:                                           # fp8.py:55-56
        raise ValueError(f"K={K} not divisible by block_k={block_k}")


def block_scaled_matmul(a, b, block_k: int = DEFAULT_BLOCK_K, weight_tile=(128, 1)) -> np.ndarray:
    """fp8.py:50-78: a (..., K) bf16, b (K, N) bf16 -> (..., N) bf16.

    weight_tile=(128, 1) is the reference's granularity (fp8.py:68);
    weight_tile=(128, 128) is the benchmark configurations' granularity.
    """
    a = np.asarray(a)
    b = np.asarray(b)
    _check_shapes(a, b, block_k)
    *leading, K = a.shape
    N = b.shape[1]
    a2 = a.reshape(-1, K).astype(np.float32)                       # fp8.py:65-66
    a_q, a_s = quantize_to_fp8(a2, block_k)
    b32 = b.astype(np.float32)
    if tuple(weight_tile) == (128, 1):
        b_q_t, b_s = quantize_to_fp8(b32.T, block_k)               # fp8.py:68
    elif tuple(weight_tile) == (128, 128):
        q, s = quantize_block2d(b32, block_k)                      # (K,N), (K/128, N/128)
        b_q_t = q.T
        b_s = np.repeat(s.T, block_k, axis=0)                      # (N, K/128)
    else:
        raise ValueError(f"unsupported weight_tile {weight_tile}")
    out = scaled_matmul(a_q, b_q_t, a_s, b_s, block_k)             # fp8.py:70-76
    return out.astype(BF16).reshape(*leading, N)                   # fp8.py:78


def backward_bf16_ste(a, b, g):
    """fp8.py:85-98: gradients of a plain bf16 matmul on the unquantised operands.

    bf16 products are exact in f32; the sums are taken in float32-or-better (here
    float64, rounded once to bf16), as a bf16 GEMM with an f32 accumulator does up
    to summation order.
    """
    a = np.asarray(a)
    b = np.asarray(b)
    g = np.asarray(g)
    *leading, K = a.shape
    N = b.shape[1]
    a2 = a.reshape(-1, K).astype(BF16).astype(np.float64)          # fp8.py:93
    g2 = g.reshape(-1, N).astype(BF16).astype(np.float64)          # fp8.py:94
    b2 = b.astype(BF16).astype(np.float64)                         # fp8.py:95
    da = (g2 @ b2.T).astype(np.float32).astype(BF16).reshape(*leading, K)   # fp8.py:96
    db = (a2.T @ g2).astype(np.float32).astype(BF16)               # fp8.py:97
    return da, db


def backward_fp8(a, b, g, block: int = DEFAULT_BLOCK_K, weight_tile=(128, 1), wgrad_grad_tile=(128, 1)):
    """Like-for-like oracle of the FP8 backward this build adds (the reference's own
    backward is `backward_bf16_ste`).  Same quantiser (fp8.py:39-47) applied along
    each GEMM's contraction:

      dgrad  da[m,k] = sum_n g[m,n] b[k,n]   g tiles 1x128 along N; b tiles 1x128
                                             along N (weight_tile (128,1)) or the
                                             shared 128x128 tiles.
      wgrad  db[k,n] = sum_m a[m,k] g[m,n]   a and g tiles 128x1 along the tokens
                                             (wgrad_grad_tile (128,128): g in 128x128 blocks).
    """
    a = np.asarray(a)
    b = np.asarray(b)
    g = np.asarray(g)
    *leading, K = a.shape
    N = b.shape[1]
    a2 = a.reshape(-1, K).astype(np.float32)
    g2 = g.reshape(-1, N).astype(np.float32)
    b32 = b.astype(np.float32)
    if N % block:
        raise ValueError(f"N={N} not divisible by block={block}")
    # dgrad: contraction over N
    g_q, g_s = quantize_to_fp8(g2, block)                          # (M,N), (M,N/128)
    if tuple(weight_tile) == (128, 1):
        w_q, w_s = quantize_to_fp8(b32, block)                     # (K,N), (K,N/128)
    else:
        w_q, s = quantize_block2d(b32, block)
        w_s = np.repeat(s, block, axis=0)[:K]                      # (K, N/128)
    da = scaled_matmul(g_q, w_q, g_s, w_s, block).astype(BF16).reshape(*leading, K)
    # wgrad: contraction over the tokens (ragged last block allowed)
    M = a2.shape[0]
    a_q, a_s = quantize_colwise(a2, block)                         # (M,K), (Mb,K)
    if tuple(wgrad_grad_tile) == (128, 1):
        gq2, gs2 = quantize_colwise(g2, block)                     # (M,N), (Mb,N)
    else:
        gq2, gs_b = quantize_block2d(g2, block)                    # (M,N), (Mb,N/128)
        gs2 = np.repeat(gs_b, block, axis=1)
    pad = (-M) % block
    aq = np.pad(a_q.astype(np.float32), ((0, pad), (0, 0))).astype(F8)
    gq = np.pad(gq2.astype(np.float32), ((0, pad), (0, 0))).astype(F8)
    db = scaled_matmul(aq.T, gq.T, a_s.T, gs2.T, block).astype(BF16)
    return da, db


def rel_frobenius(x, ref) -> float:
    """bench_fp8.py:144-152: ||x - ref||_F / ||ref||_F in float64."""
    x = np.asarray(x).astype(np.float64)
    ref = np.asarray(ref).astype(np.float64)
    return float(np.linalg.norm(x - ref) / max(np.linalg.norm(ref), 1e-300))


def tolerance_violations(x, ref, rtol: float = 2e-2, atol_rms: float = 1e-2) -> int:
    """Count of elements with |x-ref| > atol_rms*RMS(ref) + rtol*|ref| (the stated
    GEMM/gradient tolerance)."""
    x = np.asarray(x).astype(np.float64)
    ref = np.asarray(ref).astype(np.float64)
    rms = np.sqrt(np.mean(ref * ref))
    return int(np.sum(np.abs(x - ref) > atol_rms * rms + rtol * np.abs(ref)))
