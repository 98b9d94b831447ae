"""Per-block-scaled FP8 matmul: the call surface of train-gpt's `fp8.py` on B200 kernels.

`block_scaled_matmul(a, b, block_k=128)` keeps the reference's signature, error messages
and differentiation contract (train-gpt fp8.py:30-36, :50-78, :85-101): differentiable in
`a` and `b`, `block_k` static, gradients returned in the inputs' dtypes.

Keyword-only extras (defaults reproduce the reference):
  weight_tile  (128, 1)    the reference's weight-scale granularity (it quantises `b.T`
                           along K, fp8.py:68); (128, 128) is the benchmark granularity.
  backward     "bf16_ste"  the reference's straight-through bf16 backward (fp8.py:85-98);
                           "fp8" runs dgrad and wgrad as block-scaled e4m3 GEMMs as well
                           (every operand in 1x128 tiles along its contraction);
                           "fp8_blockgrad" is "fp8" with the upstream gradient quantised in
                           128x128 blocks for wgrad only: coarser, and about twice as fast there.
"""
from __future__ import annotations

import torch

from . import ops

E4M3_MAX = 448.0        # fp8.py:26
DEFAULT_BLOCK_K = 128   # fp8.py:27


def _as_bf16(t: torch.Tensor, name: str) -> torch.Tensor:
    """bf16 view of an operand.  The reference upcasts its bf16 operands to float32 before quantising
    (fp8.py:66,68); these kernels take the bf16 directly.  A wider tensor is taken only if the narrowing
    is exact, so that scales and bytes cannot silently differ from the reference's."""
    if t.dtype == torch.bfloat16:
        return t
    if not t.is_floating_point():
        raise TypeError(f"{name} must be a floating-point tensor, got {t.dtype}")
    n = t.to(torch.bfloat16)
    if not bool((n.to(t.dtype) == t).all()):
        raise TypeError(f"{name} is {t.dtype} with values bf16 cannot hold: the sm_100a kernels quantise bf16 operands "
                        "(as the reference's model does); cast explicitly if that rounding is intended")
    return n


def _check_block(block_k: int):
    if block_k != DEFAULT_BLOCK_K:
        raise ValueError(f"block_k={block_k} is not supported by the sm_100a kernels (only {DEFAULT_BLOCK_K})")


def _quantize_to_fp8(x_f32: torch.Tensor, block_k: int = DEFAULT_BLOCK_K):
    """fp8.py:39-47.  The reference only ever passes an upcast bf16 tensor (fp8.py:66,68), and the
    kernels read bf16: a float32 argument is accepted only if it holds bf16 values exactly (it is then
    narrowed back without loss); anything else raises rather than being rounded silently."""
    K = x_f32.shape[-1]
    if K % block_k != 0:
        raise ValueError(f"K={K} not divisible by block_k={block_k}")
    _check_block(block_k)
    return ops.quantize_rowwise(_as_bf16(x_f32, "x"))


class QuantizedActivation:
    """One activation in the forms the three GEMMs of a linear layer contract: the row-wise
    (1x128) pair for the forward GEMM and, made on first use and then kept, the column-wise
    (128 tokens x 1) pair for wgrad.  Passing the same object as `a_quantized=` to several
    `block_scaled_matmul` calls (q, k, v share one normed activation, model.py:63-65) makes
    each form once instead of once per call, as the reference does (bench_fp8_norm.py:91-93)."""

    def __init__(self, a: torch.Tensor, q=None, scales=None, q_col=None, scales_col=None):
        K = a.shape[-1]
        self.a2d = a.reshape(-1, K)
        self._row = None if q is None else (q.reshape(-1, K), scales.reshape(-1, K // DEFAULT_BLOCK_K))
        self._col = None if q_col is None else (q_col, scales_col)

    @classmethod
    def both(cls, a: torch.Tensor) -> "QuantizedActivation":
        """Both forms from ONE read of `a` (ops.quantize_rowcol): for an activation whose linear layer will be
        differentiated -- the forward GEMM takes the row form now, the weight-gradient GEMM the column form later."""
        K = a.shape[-1]
        a2d = a.reshape(-1, K).to(torch.bfloat16)
        q, s, qc, sc = ops.quantize_rowcol(a2d)
        return cls(a2d, q, s, qc, sc)

    def rowwise(self):
        if self._row is None:
            self._row = ops.quantize_rowwise(self.a2d.to(torch.bfloat16))
        return self._row

    def colwise(self):
        if self._col is None:
            self._col = ops.quantize_colwise(self.a2d.to(torch.bfloat16))
        return self._col


def quantize_weight(b: torch.Tensor, weight_tile=(128, 1)):
    """Quantise b (K, N) for the forward GEMM without transposing it."""
    if tuple(weight_tile) == (128, 1):
        return ops.quantize_colwise(b)
    if tuple(weight_tile) == (128, 128):
        return ops.quantize_block128(b)
    raise ValueError(f"unsupported weight_tile {weight_tile}")


def _validate(a, b, block_k):
    K = a.shape[-1]
    K_b, N = b.shape
    if K != K_b:                                                    # fp8.py:53-54
        raise ValueError(f"contracted-dim mismatch: a K={K}, b K={K_b}")
    if K % block_k != 0:                                            # fp8.py:55-56
        raise ValueError(f"K={K} not divisible by block_k={block_k}")
    _check_block(block_k)
    return K, N


def _fp8_forward(a, b, block_k=DEFAULT_BLOCK_K, weight_tile=(128, 1), a_quantized=None, return_weight=False):
    """fp8.py:50-78.  `a_quantized` = (q, scales) of `a` made earlier (e.g. by the fused
    norm+quantise kernel) skips the activation quantiser.  return_weight=True also returns the
    quantised weight pair (128x128 tiles serve the backward's dgrad unchanged)."""
    K, N = _validate(a, b, block_k)
    leading = a.shape[:-1]
    if a_quantized is None:
        a_q, a_s = ops.quantize_rowwise(_as_bf16(a.reshape(-1, K), "a"))
    elif isinstance(a_quantized, QuantizedActivation):
        a_q, a_s = a_quantized.rowwise()
    else:
        a_q, a_s = a_quantized[0].reshape(-1, K), a_quantized[1].reshape(-1, K // block_k)
    b = _as_bf16(b, "b")
    pad = (-N) % 16 if tuple(weight_tile) == (128, 1) else 0
    if pad:
        # the TMA row pitch of the (K, N) weight must be a multiple of 16 bytes: widen with
        # zero columns (their tiles quantise to zeros) and drop them from the result
        b = torch.nn.functional.pad(b, (0, pad))
    w_q, w_s = quantize_weight(b, weight_tile)
    y = ops.gemm_fwd(a_q, a_s, w_q, w_s, weight_tile)
    if pad:
        y = y[:, :N]
    y = y.reshape(*leading, N)
    return (y, (w_q, w_s)) if return_weight else y


def _fp8_backward(block_k, residuals, g, weight_tile=(128, 1), mode="bf16_ste", a_quantized=None, w_quantized=None,
                  b_slot=None):
    """fp8.py:85-98 (mode "bf16_ste"), or the same two GEMMs in block-scaled e4m3.
    `w_quantized`: the forward's 128x128-tile weight pair, reused instead of quantising again.
    `b_slot`: a gradient slot of the weight (see `_BlockScaledMatmul.backward`); the FP8 modes then write the
    weight gradient there and return None for it."""
    a, b = residuals
    K = a.shape[-1]
    N = b.shape[1]
    leading = a.shape[:-1]
    a_2d = a.reshape(-1, K).to(torch.bfloat16)
    g_2d = g.reshape(-1, N).to(torch.bfloat16)
    b_bf = b.to(torch.bfloat16)
    if mode == "bf16_ste":
        da = g_2d @ b_bf.T                                          # fp8.py:96 (cuBLAS bf16)
        db = a_2d.T @ g_2d                                          # fp8.py:97
    elif mode in ("fp8", "fp8_blockgrad"):
        if N % block_k != 0:
            raise ValueError(f"N={N} not divisible by block_k={block_k} (needed by the FP8 dgrad)")
        if mode == "fp8":
            g_q, g_s, g_qc, g_sc = ops.quantize_rowcol(g_2d)        # one read of g for both contractions
            grad_tile = (128, 1)
        else:
            g_q, g_s = ops.quantize_rowwise(g_2d)
            g_qc, g_sc = ops.quantize_block128(g_2d)
            grad_tile = (128, 128)
        if tuple(weight_tile) == (128, 1):
            w_q, w_s = ops.quantize_rowwise(b_bf)                   # tiles along N, the dgrad contraction
        elif w_quantized is not None:
            w_q, w_s = w_quantized
        else:
            w_q, w_s = ops.quantize_block128(b_bf)
        da = ops.gemm_dgrad(g_q, g_s, w_q, w_s, weight_tile)
        if isinstance(a_quantized, QuantizedActivation):
            x_qc, x_sc = a_quantized.colwise()                        # shared by every GEMM fed from this activation
        else:
            x_qc, x_sc = ops.quantize_colwise(a_2d)
        if b_slot is not None and b.dtype == torch.bfloat16:
            ops.gemm_wgrad(x_qc, x_sc, g_qc, g_sc, grad_tile=grad_tile, out=b_slot.take())
            b_slot.ready()
            return da.reshape(*leading, K).to(a.dtype), None
        db = ops.gemm_wgrad(x_qc, x_sc, g_qc, g_sc, grad_tile=grad_tile)
    else:
        raise ValueError(f"unknown backward mode {mode!r}; use 'bf16_ste', 'fp8' or 'fp8_blockgrad'")
    return da.reshape(*leading, K).to(a.dtype), db.to(b.dtype)


def _plain_2d(b) -> bool:
    # the direct weight-gradient write needs no padding of N (see _fp8_forward) and a weight as stored
    return b.dim() == 2 and b.shape[1] % 16 == 0


class _BlockScaledMatmul(torch.autograd.Function):
    """The custom VJP of fp8.py:30,101 as a torch.autograd.Function."""

    @staticmethod
    def forward(ctx, a, b, block_k, weight_tile, backward, a_quantized):
        ctx.save_for_backward(a, b)                                 # fp8.py:81-82: unquantised residuals
        ctx.cfg = (block_k, tuple(weight_tile), backward)
        ctx.aq = a_quantized if isinstance(a_quantized, QuantizedActivation) else None
        y, wq = _fp8_forward(a, b, block_k, weight_tile, a_quantized, return_weight=True)
        ctx.wq = wq if (tuple(weight_tile) == (128, 128) and backward != "bf16_ste") else None
        ctx.b_param = b if (isinstance(b, torch.nn.Parameter) and a.dim() >= 2 and _plain_2d(b)) else None
        return y

    @staticmethod
    def backward(ctx, g):
        block_k, weight_tile, mode = ctx.cfg
        # A weight may carry `grad_slot` (an object with take() -> the tensor its gradient belongs in, and
        # ready(); train_gpt_b200.dp.GradSlot): the weight-gradient GEMM then writes straight into the flat
        # gradient bucket and autograd gets None, instead of a fresh tensor that is added into a zeroed bucket.
        slot = getattr(ctx.b_param, "grad_slot", None) if ctx.b_param is not None else None
        da, db = _fp8_backward(block_k, ctx.saved_tensors, g, weight_tile, mode, ctx.aq, ctx.wq, b_slot=slot)
        return da, db, None, None, None, None


def block_scaled_matmul(a: torch.Tensor, b: torch.Tensor, block_k: int = DEFAULT_BLOCK_K, *,
                        weight_tile=(128, 1), backward: str = "bf16_ste", a_quantized=None) -> torch.Tensor:
    """Per-K-tile block-scaled FP8 matmul.

    a: (..., K), b: (K, N) -> (..., N) bf16.  Requires K % block_k == 0.
    """
    _validate(a, b, block_k)
    if backward not in ("bf16_ste", "fp8", "fp8_blockgrad"):
        raise ValueError(f"unknown backward mode {backward!r}; use 'bf16_ste', 'fp8' or 'fp8_blockgrad'")
    return _BlockScaledMatmul.apply(a, b, block_k, tuple(weight_tile), backward, a_quantized)
