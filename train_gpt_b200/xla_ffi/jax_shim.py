"""train-gpt's `fp8.py` and `kernels.py` call surface in JAX, bound to the B200 kernels through
`jax.ffi`: the file a train-gpt maintainer drops next to (or in place of) the reference's own.

    from train_gpt_b200.xla_ffi.jax_shim import block_scaled_matmul, rms_norm, _rms_norm_pure

`block_scaled_matmul(a, b, block_k=128)` keeps the reference's signature, its two ValueErrors
and its `jax.custom_vjp` with `nondiff_argnums=(2,)` (fp8.py:30-36, :50-56, :101); the forward
rule calls the quantisers and the tcgen05 GEMM instead of `_quantize_to_fp8` + `jax.nn.scaled_matmul`
(fp8.py:66-76), the backward rule is the reference's bf16 straight-through pair (fp8.py:85-98) or,
with `backward="fp8"`, the block-scaled dgrad / wgrad.  `rms_norm(x, scale, eps)` keeps
kernels.py:55-56 (positional, eps static, differentiable in x and scale).

Needs jax with the `jax.ffi` module and `libtg_xla.so` built by `build.py` next to this file.
Importing this module without them raises ImportError: there is no other path.
"""
from __future__ import annotations

import ctypes
import os
from functools import partial

import numpy as np

try:
    import jax
    import jax.numpy as jnp
    from jax import ffi as jffi
except ImportError as e:   # jax is not part of this image; the shim is source for a JAX host
    raise ImportError("train_gpt_b200.xla_ffi.jax_shim needs jax with jax.ffi") from e

E4M3_MAX = 448.0         # fp8.py:26
DEFAULT_BLOCK_K = 128    # fp8.py:27

_HERE = os.path.dirname(os.path.abspath(__file__))

# every handler xla_ffi.cc defines with XLA_FFI_DEFINE_HANDLER_SYMBOL
FFI_TARGETS = (
    "TgQuantizeRowwise", "TgQuantizeColwise", "TgQuantizeBlock128", "TgQuantizeRowcol", "TgQuantizeRowcolInto",
    "TgActQuantizeRowcol", "TgActQuantizeRowcolBwd",
    "TgRmsnormFwd", "TgRmsnormQuantFwd", "TgAddRmsnormQuantFwd", "TgRmsnormBwd", "TgRmsnormBwdAdd", "TgRmsnormBwdStatic",
    "TgSoftcapCeFwd", "TgSoftcapCeBwd", "TgSumsqBf16", "TgAdamwBf16",
    "TgGemmFwd", "TgGemmDgrad", "TgGemmWgrad",
)

_registered = False


def register(lib_path: str | None = None) -> None:
    """Load libtg_xla.so and register every handler as a CUDA FFI target (idempotent)."""
    global _registered
    if _registered:
        return
    path = lib_path or os.environ.get("TG_XLA_LIB") or os.path.join(_HERE, "libtg_xla.so")
    if not os.path.exists(path):
        raise ImportError(f"{path} not found: build it with `python -m train_gpt_b200.xla_ffi.build`")
    lib = ctypes.CDLL(path)
    for name in FFI_TARGETS:
        jffi.register_ffi_target(name, jffi.pycapsule(getattr(lib, name)), platform="CUDA")
    _registered = True


def _sds(shape, dtype):
    return jax.ShapeDtypeStruct(tuple(int(d) for d in shape), dtype)


def _cdiv(a, b):
    return -(-a // b)


# ---- quantisers (fp8.py:39-47) ------------------------------------------------------------------

def _quantize_to_fp8(x, block_k: int = DEFAULT_BLOCK_K):
    """fp8.py:39-47 on a bf16 (or upcast bf16) tensor: 1 x 128 tiles along the last axis."""
    K = x.shape[-1]
    if K % block_k != 0:
        raise ValueError(f"K={K} not divisible by block_k={block_k}")
    register()
    x = x.astype(jnp.bfloat16)
    return jffi.ffi_call("TgQuantizeRowwise", (_sds(x.shape, jnp.float8_e4m3fn),
                                               _sds((*x.shape[:-1], K // block_k), jnp.float32)))(x)


def _quantize_colwise(x):
    register()
    R, C = x.shape
    return jffi.ffi_call("TgQuantizeColwise", (_sds((R, C), jnp.float8_e4m3fn), _sds((_cdiv(R, 128), C), jnp.float32)))(x)


def _quantize_block128(x):
    register()
    R, C = x.shape
    return jffi.ffi_call("TgQuantizeBlock128", (_sds((R, C), jnp.float8_e4m3fn), _sds((_cdiv(R, 128), C // 128), jnp.float32)))(x)


def _quantize_rowcol(x):
    register()
    R, C = x.shape
    return jffi.ffi_call("TgQuantizeRowcol", (_sds((R, C), jnp.float8_e4m3fn), _sds((R, C // 128), jnp.float32),
                                              _sds((R, C), jnp.float8_e4m3fn), _sds((_cdiv(R, 128), C), jnp.float32)))(x)


# ---- GEMMs ----------------------------------------------------------------------------------------

_WORKSPACE_CAP = 1 << 28    # scratch result XLA plans for a cut contraction (float32 partial sums); 0 disables the cut


def _gemm(target, attr, a_q, a_s, b_q, b_s, M, N, gran, workspace_bytes):
    out = (_sds((M, N), jnp.bfloat16), _sds((1,), jnp.uint32), _sds((max(workspace_bytes, 16),), jnp.uint8))
    y, _status, _ws = jffi.ffi_call(target, out)(a_q, a_s, b_q, b_s, **{attr: np.int32(gran)})   # int32 attribute
    return y


def _workspace(M, N, K):
    """Upper bound of what tg_gemm_workspace_bytes can ask for (8 float32 slices), capped."""
    need = 8 * M * N * 4
    return need if (M * N <= 148 * 128 * 256 and K >= 2048 and need <= _WORKSPACE_CAP) else 0


def _fp8_forward(a, b, block_k, weight_tile=(128, 1)):
    """fp8.py:50-78."""
    K = a.shape[-1]
    K_b, N = b.shape
    if K != K_b:
        raise ValueError(f"contracted-dim mismatch: a K={K}, b K={K_b}")           # fp8.py:53-54
    if K % block_k != 0:
        raise ValueError(f"K={K} not divisible by block_k={block_k}")              # fp8.py:55-56
    if block_k != DEFAULT_BLOCK_K:
        raise ValueError(f"block_k={block_k} is not supported by the sm_100a kernels (only {DEFAULT_BLOCK_K})")
    lead = a.shape[:-1]
    a2 = a.reshape(-1, K).astype(jnp.bfloat16)                                     # fp8.py:65
    a_q, a_s = _quantize_to_fp8(a2, block_k)                                       # fp8.py:66
    b = b.astype(jnp.bfloat16)
    if tuple(weight_tile) == (128, 1):
        b_q, b_s = _quantize_colwise(b)                                            # fp8.py:68 without b.T
        gran = 1
    else:
        b_q, b_s = _quantize_block128(b)
        gran = 128
    M = a2.shape[0]
    y = _gemm("TgGemmFwd", "weight_gran", a_q, a_s, b_q, b_s, M, N, gran, _workspace(M, N, K))   # fp8.py:70-78
    return y.reshape(*lead, N)


def _fp8_backward_ste(a, b, g):
    """fp8.py:85-98: gradients of a plain bf16 matmul."""
    K = a.shape[-1]
    N = b.shape[1]
    a2 = a.reshape(-1, K).astype(jnp.bfloat16)
    g2 = g.reshape(-1, N).astype(jnp.bfloat16)
    b2 = b.astype(jnp.bfloat16)
    da = jnp.matmul(g2, b2.T, preferred_element_type=jnp.float32).astype(a.dtype).reshape(a.shape)   # fp8.py:96
    db = jnp.matmul(a2.T, g2, preferred_element_type=jnp.float32).astype(b.dtype)                    # fp8.py:97
    return da, db


def _fp8_backward_fp8(a, b, g, weight_tile):
    """The same two GEMMs in block-scaled e4m3: every operand in 1 x 128 tiles along its contraction."""
    K = a.shape[-1]
    N = b.shape[1]
    a2 = a.reshape(-1, K).astype(jnp.bfloat16)
    g2 = g.reshape(-1, N).astype(jnp.bfloat16)
    b2 = b.astype(jnp.bfloat16)
    T = a2.shape[0]
    g_q, g_s, g_qc, g_sc = _quantize_rowcol(g2)
    if tuple(weight_tile) == (128, 1):
        w_q, w_s = _quantize_to_fp8(b2)
        gran = 1
    else:
        w_q, w_s = _quantize_block128(b2)
        gran = 128
    da = _gemm("TgGemmDgrad", "weight_gran", g_q, g_s, w_q, w_s, T, K, gran, _workspace(T, K, N))
    x_qc, x_sc = _quantize_colwise(a2)
    db = _gemm("TgGemmWgrad", "grad_gran", x_qc, x_sc, g_qc, g_sc, K, N, 1, _workspace(K, N, T))
    return da.reshape(a.shape).astype(a.dtype), db.astype(b.dtype)


@partial(jax.custom_vjp, nondiff_argnums=(2, 3, 4))
def _block_scaled_matmul(a, b, block_k, weight_tile, backward):
    return _fp8_forward(a, b, block_k, weight_tile)


def _bsm_fwd(a, b, block_k, weight_tile, backward):
    return _fp8_forward(a, b, block_k, weight_tile), (a, b)                         # fp8.py:81-82


def _bsm_bwd(block_k, weight_tile, backward, res, g):
    a, b = res
    if backward == "bf16_ste":
        return _fp8_backward_ste(a, b, g)
    return _fp8_backward_fp8(a, b, g, weight_tile)


_block_scaled_matmul.defvjp(_bsm_fwd, _bsm_bwd)


def block_scaled_matmul(a, b, block_k: int = DEFAULT_BLOCK_K, *, weight_tile=(128, 1), backward: str = "bf16_ste"):
    """Per-K-tile block-scaled FP8 matmul (fp8.py:30-36).  a: (..., K), b: (K, N) -> (..., N) bf16."""
    if backward not in ("bf16_ste", "fp8"):
        raise ValueError(f"unknown backward mode {backward!r}; use 'bf16_ste' or 'fp8'")
    return _block_scaled_matmul(a, b, block_k, tuple(weight_tile), backward)


# ---- RMSNorm (kernels.py) ---------------------------------------------------------------------------

TG_NORM_FUSED, TG_NORM_PURE = 0, 1


def _norm_call(x, scale, eps, mode):
    register()
    y, _rnorm = jffi.ffi_call("TgRmsnormFwd", (_sds(x.shape, jnp.bfloat16), _sds(x.shape[:-1], jnp.float32)))(
        x.astype(jnp.bfloat16), scale.astype(jnp.bfloat16), eps=np.float32(eps), mode=np.int32(mode))
    return y


def _norm_bwd_call(x, scale, g, eps):
    register()
    return jffi.ffi_call("TgRmsnormBwdStatic", (_sds(x.shape, jnp.bfloat16), _sds(scale.shape, jnp.bfloat16)))(
        x.astype(jnp.bfloat16), scale.astype(jnp.bfloat16), g.astype(jnp.bfloat16), eps=np.float32(eps))


def _make_norm(mode):
    @partial(jax.custom_vjp, nondiff_argnums=(2,))
    def norm(x, scale, eps):
        return _norm_call(x, scale, eps, mode)

    def fwd(x, scale, eps):
        return _norm_call(x, scale, eps, mode), (x, scale)                         # kernels.py:101-102

    def bwd(eps, res, g):
        x, scale = res
        return _norm_bwd_call(x, scale, g, eps)                                    # kernels.py:104-118

    norm.defvjp(fwd, bwd)
    return norm


rms_norm = _make_norm(TG_NORM_FUSED)          # kernels.py:55-99
_rms_norm_pure = _make_norm(TG_NORM_PURE)     # kernels.py:30-33


def rms_norm_quant(x, scale, eps):
    """Norm + 1 x 128 quantise in one kernel: (q e4m3, scales f32, y bf16) for GEMMs that share the
    normed activation (model.py:63-65,72)."""
    register()
    D = x.shape[-1]
    q, s, y, _rn = jffi.ffi_call("TgRmsnormQuantFwd", (_sds(x.shape, jnp.float8_e4m3fn), _sds((*x.shape[:-1], D // 128), jnp.float32),
                                                        _sds(x.shape, jnp.bfloat16), _sds(x.shape[:-1], jnp.float32)))(
        x.astype(jnp.bfloat16), scale.astype(jnp.bfloat16), eps=np.float32(eps), mode=np.int32(TG_NORM_FUSED))
    return q, s, y
