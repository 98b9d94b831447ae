"""Generate `tests/golden/reference_vectors.npz` from the reference's own source.

Run once, in a container that has the reference checkout (its path is argv[1]):

    python tests/golden/make_golden.py /path/to/train-gpt

JAX is not installable there, so the reference modules `fp8.py` and `kernels.py`
are imported UNMODIFIED with a tiny stand-in for the `jax` package: `jax.numpy` is
NumPy, the float8/bfloat16 dtypes are ml_dtypes' (the library JAX itself uses for
those casts), `jax.lax.rsqrt` is a correctly rounded float32 rsqrt, reductions
(`mean`, `sum`) accumulate in float64 and round once to float32 (XLA leaves the
order unspecified), and `@` on bf16 arrays accumulates in float64 and rounds to
f32 then bf16 (a bf16 GEMM with an f32 accumulator).  `jax.nn.scaled_matmul` and
`pallas_call` are NOT emulated -- nothing here calls them.

What gets stored (bf16 as uint16 bit patterns, e4m3 as uint8):
  * `_quantize_to_fp8` on activations and on `b.T`           (fp8.py:39-47, :66, :68)
  * `_fp8_backward`                                           (fp8.py:85-98)
  * `_rms_norm_pure`                                          (kernels.py:30-33)
  * the custom-VJP `_bwd` of the GPU norm                     (kernels.py:104-118)
  * `cross_entropy_loss` on given capped logits               (losses.py:8-12; `model.forward`
    and `config.Config` are stubbed, log_softmax is the float64 formula rounded once)
The test-suite never imports the reference; it reads only the .npz.
"""
import functools
import importlib
import os
import sys
import types

import ml_dtypes
import numpy as np

BF16 = ml_dtypes.bfloat16
F8 = ml_dtypes.float8_e4m3fn


class Arr(np.ndarray):
    """ndarray whose `@` follows XLA's bf16 dot: wide accumulate, one rounding."""

    def __matmul__(self, other):
        out = np.asarray(self).astype(np.float64) @ np.asarray(other).astype(np.float64)
        out = out.astype(np.float32)
        if self.dtype == BF16:
            out = out.astype(BF16)
        return out.view(Arr)


def _wrap(x):
    return np.asarray(x).view(Arr)


def _install_jax_stand_in():
    jax = types.ModuleType("jax")
    jnp = types.ModuleType("jax.numpy")
    lax = types.ModuleType("jax.lax")
    nn = types.ModuleType("jax.nn")
    exp = types.ModuleType("jax.experimental")
    pallas = types.ModuleType("jax.experimental.pallas")

    jnp.float32 = np.float32
    jnp.bfloat16 = BF16
    jnp.float8_e4m3fn = F8
    jnp.abs = np.abs
    jnp.max = np.max
    jnp.maximum = np.maximum
    jnp.tile = np.tile
    jnp.take_along_axis = lambda a, i, axis: _wrap(np.take_along_axis(np.asarray(a), np.asarray(i), axis=axis))

    def log_softmax(x, axis=-1):
        x64 = np.asarray(x).astype(np.float64)
        m = x64.max(axis=axis, keepdims=True)
        return _wrap((x64 - m - np.log(np.exp(x64 - m).sum(axis=axis, keepdims=True))).astype(np.float32))

    nn.log_softmax = log_softmax

    def mean(x, axis=None, keepdims=False):
        return _wrap(np.mean(np.asarray(x).astype(np.float64), axis=axis, keepdims=keepdims).astype(np.float32))

    def sum_(x, axis=None, keepdims=False):
        return _wrap(np.sum(np.asarray(x).astype(np.float64), axis=axis, keepdims=keepdims).astype(np.float32))

    jnp.mean = mean
    jnp.sum = sum_

    def rsqrt(v):
        return _wrap((1.0 / np.sqrt(np.asarray(v, dtype=np.float32).astype(np.float64))).astype(np.float32))

    lax.rsqrt = rsqrt
    lax.optimization_barrier = lambda x: x

    class custom_vjp:
        def __init__(self, fn, nondiff_argnums=()):
            self.fn = fn
            functools.update_wrapper(self, fn)

        def __call__(self, *a, **k):
            return self.fn(*a, **k)

        def defvjp(self, fwd, bwd):
            self.fwd, self.bwd = fwd, bwd

    jax.custom_vjp = custom_vjp
    jax.Array = np.ndarray
    jax.default_backend = lambda: "cpu"
    jax.numpy, jax.lax, jax.nn, jax.experimental = jnp, lax, nn, exp
    exp.pallas = pallas
    for name, mod in [("jax", jax), ("jax.numpy", jnp), ("jax.lax", lax), ("jax.nn", nn),
                      ("jax.experimental", exp), ("jax.experimental.pallas", pallas)]:
        sys.modules[name] = mod


def main(ref_dir: str):
    _install_jax_stand_in()
    sys.path.insert(0, ref_dir)
    fp8 = importlib.import_module("fp8")
    kernels = importlib.import_module("kernels")
    out = {}
    rng = np.random.default_rng(20240607)

    # ---- quantiser on an activation with awkward tiles -------------------------------
    x = rng.standard_normal((48, 384)).astype(np.float32)
    x[rng.random(x.shape) < 0.01] *= 50.0           # outliers
    x[3, 128:256] = 0.0                              # all-zero tile -> scale 1e-30
    x[4, 0:128] = 1e-36                              # amax/448 below the 1e-30 floor
    x[5, 256:384] *= 1e-20                           # tiny but above the floor
    x[6, 7] = -0.0
    x_bf = x.astype(BF16)
    q, s = fp8._quantize_to_fp8(_wrap(x_bf).astype(np.float32), 128)
    out["q_act_in"] = x_bf.view(np.uint16)
    out["q_act_bytes"] = np.asarray(q).view(np.uint8)
    out["q_act_scales"] = np.asarray(s)

    # ---- quantiser on b.T, as the forward does (fp8.py:68) --------------------------
    b = (rng.standard_normal((256, 192)) * 0.02).astype(BF16)
    q, s = fp8._quantize_to_fp8(_wrap(b).T.astype(np.float32), 128)
    out["q_w_in"] = b.view(np.uint16)
    out["q_wt_bytes"] = np.asarray(q).view(np.uint8)       # (N, K)
    out["q_wt_scales"] = np.asarray(s)                      # (N, K/128)

    # ---- the reference's closed-form case (debug_fp8.py:105-109) --------------------
    q, s = fp8._quantize_to_fp8(_wrap(np.ones((4, 128), np.float32)), 128)
    out["q_ones_bytes"] = np.asarray(q).view(np.uint8)
    out["q_ones_scales"] = np.asarray(s)

    # ---- straight-through backward (fp8.py:85-98) -----------------------------------
    a = rng.standard_normal((2, 24, 256)).astype(BF16)
    g = rng.standard_normal((2, 24, 192)).astype(BF16)
    da, db = fp8._fp8_backward(128, (_wrap(a), _wrap(b)), _wrap(g))
    out["ste_a"] = a.view(np.uint16)
    out["ste_g"] = g.view(np.uint16)
    out["ste_da"] = np.asarray(da).view(np.uint16)
    out["ste_db"] = np.asarray(db).view(np.uint16)

    # ---- pure norm (kernels.py:30-33), 3-D input, non-uniform scale -----------------
    xn = rng.standard_normal((3, 20, 256)).astype(np.float32)
    xn[rng.random(xn.shape) < 0.005] *= 50.0
    xn = xn.astype(BF16)
    gamma = (1.0 + 0.1 * rng.standard_normal(256)).astype(BF16)
    eps = 1e-5
    y = kernels._rms_norm_pure(_wrap(xn), _wrap(gamma), eps)
    out["norm_x"] = xn.view(np.uint16)
    out["norm_gamma"] = gamma.view(np.uint16)
    out["norm_eps"] = np.float32(eps)
    out["norm_pure_y"] = np.asarray(y).view(np.uint16)

    # ---- backward of the GPU norm (kernels.py:104-118) ------------------------------
    gpu_norm = kernels._build_gpu_rms_norm()
    gy = rng.standard_normal(xn.shape).astype(BF16)
    dx, dgamma = gpu_norm.bwd(eps, (_wrap(xn), _wrap(gamma)), _wrap(gy))
    out["norm_gy"] = gy.view(np.uint16)
    out["norm_dx"] = np.asarray(dx).view(np.uint16)
    out["norm_dgamma"] = np.asarray(dgamma).view(np.uint16)

    # ---- cross-entropy on capped logits (losses.py:8-12) -----------------------------
    ce_logits = (rng.standard_normal((40, 512)) * 6.0).clip(-15, 15).astype(BF16)
    ce_targets = rng.integers(0, 512, size=(40,)).astype(np.int32)
    model_stub = types.ModuleType("model")
    model_stub.forward = lambda params, input_ids, cfg: _wrap(ce_logits)
    config_stub = types.ModuleType("config")
    config_stub.Config = object
    sys.modules["model"], sys.modules["config"] = model_stub, config_stub
    losses = importlib.import_module("losses")
    ce = losses.cross_entropy_loss(None, None, _wrap(ce_targets), None)
    del sys.modules["model"], sys.modules["config"]
    out["ce_logits"] = ce_logits.view(np.uint16)
    out["ce_targets"] = ce_targets
    out["ce_loss"] = np.float32(ce)

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1])
