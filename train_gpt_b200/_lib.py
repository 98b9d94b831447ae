"""ctypes binding of `libtrain_gpt_b200.so` (the C ABI declared in include/train_gpt_b200.h).

There is no fallback: if the library has not been built, or a launcher returns an error,
this module raises.  Build with `python -m train_gpt_b200.build`.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# TRAIN_GPT_B200_LIB points at another build of the same library (e.g. one with -G or
# different tile constants); it is never a different implementation.
LIB_PATH = os.environ.get("TRAIN_GPT_B200_LIB") or os.path.join(_PKG, "libtrain_gpt_b200.so")

TG_OK, TG_ERR_SHAPE, TG_ERR_ALIGN, TG_ERR_ARCH, TG_ERR_CUDA, TG_ERR_TOO_LARGE = 0, -1, -2, -3, -4, -5
TG_NORM_FUSED, TG_NORM_PURE = 0, 1
TG_MAJOR_K, TG_MAJOR_MN = 0, 1
TG_OUT_BF16, TG_OUT_F32 = 0, 1
TG_ACT = {"relu2": 1, "gelu": 2, "relu2_bwd": 3, "gelu_bwd": 4}

_p, _i64, _f, _i = C.c_void_p, C.c_int64, C.c_float, C.c_int


class GemmArgs(C.Structure):
    """struct tg_gemm_args"""
    _fields_ = [
        ("a", _p), ("b", _p), ("lda", _i64), ("ldb", _i64), ("a_major", _i), ("b_major", _i),
        ("sa", _p), ("sa_stride_m", _i64), ("sa_stride_kb", _i64),
        ("sb", _p), ("sb_stride_n", _i64), ("sb_stride_kb", _i64), ("sb_gran_n", _i),
        ("d", _p), ("ldd", _i64), ("out_dtype", _i),
        ("M", _i64), ("N", _i64), ("K", _i64), ("status", _p),
        ("workspace", _p), ("workspace_bytes", _i64),
    ]


# every symbol include/train_gpt_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "tg_version": (_i, []),
    "tg_last_cuda_error": (C.c_char_p, []),
    "tg_set_gemm_reserved_sms": (_i, [_i]),
    "tg_quantize_rowwise": (_i, [_p, _p, _p, _i64, _i64, _p]),
    "tg_quantize_colwise": (_i, [_p, _p, _p, _i64, _i64, _p]),
    "tg_quantize_rowcol": (_i, [_p, _p, _p, _p, _p, _i64, _i64, _p]),
    "tg_quantize_rowcol_ld": (_i, [_p, _p, _i64, _p, _i64, _p, _i64, _p, _i64, _i64, _i64, _p]),
    "tg_act_quantize_rowcol": (_i, [_p, _p, _i, _p, _p, _p, _p, _i64, _i64, _p]),
    "tg_quantize_block128": (_i, [_p, _p, _p, _i64, _i64, _p]),
    "tg_selftest_quantise_division": (_i, [_p, _p]),
    "tg_selftest_bounded_wait": (_i, [_p, _p, _i64, _p]),
    "tg_rmsnorm_fwd": (_i, [_p, _p, _f, _p, _p, _i64, _i64, _i, _p]),
    "tg_rmsnorm_quant_fwd": (_i, [_p, _p, _f, _p, _p, _p, _p, _i64, _i64, _i, _p]),
    "tg_add_rmsnorm_quant_fwd": (_i, [_p, _p, _p, _f, _p, _p, _p, _p, _p, _i64, _i64, _i, _p]),
    "tg_rmsnorm_bwd_scratch_bytes": (_i64, [_i64, _i64]),
    "tg_rmsnorm_bwd": (_i, [_p, _p, _p, _f, _p, _p, _p, _i64, _i64, _p]),
    "tg_rmsnorm_bwd_add": (_i, [_p, _p, _p, _p, _f, _p, _p, _p, _i64, _i64, _p]),
    "tg_rmsnorm_bwd_static_max_scratch_bytes": (_i64, []),
    "tg_rmsnorm_bwd_static": (_i, [_p, _p, _p, _f, _p, _p, _i64, _i64, _p]),
    "tg_softcap_ce_fwd": (_i, [_p, _p, _f, _p, _p, _p, _i64, _i64, _i64, _i64, _p]),
    "tg_softcap_ce_bwd": (_i, [_p, _p, _p, _p, _f, _p, _i64, _i64, _i64, _i64, _p]),
    "tg_sumsq_scratch_bytes": (_i64, []),
    "tg_sumsq_bf16": (_i, [_p, _i64, _p, _p, _p]),
    "tg_adamw_bf16": (_i, [_p, _p, _p, _p, _i64, _f, _f, _f, _f, _f, _p, _p, _p]),
    "tg_gemm_workspace_bytes": (_i64, [C.POINTER(GemmArgs)]),
    "tg_gemm_fp8_blockscaled": (_i, [C.POINTER(GemmArgs), _p]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library once; raise if it is missing (never fall back to another path)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: the CUDA library is not built. "
                "Run `python -m train_gpt_b200.build` (needs nvcc); there is no CPU fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


_NAMES = {TG_ERR_SHAPE: "TG_ERR_SHAPE", TG_ERR_ALIGN: "TG_ERR_ALIGN", TG_ERR_ARCH: "TG_ERR_ARCH",
          TG_ERR_CUDA: "TG_ERR_CUDA", TG_ERR_TOO_LARGE: "TG_ERR_TOO_LARGE"}


def check(rc: int, what: str) -> None:
    """Turn a launcher's status into an exception: ValueError for sizes the kernel cannot
    take, RuntimeError for everything else."""
    if rc == TG_OK:
        return
    name = _NAMES.get(rc, str(rc))
    if rc in (TG_ERR_SHAPE, TG_ERR_TOO_LARGE, TG_ERR_ALIGN):
        raise ValueError(f"{what}: {name}")
    detail = load().tg_last_cuda_error().decode() if rc == TG_ERR_CUDA else ""
    raise RuntimeError(f"{what}: {name} {detail}".strip())
