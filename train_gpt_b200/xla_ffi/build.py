"""Build `libtg_xla.so`, the XLA FFI handlers of xla_ffi.cc, next to this file.

    python -m train_gpt_b200.xla_ffi.build

Needs jax (for `jax.ffi.include_dir()`, the XLA FFI headers that ship with jaxlib), g++ and the
CUDA runtime headers; links against the in-tree libtrain_gpt_b200.so.  Where jax is missing the
build says so and exits non-zero: there is nothing else to fall back to.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
ROOT = os.path.dirname(PKG)
OUT = os.path.join(HERE, "libtg_xla.so")


def ffi_include_dir():
    """jaxlib's XLA FFI header directory, or None where jax is not installed."""
    try:
        from jax import ffi
    except ImportError:
        return None
    return ffi.include_dir()


def command(include_dir: str, cuda_home: str = "/usr/local/cuda"):
    return ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-I{include_dir}", f"-I{os.path.join(ROOT, 'include')}",
            f"-I{os.path.join(cuda_home, 'include')}", os.path.join(HERE, "xla_ffi.cc"), f"-L{PKG}", "-ltrain_gpt_b200",
            f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart", f"-Wl,-rpath,{PKG}", "-o", OUT]


def build() -> str:
    inc = ffi_include_dir()
    if inc is None:
        raise RuntimeError("jax is not installed: the XLA FFI headers (jax.ffi.include_dir()) are not available")
    from train_gpt_b200 import build as core
    core.build()
    subprocess.run(command(inc, os.environ.get("CUDA_HOME", "/usr/local/cuda")), check=True)
    return OUT


if __name__ == "__main__":
    try:
        print(build())
    except RuntimeError as e:
        print(f"not built: {e}", file=sys.stderr)
        sys.exit(1)
