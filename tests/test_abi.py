"""CPU-only checks of the drop-in boundary: the library builds, loads and exports every
symbol the public header declares, and the host-side mirrors raise the reference's errors
before touching a device."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from train_gpt_b200 import build, _lib
    build.build()
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "train_gpt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tg_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(lib):
    from train_gpt_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes prototype"
    assert sorted(_lib.SYMBOLS) == names
    assert lib.tg_version() >= 100
    assert lib.tg_set_gemm_reserved_sms(8) == 0 and lib.tg_set_gemm_reserved_sms(1000) == 8
    assert lib.tg_set_gemm_reserved_sms(0) == 64          # clamped; back to the default


def test_gemm_args_struct_matches_header_layout():
    from train_gpt_b200._lib import GemmArgs
    # 22 fields; pointers/int64 8-byte aligned, ints padded as a C compiler would
    assert ctypes.sizeof(GemmArgs) == 8 * 2 + 8 * 2 + 4 * 2 + 8 * 3 + 8 * 3 + 8 + 8 * 2 + 8 + 8 * 3 + 8 + 8 * 2
    assert GemmArgs.sa.offset == 40 and GemmArgs.d.offset == 96 and GemmArgs.status.offset == 144


def test_shape_errors_precede_any_device_work():
    from train_gpt_b200 import fp8
    a = torch.zeros(2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="contracted-dim mismatch: a K=128, b K=256"):
        fp8.block_scaled_matmul(a, torch.zeros(256, 4, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="K=192 not divisible by block_k=128"):
        fp8.block_scaled_matmul(torch.zeros(2, 192, dtype=torch.bfloat16), torch.zeros(192, 4, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="block_k=64 is not supported"):
        fp8.block_scaled_matmul(a, torch.zeros(128, 8, dtype=torch.bfloat16), 64)
    with pytest.raises(ValueError, match="unknown backward mode"):
        fp8.block_scaled_matmul(a, torch.zeros(128, 8, dtype=torch.bfloat16), backward="e5m2")


def test_no_cpu_fallback():
    from train_gpt_b200 import kernels, ops
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.quantize_rowwise(torch.zeros(4, 128, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="no CPU path"):
        kernels.rms_norm(torch.zeros(4, 128, dtype=torch.bfloat16), torch.ones(128, dtype=torch.bfloat16), 1e-5)


def test_launchers_validate_on_the_host(lib):
    # shape/alignment validation happens before any CUDA call, so it is checkable without a GPU
    from train_gpt_b200 import _lib
    assert lib.tg_quantize_rowwise(16, 16, 16, 4, 100, None) == _lib.TG_ERR_SHAPE
    assert lib.tg_quantize_rowwise(8, 16, 16, 4, 128, None) == _lib.TG_ERR_ALIGN
    assert lib.tg_quantize_rowwise(16, 16, 16, 0, 128, None) == _lib.TG_OK          # empty input
    assert lib.tg_quantize_block128(16, 16, 16, 4, 64, None) == _lib.TG_ERR_SHAPE
    assert lib.tg_rmsnorm_quant_fwd(16, 16, 1e-6, 16, 16, None, None, 4, 16384, 0, None) in (
        _lib.TG_ERR_TOO_LARGE, _lib.TG_ERR_ARCH, _lib.TG_ERR_CUDA)
    assert lib.tg_rmsnorm_fwd(16, 16, 1e-6, 16, None, 4, 100, 0, None) == _lib.TG_ERR_SHAPE
    assert lib.tg_rmsnorm_bwd_scratch_bytes(0, 128) == 0
    args = _lib.GemmArgs(a=16, b=16, lda=128, ldb=128, a_major=0, b_major=1, sa=16, sb=16, sb_gran_n=7,
                         d=16, ldd=128, M=128, N=128, K=128)
    assert lib.tg_gemm_fp8_blockscaled(ctypes.byref(args), None) == _lib.TG_ERR_SHAPE
    args.sb_gran_n = 1
    args.N = 100
    assert lib.tg_gemm_fp8_blockscaled(ctypes.byref(args), None) == _lib.TG_ERR_SHAPE


def test_nonzero_gemm_status_raises():
    """A GEMM whose bounded device wait ran out leaves a role code in its status word; reading a
    non-zero word raises and clears it.  (A host tensor stands in for the device word: no GPU.)"""
    import torch
    from train_gpt_b200 import ops
    ok = torch.zeros(1, dtype=torch.int32)
    ops.check_status(ok)                                        # zero: silent
    for code in (1, 2, 3, 4, 5, 77):
        word = torch.tensor([code], dtype=torch.int32)
        with pytest.raises(RuntimeError, match=f"status {code}"):
            ops.check_status(word)
        assert int(word.item()) == 0                            # cleared for the next check
    assert ops.status_error(0) is None
    assert "promotion warps" in str(ops.status_error(5))
    loss = torch.tensor(2.5)
    assert float(ops.poison_if_failed(loss, ok)) == 2.5
    assert torch.isnan(ops.poison_if_failed(loss, torch.tensor([3], dtype=torch.int32)))
