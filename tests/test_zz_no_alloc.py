"""The allocation-free norm backward (`tg_rmsnorm_bwd_static`) against the ordinary entry
point (`tg_rmsnorm_bwd`), called straight through the C ABI.

Some callers of this library cannot allocate device memory -- an XLA custom-call handler
only sees the buffers the compiler planned, and XLA normally owns most of the device by
then -- so they cannot supply the scratch buffer `tg_rmsnorm_bwd` asks for.  The static
variant keeps that scratch inside the library.  Both run the same kernels, so their
outputs must agree bit for bit; the check is made on two calls in a row with different
inputs, because the built-in scratch still holds the first call's partial sums when the
second one starts.

This file sorts last on purpose: a run that stops at the first failure has then already
been through every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_pair(lib, rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    gy = torch.randn(rows, cols, device="cuda", generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).to(torch.bfloat16)
    eps = 1e-5
    stream = torch.cuda.current_stream().cuda_stream

    # reference: the ordinary entry point with a caller-owned scratch buffer
    need = lib.tg_rmsnorm_bwd_scratch_bytes(rows, cols)
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    dx_ref = torch.empty_like(x)
    dg_ref = torch.empty(cols, dtype=torch.bfloat16, device="cuda")
    rc = lib.tg_rmsnorm_bwd(x.data_ptr(), gamma.data_ptr(), gy.data_ptr(), eps, dx_ref.data_ptr(), dg_ref.data_ptr(),
                            scratch.data_ptr(), rows, cols, stream)
    assert rc == 0

    # outputs are allocated by the caller (here: by torch) BEFORE the call; the call itself allocates nothing
    dx = torch.full_like(x, float("nan"))
    dg = torch.full((cols,), float("nan"), dtype=torch.bfloat16, device="cuda")
    rc = lib.tg_rmsnorm_bwd_static(x.data_ptr(), gamma.data_ptr(), gy.data_ptr(), eps, dx.data_ptr(), dg.data_ptr(),
                                   rows, cols, stream)
    assert rc == 0, lib.tg_last_cuda_error()
    torch.cuda.synchronize()
    assert torch.equal(dx.view(torch.int16), dx_ref.view(torch.int16))
    assert torch.equal(dg.view(torch.int16), dg_ref.view(torch.int16))
    assert not torch.isnan(dg.float()).any()


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    from train_gpt_b200 import _lib
    lib = _lib.load()
    assert lib.tg_rmsnorm_bwd_static_max_scratch_bytes() == 4 << 20
    _call_pair(lib, 3000, 2048, seed=1)      # fills the built-in scratch with this call's partial sums
    _call_pair(lib, 777, 1024, seed=2)       # a different shape on top of the stale contents
    _call_pair(lib, 3000, 2048, seed=3)
    _call_pair(lib, 96, 4096, seed=4)        # a row split over two warps (wider than 2048) still fits the 4 MiB for few rows


def test_static_scratch_refuses_what_does_not_fit():
    from train_gpt_b200 import _lib
    lib = _lib.load()
    rows, cols = 32768, 8192
    assert lib.tg_rmsnorm_bwd_scratch_bytes(rows, cols) > lib.tg_rmsnorm_bwd_static_max_scratch_bytes()
    x = torch.zeros(8, dtype=torch.bfloat16, device="cuda")   # never touched: the call is refused on the host
    rc = lib.tg_rmsnorm_bwd_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), 1e-5, x.data_ptr(), x.data_ptr(),
                                   rows, cols, None)
    assert rc == _lib.TG_ERR_TOO_LARGE
    assert b"4 MiB" in lib.tg_last_cuda_error()
    torch.cuda.synchronize()
