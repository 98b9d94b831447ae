"""Kernel-level operators: torch CUDA tensors in, torch CUDA tensors out, every one a
single call through the C ABI on torch's current stream.  torch is used for device
memory and streams only; no arithmetic on the path runs in torch.

Quantised tensors are `torch.float8_e4m3fn`; scales are float32.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import GemmArgs, TG_MAJOR_K, TG_MAJOR_MN, TG_NORM_FUSED, TG_NORM_PURE, TG_OUT_BF16, TG_OUT_F32

F8 = torch.float8_e4m3fn
TILE = 128


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _cdiv(a: int, b: int) -> int:
    return -(-a // b)


# ---- quantisers ---------------------------------------------------------------------------

def quantize_rowwise(x: torch.Tensor):
    """1x128 tiles along the last axis (train-gpt fp8.py:39-47 as called at :66).
    x (..., K) bf16 -> q (..., K) e4m3, scales (..., K/128) f32."""
    x = _need(x, torch.bfloat16, "x")
    K = x.shape[-1]
    if K % TILE:
        raise ValueError(f"K={K} not divisible by block_k={TILE}")
    rows = x.numel() // K if K else 0
    q = torch.empty(x.shape, dtype=F8, device=x.device)
    s = torch.empty((*x.shape[:-1], K // TILE), dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().tg_quantize_rowwise(_ptr(x), _ptr(q), _ptr(s), rows, K, _stream()), "tg_quantize_rowwise")
    return q, s


def quantize_colwise(x: torch.Tensor):
    """128x1 tiles of a 2-D tensor (what `_quantize_to_fp8(b.T)` at fp8.py:68 computes,
    without the transpose).  x (R, C) bf16 -> q (R, C) e4m3, scales (ceil(R/128), C) f32."""
    x = _need(x, torch.bfloat16, "x")
    if x.dim() != 2:
        raise ValueError("quantize_colwise takes a 2-D tensor")
    R, Cc = x.shape
    q = torch.empty((R, Cc), dtype=F8, device=x.device)
    s = torch.empty((_cdiv(R, TILE), Cc), dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().tg_quantize_colwise(_ptr(x), _ptr(q), _ptr(s), R, Cc, _stream()), "tg_quantize_colwise")
    return q, s


last_gemm_kernel_launches = 0   # kernels the most recent gemm_* call launched (1, or 2 with the split-contraction reduce)


def quantize_rowcol(x: torch.Tensor, row_out=None, col_out=None):
    """Row-wise (1x128) and column-wise (128x1) quantisation of a 2-D tensor in one pass.
    Returns (q_row, s_row, q_col, s_col), bit-identical to the two separate kernels.
    `row_out` = (q, s) / `col_out` = (q, s): write that form into these instead of fresh tensors -- column
    slices `big_q[:, c0:c0 + cols]` and `big_s[:, c0 // 128:(c0 + cols) // 128]` (row form) or
    `big_s[:, c0:c0 + cols]` (column form) of wider matrices, unit stride along a row, row pitch a multiple of
    16 bytes: several tensors' forms side by side for one GEMM."""
    x = _need(x, torch.bfloat16, "x")
    if x.dim() != 2:
        raise ValueError("quantize_rowcol takes a 2-D tensor")
    R, Cc = x.shape
    if Cc % TILE:
        raise ValueError(f"K={Cc} not divisible by block_k={TILE}")
    dense = row_out is None and col_out is None

    def form(out, s_shape, what):
        if out is None:
            return (torch.empty((R, Cc), dtype=F8, device=x.device), torch.empty(s_shape, dtype=torch.float32, device=x.device))
        q, sc = out
        if (q.dtype != F8 or sc.dtype != torch.float32 or not q.is_cuda or not sc.is_cuda
                or tuple(q.shape) != (R, Cc) or tuple(sc.shape) != s_shape):
            raise TypeError(f"{what} must be an e4m3 {(R, Cc)} and a float32 {s_shape} CUDA tensor")
        if q.stride(1) != 1 or sc.stride(1) != 1:
            raise ValueError(f"{what} tensors must have unit stride along a row")
        return q, sc

    q_row, s_row = form(row_out, (R, Cc // TILE), "row_out")
    q_col, s_col = form(col_out, (_cdiv(R, TILE), Cc), "col_out")
    lib = _lib.load()
    if dense:
        _lib.check(lib.tg_quantize_rowcol(_ptr(x), _ptr(q_row), _ptr(s_row), _ptr(q_col), _ptr(s_col), R, Cc, _stream()),
                   "tg_quantize_rowcol")
        return q_row, s_row, q_col, s_col

    def ld(t, least):                       # a one-row tensor's stride(0) is arbitrary
        return max(t.stride(0), least) if t.shape[0] > 1 else least

    _lib.check(lib.tg_quantize_rowcol_ld(_ptr(x), q_row.data_ptr(), ld(q_row, max(Cc, 16)), s_row.data_ptr(),
                                         ld(s_row, Cc // TILE), q_col.data_ptr(), ld(q_col, max(Cc, 16)),
                                         s_col.data_ptr(), ld(s_col, Cc), R, Cc, _stream()), "tg_quantize_rowcol_ld")
    return q_row, s_row, q_col, s_col


def act_quantize_rowcol(x: torch.Tensor, act: str, gate: torch.Tensor | None = None):
    """quantize_rowcol of an MLP activation computed on the fly from the pre-activation `x`:
    act "relu2" (model.py:72) or "gelu"; "relu2_bwd" / "gelu_bwd" quantise gate * act'(x), the
    gradient at the pre-activation for upstream gradient `gate`.  The activation (or its gradient)
    is rounded to bf16 once and never written to memory.  Returns (q_row, s_row, q_col, s_col)."""
    if act not in _lib.TG_ACT:
        raise ValueError(f"unknown activation {act!r}; use one of {sorted(_lib.TG_ACT)}")
    x = _need(x, torch.bfloat16, "x")
    if x.dim() != 2:
        raise ValueError("act_quantize_rowcol takes a 2-D tensor")
    bwd = act.endswith("_bwd")
    if bwd:
        if gate is None:
            raise ValueError(f"{act} needs the upstream gradient `gate`")
        gate = _need(gate, torch.bfloat16, "gate")
        if gate.shape != x.shape:
            raise ValueError(f"gate shape {tuple(gate.shape)} != x shape {tuple(x.shape)}")
    R, Cc = x.shape
    if Cc % TILE:
        raise ValueError(f"K={Cc} not divisible by block_k={TILE}")
    q_row = torch.empty((R, Cc), dtype=F8, device=x.device)
    s_row = torch.empty((R, Cc // TILE), dtype=torch.float32, device=x.device)
    q_col = torch.empty((R, Cc), dtype=F8, device=x.device)
    s_col = torch.empty((_cdiv(R, TILE), Cc), dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().tg_act_quantize_rowcol(_ptr(x), _ptr(gate) if bwd else 0, _lib.TG_ACT[act], _ptr(q_row),
                                                  _ptr(s_row), _ptr(q_col), _ptr(s_col), R, Cc, _stream()),
               "tg_act_quantize_rowcol")
    return q_row, s_row, q_col, s_col


def quantize_block128(x: torch.Tensor):
    """128x128 tiles.  x (R, C) bf16 -> q (R, C) e4m3, scales (ceil(R/128), C/128) f32."""
    x = _need(x, torch.bfloat16, "x")
    if x.dim() != 2:
        raise ValueError("quantize_block128 takes a 2-D tensor")
    R, Cc = x.shape
    if Cc % TILE:
        raise ValueError(f"C={Cc} not divisible by {TILE}")
    q = torch.empty((R, Cc), dtype=F8, device=x.device)
    s = torch.empty((_cdiv(R, TILE), Cc // TILE), dtype=torch.float32, device=x.device)
    _lib.check(_lib.load().tg_quantize_block128(_ptr(x), _ptr(q), _ptr(s), R, Cc, _stream()), "tg_quantize_block128")
    return q, s


def selftest_quantise_division(device="cuda"):
    """Exhaustive check of the quantisers' division shortcut on the device.  Returns
    (pairs checked, mismatches of x*(1/s), of the shipped one-step form, of two steps)."""
    counts = torch.zeros(4, dtype=torch.int64, device=device)
    _lib.check(_lib.load().tg_selftest_quantise_division(_ptr(counts), _stream()), "tg_selftest_quantise_division")
    return tuple(int(v) for v in counts.cpu())


def selftest_bounded_wait(limit_cycles: int = 2_000_000, device="cuda"):
    """Run the GEMM's give-up path (a barrier wait whose clock limit runs out -> abort flag -> every
    role leaves -> tensor memory freed) on a barrier that is never arrived at.  Returns
    (status code, [gave_up == 0, left_early == 2, ordinary_wait_ok == 1, teardown == 1])."""
    status = torch.zeros((1,), dtype=torch.int32, device=device)
    report = torch.zeros((4,), dtype=torch.int32, device=device)
    _lib.check(_lib.load().tg_selftest_bounded_wait(_ptr(status), _ptr(report), int(limit_cycles), _stream()),
               "tg_selftest_bounded_wait")
    return int(status.item()), [int(v) for v in report.cpu()]


# ---- RMSNorm ------------------------------------------------------------------------------

def rmsnorm_fwd(x, gamma, eps: float, pure: bool = False, want_rnorm: bool = False):
    """kernels.py:44-53 (+:66), or kernels.py:30-33 when `pure`.  Returns y [, rnorm]."""
    x = _need(x, torch.bfloat16, "x")
    gamma = _need(gamma, torch.bfloat16, "gamma")
    D = x.shape[-1]
    if gamma.shape != (D,):
        raise ValueError(f"scale shape {tuple(gamma.shape)} does not match last dim {D}")
    rows = x.numel() // D
    y = torch.empty_like(x)
    rn = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device) if want_rnorm else None
    _lib.check(_lib.load().tg_rmsnorm_fwd(_ptr(x), _ptr(gamma), float(eps), _ptr(y), _ptr(rn), rows, D,
                                          TG_NORM_PURE if pure else TG_NORM_FUSED, _stream()), "tg_rmsnorm_fwd")
    return (y, rn) if want_rnorm else y


def rmsnorm_quant_fwd(x, gamma, eps: float, pure: bool = False, want_y: bool = False, want_rnorm: bool = False):
    """Norm + 1x128 quantise in one pass.  Returns (q, scales, y or None, rnorm or None)."""
    x = _need(x, torch.bfloat16, "x")
    gamma = _need(gamma, torch.bfloat16, "gamma")
    D = x.shape[-1]
    if gamma.shape != (D,):
        raise ValueError(f"scale shape {tuple(gamma.shape)} does not match last dim {D}")
    if D % TILE:
        raise ValueError(f"K={D} not divisible by block_k={TILE}")
    rows = x.numel() // D
    q = torch.empty(x.shape, dtype=F8, device=x.device)
    s = torch.empty((*x.shape[:-1], D // TILE), dtype=torch.float32, device=x.device)
    y = torch.empty_like(x) if want_y else None
    rn = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device) if want_rnorm else None
    _lib.check(_lib.load().tg_rmsnorm_quant_fwd(_ptr(x), _ptr(gamma), float(eps), _ptr(q), _ptr(s), _ptr(y), _ptr(rn),
                                                rows, D, TG_NORM_PURE if pure else TG_NORM_FUSED, _stream()),
               "tg_rmsnorm_quant_fwd")
    return q, s, y, rn


ADD_NORM_MAX_COLS = 2048     # the widest row the fused add + norm kernels take (one warp holds a row)


def add_rmsnorm_quant_fwd(x, res, gamma, eps: float, pure: bool = False, want_q: bool = True, want_y: bool = True):
    """s = bf16(x + res) (the residual add of model.py:68 / :72), then norm + 1x128 quantise of s, one pass.
    Returns (s, q or None, scales or None, y or None).  Rows wider than ADD_NORM_MAX_COLS: ValueError."""
    x = _need(x, torch.bfloat16, "x")
    res = _need(res, torch.bfloat16, "res")
    gamma = _need(gamma, torch.bfloat16, "gamma")
    D = x.shape[-1]
    if res.shape != x.shape:
        raise ValueError("x and res shapes differ")
    if gamma.shape != (D,):
        raise ValueError(f"scale shape {tuple(gamma.shape)} does not match last dim {D}")
    if D % TILE or D > ADD_NORM_MAX_COLS:
        raise ValueError(f"K={D} must be a multiple of {TILE} and at most {ADD_NORM_MAX_COLS}")
    if not (want_q or want_y):
        raise ValueError("nothing to compute: neither the quantised nor the bf16 output is wanted")
    rows = x.numel() // D
    s = torch.empty_like(x)
    q = torch.empty(x.shape, dtype=F8, device=x.device) if want_q else None
    sc = torch.empty((*x.shape[:-1], D // TILE), dtype=torch.float32, device=x.device) if want_q else None
    y = torch.empty_like(x) if want_y else None
    _lib.check(_lib.load().tg_add_rmsnorm_quant_fwd(_ptr(x), _ptr(res), _ptr(gamma), float(eps), _ptr(s), _ptr(q), _ptr(sc),
                                                    _ptr(y), None, rows, D, TG_NORM_PURE if pure else TG_NORM_FUSED,
                                                    _stream()), "tg_add_rmsnorm_quant_fwd")
    return s, q, sc, y


def rmsnorm_bwd(x, gamma, g, eps: float, addend=None):
    """kernels.py:104-118.  Returns (dx bf16 like x, dgamma bf16 (D,)).  With `addend` (bf16 like x, rows of
    at most ADD_NORM_MAX_COLS) dx = bf16(addend + the norm's input gradient): the gradient fan-in of a
    residual junction in the same pass."""
    x = _need(x, torch.bfloat16, "x")
    gamma = _need(gamma, torch.bfloat16, "gamma")
    g = _need(g, torch.bfloat16, "g")
    if g.shape != x.shape:
        raise ValueError("g and x shapes differ")
    D = x.shape[-1]
    rows = x.numel() // D
    lib = _lib.load()
    dx = torch.empty_like(x)
    dgamma = torch.empty((D,), dtype=torch.bfloat16, device=x.device)
    nbytes = lib.tg_rmsnorm_bwd_scratch_bytes(rows, D)
    scratch = torch.empty((max(nbytes, 16),), dtype=torch.uint8, device=x.device)
    if addend is not None:
        addend = _need(addend, torch.bfloat16, "addend")
        if addend.shape != x.shape:
            raise ValueError("addend and x shapes differ")
        if D > ADD_NORM_MAX_COLS:
            raise ValueError(f"the fused add takes rows of at most {ADD_NORM_MAX_COLS}")
        _lib.check(lib.tg_rmsnorm_bwd_add(_ptr(x), _ptr(gamma), _ptr(g), _ptr(addend), float(eps), _ptr(dx), _ptr(dgamma),
                                          _ptr(scratch), rows, D, _stream()), "tg_rmsnorm_bwd_add")
        return dx, dgamma
    _lib.check(lib.tg_rmsnorm_bwd(_ptr(x), _ptr(gamma), _ptr(g), float(eps), _ptr(dx), _ptr(dgamma), _ptr(scratch),
                                  rows, D, _stream()), "tg_rmsnorm_bwd")
    return dx, dgamma


# ---- capped-logit cross-entropy -----------------------------------------------------------

def softcap_ce_fwd(logits, targets, cap: float, want_tanh: bool = True):
    """model.py:97 + losses.py:9-12 on the uncapped bf16 logits (rows, vocab).
    Returns (nll f32 (rows,), lse f32 (rows,), tanh bf16 (rows, vocab) or None)."""
    logits = _need(logits, torch.bfloat16, "logits")
    if logits.dim() != 2:
        raise ValueError("logits must be 2-D (rows, vocab)")
    if targets.dtype != torch.int32 or not targets.is_cuda or not targets.is_contiguous():
        raise TypeError("targets must be a contiguous int32 CUDA tensor")
    rows, vocab = logits.shape
    if targets.numel() != rows:
        raise ValueError("one target per row")
    lib = _lib.load()
    pitch = _cdiv(vocab, 8) * 8
    if pitch != vocab:
        # a vocabulary that is not a multiple of 8 (train-gpt's default 50257, config.py:8): the kernels
        # want a 16-byte row pitch, so the rows move to a padded buffer; the pad columns are never used
        padded = torch.empty((rows, pitch), dtype=torch.bfloat16, device=logits.device)
        padded[:, :vocab].copy_(logits)
        logits = padded
    nll = torch.empty((rows,), dtype=torch.float32, device=logits.device)
    lse = torch.empty((rows,), dtype=torch.float32, device=logits.device)
    th = torch.empty((rows, pitch), dtype=torch.bfloat16, device=logits.device) if want_tanh else None
    _lib.check(lib.tg_softcap_ce_fwd(_ptr(logits), _ptr(targets), float(cap), _ptr(th), _ptr(lse), _ptr(nll),
                                     rows, vocab, pitch, pitch, _stream()), "tg_softcap_ce_fwd")
    if th is not None and pitch != vocab:
        th = th[:, :vocab]                       # a view: the row pitch stays `pitch`
    return nll, lse, th


def softcap_ce_bwd(th, targets, lse, gscale, cap: float, in_place: bool = False):
    """Gradient of mean(nll) w.r.t. the uncapped logits; `gscale` is a float32 device scalar
    (or None for 1).  in_place=True overwrites `th` with the gradient."""
    if not th.is_cuda or th.dtype != torch.bfloat16 or th.dim() != 2 or th.stride(1) != 1:
        raise TypeError("tanh must be a 2-D bf16 CUDA tensor with unit inner stride (as softcap_ce_fwd returns it)")
    rows, vocab = th.shape
    pitch = th.stride(0)                         # > vocab for a vocabulary that is not a multiple of 8
    if in_place:
        d, d_pitch = th, pitch
    else:
        d_pitch = _cdiv(vocab, 8) * 8
        d = torch.empty((rows, d_pitch), dtype=torch.bfloat16, device=th.device)[:, :vocab]
    if gscale is not None:
        gscale = _need(gscale.reshape(1), torch.float32, "gscale")
    lib = _lib.load()
    _lib.check(lib.tg_softcap_ce_bwd(_ptr(th), _ptr(targets), _ptr(lse), _ptr(gscale), float(cap), _ptr(d),
                                     rows, vocab, pitch, d_pitch, _stream()), "tg_softcap_ce_bwd")
    return d


# ---- optimiser ------------------------------------------------------------------------------

def sumsq(x, out=None, scratch=None):
    """Sum of squares of a bf16 tensor as a float32 device scalar (one term of optax.global_norm)."""
    x = _need(x, torch.bfloat16, "x")
    lib = _lib.load()
    if out is None:
        out = torch.empty((1,), dtype=torch.float32, device=x.device)
    if scratch is None:
        scratch = torch.empty((lib.tg_sumsq_scratch_bytes(),), dtype=torch.uint8, device=x.device)
    _lib.check(lib.tg_sumsq_bf16(_ptr(x), x.numel(), _ptr(out), _ptr(scratch), _stream()), "tg_sumsq_bf16")
    return out


def adamw_step(p, g, m, v, step, lr, b1=0.9, b2=0.999, eps=1e-8, weight_decay=0.0, gscale=None):
    """optax clip + adamw on one bf16 parameter tensor, in place (p, m, v).  `step` is an int32
    device scalar holding t (1 for the first step); `gscale` a float32 device scalar or None."""
    for t, n in ((p, "p"), (g, "g"), (m, "m"), (v, "v")):
        if not t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise TypeError(f"{n} must be a contiguous bf16 CUDA tensor")
    if not (p.numel() == g.numel() == m.numel() == v.numel()):
        raise ValueError("p, g, m, v sizes differ")
    if step.dtype != torch.int32 or not step.is_cuda:
        raise TypeError("step must be an int32 CUDA scalar")
    _lib.check(_lib.load().tg_adamw_bf16(_ptr(p), _ptr(g), _ptr(m), _ptr(v), p.numel(), float(lr), float(b1), float(b2),
                                         float(eps), float(weight_decay), _ptr(step), _ptr(gscale), _stream()),
               "tg_adamw_bf16")


# ---- GEMM ---------------------------------------------------------------------------------

def set_gemm_reserved_sms(n: int) -> int:
    """Leave `n` SMs free of the persistent GEMM's thread blocks from the next launch on (for a collective
    that overlaps the GEMMs: the data-parallel gradient all-reduce).  Returns the previous setting."""
    return int(_lib.load().tg_set_gemm_reserved_sms(int(n)))


def new_status(device) -> torch.Tensor:
    """A zeroed device word for the GEMM's bounded-wait status."""
    return torch.zeros((1,), dtype=torch.int32, device=device)


# what the code a GEMM leaves in its status word says about which bounded wait ran out
STATUS_ROLES = {
    1: "the TMA producer waited for a free shared-memory stage",
    2: "the MMA issuer waited for a free accumulator buffer",
    3: "the MMA issuer waited for operands to land",
    4: "the MMA issuer waited for its last instructions to retire",
    5: "the promotion warps waited for an accumulator buffer to fill",
}

_status_words = {}


def default_status(device) -> torch.Tensor:
    """The status word every gemm_* call on `device` uses when the caller passes none: one word per
    device, allocated once (so a captured CUDA graph keeps pointing at it)."""
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    word = _status_words.get(dev)
    if word is None:
        word = _status_words[dev] = new_status(dev)
    return word


def status_error(code: int):
    """The exception for a non-zero GEMM status code, or None for 0."""
    if code == 0:
        return None
    why = STATUS_ROLES.get(int(code), "unknown role")
    return RuntimeError(f"block-scaled GEMM gave up on a bounded device wait (status {int(code)}: {why}); "
                        "its output is incomplete")


def check_status(status: torch.Tensor | None = None, device=None) -> None:
    """Read a status word (the device's default one if none is given; this synchronises with the
    work queued on it) and raise if a GEMM's bounded wait ran out since it was last zero.  The
    word is cleared so that the next check reports only newer failures."""
    word = status if status is not None else default_status(device if device is not None else "cuda")
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise status_error(code)


def poison_if_failed(value: torch.Tensor, status: torch.Tensor | None = None) -> torch.Tensor:
    """`value` with NaN in place of every element if the status word is non-zero -- a device-side
    select, no synchronisation, capturable in a CUDA graph.  The training step passes its loss through
    this, so a GEMM that gave up surfaces as a NaN loss instead of a silently wrong one."""
    word = status if status is not None else default_status(value.device)
    return torch.where(word.reshape(()) != 0, torch.full_like(value, float("nan")), value)


def gemm_blockscaled(a, b, sa, sb, *, M, N, K, a_major, b_major, sa_strides, sb_strides, sb_gran_n,
                     out_dtype=torch.bfloat16, status=None, out=None, split=True):
    """Raw call of tg_gemm_fp8_blockscaled; see include/train_gpt_b200.h for the argument
    meaning.  a, b are 2-D e4m3 tensors as stored; strides are in elements.  split=True hands
    the library the workspace it asks for (tg_gemm_workspace_bytes), so that a problem with few
    output tiles and a long contraction is cut along the contraction."""
    for t, n in ((a, "a"), (b, "b")):
        if t.dtype != F8 or t.dim() != 2 or t.stride(1) != 1:
            raise TypeError(f"{n} must be a 2-D e4m3 tensor with unit inner stride")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if status is None:
        status = default_status(a.device)      # never NULL: a bounded wait that runs out must leave a trace
    args = GemmArgs(
        a=_ptr(a), b=_ptr(b), lda=a.stride(0), ldb=b.stride(0), a_major=a_major, b_major=b_major,
        sa=_ptr(sa), sa_stride_m=sa_strides[0], sa_stride_kb=sa_strides[1],
        sb=_ptr(sb), sb_stride_n=sb_strides[0], sb_stride_kb=sb_strides[1], sb_gran_n=sb_gran_n,
        d=_ptr(out), ldd=out.stride(0), out_dtype=TG_OUT_F32 if out.dtype == torch.float32 else TG_OUT_BF16,
        M=M, N=N, K=K, status=_ptr(status), workspace=0, workspace_bytes=0)
    lib = _lib.load()
    ws = None
    if split:
        need = lib.tg_gemm_workspace_bytes(C.byref(args))
        if need > 0:
            ws = torch.empty((need,), dtype=torch.uint8, device=a.device)
            args.workspace, args.workspace_bytes = _ptr(ws), need
    _lib.check(lib.tg_gemm_fp8_blockscaled(C.byref(args), _stream()), "tg_gemm_fp8_blockscaled")
    global last_gemm_kernel_launches
    last_gemm_kernel_launches = 2 if ws is not None else 1      # a split contraction adds the reduce kernel
    return out


def gemm_fwd(x_q, x_s, w_q, w_s, weight_tile=(128, 1), out_dtype=torch.bfloat16, status=None):
    """y = x W.  x_q (M,K) rowwise-quantised with x_s (M,K/128); w_q (K,N) with
    w_s (K/128,N) [weight_tile (128,1), from quantize_colwise] or (K/128,N/128)
    [weight_tile (128,128), from quantize_block128]."""
    M, K = x_q.shape
    N = w_q.shape[1]
    nkb = x_s.shape[1]
    if tuple(weight_tile) == (128, 1):
        sb_str, gran = (1, N), 1
    else:
        sb_str, gran = (1, w_s.shape[1]), 128
    return gemm_blockscaled(x_q, w_q, x_s, w_s, M=M, N=N, K=K, a_major=TG_MAJOR_K, b_major=TG_MAJOR_MN,
                            sa_strides=(nkb, 1), sb_strides=sb_str, sb_gran_n=gran, out_dtype=out_dtype, status=status)


def gemm_dgrad(g_q, g_s, w_q, w_s, weight_tile=(128, 1), out_dtype=torch.bfloat16, status=None):
    """dx = g W^T (contracts N).  g_q (M,N) rowwise-quantised, g_s (M,N/128); w_q (K,N)
    quantised along N: w_s (K,N/128) [tile (128,1) mode: quantize_rowwise(W)] or the shared
    (K/128,N/128) [tile (128,128)]."""
    M, N = g_q.shape
    K = w_q.shape[0]
    if tuple(weight_tile) == (128, 1):
        sb_str, gran = (w_s.shape[1], 1), 1
    else:
        sb_str, gran = (w_s.shape[1], 1), 128
    return gemm_blockscaled(g_q, w_q, g_s, w_s, M=M, N=K, K=N, a_major=TG_MAJOR_K, b_major=TG_MAJOR_K,
                            sa_strides=(g_s.shape[1], 1), sb_strides=sb_str, sb_gran_n=gran, out_dtype=out_dtype,
                            status=status)


def gemm_wgrad(x_qc, x_sc, g_qc, g_sc, out_dtype=torch.bfloat16, status=None, grad_tile=(128, 1), out=None):
    """dW = x^T g (contracts the tokens).  x_qc (T,K) colwise-quantised (128 tokens x 1),
    scales (ceil(T/128),K).  g_qc (T,N) quantised either the same way, scales (ceil(T/128),N)
    [grad_tile (128,1)], or in 128x128 blocks, scales (ceil(T/128),N/128) [grad_tile (128,128)]:
    one scale per 128 output columns halves the promotion arithmetic and lets the GEMM use its
    128x256 tile.  `out`: a (K, N) bf16 or float32 tensor with unit inner stride to write into (a slice of a
    gradient bucket, say) instead of a new one."""
    T, K = x_qc.shape
    N = g_qc.shape[1]
    if out is not None and (tuple(out.shape) != (K, N) or out.stride(1) != 1 or not out.is_cuda
                            or out.dtype not in (torch.bfloat16, torch.float32)):
        raise ValueError(f"out must be a ({K}, {N}) bf16 or float32 CUDA tensor with unit inner stride")
    if tuple(grad_tile) == (128, 1):
        sb_str, gran = (1, N), 1
    else:
        sb_str, gran = (1, g_sc.shape[1]), 128
    return gemm_blockscaled(x_qc, g_qc, x_sc, g_sc, M=K, N=N, K=T, a_major=TG_MAJOR_MN, b_major=TG_MAJOR_MN,
                            sa_strides=(1, K), sb_strides=sb_str, sb_gran_n=gran, out_dtype=out_dtype, status=status, out=out)
