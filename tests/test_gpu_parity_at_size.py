"""Oracle parity of the block-scaled GEMMs and the norm backward AT THE BENCHMARKED SIZES.

The small-shape tests (test_gpu_gemm.py) compare whole outputs with the CPU oracle; the
launches the benchmark times are too large for that (a 32768 x 8192 x 2048 product is 1.1
TFLOP in float64).  Here every benchmarked launch runs at full size and a seeded SAMPLE of
its output is compared with `oracle.scaled_matmul` evaluated on just those rows / columns:

  * 128 output rows, one per residue 0..127 inside a tile, spread over the row tiles with the
    first and the last tile forced in (the last tile belongs to the last, partial wave of the
    persistent schedule), against every column;
  * 66 output columns (first, last, 64 seeded) against 2048 seeded rows.

The operands the oracle sees are the device's quantised bytes and scales, and the sampled
slices of those are first checked BIT-EXACT against the oracle's own quantiser applied to
the same slices of the bf16 input, so the chain input -> bytes -> product is covered end to
end at size.  The reference's accuracy harness runs the same real shapes
(train-gpt debug_fp8.py:112-139, bench_fp8.py:144-152,108-112).

Tolerance (the stated one): |got - ref| <= 1e-2 * RMS(ref) + 2e-2 * |ref|, zero violations,
and relative Frobenius error of the sample below 2e-3.
"""
import numpy as np
import pytest
import torch

from oracle import fp8_oracle as fo
from oracle import norm_oracle as no
from tests.gpu_util import BF16, F8, from_torch_bf16

pytestmark = pytest.mark.gpu

TOKENS = 32768
LAYER_SHAPES = [(2048, 6144), (2048, 2048), (2048, 8192), (8192, 2048)]   # (K, N) of one decoder layer


# ---- inputs -------------------------------------------------------------------------------

def _normal(shape, seed, std=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * std).to(torch.bfloat16)


def _student_t3(shape, seed):
    """Student-t with 3 degrees of freedom = N(0,1) / sqrt(chi2(3) / 3), drawn on the device."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    chi = sum(torch.randn(shape, device="cuda", generator=g) ** 2 for _ in range(3)) / 3.0
    return (torch.randn(shape, device="cuda", generator=g) / chi.sqrt()).to(torch.bfloat16)


def _host_f8(t):
    return t.contiguous().view(torch.uint8).cpu().numpy().view(F8)


def _host_bf16_rows(t, rows):
    return from_torch_bf16(t[torch.as_tensor(rows, device=t.device)])


def _host_bf16_cols(t, cols):
    return from_torch_bf16(t[:, torch.as_tensor(cols, device=t.device)])


# ---- samples ------------------------------------------------------------------------------

def _sample_rows(M, seed, n=128, tile=128):
    """n rows: residue i inside the tile for the i-th, tiles spread evenly with first and last forced."""
    tiles = -(-M // tile)
    rng = np.random.default_rng(seed)
    if M <= n:
        return np.arange(M)
    t_idx = np.unique(np.concatenate([[0, tiles - 1], rng.integers(0, tiles, size=n)]))
    rows = []
    for i in range(n):
        r = int(t_idx[i % len(t_idx)]) * tile + (i % tile)
        rows.append(min(r, M - 1))
    return np.unique(np.asarray(rows))


def _sample_cols(N, seed, n=64):
    rng = np.random.default_rng(seed + 1)
    if N <= n + 2:
        return np.arange(N)
    return np.unique(np.concatenate([[0, N - 1], rng.choice(N, size=n, replace=False)]))


def _sample_many_rows(M, seed, n=2048):
    rng = np.random.default_rng(seed + 2)
    return np.arange(M) if M <= n else np.sort(rng.choice(M, size=n, replace=False))


def _report(name, got, ref):
    got = np.asarray(got).astype(np.float64)
    ref = np.asarray(ref).astype(np.float64)
    assert np.isfinite(got).all(), name
    viol = fo.tolerance_violations(got, ref)
    frob = fo.rel_frobenius(got, ref)
    print(f"{name}: {got.size} sampled outputs, violations {viol}, rel. Frobenius {frob:.2e}")
    assert viol == 0, f"{name}: {viol} violations (rel_frob {frob:.3e})"
    assert frob < 2e-3, f"{name}: rel_frob {frob:.3e}"


def _check_sample(name, out, rows_a, a_q, a_s, b_q_t, b_s, seed):
    """out (M, N) device tensor of D = A B^T; a_q (M, Kc) / b_q_t (N, Kc) host e4m3, scales (M, Kc/128) / (N, Kc/128).
    `rows_a`: the row sample (a_q and a_s hold only those rows)."""
    got = out[torch.as_tensor(rows_a, device=out.device)].float().cpu().numpy()
    ref = fo.scaled_matmul(a_q, b_q_t, a_s, b_s)
    ref = ref.astype(BF16) if out.dtype == torch.bfloat16 else ref
    _report(name + " rows", got, ref)


def _pad_blocks(q, axis, block=128):
    pad = (-q.shape[axis]) % block
    if not pad:
        return q
    width = [(0, 0)] * q.ndim
    width[axis] = (0, pad)
    return np.pad(q.view(np.uint8), width).view(F8)      # byte 0 is +0.0 in e4m3


# ---- the three GEMMs of a linear layer, sampled ---------------------------------------------

def _forward_case(tag, x, w, seed):
    """y = x W with 1x128 activation tiles and 128x128 weight tiles (the benchmark's granularity)."""
    from train_gpt_b200 import ops
    M, K = x.shape
    N = w.shape[1]
    st = ops.new_status("cuda")
    x_q, x_s = ops.quantize_rowwise(x)
    w_q, w_s = ops.quantize_block128(w)
    y = ops.gemm_fwd(x_q, x_s, w_q, w_s, (128, 128), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    # weight: the oracle quantises all of it (K x N is small), bytes and scales must agree bit for bit
    wq_ref, ws_ref = fo.quantize_block2d(from_torch_bf16(w).astype(np.float32))
    assert np.array_equal(_host_f8(w_q).view(np.uint8), wq_ref.view(np.uint8)), tag
    assert np.array_equal(w_s.cpu().numpy(), ws_ref), tag
    b_q_t = wq_ref.T
    b_s = np.repeat(ws_ref.T, 128, axis=0)                      # (N, K/128)
    rows = _sample_rows(M, seed)
    xr_q, xr_s = fo.quantize_to_fp8(_host_bf16_rows(x, rows).astype(np.float32))
    ridx = torch.as_tensor(rows, device="cuda")
    assert np.array_equal(_host_f8(x_q[ridx]).view(np.uint8), xr_q.view(np.uint8)), tag
    assert np.array_equal(x_s[ridx].cpu().numpy(), xr_s), tag
    _check_sample(f"{tag} fwd", y, rows, xr_q, xr_s, b_q_t, b_s, seed)
    cols = _sample_cols(N, seed)
    many = _sample_many_rows(M, seed)
    midx = torch.as_tensor(many, device="cuda")
    got = y[midx][:, torch.as_tensor(cols, device="cuda")].float().cpu().numpy()
    ref = fo.scaled_matmul(_host_f8(x_q[midx]), b_q_t[cols], x_s[midx].cpu().numpy(), b_s[cols]).astype(BF16)
    _report(f"{tag} fwd cols", got, ref)


def _dgrad_case(tag, g, w, seed):
    """dx = g W^T: contraction over N; g in 1x128 tiles along N, W in its 128x128 tiles."""
    from train_gpt_b200 import ops
    M, N = g.shape
    K = w.shape[0]
    st = ops.new_status("cuda")
    g_q, g_s = ops.quantize_rowwise(g)
    w_q, w_s = ops.quantize_block128(w)
    dx = ops.gemm_dgrad(g_q, g_s, w_q, w_s, (128, 128), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    wq_ref, ws_ref = fo.quantize_block2d(from_torch_bf16(w).astype(np.float32))
    b_s = np.repeat(ws_ref, 128, axis=0)[:K]                    # (K, N/128)
    rows = _sample_rows(M, seed)
    gr_q, gr_s = fo.quantize_to_fp8(_host_bf16_rows(g, rows).astype(np.float32))
    ridx = torch.as_tensor(rows, device="cuda")
    assert np.array_equal(_host_f8(g_q[ridx]).view(np.uint8), gr_q.view(np.uint8)), tag
    _check_sample(f"{tag} dgrad", dx, rows, gr_q, gr_s, wq_ref, b_s, seed)
    cols = _sample_cols(K, seed)
    many = _sample_many_rows(M, seed)
    midx = torch.as_tensor(many, device="cuda")
    got = dx[midx][:, torch.as_tensor(cols, device="cuda")].float().cpu().numpy()
    ref = fo.scaled_matmul(_host_f8(g_q[midx]), wq_ref[cols], g_s[midx].cpu().numpy(), b_s[cols]).astype(BF16)
    _report(f"{tag} dgrad cols", got, ref)


def _wgrad_case(tag, x, g, seed, plans=(True,)):
    """dW = x^T g: contraction over the tokens; x and g in 128-token x 1 tiles.  `plans`: run with the
    library's contraction split allowed (True) and forbidden (False)."""
    from train_gpt_b200 import _lib, ops
    T, K = x.shape
    N = g.shape[1]
    x_q, x_s = ops.quantize_colwise(x)
    g_q, g_s = ops.quantize_colwise(g)
    ks = _sample_rows(K, seed, n=64)                            # sampled rows of dW = features of x
    ns = _sample_cols(N, seed)
    # sampled slices of both quantised operands against the oracle's quantiser
    xk_q, xk_s = fo.quantize_colwise(_host_bf16_cols(x, ks).astype(np.float32))
    kidx, nidx = torch.as_tensor(ks, device="cuda"), torch.as_tensor(ns, device="cuda")
    assert np.array_equal(_host_f8(x_q[:, kidx]).view(np.uint8), xk_q.view(np.uint8)), tag
    assert np.array_equal(x_s[:, kidx].cpu().numpy(), xk_s), tag
    gn_q, gn_s = fo.quantize_colwise(_host_bf16_cols(g, ns).astype(np.float32))
    assert np.array_equal(_host_f8(g_q[:, nidx]).view(np.uint8), gn_q.view(np.uint8)), tag
    assert np.array_equal(g_s[:, nidx].cpu().numpy(), gn_s), tag
    # oracle on the samples (a ragged last token block is padded with zero bytes, as the kernel's loads are)
    g_host, gs_host = _pad_blocks(_host_f8(g_q), 0), g_s.cpu().numpy()
    ref_rows = fo.scaled_matmul(_pad_blocks(xk_q, 0).T, g_host.T, xk_s.T, gs_host.T).astype(BF16)      # (|ks|, N)
    many = _sample_many_rows(K, seed)
    midx = torch.as_tensor(many, device="cuda")
    ref_cols = fo.scaled_matmul(_pad_blocks(_host_f8(x_q[:, midx]), 0).T, _pad_blocks(gn_q, 0).T,
                                x_s[:, midx].cpu().numpy().T, gn_s.T).astype(BF16)                      # (|many|, |ns|)
    for split in plans:
        st = ops.new_status("cuda")
        dw = ops.gemm_blockscaled(x_q, g_q, x_s, g_s, M=K, N=N, K=T, a_major=_lib.TG_MAJOR_MN, b_major=_lib.TG_MAJOR_MN,
                                  sa_strides=(1, K), sb_strides=(1, N), sb_gran_n=1, status=st, split=split)
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        plan = f"{ops.last_gemm_kernel_launches} launch(es)"
        _report(f"{tag} wgrad rows [{plan}]", dw[kidx].float().cpu().numpy(), ref_rows)
        _report(f"{tag} wgrad cols [{plan}]", dw[midx][:, nidx].float().cpu().numpy(), ref_cols)


# ---- ragged edges under the persistent schedule ----------------------------------------------

def test_ragged_problem_with_several_tiles_per_thread_block():
    """19237 tokens x (384 -> 640): 151 x 3 forward tiles (the last column tile half full, the last row tile
    37 rows) on 148 thread blocks, so most blocks run several tiles and hand each one to the store warp
    while they start the next; dgrad has 151 x 2 tiles, the weight gradient a ragged last token block."""
    M, K, N = 19237, 384, 640
    x, w, g = _normal((M, K), 11), _normal((K, N), 12, 0.02), _normal((M, N), 13)
    _forward_case("ragged", x, w, seed=5)
    _dgrad_case("ragged", g, w, seed=6)
    _wgrad_case("ragged", x, g, seed=7, plans=(True, False))


# ---- benchmark configuration 2: one decoder layer's linear set at 32768 tokens ---------------

@pytest.mark.parametrize("K,N", LAYER_SHAPES)
def test_decoder_layer_forward_at_size(K, N):
    _forward_case(f"layer {K}x{N}", _normal((TOKENS, K), 1), _normal((K, N), 2, 0.02), seed=K + N)


@pytest.mark.parametrize("K,N", LAYER_SHAPES)
def test_decoder_layer_dgrad_at_size(K, N):
    _dgrad_case(f"layer {K}x{N}", _normal((TOKENS, N), 3), _normal((K, N), 2, 0.02), seed=K + N)


@pytest.mark.parametrize("K,N", LAYER_SHAPES)
def test_decoder_layer_wgrad_at_size_split_and_unsplit(K, N):
    _wgrad_case(f"layer {K}x{N}", _normal((TOKENS, K), 1), _normal((TOKENS, N), 3), seed=K + N, plans=(True, False))


@pytest.mark.parametrize("K,N", [(1024, 1024), (4096, 1024), (1024, 4096), (1024, 3072)])
def test_training_configuration_wgrad_at_size_with_unequal_contraction_ranges(K, N):
    """The weight gradients of the 24-layer training configuration (d_model 1024, MLP 4096, q/k/v side by side) at
    32768 tokens.  256 contraction blocks over few output tiles: the planner cuts them into 3 ranges of 86, 85, 85
    blocks for the 1024 x 1024 one (48 tiles x 3 = 144 work items on 148 SMs) -- ranges need not be equal."""
    _wgrad_case(f"training {K}x{N}", _normal((TOKENS, K), 5), _normal((TOKENS, N), 6), seed=K + N + 1, plans=(True, False))


# ---- benchmark configuration 4: Student-t(3) activations, squares and skinny M ---------------

@pytest.mark.parametrize("n", [4096, 8192])
def test_shape_sweep_squares_student_t(n):
    x = _student_t3((n, n), 5)
    w = _normal((n, n), 6, 0.02)
    g = _normal((n, n), 7)
    _forward_case(f"square {n}", x, w, seed=n)
    _dgrad_case(f"square {n}", g, w, seed=n)
    _wgrad_case(f"square {n}", x, g, seed=n)


@pytest.mark.parametrize("m", [16, 64, 256])
def test_shape_sweep_skinny_m_student_t(m):
    """M in {16, 64, 256} with K = N = 8192: the forward and dgrad outputs are compared whole."""
    x = _student_t3((m, 8192), 8)
    w = _normal((8192, 8192), 9, 0.02)
    g = _normal((m, 8192), 10)
    _forward_case(f"skinny {m}", x, w, seed=m)
    _dgrad_case(f"skinny {m}", g, w, seed=m)
    _wgrad_case(f"skinny {m}", x, g, seed=m)


# ---- benchmark configuration 1: norm backward at 32768 x 2048 -------------------------------

def test_norm_backward_at_size():
    """dx on sampled rows (given the kernel-independent oracle rnorm) and the FULL dgamma column sums."""
    from train_gpt_b200 import ops
    rows, D, eps = 32768, 2048, 1e-6
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(rows, D, device="cuda", generator=g)
    x = torch.where(torch.rand(rows, D, device="cuda", generator=g) < 1e-3, x * 50, x).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(D, device="cuda", generator=g)).to(torch.bfloat16)
    gy = torch.randn(rows, D, device="cuda", generator=g).to(torch.bfloat16)
    dx, dgamma = ops.rmsnorm_bwd(x, gamma, gy, eps)
    torch.cuda.synchronize()
    x_h, gy_h, gamma_h = from_torch_bf16(x), from_torch_bf16(gy), from_torch_bf16(gamma)
    dx_ref, dgamma_ref = no.rms_norm_bwd(x_h, gamma_h, gy_h, eps)
    sample = _sample_many_rows(rows, 12, n=1024)
    a = from_torch_bf16(dx[torch.as_tensor(sample, device="cuda")]).astype(np.float32)
    b = dx_ref[sample].astype(np.float32)
    tol = np.abs(b) * 2.0 ** -7 + np.sqrt(np.mean(b * b)) * 2.0 ** -14      # one bf16 ulp + float32 cancellation
    bad = int((np.abs(a - b) > tol).sum())
    print(f"norm backward dx: {a.size} sampled elements, beyond one ulp {bad}, unequal {(a != b).mean():.2e}")
    assert bad == 0 and (a != b).mean() < 1e-2
    dg, dg_ref = from_torch_bf16(dgamma).astype(np.float32), dgamma_ref.astype(np.float32)
    err = np.abs(dg - dg_ref).max()
    bound = 2.0 ** -7 * np.sqrt(np.mean(dg_ref ** 2)) + 2.0 ** -7 * np.abs(dg_ref).max()
    print(f"norm backward dgamma: all {D} columns, max error {err:.3e} (bound {bound:.3e})")
    assert err <= bound
