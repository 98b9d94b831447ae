"""Parity of the tcgen05 block-scaled GEMM (forward, dgrad, wgrad) with the CPU oracle.

Tolerance (stated for this path): |got - ref| <= 1e-2 * RMS(ref) + 2e-2 * |ref| elementwise,
`ref` being the oracle's bf16 result on the SAME quantised operands (like-for-like).  The
GEMM accumulates e4m3 products in float32 inside the tensor core and promotes per 128-deep
block in float32, the oracle in float64, so differences are float32 rounding plus one bf16
output rounding; the tests also bound the Frobenius error far below the tolerance.
"""
import numpy as np
import pytest
import torch

from oracle import fp8_oracle as fo
from tests.gpu_util import BF16, F8, f8_bytes, from_torch_bf16, normal_bf16, to_torch_bf16

pytestmark = pytest.mark.gpu


def _close(got, ref, frob=2e-3):
    got = np.asarray(got).astype(np.float64)
    ref = np.asarray(ref).astype(np.float64)
    assert np.isfinite(got).all()
    assert fo.tolerance_violations(got, ref) == 0, f"rel_frob={fo.rel_frobenius(got, ref):.3e}"
    assert fo.rel_frobenius(got, ref) < frob


def _status_ok(st):
    assert int(st.item()) == 0, f"GEMM bounded wait expired, role code {int(st.item())}"


def test_ones_known_answer():
    # train-gpt debug_fp8.py:105-109: ones(4,128) @ ones(128,4) -> exactly 128
    from train_gpt_b200 import fp8
    y = fp8.block_scaled_matmul(torch.ones(4, 128, dtype=torch.bfloat16, device="cuda"),
                                torch.ones(128, 4, dtype=torch.bfloat16, device="cuda"))
    assert y.dtype == torch.bfloat16 and y.shape == (4, 4) and bool((y.float() == 128.0).all())


@pytest.mark.parametrize("M,K,N", [(128, 128, 128), (256, 384, 256), (200, 256, 144), (16, 512, 384),
                                    (2048, 256, 1536), (384, 1024, 128)])
@pytest.mark.parametrize("tile", [(128, 1), (128, 128)])
def test_forward(M, K, N, tile):
    from train_gpt_b200 import fp8, ops
    if tile == (128, 128) and N % 128:
        pytest.skip("128x128 weight tiles need N % 128 == 0")
    rng = np.random.default_rng(M * 7 + K * 3 + N)
    a = normal_bf16(rng, (M, K), outlier_p=1e-3)
    b = normal_bf16(rng, (K, N), std=0.02)
    st = ops.new_status("cuda")
    a_q, a_s = ops.quantize_rowwise(to_torch_bf16(a))
    w_q, w_s = fp8.quantize_weight(to_torch_bf16(b), tile)
    y = ops.gemm_fwd(a_q, a_s, w_q, w_s, tile, status=st)
    torch.cuda.synchronize()
    _status_ok(st)
    _close(from_torch_bf16(y), fo.block_scaled_matmul(a, b, weight_tile=tile))


def test_forward_f32_output_and_leading_dims():
    from train_gpt_b200 import fp8, ops
    rng = np.random.default_rng(3)
    a = normal_bf16(rng, (2, 70, 256))
    b = normal_bf16(rng, (256, 272), std=0.02)
    y = fp8.block_scaled_matmul(to_torch_bf16(a), to_torch_bf16(b))
    assert y.shape == (2, 70, 272)
    _close(from_torch_bf16(y), fo.block_scaled_matmul(a, b))
    a_q, a_s = ops.quantize_rowwise(to_torch_bf16(a.reshape(-1, 256)))
    w_q, w_s = fp8.quantize_weight(to_torch_bf16(b))
    y32 = ops.gemm_fwd(a_q, a_s, w_q, w_s, out_dtype=torch.float32)
    aq, as_ = fo.quantize_to_fp8(a.reshape(-1, 256).astype(np.float32))
    bq, bs = fo.quantize_to_fp8(b.astype(np.float32).T)
    ref32 = fo.scaled_matmul(aq, bq, as_, bs)
    assert fo.rel_frobenius(y32.cpu().numpy(), ref32) < 1e-5


@pytest.mark.parametrize("M,K,N", [(128, 128, 128), (200, 256, 384), (16, 384, 256), (1536, 512, 1024)])
@pytest.mark.parametrize("tile", [(128, 1), (128, 128)])
def test_fp8_backward_like_for_like(M, K, N, tile):
    from train_gpt_b200 import fp8
    rng = np.random.default_rng(M + K + N)
    a = normal_bf16(rng, (M, K))
    b = normal_bf16(rng, (K, N), std=0.02)
    g = normal_bf16(rng, (M, N))
    da, db = fp8._fp8_backward(128, (to_torch_bf16(a), to_torch_bf16(b)), to_torch_bf16(g), tile, "fp8")
    da_ref, db_ref = fo.backward_fp8(a, b, g, weight_tile=tile)
    _close(from_torch_bf16(da), da_ref)
    _close(from_torch_bf16(db), db_ref)
    # how far the FP8 gradients sit from the reference's straight-through ones (reported, bounded)
    da_ste, db_ste = fo.backward_bf16_ste(a, b, g)
    assert fo.rel_frobenius(from_torch_bf16(da), da_ste) < 0.06
    assert fo.rel_frobenius(from_torch_bf16(db), db_ste) < 0.06


def test_autograd_ste_matches_reference_vectors(golden):
    from train_gpt_b200 import fp8
    a = to_torch_bf16(np.asarray(golden["ste_a"]).view(BF16)).requires_grad_(True)
    b = to_torch_bf16(np.asarray(golden["q_w_in"]).view(BF16)).requires_grad_(True)
    g = to_torch_bf16(np.asarray(golden["ste_g"]).view(BF16))
    y = fp8.block_scaled_matmul(a, b)                 # reference defaults: tile (128,1), bf16 STE backward
    y.backward(g)
    _close(from_torch_bf16(a.grad), np.asarray(golden["ste_da"]).view(BF16), frob=4e-3)
    _close(from_torch_bf16(b.grad), np.asarray(golden["ste_db"]).view(BF16), frob=4e-3)
    assert a.grad.dtype == torch.bfloat16 and a.grad.shape == a.shape and b.grad.shape == b.shape
    _close(from_torch_bf16(y), fo.block_scaled_matmul(np.asarray(golden["ste_a"]).view(BF16), np.asarray(golden["q_w_in"]).view(BF16)))


def test_config0_single_linear_fwd_bwd():
    """Benchmark configuration 0: x (4096,768) N(0,1), W (768,3072) N(0,0.02), g (4096,3072), seed 0."""
    from train_gpt_b200 import fp8
    rng = np.random.default_rng(0)
    x = normal_bf16(rng, (4096, 768))
    w = normal_bf16(rng, (768, 3072), std=0.02)
    g = normal_bf16(rng, (4096, 3072))
    for tile in [(128, 1), (128, 128)]:
        xt, wt = to_torch_bf16(x).requires_grad_(True), to_torch_bf16(w).requires_grad_(True)
        y = fp8.block_scaled_matmul(xt, wt, weight_tile=tile, backward="fp8")
        y.backward(to_torch_bf16(g))
        _close(from_torch_bf16(y), fo.block_scaled_matmul(x, w, weight_tile=tile))
        da_ref, db_ref = fo.backward_fp8(x, w, g, weight_tile=tile)
        _close(from_torch_bf16(xt.grad), da_ref)
        _close(from_torch_bf16(wt.grad), db_ref)
    # reference-exact configuration: straight-through bf16 gradients
    xt, wt = to_torch_bf16(x).requires_grad_(True), to_torch_bf16(w).requires_grad_(True)
    fp8.block_scaled_matmul(xt, wt).backward(to_torch_bf16(g))
    da_ref, db_ref = fo.backward_bf16_ste(x, w, g)
    _close(from_torch_bf16(xt.grad), da_ref, frob=4e-3)
    _close(from_torch_bf16(wt.grad), db_ref, frob=4e-3)


def test_fused_norm_feeds_gemm():
    """q/k/v-style fan-out: one fused norm+quantise output consumed by two GEMMs equals the
    reference composition norm -> matmul per projection."""
    from train_gpt_b200 import fp8, kernels
    from oracle import norm_oracle as no
    rng = np.random.default_rng(9)
    x = normal_bf16(rng, (4, 96, 256))
    gamma = (1 + 0.1 * rng.standard_normal(256)).astype(BF16)
    w1 = normal_bf16(rng, (256, 128), std=0.02)
    w2 = normal_bf16(rng, (256, 384), std=0.02)
    nq = kernels.rms_norm_quant(to_torch_bf16(x), to_torch_bf16(gamma), 1e-5, want_y=True)
    y_np = from_torch_bf16(nq.y)
    for w in (w1, w2):
        y = fp8.block_scaled_matmul(nq.y, to_torch_bf16(w), a_quantized=nq.as_pair())
        _close(from_torch_bf16(y), fo.block_scaled_matmul(y_np, w))
    assert (y_np.view(np.uint16) != no.rms_norm(x, gamma, 1e-5).view(np.uint16)).mean() < 2e-3


def test_linearity_at_full_k():
    """Size-independent property on a large contraction (K = 8192): scaling the weight by 2 (a
    power of two: exact in bf16 and in the scales) doubles the output bit for bit."""
    from train_gpt_b200 import fp8
    g = torch.Generator(device="cuda").manual_seed(4)
    a = torch.randn(512, 8192, device="cuda", generator=g).to(torch.bfloat16)
    b = (0.02 * torch.randn(8192, 1024, device="cuda", generator=g)).to(torch.bfloat16)
    y1 = fp8.block_scaled_matmul(a, b)
    y2 = fp8.block_scaled_matmul(a, b * 2)
    assert torch.equal(y2.float(), y1.float() * 2)
    ref = a.float() @ b.float()
    assert float((y1.float() - ref).norm() / ref.norm()) < 0.05


@pytest.mark.parametrize("M,K,N", [(200, 256, 384), (1536, 512, 1024)])
def test_fp8_backward_with_block_quantised_gradient(M, K, N):
    """backward="fp8_blockgrad": wgrad with the upstream gradient in 128x128 blocks, like-for-like."""
    from train_gpt_b200 import fp8
    rng = np.random.default_rng(M + N)
    a = normal_bf16(rng, (M, K))
    b = normal_bf16(rng, (K, N), std=0.02)
    g = normal_bf16(rng, (M, N))
    da, db = fp8._fp8_backward(128, (to_torch_bf16(a), to_torch_bf16(b)), to_torch_bf16(g), (128, 128), "fp8_blockgrad")
    da_ref, db_ref = fo.backward_fp8(a, b, g, weight_tile=(128, 128), wgrad_grad_tile=(128, 128))
    _close(from_torch_bf16(da), da_ref)
    _close(from_torch_bf16(db), db_ref)


@pytest.mark.parametrize("K,N,T,gran", [(256, 384, 4096, 1), (512, 512, 8192, 1), (256, 512, 4096, 128),
                                        (256, 384, 5632, 1), (256, 512, 5632, 128)])   # 44 blocks: 5 ranges of 9, 9, 9, 9, 8
def test_wgrad_with_split_contraction_matches_unsplit_and_oracle(K, N, T, gran):
    """Few output tiles, long contraction: the library cuts the contraction when given workspace.
    The cut changes only the float32 summation order."""
    from train_gpt_b200 import ops
    rng = np.random.default_rng(K + N + T)
    x = normal_bf16(rng, (T, K))
    g = normal_bf16(rng, (T, N))
    xq, xs = ops.quantize_colwise(to_torch_bf16(x))
    if gran == 1:
        gq, gs = ops.quantize_colwise(to_torch_bf16(g))
        tile = (128, 1)
    else:
        gq, gs = ops.quantize_block128(to_torch_bf16(g))
        tile = (128, 128)
    import ctypes as C
    from train_gpt_b200 import _lib
    st = ops.new_status("cuda")
    a = ops.gemm_blockscaled(xq, gq, xs, gs, M=K, N=N, K=T, a_major=_lib.TG_MAJOR_MN, b_major=_lib.TG_MAJOR_MN,
                             sa_strides=(1, K), sb_strides=(1, gs.shape[1]), sb_gran_n=gran, out_dtype=torch.float32,
                             status=st, split=False)
    b = ops.gemm_wgrad(xq, xs, gq, gs, out_dtype=torch.float32, status=st, grad_tile=tile)
    assert int(st.item()) == 0
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-5 * float(a.abs().max()))
    assert ops.last_gemm_kernel_launches == 2         # the split path really ran: GEMM + the reduce kernel
    x_q, x_s = fo.quantize_colwise(x.astype(np.float32))
    if gran == 1:
        g_q, g_s = fo.quantize_colwise(g.astype(np.float32))
    else:
        g_q, g_sb = fo.quantize_block2d(g.astype(np.float32))
        g_s = np.repeat(g_sb, 128, axis=1)
    ref = fo.scaled_matmul(x_q.T, g_q.T, x_s.T, g_s.T)
    _close(b.cpu().numpy(), ref)



def test_bounded_wait_gives_up_and_the_cta_tears_down():
    """The path no healthy GEMM takes: a barrier wait whose limit runs out.  The self-test kernel waits
    (about a millisecond) on a barrier nobody arrives at, with the GEMM's own wait routine: it must
    RETURN with the role code in the status word, the other waiting role must leave on the abort flag
    rather than on its own, 64 times longer, limit, an ordinary wait beside them must still succeed,
    and the teardown must run (tensor memory freed) -- after which the device runs GEMMs as before."""
    from train_gpt_b200 import fp8, ops
    code, report = ops.selftest_bounded_wait(2_000_000)
    assert code == 5, code
    assert report == [0, 2, 1, 1], report
    with pytest.raises(RuntimeError, match="status 5"):
        ops.check_status(torch.tensor([code], dtype=torch.int32))
    with pytest.raises(ValueError):
        ops.selftest_bounded_wait(10 ** 12)                     # the limit itself is capped on the host
    y = fp8.block_scaled_matmul(torch.ones(4, 128, dtype=torch.bfloat16, device="cuda"),
                                torch.ones(128, 4, dtype=torch.bfloat16, device="cuda"))
    assert bool((y.float() == 128.0).all())
    ops.check_status(device="cuda")                             # the real GEMMs' shared status word stayed 0


@pytest.mark.parametrize("M,K,N", [(8, 1024, 1024), (16, 2048, 1536), (64, 1024, 2048), (136, 1024, 1152), (192, 1024, 1024),
                                    (200, 1024, 1280), (256, 2048, 1024)])
@pytest.mark.parametrize("tile", [(128, 1), (128, 128)])
def test_few_tokens_run_transposed(M, K, N, tile):
    """M <= 128 tokens against a wide weight: the library runs the problem with its operands swapped (the weight's
    N on the MMA's 128 rows, the contraction cut across SMs, a transposing reduce at the end); the larger M here
    sit just past that switch.  Forward and dgrad, bf16 and float32 outputs, against the oracle; without
    workspace the same call takes the ordinary path."""
    from train_gpt_b200 import fp8, ops
    rng = np.random.default_rng(M * 5 + K + N)
    a = normal_bf16(rng, (M, K), outlier_p=1e-3)
    b = normal_bf16(rng, (K, N), std=0.02)
    g = normal_bf16(rng, (M, N))
    st = ops.new_status("cuda")
    a_q, a_s = ops.quantize_rowwise(to_torch_bf16(a))
    w_q, w_s = fp8.quantize_weight(to_torch_bf16(b), tile)
    y = ops.gemm_fwd(a_q, a_s, w_q, w_s, tile, status=st)
    if M <= 128:
        assert ops.last_gemm_kernel_launches == 2          # the transposed path: GEMM + transposing reduce
    ref = fo.block_scaled_matmul(a, b, weight_tile=tile)
    _close(from_torch_bf16(y), ref)
    y32 = ops.gemm_fwd(a_q, a_s, w_q, w_s, tile, out_dtype=torch.float32, status=st)
    assert fo.rel_frobenius(from_torch_bf16(y32.to(torch.bfloat16)), ref) < 2e-3
    # the ordinary path (no workspace) gives the same numbers up to float32 summation order
    M_, N_ = y.shape
    sb_str = (1, N) if tile == (128, 1) else (1, w_s.shape[1])
    from train_gpt_b200 import _lib
    y_plain = ops.gemm_blockscaled(a_q, w_q, a_s, w_s, M=M, N=N, K=K, a_major=_lib.TG_MAJOR_K, b_major=_lib.TG_MAJOR_MN,
                                   sa_strides=(a_s.shape[1], 1), sb_strides=sb_str, sb_gran_n=1 if tile == (128, 1) else 128,
                                   out_dtype=torch.float32, status=st, split=False)
    assert torch.allclose(y32, y_plain, rtol=1e-5, atol=1e-5 * float(y_plain.abs().max()))
    # dgrad: dx = g W^T, the weight quantised along N
    g_q, g_s = ops.quantize_rowwise(to_torch_bf16(g))
    wd_q, wd_s = ops.quantize_rowwise(to_torch_bf16(b)) if tile == (128, 1) else (w_q, w_s)
    dx = ops.gemm_dgrad(g_q, g_s, wd_q, wd_s, tile, status=st)
    da_ref, _ = fo.backward_fp8(a, b, g, weight_tile=tile)
    _close(from_torch_bf16(dx), da_ref)
    torch.cuda.synchronize()
    _status_ok(st)


def test_wider_inputs_are_taken_only_if_they_hold_bf16_values():
    """The reference upcasts bf16 operands to float32 before quantising (fp8.py:66,68); here a float32
    operand is accepted when it is such an upcast and refused (not silently rounded) otherwise."""
    from train_gpt_b200 import fp8
    a = torch.randn(8, 128, device="cuda").to(torch.bfloat16)
    b = (0.02 * torch.randn(128, 16, device="cuda")).to(torch.bfloat16)
    y = fp8.block_scaled_matmul(a, b)
    assert torch.equal(fp8.block_scaled_matmul(a.float(), b.float()), y)
    with pytest.raises(TypeError, match="bf16 cannot hold"):
        fp8.block_scaled_matmul(a.float() + 1e-4, b)
    with pytest.raises(TypeError, match="bf16 cannot hold"):
        fp8._quantize_to_fp8(torch.full((2, 128), 1.0 + 2.0 ** -12, device="cuda"))
