"""Bit-exact parity of the CUDA quantisers with the CPU oracle (bytes and scales)."""
import numpy as np
import pytest
import torch

from oracle import fp8_oracle as fo
from tests.gpu_util import BF16, f8_bytes, normal_bf16, to_torch_bf16

pytestmark = pytest.mark.gpu


def _awkward(rng, shape):
    x = normal_bf16(rng, shape, outlier_p=0.01).astype(np.float32)
    if shape[0] > 6 and shape[1] >= 256:
        x[3, 128:256] = 0.0          # all-zero tile -> scale 1e-30, bytes 0
        x[4, 0:128] = 1e-36          # amax/448 under the floor
        x[5, -128:] *= 1e-20
        x[6, 7] = -0.0
    return x.astype(BF16)


def _bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


def test_rowwise_matches_reference_vectors(golden):
    from train_gpt_b200 import ops
    x = np.asarray(golden["q_act_in"]).view(BF16)
    q, s = ops.quantize_rowwise(to_torch_bf16(x))
    assert np.array_equal(f8_bytes(q), golden["q_act_bytes"])
    assert np.array_equal(_bits(s.cpu().numpy()), _bits(golden["q_act_scales"]))


@pytest.mark.parametrize("shape", [(1, 128), (7, 384), (300, 1024), (4096, 768), (1000, 2048)])
def test_rowwise_bit_exact(shape):
    from train_gpt_b200 import ops
    rng = np.random.default_rng(hash(shape) % 2**32)
    x = _awkward(rng, shape)
    q, s = ops.quantize_rowwise(to_torch_bf16(x))
    q_ref, s_ref = fo.quantize_to_fp8(x.astype(np.float32))
    assert np.array_equal(f8_bytes(q), q_ref.view(np.uint8))
    assert np.array_equal(_bits(s.cpu().numpy()), _bits(s_ref))


def test_rowwise_leading_dims_and_student_t():
    from train_gpt_b200 import fp8
    rng = np.random.default_rng(5)
    x = rng.standard_t(3, size=(3, 50, 256)).astype(np.float32).astype(BF16)
    q, s = fp8._quantize_to_fp8(to_torch_bf16(x).float(), 128)      # the reference passes the f32 upcast
    q_ref, s_ref = fo.quantize_to_fp8(x.astype(np.float32))
    assert q.shape == (3, 50, 256) and s.shape == (3, 50, 2)
    assert np.array_equal(f8_bytes(q), q_ref.view(np.uint8)) and np.array_equal(_bits(s.cpu().numpy()), _bits(s_ref))


def test_rowwise_nonfinite_tiles_are_flagged():
    from train_gpt_b200 import ops
    x = np.ones((2, 256), np.float32)
    x[0, 5] = np.nan
    x[1, 130] = np.inf
    q, s = ops.quantize_rowwise(to_torch_bf16(x))
    q_ref, s_ref = fo.quantize_to_fp8(x)
    s = s.cpu().numpy()
    b, b_ref = f8_bytes(q), q_ref.view(np.uint8)
    assert np.isnan(s[0, 0]) and np.isinf(s[1, 1]) and np.array_equal(np.isnan(s), np.isnan(s_ref))
    assert np.array_equal((b & 0x7F) == 0x7F, (b_ref & 0x7F) == 0x7F)     # same NaN positions
    finite = (b_ref & 0x7F) != 0x7F
    assert np.array_equal(b[finite], b_ref[finite])


def test_weight_colwise_matches_reference_vectors(golden):
    from train_gpt_b200 import fp8
    b = np.asarray(golden["q_w_in"]).view(BF16)
    q, s = fp8.quantize_weight(to_torch_bf16(b))                      # (K,N), (K/128,N)
    assert np.array_equal(f8_bytes(q).T, golden["q_wt_bytes"])
    assert np.array_equal(_bits(s.cpu().numpy().T), _bits(golden["q_wt_scales"]))


@pytest.mark.parametrize("shape", [(128, 8), (256, 192), (200, 264), (768, 3072), (1000, 2048), (16, 8192)])
def test_colwise_bit_exact(shape):
    from train_gpt_b200 import ops
    rng = np.random.default_rng(hash(shape) % 2**32)
    x = _awkward(rng, shape)
    q, s = ops.quantize_colwise(to_torch_bf16(x))
    q_ref, s_ref = fo.quantize_colwise(x.astype(np.float32))
    assert np.array_equal(f8_bytes(q), q_ref.view(np.uint8))
    assert np.array_equal(_bits(s.cpu().numpy()), _bits(s_ref))


@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (200, 256), (768, 3072)])
def test_block128_bit_exact(shape):
    from train_gpt_b200 import ops
    rng = np.random.default_rng(hash(shape) % 2**32)
    x = _awkward(rng, shape)
    q, s = ops.quantize_block128(to_torch_bf16(x))
    q_ref, s_ref = fo.quantize_block2d(x.astype(np.float32))
    assert np.array_equal(f8_bytes(q), q_ref.view(np.uint8))
    assert np.array_equal(_bits(s.cpu().numpy()), _bits(s_ref))


def test_empty_and_errors():
    from train_gpt_b200 import ops
    q, s = ops.quantize_rowwise(torch.empty(0, 128, dtype=torch.bfloat16, device="cuda"))
    assert q.shape == (0, 128) and s.shape == (0, 1)
    with pytest.raises(ValueError, match="not divisible by block_k"):
        ops.quantize_rowwise(torch.empty(4, 100, dtype=torch.bfloat16, device="cuda"))


def test_full_size_properties():
    """Config-1-sized activation (32768 x 2048 with 0.1 % x50 outliers): properties that do not
    need the oracle on 67 M elements, plus an oracle check of a strided row sample."""
    from train_gpt_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(32768, 2048, device="cuda", generator=g)
    x = torch.where(torch.rand(x.shape, device="cuda", generator=g) < 1e-3, x * 50, x).to(torch.bfloat16)
    q, s = ops.quantize_rowwise(x)
    amax = x.float().view(32768, 16, 128).abs().amax(-1)
    # torch divides by a Python scalar as a multiply by its reciprocal, so take the IEEE division on the host
    s_ref = np.maximum(amax.cpu().numpy() / np.float32(448.0), np.float32(1e-30))
    assert np.array_equal(_bits(s.cpu().numpy()), _bits(s_ref))
    deq = q.float().view(32768, 16, 128) * s[..., None]
    err = (deq - x.float().view(32768, 16, 128)).abs()
    assert bool((err <= amax[..., None] * (2.0 ** -4) + 1e-30).all())       # e4m3 half-ulp at the top binade
    assert int(q.view(torch.uint8).view(32768, 16, 128).__and__(0x7F).amax(-1).min()) == 0x7E  # every tile hits 448
    q2, s2 = ops.quantize_rowwise(x)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)  # deterministic
    rows = torch.arange(0, 32768, 257, device="cuda")
    q_ref, s_ref = fo.quantize_to_fp8(x[rows].float().cpu().numpy())
    assert np.array_equal(f8_bytes(q[rows]), q_ref.view(np.uint8))
    assert np.array_equal(_bits(s[rows].cpu().numpy()), _bits(s_ref))


def test_division_shortcut_is_exact_over_the_whole_domain():
    """Every (bf16 amax, bf16 |x| <= amax) pair: the shipped reciprocal + one-correction form
    gives the same byte as IEEE division."""
    from train_gpt_b200 import ops
    pairs, bare, shipped, two = ops.selftest_quantise_division()
    assert pairs == 1065402240        # sum over finite bf16 amax of #{x : |x| <= amax}
    assert shipped == 0 and two == 0, (pairs, bare, shipped, two)


@pytest.mark.parametrize("shape", [(128, 128), (200, 256), (1000, 2048), (4096, 768)])
def test_rowcol_equals_the_two_separate_quantisers(shape):
    from train_gpt_b200 import ops
    rng = np.random.default_rng(hash(shape) % 2**32)
    x = to_torch_bf16(_awkward(rng, shape))
    q_row, s_row, q_col, s_col = ops.quantize_rowcol(x)
    q1, s1 = ops.quantize_rowwise(x)
    q2, s2 = ops.quantize_colwise(x)
    assert torch.equal(q_row.view(torch.uint8), q1.view(torch.uint8)) and torch.equal(s_row.view(torch.int32), s1.view(torch.int32))
    assert torch.equal(q_col.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s_col.view(torch.int32), s2.view(torch.int32))


def test_rowcol_forms_into_column_slices():
    """tg_quantize_rowcol_ld: three tensors' row and column forms written side by side into wide matrices equal the
    three dense calls bit for bit, and columns nobody owns stay untouched."""
    from train_gpt_b200 import ops
    rows, widths = 300, (256, 128, 384)
    N = sum(widths)
    f8 = torch.float8_e4m3fn
    big_q = torch.full((rows, N + 128), 0x55, dtype=torch.uint8, device="cuda").view(f8)
    big_s = torch.full((rows, (N + 128) // 128), -7.0, dtype=torch.float32, device="cuda")
    big_qc = torch.full((rows, N + 128), 0x55, dtype=torch.uint8, device="cuda").view(f8)
    big_sc = torch.full(((rows + 127) // 128, N + 128), -7.0, dtype=torch.float32, device="cuda")
    off = 0
    for i, w in enumerate(widths):
        x = to_torch_bf16(normal_bf16(np.random.default_rng(40 + i), (rows, w), outlier_p=0.01))
        dense = ops.quantize_rowcol(x)
        ops.quantize_rowcol(x, row_out=(big_q[:, off:off + w], big_s[:, off // 128:(off + w) // 128]),
                            col_out=(big_qc[:, off:off + w], big_sc[:, off:off + w]))
        assert torch.equal(big_q[:, off:off + w].view(torch.uint8), dense[0].view(torch.uint8))
        assert torch.equal(big_s[:, off // 128:(off + w) // 128], dense[1])
        assert torch.equal(big_qc[:, off:off + w].view(torch.uint8), dense[2].view(torch.uint8))
        assert torch.equal(big_sc[:, off:off + w], dense[3])
        only_rows = ops.quantize_rowcol(x, row_out=(big_q[:, off:off + w], big_s[:, off // 128:(off + w) // 128]))
        assert torch.equal(only_rows[2].view(torch.uint8), dense[2].view(torch.uint8)) and torch.equal(only_rows[3], dense[3])
        off += w
    for t in (big_q, big_qc):
        assert bool((t[:, N:].view(torch.uint8) == 0x55).all())
    assert bool((big_s[:, N // 128:] == -7.0).all()) and bool((big_sc[:, N:] == -7.0).all())
    with pytest.raises(TypeError):
        ops.quantize_rowcol(x, row_out=(big_q[:, :128], big_s[:, :1]))          # wrong shape for this x
