"""GPU parity: tcgen05 FP8 GEMM vs the oracle (fp64-accumulated C loop for small cases, fp32 BLAS on the
decoded operands for large ones).  Floating-point bar: cosine >= 0.999 and max-abs <= 2e-2 x RMS(ref);
the tighter bound asserted here is one bf16 ulp of the value plus a small RMS-relative slack."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


def _fp8_operand(rng, rows, K, scale=0.02):
    """Seeded N(0, scale^2) operand quantised per tensor with scale = amax/448 (torch's E4M3 cast is
    bit-identical to the oracle's, checked in the CPU suite)."""
    import torch
    x = (rng.standard_normal((rows, K)) * scale).astype(np.float32)
    s = max(float(np.abs(x).max()) / 448.0, 1e-12)
    codes = torch.from_numpy(np.clip(x / np.float32(s), -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    return codes, np.float32(s)


def _check(D_bits, ref_f32):
    from gpu_util import cosine
    got = O.bf16_bits_to_f32(D_bits)
    rms = float(np.sqrt(np.mean(ref_f32.astype(np.float64) ** 2)))
    err = np.abs(got - ref_f32)
    assert cosine(got, ref_f32) >= 0.9999
    assert err.max() <= 2e-2 * rms
    assert (err <= np.abs(ref_f32) * 2.0 ** -8 + 2e-3 * rms).all()


def _ref(A, W, sa, sb, bias=None):
    a = O.e4m3_to_f32(A)
    w = O.e4m3_to_f32(W)
    r = (a @ w.T) * (np.float32(sa) * np.float32(sb))
    if bias is not None:
        r = r + O.bf16_bits_to_f32(bias)[None, :]
    return r.astype(np.float32)


SMALL = [(1, 128, 128), (16, 1024, 1024), (50, 2560, 1024), (50, 1024, 2048), (50, 8192, 1024), (50, 1024, 4096),
         (64, 256, 512), (100, 384, 256), (256, 4096, 1024), (33, 130, 144), (50, 1000, 1040)]


@pytest.mark.parametrize("M,N,K", SMALL)
@pytest.mark.parametrize("splits", [1, 0, 2, 8])
def test_gemm_fp8_small_m(M, N, K, splits):
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(M * 1000003 + N * 131 + K + splits)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    d_A, d_W, d_D = Dev(A), Dev(W), zeros((M, N), np.uint16)
    d_sa, d_sb = f32(sa), f32(sb)
    fvk.GemmRunner().fp8_nt_dev(d_A.ptr, d_W.ptr, d_D.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=splits)
    got = d_D.get()
    assert fvk.tensor_core_status() == 0
    _check(got, _ref(A, W, sa, sb))


def test_gemm_fp8_matches_fp64_oracle_exact_products():
    """Small integers in E4M3 make every product and partial sum exact: the result must equal the oracle bit for bit."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(5)
    M, N, K = 50, 256, 512
    vals = np.array([-4, -3, -2, -1, 0, 1, 2, 3, 4], np.float32)
    import torch
    A = torch.from_numpy(rng.choice(vals, (M, K))).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    W = torch.from_numpy(rng.choice(vals, (N, K))).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    ref = O.gemm_fp8(A, W, 0.5, 0.25, b_is_nk=True)
    d_sa, d_sb = f32(0.5), f32(0.25)
    for splits in (1, 4):
        d_A, d_W, d_D = Dev(A), Dev(W), zeros((M, N), np.uint16)
        fvk.fp8_gemm_descale_bf16out(d_A.ptr, d_W.ptr, d_D.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=splits)
        assert np.array_equal(d_D.get(), ref)


@pytest.mark.parametrize("M,N,K", [(2048, 1024, 1024), (300, 512, 256), (2048, 4096, 1024), (8192, 3072, 3072),
                                   (1000, 200, 4096), (257, 72, 128)])
def test_gemm_fp8_large_m(M, N, K):
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(M + N + K)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    d_A, d_W, d_D, d_sa, d_sb = Dev(A), Dev(W), zeros((M, N), np.uint16), f32(sa), f32(sb)
    fvk.GemmRunner().fp8_nt_dev(d_A.ptr, d_W.ptr, d_D.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0)
    got = d_D.get()
    assert fvk.tensor_core_status() == 0
    _check(got, _ref(A, W, sa, sb))


def test_gemm_bias_and_linearity():
    """bias epilogue; and D(alpha) scales linearly with the activation scale (a size-independent property)."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(11)
    M, N, K = 50, 1024, 1024
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    bias = rand_bf16(rng, (N,), 0.5)
    d_A, d_W, d_D, d_b = Dev(A), Dev(W), zeros((M, N), np.uint16), Dev(bias)
    g = fvk.GemmRunner()
    d_sa, d_sb, d_sa4 = f32(sa), f32(sb), f32(sa * 4)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_D.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, bias=d_b.ptr)
    _check(d_D.get(), _ref(A, W, sa, sb, bias))
    d_D2 = zeros((M, N), np.uint16)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_D.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_D2.ptr, M, N, K, d_sa4.ptr, d_sb.ptr, 0)   # x4 is exact in bf16
    assert np.array_equal(O.bf16_bits_to_f32(d_D.get()) * 4, O.bf16_bits_to_f32(d_D2.get()))


def test_small_bf16_projections():
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, rand_bf16, zeros
    rng = np.random.default_rng(3)
    g = fvk.GemmRunner()
    for (M, N, K) in [(50, 1024, 32), (50, 32, 1024), (10, 32, 1024), (4, 1024, 32)]:
        A, B = rand_bf16(rng, (M, K)), rand_bf16(rng, (K, N), 0.02)
        bias = rand_bf16(rng, (N,), 0.1)
        ref = O.bf16_bits_to_f32(A).astype(np.float64) @ O.bf16_bits_to_f32(B).astype(np.float64)
        d_D, d_A, d_B, d_bias = zeros((M, N), np.uint16), Dev(A), Dev(B), Dev(bias)
        g.bf16_nn(d_A.ptr, d_B.ptr, d_D.ptr, M, N, K, 0)
        got = O.bf16_bits_to_f32(d_D.get())
        rms = np.sqrt(np.mean(ref ** 2))
        assert np.abs(got - ref).max() <= np.abs(ref).max() * 2.0 ** -8 + 1e-3 * rms
        d_D2 = zeros((M, N), np.uint16)
        g.bf16_nn(d_A.ptr, d_B.ptr, d_D2.ptr, M, N, K, 0, bias=d_bias.ptr)
        got2 = O.bf16_bits_to_f32(d_D2.get())
        ref2 = ref + O.bf16_bits_to_f32(bias)[None, :]
        assert np.abs(got2 - ref2).max() <= np.abs(ref2).max() * 2.0 ** -8 + 1e-3 * rms


@pytest.mark.parametrize("M,splits", [(50, 4), (50, 1), (10, 8), (64, 2)])
def test_fused_rope_split_epilogue_equals_two_kernels(M, splits):
    """QKV GEMM with the RoPE/split/KV-append epilogue == GEMM then qkv_split_rope, byte for byte
    (the reference's own fused-vs-unfused contract, tests/test_pi05_decoder_fp4_kernels.py:45-61)."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M + splits)
    K, q_dim, k_dim, v_dim, hd, pos = 1024, 2048, 256, 256, 256, 768
    N = q_dim + k_dim + v_dim
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    inv_freq = 1.0 / (10000 ** (np.arange(0, hd, 2, dtype=np.float64) / hd))
    ph = np.arange(pos, pos + M, dtype=np.float64)[:, None] * inv_freq[None, :]
    rope = O.f32_to_bf16_bits(np.stack([np.cos(ph), np.sin(ph)], -1).reshape(M, hd).astype(np.float32))
    d_A, d_W, d_sa, d_sb, d_rope = Dev(A), Dev(W), f32(sa), f32(sb), Dev(rope)
    g = fvk.GemmRunner()
    cache0 = rand_bf16(rng, (pos + M + 2, 256))
    # two kernels
    d_qkv, d_Q1, d_K1, d_V1 = zeros((M, N), np.uint16), zeros((M, q_dim), np.uint16), Dev(cache0), Dev(cache0)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_qkv.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=splits)
    fvk.qkv_split_rope(d_qkv.ptr, d_rope.ptr, d_Q1.ptr, d_K1.ptr + pos * 512, d_V1.ptr + pos * 512, M, q_dim, k_dim,
                       v_dim, hd, 0)
    # one kernel
    d_Q2, d_K2, d_V2 = zeros((M, q_dim), np.uint16), Dev(cache0), Dev(cache0)
    g.fp8_nt_dev_rope_split(d_A.ptr, d_W.ptr, M, K, d_sa.ptr, d_sb.ptr, d_rope.ptr, d_Q2.ptr, d_K2.ptr + pos * 512,
                            d_V2.ptr + pos * 512, q_dim, k_dim, v_dim, hd, 0, splits=splits)
    assert fvk.tensor_core_status() == 0
    assert np.array_equal(d_Q1.get(), d_Q2.get())
    assert np.array_equal(d_K1.get(), d_K2.get())
    assert np.array_equal(d_V1.get(), d_V2.get())
    # and both agree with the oracle chain on the oracle's GEMM
    Kr, Vr = cache0.copy(), cache0.copy()
    Q_ref = O.qkv_split_rope(d_qkv.get(), rope, Kr, Vr, pos, q_dim, k_dim, v_dim, hd)
    assert np.array_equal(d_Q2.get(), Q_ref) and np.array_equal(d_K2.get(), Kr) and np.array_equal(d_V2.get(), Vr)


@pytest.mark.parametrize("M,splits", [(50, 2), (50, 1), (16, 8), (100, 2)])
def test_fused_geglu_epilogue_equals_two_kernels(M, splits):
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(M * 3 + splits)
    K, H = 1024, 4096
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, 2 * H, K, 0.03)
    d_A, d_W, d_sa, d_sb, d_so = Dev(A), Dev(W), f32(sa), f32(sb), f32(0.004)
    g = fvk.GemmRunner()
    d_merged, d_o1, d_o2 = zeros((M, 2 * H), np.uint16), zeros((M, H), np.uint8), zeros((M, H), np.uint8)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_merged.ptr, M, 2 * H, K, d_sa.ptr, d_sb.ptr, 0, splits=splits)
    fvk.gate_geglu_merged_fp8(d_merged.ptr, d_o1.ptr, M, H, d_so.ptr, 0)
    g.fp8_nt_dev_geglu_fp8(d_A.ptr, d_W.ptr, d_o2.ptr, M, H, K, d_sa.ptr, d_sb.ptr, d_so.ptr, 0, splits=splits)
    assert fvk.tensor_core_status() == 0
    assert np.array_equal(d_o1.get(), d_o2.get())
    assert np.array_equal(d_o2.get(), O.geglu_fp8(d_merged.get(), 0.004))
    assert (d_o2.get() != 0).mean() > 0.5


@pytest.mark.parametrize("M,splits", [(50, 2), (16, 4), (128, 1)])
def test_fused_swiglu_epilogue_equals_two_kernels(M, splits):
    """SiLU gate in the GEMM epilogue (token-major kernel): the bytes of GEMM -> gate_swiglu_merged_fp8; refused where
    that kernel does not run."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from flashrt_b200._lib import KernelError
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(M * 5 + splits)
    K, H = 1024, 2048
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, 2 * H, K, 0.03)
    d_A, d_W, d_sa, d_sb, d_so = Dev(A), Dev(W), f32(sa), f32(sb), f32(0.004)
    g = fvk.GemmRunner()
    d_merged, d_o1, d_o2 = zeros((M, 2 * H), np.uint16), zeros((M, H), np.uint8), zeros((M, H), np.uint8)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_merged.ptr, M, 2 * H, K, d_sa.ptr, d_sb.ptr, 0, splits=splits)
    fvk.gate_swiglu_merged_fp8(d_merged.ptr, d_o1.ptr, M, H, d_so.ptr, 0)
    g.fp8_nt_dev_geglu_fp8(d_A.ptr, d_W.ptr, d_o2.ptr, M, H, K, d_sa.ptr, d_sb.ptr, d_so.ptr, 0, splits=splits,
                           silu_gate=True)
    assert fvk.tensor_core_status() == 0
    assert np.array_equal(d_o1.get(), d_o2.get())
    assert np.array_equal(d_o2.get(), O.swiglu_fp8(d_merged.get(), 0.004))
    assert (d_o2.get() != 0).mean() > 0.5
    with pytest.raises(KernelError):       # more rows than the token-major kernel takes
        g.fp8_nt_dev_geglu_fp8(d_A.ptr, d_W.ptr, d_o2.ptr, 200, H, K, d_sa.ptr, d_sb.ptr, d_so.ptr, 0, silu_gate=True)


@pytest.mark.parametrize("N,K,splits", [(1024, 2048, 16), (1024, 4096, 16), (2560, 1024, 4)])
def test_split_k_over_large_clusters(N, K, splits):
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(N + K)
    M = 50
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    d_A, d_W, d_D, d_sa, d_sb = Dev(A), Dev(W), zeros((M, N), np.uint16), f32(sa), f32(sb)
    fvk.GemmRunner().fp8_nt_dev(d_A.ptr, d_W.ptr, d_D.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=splits)
    got = d_D.get()
    assert fvk.tensor_core_status() == 0
    _check(got, _ref(A, W, sa, sb))


@pytest.mark.parametrize("M,N,K", [(2048, 1024, 1024), (1000, 200, 4096), (4096, 3072, 1024), (300, 512, 256)])
def test_gemm_fp8_persistent_equals_one_tile_per_cta(M, N, K):
    """The persistent large-M kernel (two accumulators in tensor memory, overlapped epilogue) and the
    one-tile-per-CTA kernel accumulate every output in the same order: identical bytes."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M * 3 + N + K)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    bias = rand_bf16(rng, (N,), 0.3)
    d_A, d_W, d_b, d_sa, d_sb = Dev(A), Dev(W), Dev(bias), f32(sa), f32(sb)
    d_1, d_2 = zeros((M, N), np.uint16), zeros((M, N), np.uint16)
    g = fvk.GemmRunner()
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_1.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, bias=d_b.ptr)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_2.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, bias=d_b.ptr, one_tile_per_cta=True)
    assert fvk.tensor_core_status() == 0
    assert np.array_equal(d_1.get(), d_2.get())
    _check(d_1.get(), _ref(A, W, sa, sb, bias))


@pytest.mark.parametrize("M,N,K", [(2048, 1024, 1024), (512, 256, 128), (1000, 700, 512), (8192, 3072, 3072)])
def test_gemm_fp8_cta_pair_kernel(M, N, K):
    """256 x 256 tiles on CTA pairs (tcgen05 cta_group::2) against the torch reference, and against the persistent
    one-CTA kernel (same K order per output: expected identical, asserted to within the bf16 rounding of the result)."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M + 7 * N + K)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    bias = rand_bf16(rng, (N,), 0.3)
    d_A, d_W, d_b, d_sa, d_sb = Dev(A), Dev(W), Dev(bias), f32(sa), f32(sb)
    d_1, d_2 = zeros((M, N), np.uint16), zeros((M, N), np.uint16)
    g = fvk.GemmRunner()
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_1.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, bias=d_b.ptr, cta_pair=False)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_2.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, bias=d_b.ptr, cta_pair=True)
    assert fvk.tensor_core_status() == 0
    _check(d_2.get(), _ref(A, W, sa, sb, bias))
    a, b = d_1.get().astype(np.int64), d_2.get().astype(np.int64)
    assert np.abs(a - b).max() <= 1          # bf16 bit patterns at most one step apart


@pytest.mark.parametrize("M,N,K", [(2048, 1024, 1024), (1000, 200, 512), (3000, 14336 // 8, 3072)])
def test_gemm_fp8_bias_gelu_epilogue_equals_pair(M, N, K):
    """GEMM with bias + GELU + FP8 quantise in the epilogue == GEMM -> bias_gelu_quantize_fp8, byte for byte."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M + 5 * N + K)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    bias = rand_bf16(rng, (N,), 0.3)
    d_A, d_W, d_b, d_sa, d_sb, d_so = Dev(A), Dev(W), Dev(bias), f32(sa), f32(sb), f32(0.013)
    g = fvk.GemmRunner()
    d_mid, d_pair, d_fused = zeros((M, N), np.uint16), zeros((M, N), np.uint8), zeros((M, N), np.uint8)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_mid.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0)
    fvk.bias_gelu_quantize_fp8_static_bf16(d_mid.ptr, d_b.ptr, d_pair.ptr, d_so.ptr, M, N, 0)
    g.fp8_nt_dev_bias_gelu_fp8(d_A.ptr, d_W.ptr, d_fused.ptr, M, N, K, d_sa.ptr, d_sb.ptr, d_b.ptr, d_so.ptr, 0)
    assert fvk.tensor_core_status() == 0
    assert np.array_equal(d_pair.get(), d_fused.get())
    # and against the oracle
    ref = O.bias_gelu_quantize_fp8(d_mid.get(), bias, 0.013)
    assert np.array_equal(d_fused.get(), ref)
    # GELU through the hardware tanh (flags bit 7): the same codes except for last-place flips at rounding boundaries
    d_fast = zeros((M, N), np.uint8)
    g.fp8_nt_dev_bias_gelu_fp8(d_A.ptr, d_W.ptr, d_fast.ptr, M, N, K, d_sa.ptr, d_sb.ptr, d_b.ptr, d_so.ptr, 0,
                               fast_gelu=True)
    assert fvk.tensor_core_status() == 0
    f = d_fast.get()
    assert (f != ref).mean() <= 5e-3
    vr, vf = O.e4m3_to_f32(ref), O.e4m3_to_f32(f)
    assert (np.abs(vr - vf) <= np.abs(vr) * 0.13 + 2.0 ** -9).all()


@pytest.mark.parametrize("M,N,K,splits", [(50, 1024, 2048, 0), (50, 1024, 4096, 2), (10, 512, 1024, 1), (64, 1024, 256, 1),
                                          (33, 1024, 1024, 2), (1, 128, 128, 1)])
def test_gemm_fp8_gate_res_norm_epilogue_vs_pair(M, N, K, splits):
    """Projection + gated residual + adaRMS + FP8 in one launch (one cluster across the row) against the two
    separate kernels: the updated residual is identical (same operations); the FP8 codes use a row sum of squares
    accumulated in a different fixed order, so they are identical except where the pre-rounding value sits within a
    last-bit distance of a rounding boundary -- at most one code step apart, on a tiny fraction of the elements."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from flashrt_b200 import _lib
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M * 7 + N + K + splits)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    resid = rand_bf16(rng, (M, N), 1.5)
    style = rand_bf16(rng, (3 * N,), 0.3)            # [scale | shift | gate] of the next norm (gate unused here)
    gate = rand_bf16(rng, (N,), 0.7)                 # gate of this residual
    d_A, d_W, d_sa, d_sb, d_so = Dev(A), Dev(W), f32(sa), f32(sb), f32(0.011)
    d_style, d_gate = Dev(style), Dev(gate)
    g = fvk.GemmRunner()
    # pair
    d_o, d_r1, d_a1 = zeros((M, N), np.uint16), Dev(resid), zeros((M, N), np.uint8)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_o.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0)
    _lib.call("frt_b200_norm_fp8", d_r1.ptr, d_o.ptr, d_gate.ptr, 0, None, d_style.ptr, 0, d_a1.ptr, None, M, N, 1e-6,
              d_so.ptr, 0, 0)
    # fused
    d_r2, d_a2 = Dev(resid), zeros((M, N), np.uint8)
    g.fp8_nt_dev_gate_res_norm_fp8(d_A.ptr, d_W.ptr, M, N, K, d_sa.ptr, d_sb.ptr, d_r2.ptr, d_gate.ptr, d_style.ptr,
                                   d_a2.ptr, d_so.ptr, 0, splits=splits)
    assert fvk.tensor_core_status() == 0
    assert np.array_equal(d_r1.get(), d_r2.get())
    c1, c2 = d_a1.get(), d_a2.get()
    same = (c1 == c2).mean()
    assert same >= 0.995, same
    v1, v2 = O.e4m3_to_f32(c1), O.e4m3_to_f32(c2)
    assert (np.abs(v1 - v2) <= np.maximum(np.abs(v1), np.abs(v2)) * 0.13 + 2.0 ** -9).all()   # one code step at most
    # and the oracle's norm on the oracle-exact residual agrees to the same degree
    _, ref8, _ = O.norm(resid, x=d_o.get(), gate_in=gate[None, :], gate_in_stride=0, style=style[None, :],
                        style_stride=0, out="fp8", scale=0.011)
    assert (ref8 == c2).mean() >= 0.995
