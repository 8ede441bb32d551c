"""GPU parity: tcgen05 FP8 GEMM vs the oracle (fp64-accumulated C loop for small cases, fp32 BLAS on the
decoded operands for large ones).  Floating-point bar: cosine >= 0.999 and max-abs <= 2e-2 x RMS(ref);
the tighter bound asserted here is one bf16 ulp of the value plus a small RMS-relative slack."""
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
