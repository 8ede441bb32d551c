"""GPU parity of the NVFP4 path: quantisers, fused norm / GeGLU producers (byte-exact against the C oracle)
and the tcgen05 block-scaled GEMM (floating point: cosine >= 0.999, max-abs <= 2e-2 x RMS(ref), plus bit
equality where every product and partial sum is exact)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


def _edge_rows(rng, rows, D):
    """N(0,1) rows with planted edge cases: an all-zero block, exact ties at every e2m1 threshold, tiny and huge blocks."""
    x = rng.standard_normal((rows, D)).astype(np.float32)
    x[0, :16] = 0.0
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0],
                    np.float32)
    if D >= 48:
        x[1 % rows, 16:32] = ties             # amax 6 -> scale 1 -> products sit on the thresholds
        x[2 % rows, 32:48] = ties * 0.5
        x[3 % rows, 0:16] *= 1e-6
        x[4 % rows, 16:32] *= 300.0
    return O.f32_to_bf16_bits(x)


@pytest.mark.parametrize("rows,D", [(50, 1024), (257, 4096), (16, 3072), (130, 80), (1, 16)])
@pytest.mark.parametrize("family", [0, 1])
def test_quantize_nvfp4_bit_exact(rows, D, family):
    from flashrt_b200 import _lib
    from gpu_util import Dev, zeros
    rng = np.random.default_rng(rows * 7 + D + family)
    x = _edge_rows(rng, rows, D)
    ref_p, ref_sf = O.quantize_nvfp4(x, family)
    d_x, d_p, d_sf = Dev(x), zeros((rows, D // 2), np.uint8), zeros((O.nvfp4_sf_size(rows, D),), np.uint8)
    _lib.call("frt_b200_quantize_nvfp4", d_x.ptr, d_p.ptr, d_sf.ptr, rows, D, family, None, 0, 0)
    assert np.array_equal(d_sf.get(), ref_sf)
    assert np.array_equal(d_p.get(), ref_p)


def test_quantize_nvfp4_global_scale_and_shim_names():
    from flashrt_b200 import flash_rt_fp4 as fp4, flash_rt_kernels as fvk
    from flashrt_b200 import _lib
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(3)
    rows, D = 50, 2048
    x = _edge_rows(rng, rows, D)
    assert fp4.has_nvfp4()
    assert fp4.sfa_size_bytes(rows, D, False) == O.nvfp4_sf_size(rows, D)
    g = np.float32(0.0371)
    ref_p, ref_sf = O.quantize_nvfp4(x, 1, float(g))
    d_x, d_p, d_sf, d_g = Dev(x), zeros((rows, D // 2), np.uint8), zeros((O.nvfp4_sf_size(rows, D),), np.uint8), f32(g)
    assert fp4.quantize_fp4_dynamic_sfa_bf16_vec(d_x.ptr, d_p.ptr, d_sf.ptr, rows, D, False, 0,
                                                 d_global_scale=d_g.ptr) == 0
    assert np.array_equal(d_p.get(), ref_p) and np.array_equal(d_sf.get(), ref_sf)
    # family-0 name of flash_rt_kernels
    ref_p, ref_sf = O.quantize_nvfp4(x, 0)
    d_p2, d_sf2 = zeros((rows, D // 2), np.uint8), zeros((O.nvfp4_sf_size(rows, D),), np.uint8)
    fvk.quantize_bf16_to_nvfp4_swizzled(d_x.ptr, d_p2.ptr, d_sf2.ptr, rows, D, 0)
    assert np.array_equal(d_p2.get(), ref_p) and np.array_equal(d_sf2.get(), ref_sf)
    # argument checks
    assert _lib.call_status("frt_b200_quantize_nvfp4", d_x.ptr, d_p.ptr, d_sf.ptr, rows, 24, 1, None, 0, 0) == -2
    assert _lib.call_status("frt_b200_quantize_nvfp4", d_x.ptr, d_p.ptr, d_sf.ptr, rows, D, 2, None, 0, 0) == -1
    assert _lib.call_status("frt_b200_quantize_nvfp4", d_x.ptr, d_p.ptr, d_sf.ptr, 0, D, 1, None, 0, 0) == 0


@pytest.mark.parametrize("rows,H", [(50, 4096), (33, 272)])
@pytest.mark.parametrize("family", [0, 1])
def test_geglu_nvfp4_bit_exact(rows, H, family):
    from flashrt_b200 import _lib
    from gpu_util import Dev, rand_bf16, zeros
    rng = np.random.default_rng(rows + H + family)
    merged = rand_bf16(rng, (rows, 2 * H), 1.5)
    ref_p, ref_sf = O.geglu_nvfp4(merged, family)
    d_m, d_p, d_sf = Dev(merged), zeros((rows, H // 2), np.uint8), zeros((O.nvfp4_sf_size(rows, H),), np.uint8)
    _lib.call("frt_b200_geglu_nvfp4", d_m.ptr, d_p.ptr, d_sf.ptr, rows, H, family, 0, 0)
    assert np.array_equal(d_sf.get(), ref_sf)
    assert np.array_equal(d_p.get(), ref_p)


@pytest.mark.parametrize("variant", ["ada", "gate_res_ada", "res_rms", "rms"])
@pytest.mark.parametrize("rows,dim", [(50, 1024), (10, 1024), (130, 2048), (7, 272)])
@pytest.mark.parametrize("family", [0, 1])
def test_norm_nvfp4_bit_exact(variant, rows, dim, family):
    """Fused norm -> NVFP4 equals the oracle's (norm -> bf16) -> quantise, and the updated residual matches."""
    from flashrt_b200 import _lib
    from gpu_util import Dev, rand_bf16, zeros
    rng = np.random.default_rng(rows * 31 + dim + family)
    res = rand_bf16(rng, (rows, dim), 2.0)
    x = rand_bf16(rng, (rows, dim), 1.0) if variant in ("gate_res_ada", "res_rms") else None
    gate = rand_bf16(rng, (rows, dim), 0.5) if variant == "gate_res_ada" else None
    style = rand_bf16(rng, (rows, 3 * dim), 0.3) if variant in ("ada", "gate_res_ada") else None
    weight = rand_bf16(rng, (dim,), 1.0) if variant in ("res_rms", "rms") else None
    r_res, r_norm, r_gate = O.norm(res, x=x, gate_in=gate, weight=weight, style=style, out="bf16",
                                   want_gate_out=style is not None)
    ref_p, ref_sf = O.quantize_nvfp4(r_norm, family)
    d_res = Dev(res)
    d_x = Dev(x) if x is not None else None
    d_g = Dev(gate) if gate is not None else None
    d_st = Dev(style) if style is not None else None
    d_w = Dev(weight) if weight is not None else None
    d_p, d_sf = zeros((rows, dim // 2), np.uint8), zeros((O.nvfp4_sf_size(rows, dim),), np.uint8)
    d_go = zeros((rows, dim), np.uint16) if style is not None else None
    _lib.call("frt_b200_norm_nvfp4", d_res.ptr, d_x.ptr if d_x else None, d_g.ptr if d_g else None, dim,
              d_w.ptr if d_w else None, d_st.ptr if d_st else None, 3 * dim, d_p.ptr, d_sf.ptr,
              d_go.ptr if d_go else None, rows, dim, 1e-6, family, 0, 0)
    assert np.array_equal(d_res.get(), r_res)
    assert np.array_equal(d_sf.get(), ref_sf)
    assert np.array_equal(d_p.get(), ref_p)
    if d_go is not None:
        assert np.array_equal(d_go.get(), r_gate)


# ------------------------------------------------------------------ block-scaled GEMM
def _operand(rng, rows, K, scale, family=1):
    x = O.f32_to_bf16_bits((rng.standard_normal((rows, K)) * scale).astype(np.float32))
    return O.quantize_nvfp4(x, family)


def _run_gemm(Ap, Asf, Wp, Wsf, M, N, K, alpha=1.0, bias=None, splits=0):
    from flashrt_b200 import flash_rt_fp4 as fp4, flash_rt_kernels as fvk
    from gpu_util import Dev, zeros
    d = [Dev(Ap), Dev(Asf), Dev(Wp), Dev(Wsf)]
    d_D = zeros((M, N), np.uint16)
    if bias is None:
        rc = fp4.cutlass_fp4_gemm_variant(4, d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_D.ptr, M, N, K, alpha, 0.0, 0,
                                          splits=splits)
    else:
        d_b = Dev(bias)
        rc = fp4.cutlass_fp4_gemm_bias_bf16(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_b.ptr, d_D.ptr, M, N, K, 0,
                                            splits=splits)
    assert rc == 0
    out = d_D.get()
    assert fvk.tensor_core_status() == 0
    return out


def _check(D_bits, ref_f32):
    from gpu_util import cosine
    got = O.bf16_bits_to_f32(D_bits)
    rms = float(np.sqrt(np.mean(ref_f32.astype(np.float64) ** 2)))
    err = np.abs(got - ref_f32)
    assert cosine(got, ref_f32) >= 0.9999
    assert err.max() <= 2e-2 * rms
    assert (err <= np.abs(ref_f32) * 2.0 ** -8 + 2e-3 * rms).all()


def test_gemm_nvfp4_exact_products():
    """Integer-valued e2m1 elements and power-of-two scales: every product and partial sum is exact in fp32,
    so the kernel must equal the float64 oracle bit for bit -- this pins the scale-factor routing (which
    row / block each scale byte multiplies) and the nibble order."""
    rng = np.random.default_rng(11)
    M, N, K = 50, 256, 512
    ints = np.array([-4, -3, -2, -1, 0, 1, 2, 3, 4, 6, -6], np.float32)
    def make(rows):
        base = rng.choice(ints, (rows, K)).astype(np.float32)
        # per-(row, block) power-of-two factor so that every scale byte differs from its neighbours
        e = rng.integers(-3, 3, (rows, K // 16))
        e[:, 0] = 0
        x = base * np.repeat(np.exp2(e).astype(np.float32), 16, axis=1)
        # force amax of every block to 6 * 2^e so the scale is exactly 2^e in both families
        x[:, ::16] = 6.0 * np.exp2(e).astype(np.float32)
        return x
    a, w = make(M), make(N)
    Ap, Asf = O.quantize_nvfp4(a, 1)
    Wp, Wsf = O.quantize_nvfp4(w, 1)
    assert np.array_equal(O.dequantize_nvfp4(Ap, Asf), a)       # the planted values survive quantisation
    ref = O.gemm_nvfp4(Ap, Asf, Wp, Wsf, alpha=0.125)
    for splits in (1, 2):
        got = _run_gemm(Ap, Asf, Wp, Wsf, M, N, K, alpha=0.125, splits=splits)
        assert np.array_equal(got, ref)


SMALL = [(16, 1024, 1024), (50, 2560, 1024), (50, 1024, 2048), (50, 8192, 1024), (50, 1024, 4096), (64, 256, 512),
         (100, 384, 256), (256, 4096, 1024), (33, 130, 256), (200, 1000, 768)]


@pytest.mark.parametrize("M,N,K", SMALL)
@pytest.mark.parametrize("splits", [1, 0, 4])
def test_gemm_nvfp4_small_m(M, N, K, splits):
    rng = np.random.default_rng(M * 1000003 + N * 131 + K + splits)
    Ap, Asf = _operand(rng, M, K, 1.0)
    Wp, Wsf = _operand(rng, N, K, 0.02)
    got = _run_gemm(Ap, Asf, Wp, Wsf, M, N, K, splits=splits)
    _check(got, O.gemm_nvfp4(Ap, Asf, Wp, Wsf, want_f32=True))


@pytest.mark.parametrize("M,N,K", [(2048, 1024, 1024), (300, 512, 256), (2048, 4096, 1024), (1000, 200, 4096),
                                   (257, 72, 256), (4096, 3072, 3072)])
def test_gemm_nvfp4_large_m(M, N, K):
    rng = np.random.default_rng(M + N + K)
    Ap, Asf = _operand(rng, M, K, 1.0, family=0)
    Wp, Wsf = _operand(rng, N, K, 0.02)
    bias = O.f32_to_bf16_bits((rng.standard_normal(N) * 0.1).astype(np.float32))
    got = _run_gemm(Ap, Asf, Wp, Wsf, M, N, K, bias=bias)
    _check(got, O.gemm_nvfp4(Ap, Asf, Wp, Wsf, bias=bias, want_f32=True))


def test_gemm_nvfp4_rope_split_equals_pair():
    """The fused RoPE + split + KV-append epilogue is byte-identical to GEMM -> qkv_split_rope."""
    from flashrt_b200 import flash_rt_fp4 as fp4, flash_rt_kernels as fvk
    from gpu_util import Dev, rand_bf16, zeros
    rng = np.random.default_rng(21)
    S, K, q_dim, k_dim, v_dim, hd, pos = 50, 1024, 2048, 256, 256, 256, 768
    N = q_dim + k_dim + v_dim
    Ap, Asf = _operand(rng, S, K, 1.0)
    Wp, Wsf = _operand(rng, N, K, 0.02)
    rope = rand_bf16(rng, (S, hd), 0.7)
    d = [Dev(Ap), Dev(Asf), Dev(Wp), Dev(Wsf)]
    d_rope = Dev(rope)
    # pair
    d_qkv = zeros((S, N), np.uint16)
    assert fp4.cutlass_fp4_gemm_variant(0, d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_qkv.ptr, S, N, K) == 0
    q1, k1, v1 = zeros((S, q_dim), np.uint16), zeros((pos + S, k_dim), np.uint16), zeros((pos + S, v_dim), np.uint16)
    fvk.qkv_split_rope(d_qkv.ptr, d_rope.ptr, q1.ptr, k1.ptr + pos * k_dim * 2, v1.ptr + pos * v_dim * 2, S, q_dim,
                       k_dim, v_dim, hd, 0)
    # fused
    q2, k2, v2 = zeros((S, q_dim), np.uint16), zeros((pos + S, k_dim), np.uint16), zeros((pos + S, v_dim), np.uint16)
    d_pos = Dev(np.array([pos], np.int32))
    assert fp4.cutlass_fp4_gemm_rope_split(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_rope.ptr, q2.ptr, k2.ptr, v2.ptr,
                                           S, K, q_dim, k_dim, v_dim, hd, devpos=d_pos.ptr) == 0
    assert np.array_equal(q1.get(), q2.get())
    assert np.array_equal(k1.get(), k2.get())
    assert np.array_equal(v1.get(), v2.get())
    assert fvk.tensor_core_status() == 0


@pytest.mark.parametrize("M,N,K", [(2048, 1024, 1024), (1000, 200, 768), (4096, 3072, 1024)])
def test_gemm_nvfp4_persistent_equals_one_tile_per_cta(M, N, K):
    """M > 256 runs as a persistent kernel (two accumulators + the scale columns in tensor memory); the
    one-tile-per-CTA kernel accumulates in the same order: identical bytes."""
    from flashrt_b200 import flash_rt_fp4 as fp4, flash_rt_kernels as fvk
    from gpu_util import Dev, zeros
    rng = np.random.default_rng(M + N + K + 1)
    Ap, Asf = _operand(rng, M, K, 1.0)
    Wp, Wsf = _operand(rng, N, K, 0.02)
    d = [Dev(Ap), Dev(Asf), Dev(Wp), Dev(Wsf)]
    d_1, d_2 = zeros((M, N), np.uint16), zeros((M, N), np.uint16)
    assert fp4.cutlass_fp4_gemm_variant(0, d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_1.ptr, M, N, K) == 0
    assert fp4.cutlass_fp4_gemm_variant(0, d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_2.ptr, M, N, K,
                                        one_tile_per_cta=True) == 0
    assert fvk.tensor_core_status() == 0
    assert np.array_equal(d_1.get(), d_2.get())
    _check(d_1.get(), O.gemm_nvfp4(Ap, Asf, Wp, Wsf, want_f32=True))
