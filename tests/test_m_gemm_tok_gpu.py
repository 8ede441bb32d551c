"""GPU parity of the token-major small-M FP8 GEMM (activation rows on the accumulator lanes, weights on the columns,
split-K over a cluster) and of the decoder projections that fold the norm kernel between them:
  * plain GEMM over tile widths x split factors x row counts against the fp64 oracle, and bit for bit on exact products;
  * gated-residual epilogue: residual bits exact against the restated arithmetic, row statistics to fp32 accuracy;
  * in-kernel adaRMS -> FP8 producer: every produced E4M3 code exact (read back through identity weights), and the
    fused launches byte-identical to the same GEMM fed with the restated codes;
  * deferred row scale: the un-normalised operand a gated-residual launch leaves is exact against the restated
    arithmetic; the projections that apply 1 / rms and W . shift in their finish equal the plain launches bit for bit
    when the row scale is a power of two and the column term zero, and the fp64 restatement otherwise; the two launches
    in sequence reproduce norm -> quantise -> projection to FP8 accuracy."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402
from test_b_gemm_gpu import _check, _fp8_operand, _ref  # noqa: E402


def _fma32(a, b, c):
    """fp32 fused multiply-add of arrays (products of <= 24-bit significands are exact in fp64; one rounding)."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


@pytest.mark.parametrize("tile_n", [64, 128, 256])
@pytest.mark.parametrize("splits", [1, 2, 4, 8])
@pytest.mark.parametrize("M,N,K", [(50, 1024, 1024), (1, 256, 2048), (128, 512, 1024), (200, 1024, 1024),
                                   (50, 2560, 1024), (16, 1000, 4096), (50, 1024, 8192)])
def test_token_major_gemm(M, N, K, splits, tile_n):
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M * 7919 + N * 31 + K + splits * 3 + tile_n)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    bias = rand_bf16(rng, (N,), 0.2)
    d_A, d_W, d_D, d_b = Dev(A), Dev(W), zeros((M, N), np.uint16), Dev(bias)
    d_sa, d_sb = f32(sa), f32(sb)
    fvk.GemmRunner().fp8_nt_dev(d_A.ptr, d_W.ptr, d_D.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=splits,
                                tile_n=tile_n, bias=d_b.ptr)
    got = d_D.get()
    assert fvk.tensor_core_status() == 0
    _check(got, _ref(A, W, sa, sb, bias))


@pytest.mark.parametrize("splits,tile_n", [(1, 256), (4, 128), (8, 64), (2, 256)])
def test_token_major_gemm_exact_products(splits, tile_n):
    """Small integers in E4M3 make every product and partial sum exact: equal to the fp64 oracle bit for bit, and to
    the swapped kernel."""
    import torch
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(5 + splits)
    M, N, K = 50, 512, 1024
    vals = np.array([-4, -3, -2, -1, 0, 1, 2, 3, 4], np.float32)
    A = torch.from_numpy(rng.choice(vals, (M, K))).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    W = torch.from_numpy(rng.choice(vals, (N, K))).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    ref = O.gemm_fp8(A, W, 0.5, 0.25, b_is_nk=True)
    d_sa, d_sb = f32(0.5), f32(0.25)
    d_A, d_W, d_D, d_S = Dev(A), Dev(W), zeros((M, N), np.uint16), zeros((M, N), np.uint16)
    g = fvk.GemmRunner()
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_D.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=splits, tile_n=tile_n)
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_S.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=splits, swapped=True)
    assert fvk.tensor_core_status() == 0
    assert np.array_equal(d_D.get(), ref)
    assert np.array_equal(d_S.get(), ref)


@pytest.mark.parametrize("M,N,K,splits,tile_n", [(50, 1024, 2048, 8, 64), (50, 1024, 4096, 8, 64), (50, 1024, 2048, 4, 128),
                                                 (128, 512, 1024, 2, 64), (7, 1024, 4096, 0, 0), (50, 1024, 1024, 1, 128)])
def test_gated_residual_epilogue(M, N, K, splits, tile_n):
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M + N + K + splits)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    res0 = rand_bf16(rng, (M, N), 1.0)
    gate = rand_bf16(rng, (N,), 0.5)
    d_A, d_W, d_sa, d_sb = Dev(A), Dev(W), f32(sa), f32(sb)
    d_o, d_res, d_gate = zeros((M, N), np.uint16), Dev(res0), Dev(gate)
    d_stats = Dev(np.full((16, 128), -1.0, np.float32))
    g = fvk.GemmRunner()
    n_stat = g.fp8_nt_dev_gate_residual(d_A.ptr, d_W.ptr, M, N, K, d_sa.ptr, d_sb.ptr, d_res.ptr, d_gate.ptr,
                                        d_stats.ptr, 0, splits=splits, tile_n=tile_n)
    # the projection on its own with the same K split: its bf16 result is what the epilogue rounds to
    sp = splits if splits else 8
    g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_o.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=sp, tile_n=tile_n or 64)
    assert fvk.tensor_core_status() == 0
    _check(d_o.get(), _ref(A, W, sa, sb))
    o = O.bf16_bits_to_f32(d_o.get())
    r_new = _fma32(o, np.broadcast_to(O.bf16_bits_to_f32(gate), (M, N)), O.bf16_bits_to_f32(res0))
    if splits:
        assert np.array_equal(d_res.get(), O.f32_to_bf16_bits(r_new))
    else:   # the library chose the split: compare to within one bf16 step of the projection
        assert np.abs(O.bf16_bits_to_f32(d_res.get()) - r_new).max() <= 0.05
        r_new = None
    stats = d_stats.get()
    assert n_stat in (N // 64, N // 128)
    bn = N // n_stat
    assert (stats[n_stat:] == -1.0).all() and (stats[:n_stat, M:] == -1.0).all()
    if r_new is not None:
        want = (r_new.astype(np.float64) ** 2).reshape(M, n_stat, bn).sum(-1).T     # [tile][token]
        assert np.allclose(stats[:n_stat, :M], want, rtol=2e-6, atol=1e-6)


def _expected_codes(x_bits, stats, style_bits, K, eps, sa):
    """Restatement of the in-kernel adaRMS -> FP8 producer (same operations, same order)."""
    M = x_bits.shape[0]
    tot = np.zeros(M, np.float32)
    for t in range(stats.shape[0]):
        tot = (tot + stats[t, :M]).astype(np.float32)
    var = (tot / np.float32(K)).astype(np.float32) + np.float32(eps)
    rms = (np.float32(1.0) / np.sqrt(var.astype(np.float32)).astype(np.float32)).astype(np.float32)
    x = O.bf16_bits_to_f32(x_bits)
    sc = O.bf16_bits_to_f32(style_bits[:K])[None, :]
    sh = O.bf16_bits_to_f32(style_bits[K:2 * K])[None, :]
    t = (x * rms[:, None]).astype(np.float32)
    n = _fma32(t, (np.float32(1.0) + sc).astype(np.float32), np.broadcast_to(sh, t.shape))
    inv = np.float32(1.0) / np.float32(sa)
    q = np.clip((n * inv).astype(np.float32), -448.0, 448.0)
    return O.f32_to_e4m3(q)


def _producer_inputs(rng, M, K, n_stat):
    from gpu_util import rand_bf16
    x = rand_bf16(rng, (M, K), 1.5)
    style = rand_bf16(rng, (3 * K,), 0.3)
    xf = O.bf16_bits_to_f32(x).astype(np.float64)
    ssq = (xf ** 2).sum(-1)
    w = rng.random((n_stat, M)) + 0.1
    stats = np.zeros((n_stat, 128), np.float32)
    stats[:, :M] = (w / w.sum(0) * ssq[None, :]).astype(np.float32)
    return x, style, stats


@pytest.mark.parametrize("M,splits", [(50, 4), (50, 8), (50, 2), (128, 4), (3, 4)])
def test_norm_producer_codes_are_exact(M, splits):
    """Identity weights and a RoPE table of (cos, sin) = (1, 0) return the producer's E4M3 codes themselves: each must
    equal the restated arithmetic."""
    import torch
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(M * 11 + splits)
    K, n_stat = 1024, 16
    x, style, stats = _producer_inputs(rng, M, K, n_stat)
    W = np.zeros((K, K), np.uint8)
    W[np.arange(K), np.arange(K)] = 0x38                     # 1.0 in E4M3
    sa = 0.125                                               # a power of two: alpha * code value is exact in bf16
    rope = O.f32_to_bf16_bits(np.tile(np.array([1.0, 0.0], np.float32), (M, 128)))
    q_dim, k_dim, v_dim, hd = 512, 256, 256, 256
    d_x, d_st, d_sty, d_W, d_rope = Dev(x), Dev(stats), Dev(style), Dev(W), Dev(rope)
    d_sa, d_sb = f32(sa), f32(1.0)
    d_Q, d_K, d_V = zeros((M, q_dim), np.uint16), zeros((M, k_dim), np.uint16), zeros((M, v_dim), np.uint16)
    fvk.GemmRunner().norm_fp8_nt_dev_rope_split(d_x.ptr, d_st.ptr, n_stat, d_sty.ptr, d_W.ptr, M, K, d_sa.ptr, d_sb.ptr,
                                                d_rope.ptr, d_Q.ptr, d_K.ptr, d_V.ptr, q_dim, k_dim, v_dim, hd, 0,
                                                splits=splits)
    assert fvk.tensor_core_status() == 0
    got = O.bf16_bits_to_f32(np.concatenate([d_Q.get(), d_K.get(), d_V.get()], axis=1))
    want = O.e4m3_to_f32(_expected_codes(x, stats, style, K, 1e-6, sa)) * np.float32(sa)
    bad = got != want
    assert bad.mean() <= 2e-5, f"{int(bad.sum())} of {bad.size} codes differ"       # fp64-emulated fma: rare halfway cases
    assert (np.abs(want) > 0).mean() > 0.9


@pytest.mark.parametrize("M,splits", [(50, 4), (50, 0), (100, 4)])
def test_norm_producer_in_front_of_qkv_and_gate_up(M, splits):
    """The fused launches equal the same GEMM (same tile width and split) fed with the restated FP8 codes."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M * 13 + splits)
    K, n_stat, H = 1024, 8, 4096
    x, style, stats = _producer_inputs(rng, M, K, n_stat)
    xs = O.bf16_bits_to_f32(x)
    sa = float(np.abs(xs).max()) * 4.0 / 448.0
    codes = _expected_codes(x, stats, style, K, 1e-6, sa)
    g = fvk.GemmRunner()
    d_x, d_st, d_sty, d_A = Dev(x), Dev(stats), Dev(style), Dev(codes)
    d_sa = f32(sa)
    # ---- QKV
    q_dim, k_dim, v_dim, hd, pos = 2048, 256, 256, 256, 5
    Wq, sb = _fp8_operand(rng, q_dim + k_dim + v_dim, K, 0.02)
    inv_freq = 1.0 / (10000 ** (np.arange(0, hd, 2, dtype=np.float64) / hd))
    ph = np.arange(pos, pos + M, dtype=np.float64)[:, None] * inv_freq[None, :]
    rope = O.f32_to_bf16_bits(np.stack([np.cos(ph), np.sin(ph)], -1).reshape(M, hd).astype(np.float32))
    d_W, d_sb, d_rope = Dev(Wq), f32(sb), Dev(rope)
    outs = []
    for fused in (False, True):
        d_Q, d_K, d_V = zeros((M, q_dim), np.uint16), zeros((M + pos, k_dim), np.uint16), zeros((M + pos, v_dim), np.uint16)
        tail = (d_rope.ptr, d_Q.ptr, d_K.ptr + pos * k_dim * 2, d_V.ptr + pos * v_dim * 2, q_dim, k_dim, v_dim, hd, 0)
        if fused:
            g.norm_fp8_nt_dev_rope_split(d_x.ptr, d_st.ptr, n_stat, d_sty.ptr, d_W.ptr, M, K, d_sa.ptr, d_sb.ptr, *tail,
                                         splits=splits)
        else:
            g.fp8_nt_dev_rope_split(d_A.ptr, d_W.ptr, M, K, d_sa.ptr, d_sb.ptr, *tail, splits=splits)
        outs.append((d_Q.get(), d_K.get(), d_V.get()))
    assert fvk.tensor_core_status() == 0
    mism = sum(int((a != b).sum()) for a, b in zip(*outs))
    assert mism <= 40, mism            # a code that differs from the restatement (fma emulation) touches one output row
    assert (outs[1][0] != 0).mean() > 0.9
    # ---- gate|up
    Wg, sbg = _fp8_operand(rng, 2 * H, K, 0.03)
    d_Wg, d_sbg, d_so = Dev(Wg), f32(sbg), f32(0.004)
    d_o1, d_o2 = zeros((M, H), np.uint8), zeros((M, H), np.uint8)
    g.fp8_nt_dev_geglu_fp8(d_A.ptr, d_Wg.ptr, d_o1.ptr, M, H, K, d_sa.ptr, d_sbg.ptr, d_so.ptr, 0, splits=splits)
    g.norm_fp8_nt_dev_geglu_fp8(d_x.ptr, d_st.ptr, n_stat, d_sty.ptr, d_Wg.ptr, d_o2.ptr, M, H, K, d_sa.ptr, d_sbg.ptr,
                                d_so.ptr, 0, splits=splits)
    assert fvk.tensor_core_status() == 0
    assert int((d_o1.get() != d_o2.get()).sum()) <= 40
    assert (d_o2.get() != 0).mean() > 0.5


@pytest.mark.parametrize("M,N,K,splits,tile_n", [(50, 1024, 2048, 4, 64), (50, 1024, 4096, 8, 64), (128, 512, 1024, 2, 128),
                                                 (3, 1024, 1024, 0, 0)])
def test_gated_residual_also_leaves_the_next_operand(M, N, K, splits, tile_n):
    """q8_out = e4m3(clamp(bf16(residual) * (1 + next_scale) / scale)): every code exact; residual and statistics are
    the ones the launch without the extra output writes."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M * 3 + N + K + splits)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    res0, gate, mod = rand_bf16(rng, (M, N), 1.0), rand_bf16(rng, (N,), 0.5), rand_bf16(rng, (N,), 0.3)
    q8s = 0.013
    d_A, d_W, d_sa, d_sb, d_gate, d_mod, d_q8s = Dev(A), Dev(W), f32(sa), f32(sb), Dev(gate), Dev(mod), f32(q8s)
    g = fvk.GemmRunner()
    outs = []
    for with_q8 in (False, True):
        d_res, d_stats, d_q8 = Dev(res0), Dev(np.full((16, 128), -1.0, np.float32)), zeros((M, N), np.uint8)
        kw = dict(next_scale=d_mod.ptr, q8_out=d_q8.ptr, d_scale_q8=d_q8s.ptr) if with_q8 else {}
        n = g.fp8_nt_dev_gate_residual(d_A.ptr, d_W.ptr, M, N, K, d_sa.ptr, d_sb.ptr, d_res.ptr, d_gate.ptr,
                                       d_stats.ptr, 0, splits=splits, tile_n=tile_n, **kw)
        outs.append((n, d_res.get(), d_stats.get(), d_q8.get()))
    assert fvk.tensor_core_status() == 0
    assert outs[0][0] == outs[1][0]
    assert np.array_equal(outs[0][1], outs[1][1]) and np.array_equal(outs[0][2], outs[1][2])
    r = O.bf16_bits_to_f32(outs[1][1])
    one_s = (np.float32(1.0) + O.bf16_bits_to_f32(mod)).astype(np.float32)[None, :]
    inv = np.float32(1.0) / np.float32(q8s)
    want = O.f32_to_e4m3(np.clip(((r * one_s).astype(np.float32) * inv).astype(np.float32), -448.0, 448.0))
    assert np.array_equal(outs[1][3], want)
    assert (want != 0).mean() > 0.9


def _identity_rope(M, hd):
    return O.f32_to_bf16_bits(np.tile(np.array([1.0, 0.0], np.float32), (M, hd // 2)))


@pytest.mark.parametrize("M,splits,tile_n", [(50, 4, 64), (50, 2, 128), (128, 1, 128), (7, 0, 0)])
def test_row_scaled_projections(M, splits, tile_n):
    """1 / rms a power of two and a zero column term: bit-equal to the plain launch with the scale folded into the
    operand scale.  Random statistics and column terms: the fp64 restatement bf16(alpha * acc * rms + c)."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(M * 17 + splits)
    K, H, hd = 1024, 2048, 256
    q_dim, k_dim, v_dim = 1024, 256, 256
    N = q_dim + k_dim + v_dim
    A, sa = _fp8_operand(rng, M, K, 1.0)
    Wq, sbq = _fp8_operand(rng, N, K, 0.02)
    Wg, sbg = _fp8_operand(rng, 2 * H, K, 0.03)
    g = fvk.GemmRunner()
    d_A, d_Wq, d_Wg, d_sbq, d_sbg, d_so = Dev(A), Dev(Wq), Dev(Wg), f32(sbq), f32(sbg), f32(0.004)
    d_rope = Dev(_identity_rope(M, hd))
    kw = dict(splits=splits, tile_n=tile_n)
    kw_gu = dict(splits=splits, tile_n=max(tile_n, 128) if tile_n else 0)       # a GeGLU tile is gate + up columns

    def qkv(rowscale, d_sa, stats=None, n_stat=0, col=None):
        d_Q, d_K, d_V = zeros((M, q_dim), np.uint16), zeros((M, k_dim), np.uint16), zeros((M, v_dim), np.uint16)
        tail = (d_rope.ptr, d_Q.ptr, d_K.ptr, d_V.ptr, q_dim, k_dim, v_dim, hd, 0)
        if rowscale:
            g.fp8_nt_dev_rope_split_rowscale(d_A.ptr, d_Wq.ptr, M, K, d_sa.ptr, d_sbq.ptr, stats.ptr, n_stat, col.ptr,
                                             *tail, eps=0.0, **kw)
        else:
            g.fp8_nt_dev_rope_split(d_A.ptr, d_Wq.ptr, M, K, d_sa.ptr, d_sbq.ptr, *tail, **kw)
        return np.concatenate([d_Q.get(), d_K.get(), d_V.get()], axis=1)

    def gu(rowscale, d_sa, stats=None, n_stat=0, col=None):
        d_o = zeros((M, H), np.uint8)
        if rowscale:
            g.fp8_nt_dev_geglu_fp8_rowscale(d_A.ptr, d_Wg.ptr, d_o.ptr, M, H, K, d_sa.ptr, d_sbg.ptr, stats.ptr, n_stat,
                                            col.ptr, d_so.ptr, 0, eps=0.0, **kw_gu)
        else:
            g.fp8_nt_dev_geglu_fp8(d_A.ptr, d_Wg.ptr, d_o.ptr, M, H, K, d_sa.ptr, d_sbg.ptr, d_so.ptr, 0, **kw_gu)
        return d_o.get()

    # ---- exact: sum of squares 16 K in two statistics rows -> 1 / rms = 0.25; operand scale x 4 cancels it
    stats = np.zeros((2, 128), np.float32)
    stats[:, :M] = 8.0 * K
    d_st, d_sa, d_sa4 = Dev(stats), f32(sa), f32(sa * 4.0)
    zq, zg = Dev(np.zeros(N, np.float32)), Dev(np.zeros(2 * H, np.float32))
    assert np.array_equal(qkv(True, d_sa4, d_st, 2, zq), qkv(False, d_sa))
    assert np.array_equal(gu(True, d_sa4, d_st, 2, zg), gu(False, d_sa))
    # ---- general
    n_stat = 16
    stats = np.zeros((n_stat, 128), np.float32)
    stats[:, :M] = rng.random((n_stat, M)).astype(np.float32) * K / 4.0
    rms = 1.0 / np.sqrt(stats[:, :M].astype(np.float64).sum(0) / K)
    cq, cg = rng.standard_normal(N).astype(np.float32), rng.standard_normal(2 * H).astype(np.float32) * 0.5
    d_st = Dev(stats)
    got = qkv(True, d_sa, d_st, n_stat, Dev(cq))
    want = (_ref(A, Wq, sa, sbq).astype(np.float64) * rms[:, None] + cq[None, :]).astype(np.float32)
    _check(got, want)
    got8 = O.e4m3_to_f32(gu(True, d_sa, d_st, n_stat, Dev(cg)))
    y = _ref(A, Wg, sa, sbg).astype(np.float64) * rms[:, None] + cg[None, :]
    merged = O.f32_to_bf16_bits(y.astype(np.float32))
    want8 = O.e4m3_to_f32(O.geglu_fp8(merged, 0.004))
    assert fvk.tensor_core_status() == 0
    # a bf16 step of the gate / up value moves the product by < 1 %; an E4M3 step is 6-12 %: codes agree or neighbour
    close = np.abs(got8 - want8) <= np.abs(want8) * 0.13 + 1e-3
    assert close.all()
    assert (got8 == want8).mean() > 0.97
    assert (want8 != 0).mean() > 0.5


def test_deferred_row_scale_reproduces_norm_then_projection():
    """o-projection + gated residual + un-normalised operand, then the row-scaled QKV projection, against the restated
    norm (fp64) -> projection of the un-quantised normalised rows: equal to FP8 accuracy (the only rounding that
    differs from the in-kernel norm producer is where the E4M3 quantisation sits)."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(77)
    M, D, K0, hd = 50, 1024, 2048, 256
    q_dim, k_dim, v_dim = 2048, 256, 256
    N = q_dim + k_dim + v_dim
    A, sa = _fp8_operand(rng, M, K0, 1.0)
    Wo, sbo = _fp8_operand(rng, D, K0, 0.02)
    Wq, sbq = _fp8_operand(rng, N, D, 0.02)
    res0, gate, style = rand_bf16(rng, (M, D), 1.0), rand_bf16(rng, (D,), 0.5), rand_bf16(rng, (3 * D,), 0.3)
    sc = O.bf16_bits_to_f32(style[:D]).astype(np.float64)
    sh = O.bf16_bits_to_f32(style[D:2 * D]).astype(np.float64)
    g = fvk.GemmRunner()
    d_res, d_stats, d_q8 = Dev(res0), zeros((16, 128), np.float32), zeros((M, D), np.uint8)
    # scale of the un-normalised operand from the values themselves, as calibration does
    o = _ref(A, Wo, sa, sbo)
    r_est = O.bf16_bits_to_f32(res0) + o * O.bf16_bits_to_f32(gate)[None, :]
    q8s = float(np.abs(r_est * (1 + sc)[None, :]).max() / 448.0)
    wq = O.e4m3_to_f32(Wq).astype(np.float64) * sbq
    col = (wq @ sh).astype(np.float32)
    d_A, d_Wo, d_Wq, d_gate, d_style, d_col = Dev(A), Dev(Wo), Dev(Wq), Dev(gate), Dev(style), Dev(col)
    d_sa, d_sbo, d_sbq, d_q8s, d_rope = f32(sa), f32(sbo), f32(sbq), f32(q8s), Dev(_identity_rope(M, hd))
    n_stat = g.fp8_nt_dev_gate_residual(d_A.ptr, d_Wo.ptr, M, D, K0, d_sa.ptr, d_sbo.ptr, d_res.ptr, d_gate.ptr,
                                        d_stats.ptr, 0, splits=4, tile_n=64, next_scale=d_style.ptr, q8_out=d_q8.ptr,
                                        d_scale_q8=d_q8s.ptr)
    d_Q, d_K, d_V = zeros((M, q_dim), np.uint16), zeros((M, k_dim), np.uint16), zeros((M, v_dim), np.uint16)
    g.fp8_nt_dev_rope_split_rowscale(d_q8.ptr, d_Wq.ptr, M, D, d_q8s.ptr, d_sbq.ptr, d_stats.ptr, n_stat, d_col.ptr,
                                     d_rope.ptr, d_Q.ptr, d_K.ptr, d_V.ptr, q_dim, k_dim, v_dim, hd, 0, splits=4,
                                     tile_n=64)
    assert fvk.tensor_core_status() == 0
    got = O.bf16_bits_to_f32(np.concatenate([d_Q.get(), d_K.get(), d_V.get()], axis=1))
    x = O.bf16_bits_to_f32(d_res.get()).astype(np.float64)
    rms = 1.0 / np.sqrt((x ** 2).mean(-1) + 1e-6)
    y = x * rms[:, None] * (1 + sc)[None, :] + sh[None, :]
    want = y @ wq.T
    # the same projection with the reference's quantisation point: in-kernel norm producer, scale from the normalised rows
    sa_n = float(np.abs(y).max() / 448.0)
    d_san = f32(sa_n)
    g.norm_fp8_nt_dev_rope_split(d_res.ptr, d_stats.ptr, n_stat, d_style.ptr, d_Wq.ptr, M, D, d_san.ptr, d_sbq.ptr,
                                 d_rope.ptr, d_Q.ptr, d_K.ptr, d_V.ptr, q_dim, k_dim, v_dim, hd, 0, splits=4, tile_n=64)
    assert fvk.tensor_core_status() == 0
    ref_path = O.bf16_bits_to_f32(np.concatenate([d_Q.get(), d_K.get(), d_V.get()], axis=1))
    from gpu_util import cosine
    assert cosine(got, want.astype(np.float32)) >= 0.9995
    out_rms = float(np.sqrt((want ** 2).mean()))
    err_deferred = float(np.sqrt(((got - want) ** 2).mean())) / out_rms
    err_reference_point = float(np.sqrt(((ref_path - want) ** 2).mean())) / out_rms
    assert err_deferred <= 3e-2                                    # E4M3 rounding of 1024 operand elements per sum
    assert err_deferred <= 1.15 * err_reference_point + 1e-3       # no worse than quantising behind the row scale
    assert np.abs(got - want).max() <= 6.0 * err_deferred * out_rms + 1e-2


@pytest.mark.parametrize("M,splits", [(50, 2), (128, 4)])
def test_hardware_tanh_gelu_matches_the_exact_finish(M, splits):
    """flags bit 7: GELU through tanh.approx (2^-11 relative).  The FP8 codes are those of the exact finish except for
    last-place flips at rounding boundaries; no code moves by more than one step."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(M + splits)
    K, H = 1024, 4096
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, 2 * H, K, 0.03)
    d_A, d_W, d_sa, d_sb, d_so = Dev(A), Dev(W), f32(sa), f32(sb), f32(0.004)
    d_exact, d_fast = zeros((M, H), np.uint8), zeros((M, H), np.uint8)
    g = fvk.GemmRunner()
    g.fp8_nt_dev_geglu_fp8(d_A.ptr, d_W.ptr, d_exact.ptr, M, H, K, d_sa.ptr, d_sb.ptr, d_so.ptr, 0, splits=splits)
    g.fp8_nt_dev_geglu_fp8(d_A.ptr, d_W.ptr, d_fast.ptr, M, H, K, d_sa.ptr, d_sb.ptr, d_so.ptr, 0, splits=splits,
                           fast_gelu=True)
    assert fvk.tensor_core_status() == 0
    e, f = d_exact.get(), d_fast.get()
    assert (e != f).mean() <= 5e-3
    ve, vf = O.e4m3_to_f32(e), O.e4m3_to_f32(f)
    assert (np.abs(ve - vf) <= np.abs(ve) * 0.13 + 2.0 ** -9).all()        # one E4M3 step at most
    assert (e != 0).mean() > 0.5


def test_refusals():
    from flashrt_b200 import flash_rt_kernels as fvk
    from flashrt_b200._lib import KernelError
    from gpu_util import zeros
    g = fvk.GemmRunner()
    z = zeros((256, 1024), np.uint16)
    with pytest.raises(KernelError):       # more rows than one accumulator tile
        g.fp8_nt_dev_gate_residual(z.ptr, z.ptr, 129, 1024, 1024, 0, 0, z.ptr, z.ptr, z.ptr, 0)
    with pytest.raises(KernelError):       # K not in whole 128-byte blocks
        g.fp8_nt_dev_gate_residual(z.ptr, z.ptr, 50, 1024, 1000, 0, 0, z.ptr, z.ptr, z.ptr, 0)
    with pytest.raises(KernelError):       # K-slice that cannot stay resident
        g.norm_fp8_nt_dev_geglu_fp8(z.ptr, z.ptr, 4, z.ptr, z.ptr, z.ptr, 50, 4096, 4096, z.ptr, z.ptr, z.ptr, 0,
                                    splits=2)


@pytest.mark.parametrize("M,N,K,splits", [(50, 2560, 1024, 0), (50, 1024, 2048, 4), (16, 8192, 1024, 0), (128, 1024, 4096, 8),
                                          (200, 3072, 3072, 0), (1, 256, 128, 1), (2048, 1024, 1024, 0),
                                          (1000, 384, 512, 0), (8192, 3072, 3072, 0), (300, 14336, 3072, 0)])
def test_fp8_nn_dev_kn_weights_equal_nt_on_the_transpose(M, N, K, splits):
    """GemmRunner.fp8_nn_dev -- weights stored (K, N), the reference's default layout -- gives the bytes of fp8_nt_dev on
    the transposed weights (same kernel, same accumulation order; only the operand descriptor differs), and both
    agree with the fp64 oracle."""
    from flashrt_b200 import flash_rt_kernels as fvk
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(M + 3 * N + 7 * K)
    A, sa = _fp8_operand(rng, M, K, 1.0)
    W, sb = _fp8_operand(rng, N, K, 0.02)
    bias = rand_bf16(rng, (N,), 0.2)
    d_A, d_W, d_Wt, d_b = Dev(A), Dev(W), Dev(np.ascontiguousarray(W.T)), Dev(bias)
    d_sa, d_sb = f32(sa), f32(sb)
    d_nt, d_nn = zeros((M, N), np.uint16), zeros((M, N), np.uint16)
    g = fvk.GemmRunner()
    tile = 128 if (M <= 256 and N % 256) else (256 if M <= 256 else 0)
    if M <= 256:
        g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_nt.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=splits, bias=d_b.ptr, tile_n=tile)
        g.fp8_nn_dev(d_A.ptr, d_Wt.ptr, d_nn.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, splits=splits, bias=d_b.ptr, tile_n=tile)
    else:
        g.fp8_nt_dev(d_A.ptr, d_W.ptr, d_nt.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, bias=d_b.ptr, cta_pair=False)
        g.fp8_nn_dev(d_A.ptr, d_Wt.ptr, d_nn.ptr, M, N, K, d_sa.ptr, d_sb.ptr, 0, bias=d_b.ptr)
    assert fvk.tensor_core_status() == 0
    _check(d_nn.get(), _ref(A, W, sa, sb, bias))
    assert np.array_equal(d_nt.get(), d_nn.get())
