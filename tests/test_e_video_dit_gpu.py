"""GPU parity, bit-exact: video-DiT (Wan-shape) fused producers vs the C oracle; M = 2 x 20 280 rows checked
through row sampling and size-independent properties."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


@pytest.fixture(scope="module")
def fvk():
    from flashrt_b200 import flash_rt_kernels as m
    return m


def _bf(rng, shape, scale=1.0):
    return O.f32_to_bf16_bits((rng.standard_normal(shape) * scale).astype(np.float32))


@pytest.mark.parametrize("rows,dim", [(1, 64), (37, 3072), (300, 4096), (5, 8192)])
@pytest.mark.parametrize("per_token", [False, True])
def test_ada_layer_norm_fp8_and_bf16(fvk, rows, dim, per_token):
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(rows + dim + per_token)
    x = _bf(rng, (rows, dim), 1.5)
    x[:, 0] = O.f32_to_bf16_bits(np.full(rows, 3.0, np.float32))        # non-zero mean
    sc, sh = _bf(rng, (rows if per_token else 1, dim), 0.3), _bf(rng, (rows if per_token else 1, dim), 0.3)
    stride = dim if per_token else 0
    qs = 0.02
    d_x, d_sc, d_sh, d_s = Dev(x), Dev(sc), Dev(sh), f32(qs)
    d_o8, d_o16 = zeros((rows, dim), np.uint8), zeros((rows, dim), np.uint16)
    fvk.ada_layer_norm_fp8(d_x.ptr, d_sc.ptr, d_sh.ptr, d_o8.ptr, d_s.ptr, rows, dim, 1e-6, 0, mod_stride=stride)
    (fvk.ada_layer_norm_bf16_per_token if per_token else fvk.ada_layer_norm_bf16)(
        d_x.ptr, d_sc.ptr, d_sh.ptr, d_o16.ptr, rows, dim, 1e-6, 0)
    assert np.array_equal(d_o8.get(), O.layer_norm(x, scale=sc, shift=sh, mod_stride=stride, out="fp8", qscale=qs))
    ref16 = O.layer_norm(x, scale=sc, shift=sh, mod_stride=stride, out="bf16")
    assert np.array_equal(d_o16.get(), ref16)
    # the FP8 output is the quantisation of the bf16 output (the reference's "round through bf16" contract)
    assert np.array_equal(d_o8.get(), O.quantize_fp8_static(ref16, qs))


def test_affine_layer_norm(fvk):
    from gpu_util import Dev, zeros
    rng = np.random.default_rng(5)
    rows, dim = 33, 3072
    x, w, b = _bf(rng, (rows, dim)), _bf(rng, (dim,)), _bf(rng, (dim,), 0.2)
    d_x, d_w, d_b, d_o = Dev(x), Dev(w), Dev(b), zeros((rows, dim), np.uint16)
    fvk.layer_norm(d_x.ptr, d_w.ptr, d_b.ptr, d_o.ptr, rows, dim, 1e-6, 0)
    assert np.array_equal(d_o.get(), O.layer_norm(x, weight=w, bias=b, out="bf16"))


@pytest.mark.parametrize("B,L,N,D_h,seq_len", [(1, 5, 2, 64, 5), (2, 40, 24, 128, 40), (1, 9, 24, 128, 6)])
def test_qkv_split_norm_rope(fvk, B, L, N, D_h, seq_len):
    from gpu_util import Dev, zeros
    rng = np.random.default_rng(B + L + N)
    dim = N * D_h
    packed = _bf(rng, (B * L, 3 * dim))
    wq, wk = _bf(rng, (dim,), 1.0), _bf(rng, (dim,), 1.0)
    ang = rng.uniform(0, 6.28, (L, D_h // 2))
    fre, fim = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    d = [Dev(a) for a in (packed, wq, wk, fre, fim)]
    d_q, d_k = zeros((B * L, dim), np.uint16), zeros((B * L, dim), np.uint16)
    fvk.qkv_split_norm_rope_bf16(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d[4].ptr, d_q.ptr, d_k.ptr, B, L, N, D_h,
                                 seq_len, 1e-6, 0)
    q_ref, k_ref = O.qkv_split_norm_rope(packed, wq, wk, fre, fim, B, L, N, D_h, seq_len)
    assert np.array_equal(d_q.get(), q_ref)
    assert np.array_equal(d_k.get(), k_ref)
    assert np.array_equal(d[0].get(), packed)                 # V stays where it is


@pytest.mark.parametrize("M,N", [(3, 64), (100, 14336)])
def test_bias_gelu_quantize_and_residuals(fvk, M, N):
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(M + N)
    x, bias = _bf(rng, (M, N), 2.0), _bf(rng, (N,), 0.5)
    d_x, d_b, d_o, d_s = Dev(x), Dev(bias), zeros((M, N), np.uint8), f32(0.01)
    fvk.bias_gelu_quantize_fp8_static_bf16(d_x.ptr, d_b.ptr, d_o.ptr, d_s.ptr, M, N, 0)
    assert np.array_equal(d_o.get(), O.bias_gelu_quantize_fp8(x, bias, 0.01))
    fvk.bias_gelu_quantize_fp8_static_bf16(d_x.ptr, 0, d_o.ptr, d_s.ptr, M, N, 0)
    assert np.array_equal(d_o.get(), O.bias_gelu_quantize_fp8(x, None, 0.01))
    res, gate = _bf(rng, (M, N)), _bf(rng, (M, N), 0.5)
    d_r, d_g = Dev(res), Dev(gate)
    fvk.bias_gate_mul_residual_bf16(d_r.ptr, d_x.ptr, d_b.ptr, d_g.ptr, M, N, 0)
    assert np.array_equal(d_r.get(), O.bias_gate_mul_residual(res, x, bias, gate, N))
    d_r = Dev(res)
    fvk.add_bias_bf16(d_r.ptr, d_b.ptr, M, N, 0)
    assert np.array_equal(d_r.get(), O.bias_gate_mul_residual(res, None, bias, None, 0))


def test_adaln_modulation6(fvk):
    from gpu_util import Dev, zeros
    rng = np.random.default_rng(2)
    B, S, D = 2, 7, 3072
    params = rng.standard_normal((B, S, 6, D)).astype(np.float32)
    lm = rng.standard_normal((6, D)).astype(np.float32)
    d_p, d_l = Dev(params), Dev(lm)
    outs = [zeros((B * S, D), np.uint16) for _ in range(6)]
    fvk.adaln_modulation6_bf16(d_p.ptr, d_l.ptr, *[o.ptr for o in outs], B, S, D, 0)
    ref = O.adaln_modulation6(params.reshape(B * S, 6, D), lm)
    for j in range(6):
        assert np.array_equal(outs[j].get(), ref[j])


def test_full_size_rows_idempotent_and_sampled(fvk):
    """BASELINE size (2 x 20 280 rows of 3072): sampled rows equal the oracle; a second run gives the same bytes."""
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(9)
    rows, dim = 40560, 3072
    x = _bf(rng, (rows, dim))
    sc, sh = _bf(rng, (1, dim), 0.3), _bf(rng, (1, dim), 0.3)
    d_x, d_sc, d_sh, d_s, d_o = Dev(x), Dev(sc), Dev(sh), f32(0.02), zeros((rows, dim), np.uint8)
    fvk.ada_layer_norm_fp8(d_x.ptr, d_sc.ptr, d_sh.ptr, d_o.ptr, d_s.ptr, rows, dim, 1e-6, 0)
    a = d_o.get().copy()
    fvk.ada_layer_norm_fp8(d_x.ptr, d_sc.ptr, d_sh.ptr, d_o.ptr, d_s.ptr, rows, dim, 1e-6, 0)
    assert np.array_equal(a, d_o.get())
    idx = rng.choice(rows, 64, replace=False)
    assert np.array_equal(a[idx], O.layer_norm(x[idx], scale=sc, shift=sh, mod_stride=0, out="fp8", qscale=0.02))
