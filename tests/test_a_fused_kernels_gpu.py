"""GPU parity, bit-exact: fused norm / quantise / activation / RoPE kernels vs the C oracle.

Calls go through the reference-named shim (``flashrt_b200.flash_rt_kernels``), i.e. through the C-ABI.
The bar for these kernels is byte equality of every output (FP8 codes, bf16 bits).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


@pytest.fixture(scope="module")
def fvk():
    from flashrt_b200 import flash_rt_kernels as m
    return m


def _mk(rng, rows, dim, scale=1.0):
    from gpu_util import rand_bf16
    return rand_bf16(rng, (rows, dim), scale)


DIMS = [64, 1024, 2048, 3072, 4096, 8192]
ROWS = [1, 50, 257]


@pytest.mark.parametrize("dim", DIMS)
@pytest.mark.parametrize("rows", ROWS)
def test_residual_add_rms_norm_fp8(fvk, rows, dim):
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(rows * 10007 + dim)
    res, x, w = _mk(rng, rows, dim), _mk(rng, rows, dim, 0.5), _mk(rng, 1, dim)[0]
    scale = 0.0123
    r_ref, o_ref, _ = O.norm(res, x=x, weight=w, out="fp8", scale=scale)
    d_res, d_x, d_w, d_o, d_s = Dev(res), Dev(x), Dev(w), zeros((rows, dim), np.uint8), f32(scale)
    fvk.residual_add_rms_norm_fp8(d_res.ptr, d_x.ptr, d_w.ptr, d_o.ptr, rows, dim, 1e-6, d_s.ptr, 0)
    assert np.array_equal(d_res.get(), r_ref)
    assert np.array_equal(d_o.get(), o_ref)


@pytest.mark.parametrize("dim", [1024, 3072])
@pytest.mark.parametrize("rows", ROWS)
def test_residual_add_rms_norm_bf16_and_rms_norm(fvk, rows, dim):
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(rows * 31 + dim)
    res, x, w = _mk(rng, rows, dim), _mk(rng, rows, dim, 0.5), _mk(rng, 1, dim)[0]
    r_ref, o_ref, _ = O.norm(res, x=x, weight=w, out="bf16")
    d_res, d_x, d_w, d_o = Dev(res), Dev(x), Dev(w), zeros((rows, dim), np.uint16)
    fvk.residual_add_rms_norm(d_res.ptr, d_x.ptr, d_w.ptr, d_o.ptr, rows, dim)
    assert np.array_equal(d_res.get(), r_ref)
    assert np.array_equal(d_o.get(), o_ref)
    # plain rms_norm / rms_norm_fp8 (input untouched)
    _, o2_ref, _ = O.norm(res, weight=w, out="bf16")
    d_in, d_o2 = Dev(res), zeros((rows, dim), np.uint16)
    fvk.rms_norm(d_in.ptr, d_w.ptr, d_o2.ptr, rows, dim)
    assert np.array_equal(d_o2.get(), o2_ref)
    assert np.array_equal(d_in.get(), res)
    _, o3_ref, _ = O.norm(res, weight=w, out="fp8", scale=0.02)
    d_o3, d_s = zeros((rows, dim), np.uint8), f32(0.02)
    fvk.rms_norm_fp8(d_in.ptr, d_w.ptr, d_o3.ptr, rows, dim, 1e-6, d_s.ptr)
    assert np.array_equal(d_o3.get(), o3_ref)


@pytest.mark.parametrize("dim", [1024, 2048])
@pytest.mark.parametrize("rows", ROWS)
@pytest.mark.parametrize("shared_style", [False, True])
def test_ada_rms_norm_style_fp8_and_bf16(fvk, rows, dim, shared_style):
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(rows * 7 + dim + shared_style)
    x = _mk(rng, rows, dim)
    ones = O.f32_to_bf16_bits(np.ones(dim, np.float32))
    style = _mk(rng, 1 if shared_style else rows, 3 * dim, 0.3)
    ss = 0 if shared_style else 3 * dim
    scale = 0.017
    _, o_ref, g_ref = O.norm(x, weight=ones, style=style, style_stride=ss, out="fp8", want_gate_out=True,
                             scale=scale)
    d_x, d_w, d_st = Dev(x), Dev(ones), Dev(style)
    d_o, d_g, d_s = zeros((rows, dim), np.uint8), zeros((rows, dim), np.uint16), f32(scale)
    fvk.ada_rms_norm_style_fp8(d_x.ptr, d_w.ptr, d_st.ptr, d_o.ptr, d_g.ptr, rows, dim, 1e-6, d_s.ptr, 0,
                               style_stride=ss)
    assert np.array_equal(d_o.get(), o_ref)
    assert np.array_equal(d_g.get(), g_ref)
    _, ob_ref, _ = O.norm(x, weight=ones, style=style, style_stride=ss, out="bf16", want_gate_out=True)
    d_ob = zeros((rows, dim), np.uint16)
    fvk.ada_rms_norm_style(d_x.ptr, d_w.ptr, d_st.ptr, d_ob.ptr, d_g.ptr, rows, dim, style_stride=ss)
    assert np.array_equal(d_ob.get(), ob_ref)


@pytest.mark.parametrize("dim", [1024, 4096])
@pytest.mark.parametrize("rows", ROWS)
def test_gate_residual_ada_norm_fp8_in_place_gate(fvk, rows, dim):
    """The reference call site passes the same buffer as gate (in) and gate_out (pipeline_rtx.py:1619-1627)."""
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(rows + dim)
    res, x, gate = _mk(rng, rows, dim), _mk(rng, rows, dim, 0.7), _mk(rng, rows, dim, 0.5)
    ones = O.f32_to_bf16_bits(np.ones(dim, np.float32))
    style = _mk(rng, rows, 3 * dim, 0.3)
    scale = 0.02
    r_ref, o_ref, g_ref = O.norm(res, x=x, gate_in=gate, gate_in_stride=dim, weight=ones, style=style,
                                 style_stride=3 * dim, out="fp8", want_gate_out=True, scale=scale)
    d_res, d_x, d_gate, d_w, d_st = Dev(res), Dev(x), Dev(gate), Dev(ones), Dev(style)
    d_o, d_s = zeros((rows, dim), np.uint8), f32(scale)
    fvk.gate_residual_ada_norm_fp8(d_res.ptr, d_x.ptr, d_gate.ptr, d_w.ptr, d_st.ptr, d_o.ptr, d_gate.ptr, rows,
                                   dim, 1e-6, d_s.ptr, 0)
    assert np.array_equal(d_res.get(), r_ref)
    assert np.array_equal(d_o.get(), o_ref)
    assert np.array_equal(d_gate.get(), g_ref)


def test_norm_edge_cases(fvk):
    """Zero rows is a no-op; an all-zero row gives zeros (eps keeps rms finite); huge values saturate at +-448."""
    from gpu_util import Dev, f32, zeros
    from flashrt_b200._lib import KernelError
    dim = 1024
    d_w = Dev(O.f32_to_bf16_bits(np.ones(dim, np.float32)))
    d_s = f32(1e-3)
    fvk.rms_norm_fp8(d_w.ptr, d_w.ptr, d_w.ptr, 0, dim, 1e-6, d_s.ptr)      # rows == 0
    x = np.zeros((2, dim), np.float32)
    x[1, :] = 3.0e4
    xb = O.f32_to_bf16_bits(x)
    _, o_ref, _ = O.norm(xb, out="fp8", scale=1e-3)
    d_x, d_o = Dev(xb), zeros((2, dim), np.uint8)
    fvk.rms_norm_fp8(d_x.ptr, d_w.ptr, d_o.ptr, 2, dim, 1e-6, d_s.ptr)
    got = d_o.get()
    assert np.array_equal(got, o_ref)
    assert (got[0] == 0).all() and (got[1] == 0x7E).all()
    with pytest.raises(KernelError):
        fvk.rms_norm_fp8(d_x.ptr, d_w.ptr, d_o.ptr, 2, 1020, 1e-6, d_s.ptr)  # dim % 8 != 0
    with pytest.raises(KernelError):
        fvk.rms_norm_fp8(d_x.ptr + 2, d_w.ptr, d_o.ptr, 2, dim, 1e-6, d_s.ptr)  # misaligned


@pytest.mark.parametrize("rows,H", [(1, 8), (50, 4096), (333, 1024), (2048, 4096)])
def test_geglu_fp8_and_bf16(fvk, rows, H):
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(rows + H)
    merged = _mk(rng, rows, 2 * H, 2.0)
    merged.reshape(-1)[:6] = O.f32_to_bf16_bits(np.array([0.0, -0.0, 50.0, -50.0, 1e-30, -300.0], np.float32))
    scale = 0.03
    ref8 = O.geglu_fp8(merged, scale)
    ref16 = O.geglu_bf16(merged)
    d_m, d_o8, d_o16, d_s = Dev(merged), zeros((rows, H), np.uint8), zeros((rows, H), np.uint16), f32(scale)
    fvk.gate_geglu_merged_fp8(d_m.ptr, d_o8.ptr, rows, H, d_s.ptr, 0)
    fvk.gate_geglu_merged(d_m.ptr, d_o16.ptr, rows, H, 0)
    assert np.array_equal(d_o8.get(), ref8)
    assert np.array_equal(d_o16.get(), ref16)


@pytest.mark.parametrize("rows,H", [(1, 8), (50, 4096), (333, 1024)])
def test_swiglu_fp8_and_bf16(fvk, rows, H):
    """SiLU gate on the merged [gate | up] layout: byte-exact against the C oracle."""
    from gpu_util import Dev, f32, zeros
    rng = np.random.default_rng(rows * 3 + H)
    merged = _mk(rng, rows, 2 * H, 2.0)
    merged.reshape(-1)[:6] = O.f32_to_bf16_bits(np.array([0.0, -0.0, 50.0, -50.0, 1e-30, -300.0], np.float32))
    scale = 0.03
    d_m, d_o8, d_o16, d_s = Dev(merged), zeros((rows, H), np.uint8), zeros((rows, H), np.uint16), f32(scale)
    fvk.gate_swiglu_merged_fp8(d_m.ptr, d_o8.ptr, rows, H, d_s.ptr, 0)
    fvk.gate_swiglu_merged(d_m.ptr, d_o16.ptr, rows, H, 0)
    assert np.array_equal(d_o8.get(), O.swiglu_fp8(merged, scale))
    assert np.array_equal(d_o16.get(), O.swiglu_bf16(merged))
    assert not np.array_equal(d_o16.get(), O.geglu_bf16(merged))


@pytest.mark.parametrize("n", [8, 50 * 2048, 50 * 2048 + 3, 1 << 22])
def test_quantize_fp8_static_and_device(fvk, n):
    from gpu_util import Dev, f32, rand_bf16, zeros
    rng = np.random.default_rng(n)
    x = rand_bf16(rng, (n,), 3.0)
    scale = 0.011
    ref = O.quantize_fp8_static(x, scale)
    d_x, d_o, d_s = Dev(x), zeros((n,), np.uint8), f32(scale)
    fvk.quantize_fp8_static(d_x.ptr, d_o.ptr, d_s.ptr, n, 0)
    assert np.array_equal(d_o.get(), ref)
    # device-computed scale: max(amax/448, 1e-12), written back, then the same quantisation
    s_ref = O.amax_scale(x)
    d_s2 = f32(123.0)
    fvk.quantize_fp8_device(d_x.ptr, d_o.ptr, d_s2.ptr, n, 0)
    assert d_s2.get()[0] == np.float32(s_ref)
    assert np.array_equal(d_o.get(), O.quantize_fp8_static(x, s_ref))
    # running max of scales
    d_acc = f32(s_ref / 2)
    fvk.fp8_accumulate_scale_max(d_s2.ptr, d_acc.ptr, 0)
    assert d_acc.get()[0] == np.float32(s_ref)
    d_acc2 = f32(s_ref * 2)
    fvk.fp8_accumulate_scale_max(d_s2.ptr, d_acc2.ptr, 0)
    assert d_acc2.get()[0] == np.float32(s_ref * 2)


def test_quantize_all_zero_input_uses_scale_floor(fvk):
    from gpu_util import Dev, f32, zeros
    x = np.zeros(1024, np.uint16)
    d_x, d_o, d_s = Dev(x), zeros((1024,), np.uint8), f32(5.0)
    fvk.quantize_fp8_device(d_x.ptr, d_o.ptr, d_s.ptr, 1024, 0)
    assert d_s.get()[0] == np.float32(1e-12)
    assert (d_o.get() == 0).all()


@pytest.mark.parametrize("rows,dim", [(50, 1024), (50, 32), (7, 4096)])
def test_adds(fvk, rows, dim):
    from gpu_util import Dev
    rng = np.random.default_rng(rows * dim)
    res, x, gate = _mk(rng, rows, dim), _mk(rng, rows, dim), _mk(rng, rows, dim)
    bias = _mk(rng, 1, dim)[0]
    n = rows * dim
    d_x, d_gate, d_bias = Dev(x), Dev(gate), Dev(bias)     # keep every device buffer alive across the launch
    d = Dev(res)
    fvk.residual_add(d.ptr, d_x.ptr, n, 0)
    assert np.array_equal(d.get(), O.add(res, x, mode=0))
    d = Dev(res)
    fvk.bias_residual(d.ptr, d_x.ptr, d_bias.ptr, rows, dim, 0)
    assert np.array_equal(d.get(), O.add(res, x, aux=bias, mode=1))
    d = Dev(res)
    fvk.gate_mul_residual(d.ptr, d_x.ptr, d_gate.ptr, n, 0)
    assert np.array_equal(d.get(), O.add(res, x, aux=gate, aux_stride=dim, mode=2))


@pytest.mark.parametrize("seq,pos,use_devpos", [(50, 768, False), (50, 768, True), (10, 0, True), (1, 5, True)])
def test_qkv_split_rope_appends_to_cache(fvk, seq, pos, use_devpos):
    from gpu_util import Dev
    rng = np.random.default_rng(seq + pos)
    q_dim, k_dim, v_dim, hd = 2048, 256, 256, 256
    total = pos + seq + 3
    qkv = _mk(rng, seq, q_dim + k_dim + v_dim)
    inv_freq = 1.0 / (10000 ** (np.arange(0, hd, 2, dtype=np.float64) / hd))
    ph = (np.arange(pos, pos + seq, dtype=np.float64))[:, None] * inv_freq[None, :]
    rope = O.f32_to_bf16_bits(np.stack([np.cos(ph), np.sin(ph)], -1).reshape(seq, hd).astype(np.float32))
    Kc, Vc = _mk(rng, total, k_dim), _mk(rng, total, v_dim)
    Kr, Vr = Kc.copy(), Vc.copy()
    Q_ref = O.qkv_split_rope(qkv, rope, Kr, Vr, pos, q_dim, k_dim, v_dim, hd)
    d_qkv, d_rope, d_K, d_V = Dev(qkv), Dev(rope), Dev(Kc), Dev(Vc)
    d_Q = Dev(np.zeros((seq, q_dim), np.uint16))
    if use_devpos:
        d_pos = Dev(np.array([pos], np.int32))
        fvk.qkv_split_rope_devpos(d_qkv.ptr, d_rope.ptr, d_Q.ptr, d_K.ptr, d_V.ptr, d_pos.ptr, seq, q_dim, k_dim,
                                  v_dim, hd, 0)
    else:
        fvk.qkv_split_rope(d_qkv.ptr, d_rope.ptr, d_Q.ptr, d_K.ptr + pos * k_dim * 2, d_V.ptr + pos * v_dim * 2,
                           seq, q_dim, k_dim, v_dim, hd, 0)
    assert np.array_equal(d_Q.get(), Q_ref)
    assert np.array_equal(d_K.get(), Kr)       # rows outside [pos, pos+seq) untouched
    assert np.array_equal(d_V.get(), Vr)
