"""CPU suite: pins the oracle (C kernels + torch block restatement) against
  * outputs of the reference's own torch ground-truth functions (tests/golden/cfg0_block.npz),
  * torch's E4M3 / bf16 conversions (bit-exact),
  * plain fp32 / fp64 formulas of each fused kernel (to rounding tolerance).
"""
import os
import zlib

import numpy as np
import pytest
import torch

from oracle import block_ref as R
from oracle import oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden", "cfg0_block.npz")


def _crc(t):
    return zlib.crc32(t.contiguous().numpy().tobytes())


@pytest.fixture(scope="module")
def cfg0():
    S, P = 50, 768
    ck = R.synthetic_checkpoint(seed=0, layers=1)
    pk, pv = R.synthetic_prefix_kv(seed=1, layers=1, prefix_len=P)
    x = torch.randn(S, R.DEC_D, generator=torch.Generator().manual_seed(2))
    cond = R.conditioning(ck, 0.5)[None, :]
    return dict(S=S, P=P, ck=ck, pk=pk, pv=pv, x=x, cond=cond, gold=np.load(GOLD))


def test_seeded_inputs_regenerate(cfg0):
    c = cfg0
    got = [_crc(c["x"]), _crc(c["cond"]), _crc(c["ck"]["decoder_attn_qkv_w"][0]), _crc(c["pk"]), _crc(c["pv"])]
    assert got == [int(v) for v in c["gold"]["crc"]]


def test_block_restatement_matches_reference_ground_truth(cfg0):
    """oracle.block_ref.decoder_block (device layout, adjacent-pair RoPE) == the reference's catalog functions
    (HF layout, rotate-half RoPE) on configuration 0."""
    c = cfg0
    ck = c["ck"]
    sa = (c["cond"] @ ck["decoder_pre_attn_norm_mod_w"][0] + ck["decoder_pre_attn_norm_mod_b"][0])[0]
    sf = (c["cond"] @ ck["decoder_pre_ffn_norm_mod_w"][0] + ck["decoder_pre_ffn_norm_mod_b"][0])[0]
    tab = R.rope_table(np.arange(c["P"], c["P"] + c["S"]))
    out, parts = R.decoder_block(c["x"], ck, 0, sa, sf, c["pk"][0], c["pv"][0], tab, return_parts=True)
    g = c["gold"]
    for name, got in (("out", out), ("x1", parts["x1"]), ("h", parts["h"]), ("h2", parts["h2"]),
                      ("attn", parts["attn"])):
        ref = torch.from_numpy(g[name])
        assert torch.allclose(got, ref, rtol=2e-4, atol=2e-5), name
    assert np.array_equal(g["out"], g["out_via_decoder_ffn_ref"])
    # q / k agree up to the head-dim permutation that relates the two RoPE forms
    q_hf = torch.from_numpy(g["q_hf"])                       # (S, 8, 256) first halves | second halves
    q_il = parts["q"]                                        # pairs adjacent
    assert torch.allclose(q_il[..., 0::2], q_hf[..., :128], rtol=2e-4, atol=2e-5)
    assert torch.allclose(q_il[..., 1::2], q_hf[..., 128:], rtol=2e-4, atol=2e-5)


def test_rope_interleave_identity():
    """rotate-half on HF-layout projections == adjacent-pair rotation on row-interleaved projections
    (the identity the reference tests in tests/test_structures_adarms_stack_region.py:208-221)."""
    g = torch.Generator().manual_seed(3)
    S, H, hd, D = 7, 2, 256, 64
    w_hf = torch.randn(H * hd, D, generator=g)
    x = torch.randn(S, D, generator=g)
    tab = R.rope_table(np.arange(100, 100 + S), hd)
    q_hf = R.rope_rotate_half((x @ w_hf.t()).reshape(S, H, hd), tab)
    q_il = R.rope_adjacent_pairs((x @ R.interleave_qk_rows(w_hf, H).t()).reshape(S, H, hd), tab)
    assert torch.allclose(q_il[..., 0::2], q_hf[..., :hd // 2], atol=1e-5)
    assert torch.allclose(q_il[..., 1::2], q_hf[..., hd // 2:], atol=1e-5)


def test_deferred_row_scale_restatement(cfg0):
    """``Fp8Linears.deferred`` (operand quantised in front of the row scale, 1 / rms and W . shift applied behind the
    product) is the same sum as quantising the adaRMS output: equal to the un-quantised projection of the normalised
    rows to FP8 accuracy, and no further from it than the reference's quantisation point."""
    ck, x = cfg0["ck"], cfg0["x"].to(torch.bfloat16).float()
    style = torch.randn(3 * R.DEC_D, generator=torch.Generator().manual_seed(5)) * 0.3
    h, _ = R.ada_rms(x, style)
    scale = style[:R.DEC_D]
    act = torch.zeros(1, 1, 4)
    act[0, 0, 0] = h.abs().max() / 448.0
    raw = torch.zeros(1, 1, 2)
    raw[0, 0, 0] = (x * (1 + scale)).abs().max() / 448.0
    lin = R.Fp8Linears(ck, 1, act, raw_scale=raw)
    w = lin.w[("decoder_attn_qkv_w", 0)]
    want = h @ w
    (got,) = lin.deferred(x, style, 0, 0, 0, ("decoder_attn_qkv_w",))
    ref_point = lin(lin.act(h, 0, 0, "qkv"), "decoder_attn_qkv_w", 0)
    rms = float(want.pow(2).mean().sqrt())
    e_def = float((got - want).pow(2).mean().sqrt()) / rms
    e_ref = float((ref_point - want).pow(2).mean().sqrt()) / rms
    assert e_def <= 3e-2 and e_def <= 1.15 * e_ref + 1e-3
    # without the FP8 rounding the two forms are the same number
    rs = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    exact = ((x * (1 + scale)) @ w) * rs + style[R.DEC_D:2 * R.DEC_D] @ w
    assert torch.allclose(exact, want, rtol=1e-4, atol=1e-4 * rms)


def test_time_schedule_and_embedding():
    ts = R.time_schedule(10)
    assert ts[0] == 1.0 and abs(ts[-1] - 0.1) < 1e-6 and len(ts) == 10
    e = R.time_embedding(0.5)
    assert e.shape == (1024,)
    # first period is 4e-3: sin(2 pi 0.5 / 4e-3) = sin(250 pi) ~ 0; last period 4.0: sin(pi/4)
    assert abs(float(e[511]) - np.sin(2 * np.pi * 0.5 / 4.0)) < 1e-5
    assert abs(float(e[1023]) - np.cos(2 * np.pi * 0.5 / 4.0)) < 1e-5


# ------------------------------------------------------------------ formats
def test_e4m3_and_bf16_conversions_bit_exact_vs_torch():
    lut = O.e4m3_lut()
    t = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(lut, nan=999.0), np.nan_to_num(t, nan=999.0))
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(60000, generator=g) * torch.exp(torch.randn(60000, generator=g) * 4)).clamp(-448, 448)
    mids = torch.tensor([(lut[c] + lut[c + 1]) / 2 for c in range(0, 0x7E)])
    x = torch.cat([x, mids, -mids, torch.tensor([0.0, -0.0, 448.0, -448.0, 2.0 ** -10, 2.0 ** -9, 1e-30])])
    assert np.array_equal(O.f32_to_e4m3(x.numpy()), x.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    y = torch.randn(100000, generator=g) * torch.exp(torch.randn(100000, generator=g) * 10)
    assert np.array_equal(O.f32_to_bf16_bits(y.numpy()), y.to(torch.bfloat16).view(torch.uint16).numpy())


def test_det_exp_and_gelu_accuracy():
    L = O.lib()
    xs = np.linspace(-90, 90, 20001).astype(np.float32)
    e = np.array([L.orc_det_expf(float(v)) for v in xs], dtype=np.float64)
    tr = np.exp(np.clip(xs.astype(np.float64), -87, 88))
    assert (np.abs(e - tr) / tr).max() < 2.0 ** -22
    gs = np.linspace(-12, 12, 20001).astype(np.float32)
    gg = np.array([L.orc_det_gelu_tanh(float(v)) for v in gs], dtype=np.float64)
    tg = torch.nn.functional.gelu(torch.tensor(gs, dtype=torch.float64), approximate="tanh").numpy()
    assert np.abs(gg - tg).max() < 2e-6


# ------------------------------------------------------------------ fused kernels vs plain formulas
def _bf(rng, shape, scale=1.0):
    return O.f32_to_bf16_bits((rng.standard_normal(shape) * scale).astype(np.float32))


def test_norm_oracle_vs_plain_formula():
    rng = np.random.default_rng(0)
    rows, dim = 9, 1024
    res, x, gate = _bf(rng, (rows, dim)), _bf(rng, (rows, dim), 0.5), _bf(rng, (rows, dim), 0.5)
    style = _bf(rng, (rows, 3 * dim), 0.3)
    scale = 0.02
    r_out, o8, g_out = O.norm(res, x=x, gate_in=gate, gate_in_stride=dim, style=style, style_stride=3 * dim,
                              out="fp8", want_gate_out=True, scale=scale)
    rf, xf, gf, sf = (O.bf16_bits_to_f32(a).astype(np.float64) for a in (res, x, gate, style))
    r = rf + xf * gf
    assert np.array_equal(r_out, O.f32_to_bf16_bits(r.astype(np.float32)))
    rb = O.bf16_bits_to_f32(r_out).astype(np.float64)
    rms = 1.0 / np.sqrt((r ** 2).mean(-1, keepdims=True) + 1e-6)
    y = rb * rms * (1 + sf[:, :dim]) + sf[:, dim:2 * dim]
    want = np.clip(y / scale, -448, 448)
    got = O.e4m3_to_f32(o8).astype(np.float64)
    # an E4M3 code is at most half a step (2^-4 relative) from the value it encodes
    assert (np.abs(got - want) <= np.abs(want) * 2.0 ** -4 + 2.0 ** -10).all()
    assert (np.abs(got - want) > np.abs(want) * 2.0 ** -4 * 0.999 + 2.0 ** -10).sum() == 0
    assert np.array_equal(g_out, style[:, 2 * dim:])
    # shared (stride 0) style row == the same row repeated
    _, o_shared, _ = O.norm(res, style=style[:1], style_stride=0, out="bf16")
    _, o_rep, _ = O.norm(res, style=np.repeat(style[:1], rows, 0), style_stride=3 * dim, out="bf16")
    assert np.array_equal(o_shared, o_rep)


def test_geglu_quantize_adds_oracle_vs_plain_formula():
    rng = np.random.default_rng(1)
    merged = _bf(rng, (5, 2 * 64), 2.0)
    o16 = O.geglu_bf16(merged)
    m = torch.from_numpy(O.bf16_bits_to_f32(merged))
    ref = torch.nn.functional.gelu(m[:, :64].double(), approximate="tanh") * m[:, 64:].double()
    got = torch.from_numpy(O.bf16_bits_to_f32(o16)).double()
    assert (got - ref).abs().max() <= ref.abs().max() * 2.0 ** -8
    ref = torch.nn.functional.silu(m[:, :64].double()) * m[:, 64:].double()        # the SiLU-gated sibling
    got = torch.from_numpy(O.bf16_bits_to_f32(O.swiglu_bf16(merged))).double()
    assert (got - ref).abs().max() <= ref.abs().max() * 2.0 ** -8
    q = O.e4m3_to_f32(O.swiglu_fp8(merged, 0.05)) * 0.05
    assert np.abs(q - np.clip(ref.numpy(), -22.4, 22.4)).max() <= np.abs(ref.numpy()).max() * 2.0 ** -4
    x = _bf(rng, (1000,), 3.0)
    s = O.amax_scale(x)
    assert s == np.float32(np.abs(O.bf16_bits_to_f32(x)).max() / np.float32(448.0))
    q = O.quantize_fp8_static(x, s)
    assert np.array_equal(q, O.f32_to_e4m3(np.clip(O.bf16_bits_to_f32(x) * (np.float32(1.0) / np.float32(s)), -448, 448)))
    assert O.amax_scale(np.zeros(16, np.uint16)) == np.float32(1e-12)
    a, b = _bf(rng, (3, 16)), _bf(rng, (3, 16))
    assert np.array_equal(O.add(a, b, mode=0), O.f32_to_bf16_bits(O.bf16_bits_to_f32(a) + O.bf16_bits_to_f32(b)))


def test_rope_split_oracle_vs_torch():
    rng = np.random.default_rng(2)
    seq, pos, hd = 6, 3, 256
    qkv = _bf(rng, (seq, 2048 + 256 + 256))
    tab = R.rope_table(np.arange(pos, pos + seq)).to(torch.bfloat16)
    rope = tab.view(torch.uint16).numpy()
    Kc, Vc = np.zeros((pos + seq, 256), np.uint16), np.zeros((pos + seq, 256), np.uint16)
    Q = O.qkv_split_rope(qkv, rope, Kc, Vc, pos, 2048, 256, 256, hd)
    f = torch.from_numpy(O.bf16_bits_to_f32(qkv))
    q_ref = R.rope_adjacent_pairs(f[:, :2048].reshape(seq, 8, hd), tab.float()).reshape(seq, 2048)
    k_ref = R.rope_adjacent_pairs(f[:, 2048:2304].reshape(seq, 1, hd), tab.float()).reshape(seq, 256)
    assert np.abs(O.bf16_bits_to_f32(Q) - q_ref.numpy()).max() <= np.abs(q_ref.numpy()).max() * 2.0 ** -8
    assert np.abs(O.bf16_bits_to_f32(Kc[pos:]) - k_ref.numpy()).max() <= np.abs(k_ref.numpy()).max() * 2.0 ** -8
    assert np.array_equal(Vc[pos:], qkv[:, 2304:]) and (Kc[:pos] == 0).all() and (Vc[:pos] == 0).all()


def test_gemm_and_attention_oracles_vs_torch():
    rng = np.random.default_rng(4)
    A = rng.integers(0, 0x7E, (5, 64)).astype(np.uint8)
    W = rng.integers(0, 0x7E, (7, 64)).astype(np.uint8)
    D, Df = O.gemm_fp8(A, W, 0.5, 0.25, b_is_nk=True, want_f32=True)
    ref = (O.e4m3_to_f32(A).astype(np.float64) @ O.e4m3_to_f32(W).astype(np.float64).T) * 0.125
    assert np.allclose(Df, ref, rtol=1e-6)
    D2 = O.gemm_fp8(A, np.ascontiguousarray(W.T), 0.5, 0.25, b_is_nk=False)
    assert np.array_equal(D, D2)
    q, k, v = _bf(rng, (1, 5, 8, 64)), _bf(rng, (1, 11, 1, 64)), _bf(rng, (1, 11, 1, 64))
    out, lse = O.attention(q, k, v, 0.125)
    tq, tk, tv = (torch.from_numpy(O.bf16_bits_to_f32(a)) for a in (q, k, v))
    ref = R.attention(tq[0], tk[0], tv[0], 0.125)
    assert torch.allclose(torch.from_numpy(out[0]), ref, atol=1e-5)


def test_video_dit_oracle_vs_plain_formulas():
    rng = np.random.default_rng(7)
    rows, dim = 6, 3072
    x = _bf(rng, (rows, dim), 1.5)
    sc, sh = _bf(rng, (1, dim), 0.3), _bf(rng, (1, dim), 0.3)
    got = torch.from_numpy(O.bf16_bits_to_f32(O.layer_norm(x, scale=sc, shift=sh, out="bf16"))).double()
    xf = torch.from_numpy(O.bf16_bits_to_f32(x)).double()
    n = (xf - xf.mean(-1, keepdim=True)) * torch.rsqrt(xf.var(-1, keepdim=True, unbiased=False) + 1e-6)
    ref = n * (1 + torch.from_numpy(O.bf16_bits_to_f32(sc)).double()) + torch.from_numpy(O.bf16_bits_to_f32(sh)).double()
    assert (got - ref).abs().max() <= ref.abs().max() * 2.0 ** -8
    # tanh-form GELU
    L = O.lib()
    gs = np.linspace(-10, 10, 4001).astype(np.float32)
    gg = np.array([L.orc_det_gelu_tanh_form(float(v)) for v in gs], dtype=np.float64)
    tg = torch.nn.functional.gelu(torch.tensor(gs, dtype=torch.float64), approximate="tanh").numpy()
    assert np.abs(gg - tg).max() < 3e-6
    # q/k RMSNorm over the full width + complex-pair rotation
    B, Lt, N, Dh = 1, 3, 2, 64
    packed = _bf(rng, (B * Lt, 3 * N * Dh))
    wq, wk = _bf(rng, (N * Dh,)), _bf(rng, (N * Dh,))
    ang = rng.uniform(0, 6.28, (Lt, Dh // 2))
    q, k = O.qkv_split_norm_rope(packed, wq, wk, np.cos(ang), np.sin(ang), B, Lt, N, Dh, seq_len=2)
    pf = torch.from_numpy(O.bf16_bits_to_f32(packed)).double()
    qf = pf[:, :N * Dh]
    qn = qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + 1e-6) * torch.from_numpy(O.bf16_bits_to_f32(wq)).double()
    qc = torch.view_as_complex(qn.reshape(Lt, N, Dh // 2, 2).contiguous())
    rot = torch.polar(torch.ones(Lt, Dh // 2, dtype=torch.float64), torch.from_numpy(ang))
    ref = torch.view_as_real(qc * rot[:, None, :]).reshape(Lt, N * Dh)
    got = torch.from_numpy(O.bf16_bits_to_f32(q)).double()
    assert (got[:2] - ref[:2]).abs().max() <= 2.0 ** -7 * ref.abs().max()
    assert (got[2] - qn[2]).abs().max() <= 2.0 ** -7 * qn.abs().max()       # row beyond seq_len: not rotated


# ---------------------------------------------------------------- NVFP4 restatement
def test_nvfp4_sf_layout_matches_cutlass_table():
    """The closed-form scale-factor offset equals CUTLASS's Sm1xxBlockScaledConfig<16> layout (fixture generated
    by tests/golden/make_sf_layout_golden.py) for SFA and SFB, including ragged rows and K not a multiple of 64."""
    import os
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "sf_layout.npz"))
    cases = sorted(k[5:] for k in z.files if k.startswith("offs_"))
    assert len(cases) >= 6
    for c in cases:
        rows, K, _ = (int(v) for v in c.split("_"))
        assert O.nvfp4_sf_size(rows, K) == int(z["size_" + c][0])
        table = O.nvfp4_sf_offsets(rows, K)
        assert np.array_equal(table, z["offs_" + c])
        for r, b in [(0, 0), (rows - 1, K // 16 - 1), (rows // 2, 1)]:
            assert O.lib().orc_nvfp4_sf_offset(r, b, K) == table[r, b]


def test_nvfp4_scale_conversions():
    L = O.lib()
    vals = np.array([L.orc_ue4m3_to_f32(c) for c in range(0x7F)], np.float64)
    assert (np.diff(vals) > 0).all() and vals[0] == 0 and vals[0x38] == 1.0 and vals[0x7E] == 448.0
    # the unsigned E4M3 decode agrees with the signed E4M3 table on non-negative codes
    assert np.array_equal(vals.astype(np.float32), O.e4m3_lut()[:0x7F])
    rng = np.random.default_rng(0)
    samples = np.concatenate([np.exp(rng.uniform(np.log(1e-4), np.log(240.0), 4000)), vals[1:0x78],
                              vals[1:0x78] * (1 + 1e-6), [240.0]]).astype(np.float32)
    for v in samples:
        c = L.orc_ue4m3_ceil(float(v))
        if v > 240.0:
            assert c == 0xFE
            continue
        assert vals[c] >= v                      # never below the input ...
        assert c == 1 or vals[c - 1] < v         # ... and the smallest such code
    assert L.orc_ue4m3_ceil(0.0) == 0 and L.orc_ue4m3_ceil(-1.0) == 0 and L.orc_ue4m3_ceil(241.0) == 0xFE


def test_nvfp4_quantise_conventions():
    """Ties and zero blocks behave as the two reference conventions say (nvfp4_convert.cuh:31-45,78-105;
    quantize_fp4_sfa.cu:31-50,89-108)."""
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0],
                    np.float32)[None, :]
    pa, sa = O.quantize_nvfp4(ties, 0)
    pb, sb = O.quantize_nvfp4(ties, 1)
    assert sa[0] == 0x38 and sb[0] == 0x38                      # amax 6 -> scale 1.0 in both families
    codes = lambda p: np.stack([p[0] & 15, p[0] >> 4], 1).ravel()
    assert list(codes(pa)) == [1, 2, 3, 4, 5, 6, 7, 7, 9, 10, 11, 12, 13, 14, 15, 15]   # '<': tie -> larger magnitude
    assert list(codes(pb)) == [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15]    # '<=': tie -> smaller; -0.25 -> -0
    zero = np.zeros((1, 16), np.float32)
    pa, sa = O.quantize_nvfp4(zero, 0)
    pb, sb = O.quantize_nvfp4(zero, 1)
    assert sa[0] == 0 and (pa == 0).all()
    assert sb[0] == 0 and (pb == 0x77).all()                    # 0 * inf = NaN falls through to code 7; scale 0 keeps it inert
    assert (O.dequantize_nvfp4(pb, sb) == 0).all()
    # the widest e2m1 gap (4 -> 6) is two scale units, the scale at most amax / 6 * (1 + 1/8)
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((64, 256)) * 3).astype(np.float32)
    for fam in (0, 1):
        p, s = O.quantize_nvfp4(x, fam)
        d = O.dequantize_nvfp4(p, s)
        blk_amax = np.abs(x).reshape(64, 16, 16).max(-1)
        err = np.abs(d - x).reshape(64, 16, 16).max(-1)
        assert (err <= blk_amax / 6.0 * 1.13 + 1e-6).all()
    # global scale: x / g quantised, dequantised value * g
    p, s = O.quantize_nvfp4(x, 1, 0.5)
    assert np.allclose(O.dequantize_nvfp4(p, s, 0.5), x, atol=np.abs(x).max() / 6)


def test_nvfp4_gemm_oracle_shapes():
    rng = np.random.default_rng(2)
    a = O.f32_to_bf16_bits(rng.standard_normal((5, 64)).astype(np.float32))
    w = O.f32_to_bf16_bits(rng.standard_normal((7, 64)).astype(np.float32))
    Ap, Asf = O.quantize_nvfp4(a, 1)
    Wp, Wsf = O.quantize_nvfp4(w, 1)
    D = O.gemm_nvfp4(Ap, Asf, Wp, Wsf, want_f32=True)
    ref = O.bf16_bits_to_f32(a) @ O.bf16_bits_to_f32(w).T
    assert D.shape == (5, 7)
    from_cos = float((D.ravel() @ ref.ravel()) / (np.linalg.norm(D) * np.linalg.norm(ref)))
    assert from_cos > 0.98


def test_nvfp4_family1_matches_the_references_torch_reference():
    """Golden vectors produced by the reference's own ``fake_nvfp4`` (tests/test_fp4_integration_meta.py, executed
    unchanged by tests/golden/make_nvfp4_golden.py): quantise + dequantise of the family-1 restatement must equal
    them bit for bit, including an all-zero block, ties on every e2m1 threshold and a block whose scale rounds to 0."""
    import os
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "nvfp4_fake_quant.npz"))
    names = [k[3:] for k in z.files if k.startswith("in_")]
    assert len(names) >= 4
    for n in names:
        x = np.ascontiguousarray(z["in_" + n], np.float32)
        packed, sf = O.quantize_nvfp4(x, 1)
        assert np.array_equal(O.dequantize_nvfp4(packed, sf), z["out_" + n]), n
        # the same inputs as bf16 bit patterns (the device kernels' input type) give the same codes
        p2, s2 = O.quantize_nvfp4(O.f32_to_bf16_bits(x), 1)
        assert np.array_equal(p2, packed) and np.array_equal(s2, sf), n


def test_wan_ref_building_blocks_match_reference_catalog():
    """The helpers the video-DiT restatement is made of agree with the reference's own catalog ground truth
    (tests/golden/wan_parts.npz, generated by tests/golden/make_wan_golden.py): full-width q/k RMSNorm + complex-pair
    RoPE (qk_norm_rope_ref, projection scope, interleaved layout), affine LayerNorm (norm_fused_ref), modulated
    affine-free LayerNorm -> projections (modnorm_qkv_chain_ref), LN -> fc1 -> GELU(tanh) -> fc2 + x (vision_ffn_ref)."""
    import importlib.util
    import os
    import torch
    from oracle import wan_ref as W
    here = os.path.dirname(__file__)
    spec = importlib.util.spec_from_file_location("make_wan_golden", os.path.join(here, "golden", "make_wan_golden.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    i = gen.inputs()
    z = np.load(os.path.join(here, "golden", "wan_parts.npz"))
    B, L, D, H, HD = gen.B, gen.L, gen.D, gen.H, gen.HD
    close = lambda a, name: np.testing.assert_allclose(a.numpy(), z[name], rtol=2e-5, atol=2e-5, err_msg=name)  # noqa: E731
    q = W._rope(W._rms(i["q"].reshape(B, L, D), i["wq_norm"]).reshape(B, L, H, HD), i["cos"], i["sin"])
    k = W._rope(W._rms(i["k"].reshape(B, L, D), i["wk_norm"]).reshape(B, L, H, HD), i["cos"], i["sin"])
    close(q, "qk_norm_rope_q")
    close(k, "qk_norm_rope_k")
    close(W._ln(i["x"]) * i["ln_w"] + i["ln_b"], "norm_fused")
    scale, shift = torch.from_numpy(z["silu_cond_affine"]).chunk(2, dim=-1)
    h = W._ln(i["x"]) * (1 + scale[:, None]) + shift[:, None]
    close(h @ i["w_q"].t() + i["b_q"], "modnorm_q")
    close(h @ i["w_k"].t() + i["b_k"], "modnorm_k")
    close(h @ i["w_v"].t() + i["b_v"], "modnorm_v")
    ff = torch.nn.functional.gelu(W._ln(i["x"]) @ i["w_fc1"].t() + i["b_fc1"], approximate="tanh")
    close(i["x"] + (ff @ i["w_fc2"].t() + i["b_fc2"]), "vision_ffn")
