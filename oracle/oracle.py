"""TEST INFRASTRUCTURE ONLY — numpy front-end of the C oracle (``oracle_kernels.c``).

Only ``tests/``, the smoke check and the benchmark's CPU-baseline leg import
this module.  Arrays are numpy: bf16 tensors travel as ``uint16`` bit patterns,
FP8 E4M3 tensors as ``uint8`` codes.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` next to its source (gcc, a second or two)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "oracle_kernels.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "liboracle.so"])
    return so


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(so):
            build()
        L = C.CDLL(so)
        L.orc_f32_to_bf16.restype = C.c_uint16
        L.orc_f32_to_bf16.argtypes = [C.c_float]
        L.orc_bf16_to_f32.restype = C.c_float
        L.orc_bf16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_e4m3.restype = C.c_uint8
        L.orc_f32_to_e4m3.argtypes = [C.c_float]
        L.orc_e4m3_to_f32.restype = C.c_float
        L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_det_expf.restype = C.c_float
        L.orc_det_expf.argtypes = [C.c_float]
        L.orc_det_gelu_tanh.restype = C.c_float
        L.orc_det_gelu_tanh.argtypes = [C.c_float]
        L.orc_amax_scale.restype = C.c_float
        L.orc_det_gelu_tanh_form.restype = C.c_float
        L.orc_det_gelu_tanh_form.argtypes = [C.c_float]
        L.orc_ue4m3_to_f32.restype = C.c_float
        L.orc_ue4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_ue4m3_ceil.restype = C.c_uint8
        L.orc_ue4m3_ceil.argtypes = [C.c_float]
        L.orc_nvfp4_sf_offset.restype = C.c_longlong
        L.orc_nvfp4_sf_offset.argtypes = [C.c_longlong, C.c_int, C.c_int]
        L.orc_nvfp4_sf_size.restype = C.c_longlong
        L.orc_nvfp4_sf_size.argtypes = [C.c_longlong, C.c_int]
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _u16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16, a.dtype
    return a


# ---------------------------------------------------------------- format helpers
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    r[nan] = 0x7FFF
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


_E4M3_LUT = None


def e4m3_lut() -> np.ndarray:
    global _E4M3_LUT
    if _E4M3_LUT is None:
        L = lib()
        _E4M3_LUT = np.array([L.orc_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
    return _E4M3_LUT


def e4m3_to_f32(codes: np.ndarray) -> np.ndarray:
    return e4m3_lut()[np.ascontiguousarray(codes, dtype=np.uint8)]


def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    L = lib()
    flat = np.ascontiguousarray(x, dtype=np.float32).ravel()
    return np.array([L.orc_f32_to_e4m3(float(v)) for v in flat], dtype=np.uint8).reshape(np.shape(x))


# ---------------------------------------------------------------- kernels
def norm(residual, x=None, gate_in=None, gate_in_stride=None, weight=None, style=None, style_stride=None,
         out="fp8", want_gate_out=False, eps=1e-6, scale=1.0):
    """Fused (gated-)residual + RMS/adaRMS norm.  Returns (residual_out, out, gate_out)."""
    res = _u16(residual).copy()
    rows, dim = res.shape
    x = None if x is None else _u16(x)
    gate_in = None if gate_in is None else _u16(gate_in)
    weight = None if weight is None else _u16(weight)
    style = None if style is None else _u16(style)
    if gate_in is not None and gate_in_stride is None:
        gate_in_stride = dim if gate_in.ndim == 2 and gate_in.shape[0] > 1 else 0
    if style is not None and style_stride is None:
        style_stride = 3 * dim if style.ndim == 2 and style.shape[0] > 1 else 0
    o8 = np.zeros((rows, dim), np.uint8) if out == "fp8" else None
    o16 = np.zeros((rows, dim), np.uint16) if out != "fp8" else None
    g = np.zeros((rows, dim), np.uint16) if (want_gate_out and style is not None) else None
    lib().orc_norm(_p(res), _p(x), _p(gate_in), C.c_longlong(gate_in_stride or 0), _p(weight), _p(style),
                   C.c_longlong(style_stride or 0), _p(o8), _p(o16), _p(g), C.c_int(rows), C.c_int(dim),
                   C.c_float(eps), C.c_float(scale))
    return res, (o8 if out == "fp8" else o16), g


def geglu_fp8(merged, scale):
    merged = _u16(merged)
    rows, two_h = merged.shape
    out = np.zeros((rows, two_h // 2), np.uint8)
    lib().orc_geglu_fp8(_p(merged), _p(out), C.c_int(rows), C.c_int(two_h // 2), C.c_float(scale))
    return out


def swiglu_fp8(merged, scale):
    """silu(gate) * up -> E4M3 on the merged [gate | up] layout (csrc/kernels/activation.cu:291-306)."""
    merged = _u16(merged)
    rows, two_h = merged.shape
    out = np.zeros((rows, two_h // 2), np.uint8)
    lib().orc_swiglu_fp8(_p(merged), _p(out), C.c_int(rows), C.c_int(two_h // 2), C.c_float(scale))
    return out


def swiglu_bf16(merged):
    merged = _u16(merged)
    rows, two_h = merged.shape
    out = np.zeros((rows, two_h // 2), np.uint16)
    lib().orc_swiglu_bf16(_p(merged), _p(out), C.c_int(rows), C.c_int(two_h // 2))
    return out


def geglu_bf16(merged):
    merged = _u16(merged)
    rows, two_h = merged.shape
    out = np.zeros((rows, two_h // 2), np.uint16)
    lib().orc_geglu_bf16(_p(merged), _p(out), C.c_int(rows), C.c_int(two_h // 2))
    return out


def quantize_fp8_static(x, scale):
    x = _u16(x)
    out = np.zeros(x.shape, np.uint8)
    lib().orc_quantize_fp8_static(_p(x), _p(out), C.c_longlong(x.size), C.c_float(scale))
    return out


def amax_scale(x) -> float:
    x = _u16(x)
    return float(lib().orc_amax_scale(_p(x), C.c_longlong(x.size)))


def add(res, x, aux=None, aux_stride=0, mode=0):
    res = _u16(res).copy()
    x = _u16(x)
    r2 = res.reshape(-1, res.shape[-1]) if res.ndim > 1 else res.reshape(1, -1)
    rows, dim = r2.shape
    aux = None if aux is None else _u16(aux)
    lib().orc_add(_p(res), _p(x), _p(aux), C.c_longlong(aux_stride), C.c_int(rows), C.c_int(dim), C.c_int(mode))
    return res


def qkv_split_rope(qkv, rope, K_cache, V_cache, pos, q_dim, k_dim, v_dim, head_dim):
    """Returns Q; K_cache / V_cache (uint16 arrays) are updated in place at rows pos..pos+seq."""
    qkv = _u16(qkv)
    rope = _u16(rope)
    seq = qkv.shape[0]
    Q = np.zeros((seq, q_dim), np.uint16)
    assert K_cache.dtype == np.uint16 and V_cache.dtype == np.uint16
    assert K_cache.flags.c_contiguous and V_cache.flags.c_contiguous
    lib().orc_qkv_split_rope(_p(qkv), _p(rope), _p(Q), _p(K_cache), _p(V_cache), C.c_int(pos), C.c_int(seq),
                             C.c_int(q_dim), C.c_int(k_dim), C.c_int(v_dim), C.c_int(head_dim))
    return Q


def gemm_fp8(A, B, sa, sb, b_is_nk=True, want_f32=False):
    """bf16 (and optionally fp32) result of (sa*sb) * A(M,K) . B, fp64 accumulate."""
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    M, K = A.shape
    N = B.shape[0] if b_is_nk else B.shape[1]
    D = np.zeros((M, N), np.uint16)
    Df = np.zeros((M, N), np.float32) if want_f32 else None
    lib().orc_gemm_fp8(_p(A), _p(B), _p(D), _p(Df), C.c_int(M), C.c_int(N), C.c_int(K), C.c_float(sa),
                       C.c_float(sb), C.c_int(1 if b_is_nk else 0))
    return (D, Df) if want_f32 else D


# ---------------------------------------------------------------- attention (numpy, fp64)
def attention(q_bits, k_bits, v_bits, scale, kv_len=None):
    """Masked-softmax attention restated from the reference's torch ground truth
    (flash_rt/structures/catalog/attention_core/reference.py:8-36; call site
    flash_rt/hardware/rtx/attn_backend.py:633-660: non-causal, the query heads of a group share
    one KV head, keys = prefix followed by the fresh tokens).

    q (B, Sq, Hq, D), k / v (B, Skv, Hkv, D) as bf16 bit patterns; returns (out fp32 (B, Sq, Hq, D),
    lse fp64 (B, Hq, Sq)).  Only the first ``kv_len`` keys count when given.
    """
    q = bf16_bits_to_f32(q_bits).astype(np.float64)
    k = bf16_bits_to_f32(k_bits).astype(np.float64)
    v = bf16_bits_to_f32(v_bits).astype(np.float64)
    B, Sq, Hq, D = q.shape
    Hkv = k.shape[2]
    g = Hq // Hkv
    if kv_len is not None:
        k, v = k[:, :kv_len], v[:, :kv_len]
    out = np.zeros((B, Sq, Hq, D), np.float64)
    lse = np.zeros((B, Hq, Sq), np.float64)
    for b in range(B):
        for h in range(Hq):
            s = (q[b, :, h, :] @ k[b, :, h // g, :].T) * scale
            m = s.max(-1, keepdims=True)
            p = np.exp(s - m)
            l = p.sum(-1, keepdims=True)
            out[b, :, h, :] = (p / l) @ v[b, :, h // g, :]
            lse[b, h, :] = (m + np.log(l))[:, 0]
    return out.astype(np.float32), lse


# ---------------------------------------------------------------- video-DiT producers
def layer_norm(x, weight=None, bias=None, scale=None, shift=None, mod_stride=0, out="bf16", eps=1e-6, qscale=1.0):
    x = _u16(x)
    rows, dim = x.shape
    o8 = np.zeros((rows, dim), np.uint8) if out == "fp8" else None
    o16 = np.zeros((rows, dim), np.uint16) if out != "fp8" else None
    a = [None if t is None else _u16(t) for t in (weight, bias, scale, shift)]
    lib().orc_layer_norm(_p(x), _p(a[0]), _p(a[1]), _p(a[2]), _p(a[3]), C.c_longlong(mod_stride), _p(o8), _p(o16),
                         C.c_int(rows), C.c_int(dim), C.c_float(eps), C.c_float(qscale))
    return o8 if out == "fp8" else o16


def qkv_split_norm_rope(packed, wq, wk, fre, fim, B, L, N, D_h, seq_len, eps=1e-6):
    packed, wq, wk = _u16(packed), _u16(wq), _u16(wk)
    fre = np.ascontiguousarray(fre, np.float32)
    fim = np.ascontiguousarray(fim, np.float32)
    dim = N * D_h
    q = np.zeros((B * L, dim), np.uint16)
    k = np.zeros((B * L, dim), np.uint16)
    lib().orc_qkv_split_norm_rope(_p(packed), _p(wq), _p(wk), _p(fre), _p(fim), _p(q), _p(k), C.c_int(B), C.c_int(L),
                                  C.c_int(N), C.c_int(D_h), C.c_int(seq_len), C.c_float(eps))
    return q, k


def bias_gelu_quantize_fp8(x, bias, scale):
    x = _u16(x)
    M, N = x.shape
    out = np.zeros((M, N), np.uint8)
    lib().orc_bias_gelu_quantize_fp8(_p(x), _p(None if bias is None else _u16(bias)), _p(out), C.c_longlong(M),
                                     C.c_int(N), C.c_float(scale))
    return out


def bias_gate_mul_residual(res, x, bias, gate, gate_stride):
    res = _u16(res).copy()
    rows, dim = res.shape
    lib().orc_bias_gate_mul_residual(_p(res), _p(None if x is None else _u16(x)), _p(None if bias is None else _u16(bias)),
                                     _p(None if gate is None else _u16(gate)), C.c_longlong(gate_stride),
                                     C.c_longlong(rows), C.c_int(dim))
    return res


def adaln_modulation6(params, layer_mod):
    params = np.ascontiguousarray(params, np.float32)
    layer_mod = np.ascontiguousarray(layer_mod, np.float32)
    BS, six, D = params.reshape(-1, 6, params.shape[-1]).shape
    out = np.zeros((6, BS, D), np.uint16)
    lib().orc_adaln_modulation6(_p(params), _p(layer_mod), _p(out), C.c_longlong(BS), C.c_int(D))
    return out


# ---------------------------------------------------------------- NVFP4
E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def nvfp4_sf_size(rows: int, K: int) -> int:
    return int(lib().orc_nvfp4_sf_size(rows, K))


def nvfp4_sf_offsets(rows: int, K: int) -> np.ndarray:
    """(rows, K/16) table of scale-byte offsets."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    b = np.arange(K // 16, dtype=np.int64)[None, :]
    katoms = (K + 63) // 64
    return ((r // 128) * katoms + b // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4


def quantize_nvfp4(x, family: int, global_scale: float = 1.0):
    """x: bf16 bit patterns (uint16) or float32, shape (rows, D).  Returns (packed (rows, D/2), sf bytes)."""
    x = np.ascontiguousarray(x)
    rows, D = x.shape
    packed = np.zeros((rows, D // 2), np.uint8)
    sf = np.zeros(nvfp4_sf_size(rows, D), np.uint8)
    fn = lib().orc_nvfp4_quantize_bf16 if x.dtype == np.uint16 else lib().orc_nvfp4_quantize_f32
    assert x.dtype in (np.uint16, np.float32)
    fn(_p(x), _p(packed), _p(sf), C.c_longlong(rows), C.c_int(D), C.c_int(family), C.c_float(global_scale))
    return packed, sf


def dequantize_nvfp4(packed, sf, global_scale: float = 1.0) -> np.ndarray:
    packed = np.ascontiguousarray(packed, np.uint8)
    sf = np.ascontiguousarray(sf, np.uint8)
    rows, half = packed.shape
    out = np.zeros((rows, 2 * half), np.float32)
    lib().orc_nvfp4_dequantize(_p(packed), _p(sf), _p(out), C.c_longlong(rows), C.c_int(2 * half),
                               C.c_float(global_scale))
    return out


def geglu_nvfp4(merged, family: int = 1):
    merged = _u16(merged)
    rows, two_h = merged.shape
    H = two_h // 2
    packed = np.zeros((rows, H // 2), np.uint8)
    sf = np.zeros(nvfp4_sf_size(rows, H), np.uint8)
    lib().orc_geglu_nvfp4(_p(merged), _p(packed), _p(sf), C.c_int(rows), C.c_int(H), C.c_int(family))
    return packed, sf


def gemm_nvfp4(a_packed, a_sf, w_packed, w_sf, alpha: float = 1.0, bias=None, want_f32: bool = False):
    """D = alpha * dequant(A) . dequant(W)^T (+ bias), float64 accumulation, bf16 bits out (or float32)."""
    A = dequantize_nvfp4(a_packed, a_sf).astype(np.float64)
    W = dequantize_nvfp4(w_packed, w_sf).astype(np.float64)
    D = (A @ W.T) * float(alpha)
    if bias is not None:
        D = D + bf16_bits_to_f32(_u16(bias)).astype(np.float64)[None, :]
    D = D.astype(np.float32)
    return D if want_f32 else f32_to_bf16_bits(D)


def cfg_combine(residual, v_cond, v_uncond, beta: float):
    """residual + (v_uncond + beta * (v_cond - v_uncond)); bf16 bit patterns (uint16) or float32 arrays."""
    r = np.ascontiguousarray(residual).copy()
    vc, vu = np.ascontiguousarray(v_cond), np.ascontiguousarray(v_uncond)
    assert r.dtype == vc.dtype == vu.dtype and r.dtype in (np.uint16, np.float32)
    fn = lib().orc_cfg_combine_bf16 if r.dtype == np.uint16 else lib().orc_cfg_combine_f32
    fn(_p(r), _p(vc), _p(vu), C.c_float(beta), C.c_longlong(r.size))
    return r
