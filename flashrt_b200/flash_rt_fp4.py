"""Stand-in for the reference's ``flash_rt.flash_rt_fp4`` pybind module (``csrc/fp4_bindings.cpp``) for the
denoise path, backed by the sm_100a C-ABI library.

Same names and argument order; every pointer is a Python ``int`` holding a device address.  The 16-bit
activation type of this library is **bf16** (the reference's Pi0.5 NVFP4 decoder keeps an fp16 residual
stream, its GR00T path a bf16 one): the ``*_bf16`` names are the native ones.  The reference's ``*_fp16`` names
exist too, but pointers carry no type and an fp16 buffer read as bf16 gives silently wrong numbers, so every
``*_fp16`` name REFUSES (:class:`NotBuilt`) unless the caller states ``io_dtype="bf16"`` -- i.e. that the buffers it
passes hold bf16 -- and ``STREAM_DTYPE`` is exported for frontends to check before they allocate.

Functions that return ``int`` in the reference return the C-ABI status (0 = success); ``void`` ones raise
:class:`flashrt_b200._lib.KernelError`.  One GEMM kernel serves every ``variant`` index.
"""
from __future__ import annotations

import ctypes as C

from . import _lib
from ._lib import KernelError, call, call_status  # noqa: F401
from .flash_rt_kernels import NotBuilt, _f

STREAM_DTYPE = "bfloat16"
FAMILY = 1      # flash_rt_fp4 convention: RN-even E4M3 block scale, '<=' thresholds


def _fp16_name(fn, name: str):
    """The reference binding ``name`` (fp16 buffers there) served by the bf16 kernel ``fn``: callable only with
    ``io_dtype="bf16"``, the caller's statement that its 16-bit buffers hold bf16."""
    def wrapper(*args, io_dtype=None, **kw):
        if io_dtype != "bf16":
            raise NotBuilt(f"flash_rt_fp4.{name}: this library's 16-bit activations are bf16; an fp16 buffer would be "
                           f"mis-read.  Allocate bf16 buffers and call {fn.__name__}, or pass io_dtype=\"bf16\" to "
                           f"state that the buffers hold bf16 (STREAM_DTYPE = {STREAM_DTYPE!r}).")
        return fn(*args, **kw)
    import inspect
    sig = inspect.signature(fn)
    params = [q for q in sig.parameters.values() if q.kind != q.VAR_KEYWORD]
    params.append(inspect.Parameter("io_dtype", inspect.Parameter.KEYWORD_ONLY, default=None))
    params += [q for q in sig.parameters.values() if q.kind == q.VAR_KEYWORD]
    wrapper.__signature__ = sig.replace(parameters=params)     # same positional names and order as the reference binding
    wrapper.__name__ = name
    wrapper.__doc__ = f"``{name}`` of csrc/fp4_bindings.cpp on bf16 buffers (requires io_dtype=\"bf16\"); see {fn.__name__}."
    return wrapper


def has_nvfp4() -> bool:                                   # csrc/fp4_bindings.cpp:466
    return call_status("frt_b200_sm_version") >= 100


def sfa_size_bytes(rows, D, is_sfb=False) -> int:          # csrc/fp4_bindings.cpp:349-352
    out = C.c_longlong(0)
    call("frt_b200_nvfp4_sf_bytes", rows, D, C.byref(out))
    return int(out.value)


def cutlass_fp4_gemm_num_variants() -> int:                # csrc/fp4_bindings.cpp:463
    return 11


def cutlass_fp4_gemm_variant_name(idx) -> str:             # csrc/fp4_bindings.cpp:461
    return "b200_tcgen05_mxf4nvf4_128xNx256 (one kernel for every index)"


# ------------------------------------------------------------------ quantisers
def quantize_fp4_dynamic_sfa_bf16_vec(src, packed, sfa, N, D, is_sfb=False, stream=0, *, pdl=False,
                                      d_global_scale=0) -> int:   # csrc/fp4_bindings.cpp:1124-1137
    return call_status("frt_b200_quantize_nvfp4", src, packed, sfa, N, D, FAMILY, d_global_scale or None,
                       _f(pdl), stream)


quantize_fp4_dynamic_sfa_fp16 = _fp16_name(quantize_fp4_dynamic_sfa_bf16_vec, "quantize_fp4_dynamic_sfa_fp16")       # csrc/fp4_bindings.cpp:299-315
quantize_fp4_dynamic_sfa_fp16_vec = _fp16_name(quantize_fp4_dynamic_sfa_bf16_vec, "quantize_fp4_dynamic_sfa_fp16_vec")   # csrc/fp4_bindings.cpp:317-333


def gate_geglu_fp4_sfa_vec_bf16(merged, packed, sfa, seq_len, half_dim, stream=0, *, pdl=False) -> int:
    return call_status("frt_b200_geglu_nvfp4", merged, packed, sfa, seq_len, half_dim, FAMILY, _f(pdl), stream)


gate_geglu_fp4_sfa_vec_fp16 = _fp16_name(gate_geglu_fp4_sfa_vec_bf16, "gate_geglu_fp4_sfa_vec_fp16")               # csrc/fp4_bindings.cpp:739-753


def gate_geglu_fp4_sfa_bf16(merged, packed, sfa, seq_len, half_dim, stream=0, *, pdl=False):   # :711-723
    call("frt_b200_geglu_nvfp4", merged, packed, sfa, seq_len, half_dim, FAMILY, _f(pdl), stream)


gate_geglu_fp4_sfa_fp16 = _fp16_name(gate_geglu_fp4_sfa_bf16, "gate_geglu_fp4_sfa_fp16")


gate_geglu_fp4_sfa_v2_fp16 = _fp16_name(gate_geglu_fp4_sfa_bf16, "gate_geglu_fp4_sfa_v2_fp16")                    # csrc/fp4_bindings.cpp:725-737


# ------------------------------------------------------------------ fused norms -> NVFP4
def pi05_adarms_fp4_sfa_bf16(x, style, packed, sfa, gate, seq_len, dim, stream=0, *, pdl=False, style_stride=None,
                             eps=1e-6):
    """adaRMS(style) -> NVFP4 + gate copy (csrc/fp4_bindings.cpp:547-570); any seq_len, dim % 16 == 0."""
    ss = 3 * dim if style_stride is None else style_stride
    call("frt_b200_norm_nvfp4", x, None, None, 0, None, style, ss, packed, sfa, gate or None, seq_len, dim, eps,
         FAMILY, _f(pdl), stream)


def pi05_gate_res_adarms_fp4_sfa_bf16(x, prev_gate, residual, style, packed, sfa, gate, seq_len, dim, stream=0, *,
                                      pdl=False, style_stride=None, gate_stride=None, eps=1e-6):
    """residual += x * prev_gate; adaRMS(style) -> NVFP4 + next gate (csrc/fp4_bindings.cpp:572-600)."""
    ss = 3 * dim if style_stride is None else style_stride
    gs = dim if gate_stride is None else gate_stride
    call("frt_b200_norm_nvfp4", residual, x, prev_gate, gs, None, style, ss, packed, sfa, gate or None, seq_len,
         dim, eps, FAMILY, _f(pdl), stream)


pi05_adarms_fp4_sfa_fp16 = _fp16_name(pi05_adarms_fp4_sfa_bf16, "pi05_adarms_fp4_sfa_fp16")                              # :547-570
pi05_adarms_fp4_sfa_native_fp16 = _fp16_name(pi05_adarms_fp4_sfa_bf16, "pi05_adarms_fp4_sfa_native_fp16")                       # :602-625
pi05_gate_res_adarms_fp4_sfa_fp16 = _fp16_name(pi05_gate_res_adarms_fp4_sfa_bf16, "pi05_gate_res_adarms_fp4_sfa_fp16")            # :572-600
pi05_gate_res_adarms_fp4_sfa_native_fp16 = _fp16_name(pi05_gate_res_adarms_fp4_sfa_bf16, "pi05_gate_res_adarms_fp4_sfa_native_fp16")     # :627-657


def rms_norm_fp4_sfa_bf16(x, packed, sfa, seq_len, dim, stream=0, *, weight=0, pdl=False, eps=1e-6):   # :501-513
    # the reference's kernel has no weight operand (the norm weight is folded into the next projection); `weight`
    # is an extension of this library
    call("frt_b200_norm_nvfp4", x, None, None, 0, weight or None, None, 0, packed, sfa, None, seq_len, dim, eps,
         FAMILY, _f(pdl), stream)


rms_norm_fp4_sfa_fp16 = _fp16_name(rms_norm_fp4_sfa_bf16, "rms_norm_fp4_sfa_fp16")


def residual_add_rms_norm_fp4_sfa_bf16(residual, x, packed, sfa, seq_len, dim, stream=0, *, weight=0, pdl=False,
                                       eps=1e-6):                                                    # :531-545
    call("frt_b200_norm_nvfp4", residual, x, None, 0, weight or None, None, 0, packed, sfa, None, seq_len, dim,
         eps, FAMILY, _f(pdl), stream)


residual_add_rms_norm_fp4_sfa_fp16 = _fp16_name(residual_add_rms_norm_fp4_sfa_bf16, "residual_add_rms_norm_fp4_sfa_fp16")


residual_add_rms_norm_fp4_sfa_v2_fp16 = _fp16_name(residual_add_rms_norm_fp4_sfa_bf16, "residual_add_rms_norm_fp4_sfa_v2_fp16")                           # :515-529


# ------------------------------------------------------------------ GEMM
def cutlass_fp4_gemm_variant(idx, A, SFA, B, SFB, D, M, N, K, alpha=1.0, beta=0.0, stream=0, *, pdl=False,
                             splits=0, d_alpha=0, one_tile_per_cta=False) -> int:
    """D (M, N) bf16 = alpha * (A.SFA) (B.SFB)^T (csrc/fp4_bindings.cpp:355-370); beta must be 0."""
    if beta != 0.0:
        raise NotBuilt("NVFP4 GEMM with beta != 0 (the decoder path calls with beta = 0)")
    return call_status("frt_b200_gemm_nvfp4_nt", A, SFA, B, SFB, D, M, N, K, alpha, d_alpha or None, None, splits,
                       _f(pdl) | (2 if one_tile_per_cta else 0), stream)


def cutlass_fp4_sq_bf16(A, SFA, B, SFB, D, M, N, K, alpha=1.0, beta=0.0, stream=0, **kw) -> int:   # :85-99
    return cutlass_fp4_gemm_variant(0, A, SFA, B, SFB, D, M, N, K, alpha, beta, stream, **kw)


cutlass_fp4_sq_fp16 = _fp16_name(cutlass_fp4_sq_bf16, "cutlass_fp4_sq_fp16")


def cutlass_fp4_gemm_bias_bf16(A, SFA, B, SFB, bias, D, M, N, K, stream=0, *, pdl=False, splits=0) -> int:
    """D = A @ B^T + bias[N] (csrc/fp4_bindings.cpp:1139-1155)."""
    return call_status("frt_b200_gemm_nvfp4_nt", A, SFA, B, SFB, D, M, N, K, 1.0, None, bias or None, splits,
                       _f(pdl), stream)


def cutlass_fp4_gemm_rope_split(A, SFA, B, SFB, rope, Q, Kc, Vc, M, K, q_dim, k_dim, v_dim, head_dim, devpos=0,
                                alpha=1.0, stream=0, *, pdl=False, splits=0) -> int:
    """QKV projection with RoPE + split + KV append in the epilogue (no single reference entry point: stands for
    cutlass_fp4_gemm_variant + qkv_split_rope_kvcache_fp16, flash_rt/models/pi05/pipeline_thor.py:366-385)."""
    return call_status("frt_b200_gemm_nvfp4_nt_rope_split", A, SFA, B, SFB, M, K, alpha, rope, Q, Kc, Vc,
                       devpos or None, q_dim, k_dim, v_dim, head_dim, splits, _f(pdl), stream)


def __getattr__(name):
    raise _missing(name)


def _missing(name):
    from .flash_rt_kernels import _NotBuiltAttr
    return _NotBuiltAttr(f"flash_rt_fp4.{name} is not part of the B200 denoise path")
