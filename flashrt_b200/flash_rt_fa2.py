"""Drop-in stand-in for the reference's ``flash_rt.flash_rt_fa2`` pybind module
(``csrc/fa2_bindings.cpp:139-183``): same names and argument lists, served by the
tcgen05 attention kernel of ``libflashrt_b200.so``.

The split-KV scratch arguments of the reference (``softmax_lse_accum``, ``o_accum``) keep
their meaning: when given, the kv splits combine through them (plus a small arrival-counter
buffer); when absent, the splits combine inside a thread-block cluster through distributed
shared memory.
"""
from __future__ import annotations

import ctypes as C

from ._lib import call, call_status, KernelError  # noqa: F401


def _s3(t):
    return (C.c_longlong * 3)(int(t[0]), int(t[1]), int(t[2]))


_COUNTERS = {}


def _default_counters(n_words: int) -> int:
    """Arrival counters for the split-KV-through-scratch path when the caller passes the reference's scratch
    buffers but no counters: one zeroed int32 buffer per device, created on first use (outside graph capture)."""
    import torch
    dev = torch.cuda.current_device()
    buf = _COUNTERS.get(dev)
    if buf is None or buf.numel() < n_words:
        buf = torch.zeros(max(n_words, 4096), dtype=torch.int32, device=f"cuda:{dev}")
        _COUNTERS[dev] = buf
    return buf.data_ptr()


def _fwd(Q, K, V, O, softmax_lse, seqused_k, lse_accum, o_accum, batch, seqlen_q, seqlen_k, num_heads_q,
         num_heads_kv, head_dim, q_strides, k_strides, v_strides, o_strides, softmax_scale, stream, *, pdl=False,
         kv_splits=0, out_fp8=0, out_scale=0, kv_static_rows=0, counters=0, flags=0):
    if lse_accum and o_accum and not counters:
        g = num_heads_q // num_heads_kv
        counters = _default_counters(2 * ((seqlen_q * g + 127) // 128) * num_heads_kv * batch)
    if not (lse_accum and o_accum):
        lse_accum = o_accum = counters = 0
    call("frt_b200_attention_fwd_bf16", Q, K, V, O, out_fp8 or None, out_scale or None, softmax_lse or None,
         seqused_k or None, batch, seqlen_q, seqlen_k, num_heads_q, num_heads_kv, head_dim,
         C.cast(_s3(q_strides), C.c_void_p), C.cast(_s3(k_strides), C.c_void_p),
         C.cast(_s3(v_strides), C.c_void_p), C.cast(_s3(o_strides), C.c_void_p),
         softmax_scale, kv_splits, kv_static_rows, o_accum or None, lse_accum or None, counters or None,
         (1 if pdl else 0) | (flags & ~1), stream)


def fwd_bf16(Q, K, V, O, softmax_lse, softmax_lse_accum=0, o_accum=0, batch=1, seqlen_q=0, seqlen_k=0,
             num_heads_q=1, num_heads_kv=1, head_dim=0, q_strides=(0, 0, 0), k_strides=(0, 0, 0),
             v_strides=(0, 0, 0), o_strides=(0, 0, 0), softmax_scale=1.0, num_sms=0, stream=0, **kw):
    """``fa2.fwd_bf16`` (csrc/fa2_bindings.cpp:173-183).  ``softmax_lse_accum`` / ``o_accum`` are the reference's
    split-kv scratch buffers ((splits, batch, heads, seqlen_q[, head_dim]) fp32, sized for at least 8 splits);
    when both are given the kv splits combine through them, otherwise through the thread-block cluster."""
    _fwd(Q, K, V, O, softmax_lse, 0, softmax_lse_accum, o_accum, batch, seqlen_q, seqlen_k, num_heads_q,
         num_heads_kv, head_dim, q_strides, k_strides, v_strides, o_strides, softmax_scale, stream, **kw)


def fwd_bf16_seqused(Q, K, V, O, softmax_lse, seqused_k, batch, seqlen_q, seqlen_k, num_heads_q, num_heads_kv,
                     head_dim, q_strides, k_strides, v_strides, o_strides, softmax_scale=1.0, num_sms=0, stream=0,
                     **kw):
    """``fa2.fwd_bf16_seqused`` (csrc/fa2_bindings.cpp:142-150): only the first ``*seqused_k`` keys count."""
    _fwd(Q, K, V, O, softmax_lse, seqused_k, 0, 0, batch, seqlen_q, seqlen_k, num_heads_q, num_heads_kv, head_dim,
         q_strides, k_strides, v_strides, o_strides, softmax_scale, stream, **kw)


def fwd_bf16_seqused_splitkv(Q, K, V, O, softmax_lse, seqused_k, softmax_lse_accum=0, o_accum=0, batch=1,
                             seqlen_q=0, seqlen_k=0, num_heads_q=1, num_heads_kv=1, head_dim=0,
                             q_strides=(0, 0, 0), k_strides=(0, 0, 0), v_strides=(0, 0, 0), o_strides=(0, 0, 0),
                             softmax_scale=1.0, num_sms=0, stream=0, **kw):
    """``fa2.fwd_bf16_seqused_splitkv`` (csrc/fa2_bindings.cpp:152-160)."""
    _fwd(Q, K, V, O, softmax_lse, seqused_k, softmax_lse_accum, o_accum, batch, seqlen_q, seqlen_k, num_heads_q,
         num_heads_kv, head_dim, q_strides, k_strides, v_strides, o_strides, softmax_scale, stream, **kw)


def attention_status(reset: bool = True) -> int:
    return call_status("frt_b200_attention_status", 1 if reset else 0)


def fwd_bf16_static_scratch(Q, K, V, O, softmax_lse, batch, seqlen_q, seqlen_k, num_heads_q, num_heads_kv, head_dim,
                            q_strides, k_strides, v_strides, o_strides, softmax_scale=1.0, stream=0, *, seqused_k=0,
                            kv_splits=0, kv_static_rows=0, out_fp8=0, out_scale=0, pdl=False):
    """Split-KV attention for callers that cannot allocate device memory at the call site (no counterpart in the
    reference): the partials live in a fixed array inside the library instead of caller-provided buffers.  Raises
    :class:`KernelError` (status -4) when the shape exceeds that array (8 splits, 512 query rows x heads, head_dim
    256).  Make the first call on a device outside stream capture; do not let two calls overlap on the GPU."""
    call("frt_b200_attention_fwd_bf16_static_scratch", Q, K, V, O, out_fp8 or None, out_scale or None,
         softmax_lse or None, seqused_k or None, batch, seqlen_q, seqlen_k, num_heads_q, num_heads_kv, head_dim,
         C.cast(_s3(q_strides), C.c_void_p), C.cast(_s3(k_strides), C.c_void_p),
         C.cast(_s3(v_strides), C.c_void_p), C.cast(_s3(o_strides), C.c_void_p),
         softmax_scale, kv_splits, kv_static_rows, 1 if pdl else 0, stream)
