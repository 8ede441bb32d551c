"""Drop-in stand-in for the reference's ``flash_rt.flash_rt_kernels`` pybind module
(``csrc/bindings.cpp``) for the denoise hot path, backed by the sm_100a C-ABI library.

Same names, same positional / keyword arguments, same calling convention: every
pointer is a Python ``int`` holding a device address, ``stream`` is an ``int``
(0 = default stream), scales are device ``float*`` passed as ``int`` (``d_scale``).
Functions the reference declares ``void`` raise :class:`flashrt_b200._lib.KernelError`
on a non-zero status instead of failing silently.  Entry points of the reference that
lie outside the denoise path raise :class:`NotBuilt` (the analogue of the reference's
"extension not built" refusal, ``flash_rt/_extensions.py:67-108``).

Optional keyword ``pdl=True`` (not in the reference) launches with programmatic
dependent launch; the B200 pipeline uses it, reference call sites never pass it.
"""
from __future__ import annotations

from . import _lib
from ._lib import KernelError, call, call_status  # noqa: F401  (re-exported)


class NotBuilt(RuntimeError):
    """Raised for reference entry points that this library does not provide."""


class _NotBuiltAttr(NotBuilt, AttributeError):
    """Module-attribute form, so that ``hasattr(fvk, name)`` answers False instead of raising."""


def _f(pdl: bool) -> int:
    return 1 if pdl else 0


# ------------------------------------------------------------------ norms (csrc/bindings.cpp:854-947,1144-1162)
def rms_norm(x, weight, out, seq_len, dim, eps=1e-6, stream=0, *, pdl=False):
    call("frt_b200_norm_bf16", x, None, None, 0, weight, None, 0, out, None, seq_len, dim, eps, _f(pdl), stream)


def rms_norm_fp8(x, weight, out, seq_len, dim, eps=1e-6, d_scale=0, stream=0, *, pdl=False):
    call("frt_b200_norm_fp8", x, None, None, 0, weight, None, 0, out, None, seq_len, dim, eps, d_scale, _f(pdl),
         stream)


def ada_rms_norm_style(x, weight, style, out, gate_out, seq_len, dim, eps=1e-6, stream=0, *, pdl=False,
                       style_stride=None):
    ss = 3 * dim if style_stride is None else style_stride
    call("frt_b200_norm_bf16", x, None, None, 0, weight, style, ss, out, gate_out or None, seq_len, dim, eps,
         _f(pdl), stream)


def ada_rms_norm_style_fp8(x, weight, style, out, gate_out, seq_len, dim, eps=1e-6, d_scale=0, stream=0, *,
                           pdl=False, style_stride=None):
    ss = 3 * dim if style_stride is None else style_stride
    call("frt_b200_norm_fp8", x, None, None, 0, weight, style, ss, out, gate_out or None, seq_len, dim, eps,
         d_scale, _f(pdl), stream)


def residual_add_rms_norm_fp8(residual, x, weight, out, seq_len, dim, eps=1e-6, d_scale=0, stream=0, *,
                              pdl=False):
    call("frt_b200_norm_fp8", residual, x, None, 0, weight, None, 0, out, None, seq_len, dim, eps, d_scale,
         _f(pdl), stream)


def residual_add_rms_norm(residual, x, weight, out, seq_len, dim, eps=1e-6, stream=0, *, pdl=False):
    call("frt_b200_norm_bf16", residual, x, None, 0, weight, None, 0, out, None, seq_len, dim, eps, _f(pdl),
         stream)


def gate_residual_ada_norm_fp8(residual, x, gate, weight, style, out, gate_out, seq_len, dim, eps=1e-6,
                               d_scale=0, stream=0, *, pdl=False, style_stride=None, gate_stride=None):
    ss = 3 * dim if style_stride is None else style_stride
    gs = dim if gate_stride is None else gate_stride
    call("frt_b200_norm_fp8", residual, x, gate, gs, weight, style, ss, out, gate_out or None, seq_len, dim, eps,
         d_scale, _f(pdl), stream)


# ------------------------------------------------------------------ NVFP4 producers of this module (family 0:
# ceil-rounded UE4M3 block scale, '<' thresholds; csrc/bindings.cpp:1277-1285,1475-1590)
def quantize_bf16_to_nvfp4_swizzled(input, fp4_data, scale_factors, rows, cols, stream=0, *, pdl=False):
    call("frt_b200_quantize_nvfp4", input, fp4_data, scale_factors, rows, cols, 0, None, _f(pdl), stream)


quantize_bf16_to_nvfp4_swizzled_v2 = quantize_bf16_to_nvfp4_swizzled


def rms_norm_to_nvfp4_swizzled_bf16(x, weight, packed, sf_swz, rows, cols, eps=1e-6, stream=0, *, pdl=False):
    call("frt_b200_norm_nvfp4", x, None, None, 0, weight, None, 0, packed, sf_swz, None, rows, cols, eps, 0,
         _f(pdl), stream)


rms_norm_to_nvfp4_swizzled_bf16_v2 = rms_norm_to_nvfp4_swizzled_bf16
rms_norm_to_nvfp4_swizzled_bf16_v3 = rms_norm_to_nvfp4_swizzled_bf16


def residual_add_rms_norm_to_nvfp4_swizzled_bf16(h_in, attn_proj, h_post, weight, packed, sf_swz, rows, cols,
                                                 eps=1e-6, stream=0, *, pdl=False):
    """h_post = h_in + attn_proj; NVFP4(rms_norm(h_post) * weight).  The kernel updates in place, so a distinct
    h_post is first filled with h_in."""
    if h_post != h_in:
        call("frt_b200_copy", h_post, h_in, rows * cols * 2, stream)
        pdl = False
    call("frt_b200_norm_nvfp4", h_post, attn_proj, None, 0, weight, None, 0, packed, sf_swz, None, rows, cols, eps,
         0, _f(pdl), stream)


residual_add_rms_norm_to_nvfp4_swizzled_bf16_v2 = residual_add_rms_norm_to_nvfp4_swizzled_bf16


# ------------------------------------------------------------------ activation (csrc/bindings.cpp:1031-1044)
def gate_geglu_merged(merged, out, seq, half_dim, stream=0, *, pdl=False):
    call("frt_b200_geglu_bf16", merged, out, seq, half_dim, _f(pdl), stream)


def gate_geglu_merged_fp8(merged, out, seq, half_dim, d_scale=0, stream=0, *, pdl=False):
    call("frt_b200_geglu_fp8", merged, out, seq, half_dim, d_scale, _f(pdl), stream)


def gate_swiglu_merged(merged, out, seq, half_dim, stream=0, *, pdl=False):
    """silu(gate) * up of a merged (seq, 2 * half_dim) bf16 buffer -> bf16: the arithmetic of the reference's
    ``silu_mul_split_fp8_fp16`` family (csrc/kernels/activation.cu:291-306) on the [gate | up] layout of
    ``gate_geglu_merged``."""
    call("frt_b200_geglu_bf16", merged, out, seq, half_dim, _f(pdl) | 2, stream)


def gate_swiglu_merged_fp8(merged, out, seq, half_dim, d_scale, stream=0, *, pdl=False):
    """The same with the static FP8 quantisation of ``gate_geglu_merged_fp8`` behind it."""
    call("frt_b200_geglu_fp8", merged, out, seq, half_dim, d_scale, _f(pdl) | 2, stream)


# ------------------------------------------------------------------ RoPE (csrc/bindings.cpp:1071-1099)
def qkv_split_rope(qkv, rope_weights, Q, K, V, seq, q_dim, k_dim, v_dim, head_dim, stream=0, *, pdl=False):
    call("frt_b200_qkv_split_rope", qkv, rope_weights, Q, K, V, None, seq, q_dim, k_dim, v_dim, head_dim, _f(pdl),
         stream)


def qkv_split_rope_devpos(qkv, rope_weights, Q, K, V, devpos, seq, q_dim, k_dim, v_dim, head_dim, stream=0, *,
                          pdl=False):
    call("frt_b200_qkv_split_rope", qkv, rope_weights, Q, K, V, devpos, seq, q_dim, k_dim, v_dim, head_dim,
         _f(pdl), stream)


# ------------------------------------------------------------------ classifier-free guidance (csrc/bindings.cpp:1133-1141)
def cfg_combine_into_residual(residual, v_cond, v_uncond, beta, n, stream=0, *, pdl=False, f32=False):
    """residual += v_uncond + beta * (v_cond - v_uncond).  ``f32=True`` (not in the reference): fp32 arrays."""
    call("frt_b200_cfg_combine_into_residual", residual, v_cond, v_uncond, float(beta), n, 1 if f32 else 0, _f(pdl),
         stream)


# ------------------------------------------------------------------ elementwise (csrc/bindings.cpp:1103-1119)
def gate_mul_residual(residual, x, gate, n, stream=0, *, pdl=False):
    # flat form of the reference: gate has the same n elements as residual
    call("frt_b200_gate_mul_residual", residual, x, gate, n, 1, n, _f(pdl), stream)


def bias_residual(residual, x, bias, seq_len, dim, stream=0, *, pdl=False):
    call("frt_b200_bias_residual", residual, x, bias, seq_len, dim, _f(pdl), stream)


def residual_add(residual, x, n, stream=0, *, pdl=False):
    call("frt_b200_residual_add", residual, x, n, _f(pdl), stream)


def gpu_copy(dst, src, nbytes, stream=0):
    call("frt_b200_copy", dst, src, nbytes, stream)


# ------------------------------------------------------------------ video-DiT producers (csrc/bindings.cpp:879,1122,2802-2826,3427-3726)
def layer_norm(x, weight, bias, out, seq_len, dim, eps=1e-6, stream=0, *, pdl=False):
    call("frt_b200_layer_norm", x, weight, bias or None, None, None, 0, None, out, None, seq_len, dim, eps, _f(pdl),
         stream)


def ada_layer_norm_bf16(x, scale, shift, out, seq_len, dim, eps=1e-6, stream=0, *, pdl=False):
    """scale / shift: one (dim,) row shared by all tokens."""
    call("frt_b200_layer_norm", x, None, None, scale, shift, 0, None, out, None, seq_len, dim, eps, _f(pdl), stream)


def ada_layer_norm_bf16_per_token(x, scale, shift, out, seq_len, dim, eps=1e-6, stream=0, *, pdl=False):
    """scale / shift: (seq_len, dim), one row per token."""
    call("frt_b200_layer_norm", x, None, None, scale, shift, dim, None, out, None, seq_len, dim, eps, _f(pdl), stream)


def ada_layer_norm_fp8(x_bf16, scale_bf16, shift_bf16, out_fp8, act_scale, seq_len, dim, eps=1e-6, stream=0, *,
                       pdl=False, mod_stride=0):
    call("frt_b200_layer_norm", x_bf16, None, None, scale_bf16, shift_bf16, mod_stride, out_fp8, None, act_scale,
         seq_len, dim, eps, _f(pdl), stream)


def qkv_split_norm_rope_bf16(packed_qkv, norm_q_w, norm_k_w, freqs_re, freqs_im, q_rope_out, k_rope_out, B, L_v, N,
                             D_h, seq_len, eps=1e-6, stream=0, *, pdl=False, ext_ssq_q=0, ext_ssq_k=0, full_dim=0):
    call("frt_b200_qkv_split_norm_rope", packed_qkv, norm_q_w, norm_k_w, freqs_re, freqs_im, q_rope_out, k_rope_out,
         B, L_v, N, D_h, seq_len, eps, ext_ssq_q or None, ext_ssq_k or None, full_dim, _f(pdl), stream)


def row_sumsq(x, row_stride, col0, ncols, out, rows, stream=0, *, pdl=False):
    call("frt_b200_row_sumsq", x, row_stride, col0, ncols, out, rows, _f(pdl), stream)


def rms_norm_ext(x, x_stride, weight, ssq, out, out_stride, rows, dim, full_dim, eps=1e-6, stream=0, *, pdl=False):
    call("frt_b200_rms_norm_ext", x, x_stride, weight, ssq, out, out_stride, rows, dim, full_dim, eps, _f(pdl), stream)


def bias_gelu_quantize_fp8_static_bf16(in_bf16, bias_bf16, out_fp8, act_scale, M, N, stream=0, *, pdl=False):
    call("frt_b200_bias_gelu_quantize_fp8", in_bf16, bias_bf16 or None, out_fp8, act_scale, M, N, _f(pdl), stream)


def bias_gate_mul_residual_bf16(residual, x, bias, gate, seq_len, dim, stream=0, *, pdl=False, gate_stride=None):
    gs = dim if gate_stride is None else gate_stride
    call("frt_b200_bias_gate_mul_residual", residual, x, bias or None, gate, gs, seq_len, dim, _f(pdl), stream)


def add_bias_bf16(x, b, S, D, stream=0, *, pdl=False):
    call("frt_b200_add_bias", x, b, S, D, _f(pdl), stream)


def adaln_modulation6_bf16(adaln_params, layer_modulation, out0, out1, out2, out3, out4, out5, B, S, D, stream=0, *,
                           pdl=False):
    call("frt_b200_adaln_modulation6", adaln_params, layer_modulation, out0, out1, out2, out3, out4, out5, B, S, D,
         _f(pdl), stream)


# ------------------------------------------------------------------ quantise (csrc/bindings.cpp:1191-1211)
def quantize_fp8_static(input, output, d_scale, n, stream=0, *, pdl=False):  # noqa: A002 (reference kwarg name)
    call("frt_b200_quantize_fp8_static", input, output, d_scale, n, _f(pdl), stream)


def quantize_fp8_device(input, output, d_scale, n, stream=0):  # noqa: A002
    call("frt_b200_quantize_fp8_device", input, output, d_scale, n, stream)


def fp8_accumulate_scale_max(src_scale, dst_scale, stream=0):
    call("frt_b200_fp8_accumulate_scale_max", src_scale, dst_scale, stream)


# ------------------------------------------------------------------ GEMM (csrc/bindings.cpp:605-803,2062-2069)
def fp8_gemm_descale_bf16out(A, B, C, M, N, K, act_descale, w_descale, stream=0, *, pdl=False, splits=0):
    """C(M,N) bf16 = act_descale * w_descale * A(M,K) . B(N,K)^T  (B = weights, K contiguous)."""
    call("frt_b200_gemm_fp8_nt", A, B, C, M, N, K, act_descale, w_descale, 1.0, None, splits, _f(pdl), stream)


def _tile_hint(tile_n: int) -> int:
    """flags bits 8-9 of the small-M FP8 GEMM entry points: pinned tile width of the token-major kernel."""
    return {0: 0, 64: 1, 128: 2, 256: 3}[int(tile_n)] << 8


class GemmRunner:
    """Stand-in for the reference's cuBLASLt ``GemmRunner`` (``csrc/gemm/gemm_runner.h``).

    Only the methods the denoise path calls exist.  There is nothing to autotune (the
    kernel is chosen from the shape), so the ``autotune_*`` methods accept the
    reference's arguments and return immediately.
    """

    def fp8_nt_dev(self, A, B, D, M, N, K, d_scale_a, d_scale_b, stream=0, *, pdl=False, splits=0, bias=None,
                   one_tile_per_cta=False, cta_pair=None, swapped=False, tile_n=0):
        """D(M,N) bf16 = sa*sb * A(M,K) . B(N,K)^T — weights stored (N,K), the ``fp8_layout == "nk"`` form.
        ``one_tile_per_cta`` selects the non-persistent large-M kernel (same result; kept for comparison runs);
        ``cta_pair`` True / False forces / forbids the 256 x 256-tile kernel on CTA pairs (M > 256, N >= 256; by
        default the library uses it for tile lists of at least two waves at K >= 2048).  M <= 256: ``swapped``
        keeps the weights-on-lanes kernel instead of the token-major one, ``tile_n`` (64 / 128 / 256) pins the
        token-major kernel's tile width."""
        call("frt_b200_gemm_fp8_nt", A, B, D, M, N, K, d_scale_a, d_scale_b, 1.0, bias, splits,
             _f(pdl) | (2 if one_tile_per_cta else 0) | (8 if cta_pair else 0) | (32 if cta_pair is False else 0)
             | (16 if swapped else 0)
             | _tile_hint(tile_n), stream)

    # -- the decoder's projections with the norm kernel between them folded in ------------------------------
    def fp8_nt_dev_gate_residual(self, A, B, M, N, K, d_scale_a, d_scale_b, residual, gate, stats_out, stream=0, *,
                                 pdl=False, splits=0, tile_n=0, next_scale=0, q8_out=0, d_scale_q8=0) -> int:
        """``fp8_nt_dev`` + the first pass of ``gate_residual_ada_norm_fp8``: residual <- residual + o * gate and
        the per-tile row sums of squares into ``stats_out`` (rows of 128 floats).  Returns the number of rows
        written, which the consuming ``norm_fp8_nt_dev_*`` / ``fp8_nt_dev_*_rowscale`` call takes as ``n_stat``.
        With ``q8_out``: also the next projection's FP8 operand e4m3(residual * (1 + next_scale) / *d_scale_q8),
        i.e. the norm's output without its per-row 1 / rms, which ``fp8_nt_dev_*_rowscale`` applies afterwards."""
        import ctypes
        n = ctypes.c_int(0)
        call("frt_b200_gemm_fp8_nt_gate_residual_q8", A, B, M, N, K, d_scale_a, d_scale_b, residual, gate,
             stats_out or None, ctypes.addressof(n), next_scale or None, q8_out or None, d_scale_q8 or None, splits,
             _f(pdl) | _tile_hint(tile_n), stream)
        return n.value

    def fp8_nt_dev_rope_split_rowscale(self, A, B, M, K, d_scale_a, d_scale_b, stats, n_stat, col_term, rope_weights,
                                       Q, Kc, Vc, q_dim, k_dim, v_dim, head_dim, stream=0, *, eps=1e-6, devpos=0,
                                       pdl=False, splits=0, tile_n=0):
        """QKV projection of an operand left by ``fp8_nt_dev_gate_residual(q8_out=...)``: the row's 1 / rms (from
        ``stats``) and ``col_term`` = W . shift are applied in the finish, then ``qkv_split_rope[_devpos]``."""
        call("frt_b200_gemm_fp8_nt_rope_split_rowscale", A, B, M, K, d_scale_a, d_scale_b, stats, n_stat, eps,
             col_term, rope_weights, Q, Kc, Vc, devpos or None, q_dim, k_dim, v_dim, head_dim, splits,
             _f(pdl) | _tile_hint(tile_n), stream)

    def fp8_nt_dev_geglu_fp8_rowscale(self, A, B, out, M, half_dim, K, d_scale_a, d_scale_b, stats, n_stat, col_term,
                                      d_scale_out, stream=0, *, eps=1e-6, pdl=False, splits=0, tile_n=0, fast_gelu=False):
        """gate|up projection of such an operand, ``gate_geglu_merged_fp8`` behind it (``fast_gelu``: the GELU through
        the hardware tanh)."""
        call("frt_b200_gemm_fp8_nt_geglu_fp8_rowscale", A, B, out, M, half_dim, K, d_scale_a, d_scale_b, stats, n_stat,
             eps, col_term, d_scale_out, splits, _f(pdl) | (128 if fast_gelu else 0) | _tile_hint(tile_n), stream)

    def norm_fp8_nt_dev_rope_split(self, x, stats, n_stat, style, B, M, K, d_scale_a, d_scale_b, rope_weights, Q, Kc,
                                   Vc, q_dim, k_dim, v_dim, head_dim, stream=0, *, eps=1e-6, devpos=0, pdl=False,
                                   splits=0, tile_n=0):
        """Second pass of ``gate_residual_ada_norm_fp8`` (adaRMS -> FP8 from the residual rows and the sums of
        squares in ``stats``) produced inside the QKV projection, then ``qkv_split_rope[_devpos]``."""
        call("frt_b200_norm_gemm_fp8_nt_rope_split", x, stats, n_stat, style, eps, B, M, K, d_scale_a, d_scale_b,
             rope_weights, Q, Kc, Vc, devpos or None, q_dim, k_dim, v_dim, head_dim, splits,
             _f(pdl) | _tile_hint(tile_n), stream)

    def norm_fp8_nt_dev_geglu_fp8(self, x, stats, n_stat, style, B, out, M, half_dim, K, d_scale_a, d_scale_b,
                                  d_scale_out, stream=0, *, eps=1e-6, pdl=False, splits=0, tile_n=0, fast_gelu=False):
        """The same producer in front of the gate|up projection, ``gate_geglu_merged_fp8`` behind it."""
        call("frt_b200_norm_gemm_fp8_nt_geglu_fp8", x, stats, n_stat, style, eps, B, out, M, half_dim, K, d_scale_a,
             d_scale_b, d_scale_out, splits, _f(pdl) | (128 if fast_gelu else 0) | _tile_hint(tile_n), stream)

    def fp8_nt_dev_gate_res_norm_fp8(self, A, B, M, N, K, d_scale_a, d_scale_b, residual, gate, style, out, d_scale_out,
                                     stream=0, *, eps=1e-6, pdl=False, splits=0):
        """``fp8_nt_dev`` followed by ``gate_residual_ada_norm_fp8`` (unit norm weight, shared gate / style rows) in
        one launch: the projection's result never leaves the chip before the next GEMM's FP8 input is written."""
        call("frt_b200_gemm_fp8_nt_gate_res_norm_fp8", A, B, M, N, K, d_scale_a, d_scale_b, residual, gate, style, out,
             d_scale_out, eps, splits, _f(pdl), stream)

    def fp8_nt_dev_bias_gelu_fp8(self, A, B, out, M, N, K, d_scale_a, d_scale_b, bias, d_scale_out, stream=0, *,
                                 pdl=False, fast_gelu=False):
        """``fp8_nt_dev`` followed by ``bias_gelu_quantize_fp8_static_bf16`` (csrc/bindings.cpp:3427-3440) in one
        launch, M > 256: the video-DiT FFN-up projection writes its FP8 mid-activation directly."""
        call("frt_b200_gemm_fp8_nt_bias_gelu_fp8", A, B, out, M, N, K, d_scale_a, d_scale_b, bias or None,
             d_scale_out, _f(pdl) | (128 if fast_gelu else 0), stream)

    # -- fused forms (no reference counterpart as single calls; each equals two reference calls) ------------
    def fp8_nt_dev_rope_split(self, A, B, M, K, d_scale_a, d_scale_b, rope_weights, Q, Kc, Vc, q_dim, k_dim, v_dim,
                              head_dim, stream=0, *, devpos=0, pdl=False, splits=0, swapped=False, tile_n=0):
        """``fp8_nt_dev`` into a (M, q+k+v) buffer followed by ``qkv_split_rope[_devpos]``, in one launch."""
        call("frt_b200_gemm_fp8_nt_rope_split", A, B, M, K, d_scale_a, d_scale_b, rope_weights, Q, Kc, Vc,
             devpos or None, q_dim, k_dim, v_dim, head_dim, splits,
             _f(pdl) | (16 if swapped else 0) | _tile_hint(tile_n), stream)

    def fp8_nt_dev_geglu_fp8(self, A, B, out, M, half_dim, K, d_scale_a, d_scale_b, d_scale_out, stream=0, *,
                             pdl=False, splits=0, swapped=False, tile_n=0, silu_gate=False, fast_gelu=False):
        """``fp8_nt_dev`` into a merged (M, 2*half) buffer followed by ``gate_geglu_merged_fp8``, in one launch.
        ``silu_gate``: SiLU instead of GELU on the gate (``gate_swiglu_merged_fp8`` behind the GEMM; M <= 128)."""
        call("frt_b200_gemm_fp8_nt_geglu_fp8", A, B, out, M, half_dim, K, d_scale_a, d_scale_b, d_scale_out, splits,
             _f(pdl) | (16 if swapped else 0) | (64 if silu_gate else 0) | (128 if fast_gelu else 0) | _tile_hint(tile_n),
             stream)

    def fp8_nn_dev(self, A, B, D, M, N, K, d_scale_a, d_scale_b, stream=0, *, pdl=False, splits=0, bias=None,
                   tile_n=0):
        """D(M,N) bf16 = sa*sb * A(M,K) . B(K,N) — weights stored (K,N), the reference's default ``fp8_layout == "kn"``
        form (csrc/bindings.cpp:706-716).  Same result as ``fp8_nt_dev`` on the transposed weights.  K % 128 == 0,
        N % 16 == 0, N >= 128."""
        call("frt_b200_gemm_fp8_nn", A, B, D, M, N, K, d_scale_a, d_scale_b, 1.0, bias, splits,
             _f(pdl) | _tile_hint(tile_n), stream)

    def bf16_nn(self, A, B, D, M, N, K, stream=0, *, pdl=False, bias=None, accumulate=False, a_f32=False,
                d_f32=False):
        if not (N <= 64 or K <= 64):
            raise NotBuilt("bf16_nn is provided for the 32<->1024 action projections only (N <= 64 or K <= 64)")
        call("frt_b200_gemm_bf16_nn_small", A, B, D, bias, M, N, K, 1 if accumulate else 0,
             (1 if a_f32 else 0) | (2 if d_f32 else 0), _f(pdl), stream)

    # the reference measures cuBLASLt algorithms here; nothing to do for a shape-selected kernel
    def autotune_bf16_nn(self, *a, **k):
        return 0

    def autotune_fp8_nn_dev(self, *a, **k):
        return 0

    def autotune_fp8_nt_dev(self, *a, **k):
        return 0


# ------------------------------------------------------------------ capability probes (csrc/bindings.cpp:2424-2459)
def has_cutlass_sm100() -> bool:
    """The reference reports whether its CUTLASS Sm100 kernels were compiled in; here the tcgen05 path is
    the only path."""
    return True


def has_nvfp4() -> bool:
    return False


def get_sm_version() -> int:
    v = _lib.call_status("frt_b200_sm_version")
    if v < 0:
        raise KernelError(f"frt_b200_sm_version failed: status {v}")
    return v


def tensor_core_status(reset: bool = True) -> int:
    """0 unless a bounded wait inside a tensor-core kernel gave up (see ``frt_b200_gemm_status``)."""
    r = 1 if reset else 0
    return (_lib.call_status("frt_b200_gemm_status", r) or _lib.call_status("frt_b200_attention_status", r)
            or _lib.call_status("frt_b200_expert_loop_status", r))


def __getattr__(name: str):
    if name.startswith("__"):
        raise AttributeError(name)
    raise _NotBuiltAttr(f"flash_rt_kernels.{name} is outside the denoise hot path and is not provided by flashrt_b200")
