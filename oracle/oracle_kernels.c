/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement (plain C, scalar) of the
 * reference's fused norm / quantise / activation / RoPE kernels on the denoise
 * hot path.  Nothing in the shipped library links or calls this file; only the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Each function restates one reference kernel (cited by file:line inside
 * FlashRT) with every fp32 operation individually rounded, in a fixed order:
 *
 *   - The reference is built with --use_fast_math (CMakeLists.txt:376), so its
 *     own binaries use approximate reciprocal / rsqrt / exp and compiler-chosen
 *     FMA contraction; those are not reproducible from source on a CPU.  This
 *     restatement keeps the reference's algorithm and rounding POINTS (what is
 *     rounded to bf16 and when, what is summed unrounded, multiply by the fp32
 *     reciprocal of the scale, clamp to +-448, RN-even E4M3 conversion) and
 *     pins the remaining freedom to correctly rounded IEEE operations:
 *     1/s by division, rsqrt as 1/sqrtf, exp by the explicit polynomial below,
 *     a*b+c as one fma where noted.
 *   - Reduction order is a property of launch geometry, not of the algorithm.
 *     The order used here is: each group of 8 consecutive elements is summed by
 *     a sequential fma chain; 32 such partial sums are combined by an
 *     xor-butterfly (offsets 16, 8, 4, 2, 1); the per-32-group totals are added
 *     in increasing order.  (The reference: 256 threads stride over bf16 pairs,
 *     shfl_down tree, csrc/kernels/common.cuh:61-97.)
 *
 * Pinning: checked against vectors produced by importing the reference's own
 * torch ground-truth functions (flash_rt/structures/catalog/ * /reference.py)
 * -- see tests/golden/ -- to fp32 tolerance, and bit-exactly against E4M3 /
 * bf16 conversions of torch.
 *
 * Build: gcc -O2 -ffp-contract=off -mfma -shared -fPIC (see oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ formats */
static inline float bf16_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
/* round-to-nearest-even; NaN -> 0x7fff (cvt.rn.bf16.f32 canonical NaN) */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}
uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_bf16_to_f32(uint16_t b) { return bf16_to_f32(b); }

/* fp32 -> E4M3 (bias 7, 3 mantissa bits, max finite 448 = 0x7e, no inf),
 * round-to-nearest-even, saturating to +-448; NaN -> 0x7f. */
static inline uint8_t f32_to_e4m3(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(sign | 0x7f);
    float af;
    memcpy(&af, &a, 4);
    if (af >= 448.0f) {
        /* values above 448 saturate; the halfway point to the non-existent 480
         * also saturates under satfinite */
        return (uint8_t)(sign | 0x7e);
    }
    int e = (int)(a >> 23) - 127; /* unbiased fp32 exponent */
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    int shift; /* bits to drop from the 24-bit significand */
    int eb;    /* biased e4m3 exponent of the result before rounding carry */
    if (a == 0) return sign;
    if (e >= -6) {
        shift = 20; /* keep 1+3 bits */
        eb = e + 7;
    } else {
        /* subnormal target: value = q * 2^-9, q in [0,8) */
        shift = 20 + (-6 - e);
        eb = 0;
        if (shift > 25) return sign; /* below half the smallest subnormal */
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    uint32_t code;
    if (eb == 0) {
        code = q; /* q == 8 becomes exponent 1, mantissa 0 = smallest normal */
    } else {
        /* q in [8,16]; q == 16 carries into the exponent */
        code = ((uint32_t)eb << 3) + (q - 8u);
    }
    if (code > 0x7e) code = 0x7e;
    return (uint8_t)(sign | code);
}
uint8_t orc_f32_to_e4m3(float f) { return f32_to_e4m3(f); }

static inline float e4m3_to_f32(uint8_t c) {
    int s = c & 0x80;
    int e = (c >> 3) & 0xf;
    int m = c & 7;
    float v;
    if (e == 0) v = ldexpf((float)m, -9);
    else if (e == 15 && m == 7) v = NAN;
    else v = ldexpf((float)(8 + m), e - 10);
    return s ? -v : v;
}
float orc_e4m3_to_f32(uint8_t c) { return e4m3_to_f32(c); }

/* fminf/fmaxf with CUDA semantics: the non-NaN operand wins */
static inline float clamp448(float v) {
    float t = (v != v) ? -448.0f : (v > -448.0f ? v : -448.0f);
    return t < 448.0f ? t : 448.0f;
}

/* ------------------------------------------------------------------ exp / gelu
 * e^x: clamp to [-87, 88]; n = rint(x*log2e); r = x - n*ln2 (two-piece,
 * fma); degree-7 Horner with fma; multiply by 2^n. */
static inline float det_expf(float x) {
    x = x != x ? -87.0f : x; /* fmaxf(NaN,-87) = -87 */
    x = x > -87.0f ? x : -87.0f;
    x = x < 88.0f ? x : 88.0f;
    float n = rintf(x * 1.4426950408889634f);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.4286068203094173e-06f, r);
    float p = 1.9841269841269841e-04f;
    p = fmaf(p, r, 1.3888888888888889e-03f);
    p = fmaf(p, r, 8.3333333333333332e-03f);
    p = fmaf(p, r, 4.1666666666666664e-02f);
    p = fmaf(p, r, 1.6666666666666666e-01f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    uint32_t sb = (uint32_t)((int)n + 127) << 23;
    float s;
    memcpy(&s, &sb, 4);
    return p * s;
}
float orc_det_expf(float x) { return det_expf(x); }

/* gelu_tanh(g) = g / (1 + exp(-1.5957691216057308 g (1 + 0.044715 g^2)))
 * csrc/kernels/activation.cu:262 */
static inline float det_gelu_tanh(float g) {
    float inner = fmaf(0.044715f * g, g, 1.0f);
    float arg = (-1.5957691216057308f * g) * inner;
    float e = det_expf(arg);
    return g / (1.0f + e);
}
float orc_det_gelu_tanh(float g) { return det_gelu_tanh(g); }

/* ------------------------------------------------------------------ row sum of squares */
static float row_ssq_tree(const float* r, int dim) {
    int nthreads = ((dim / 8 + 31) / 32) * 32;
    int nwarps = nthreads / 32;
    float tot = 0.0f;
    for (int w = 0; w < nwarps; ++w) {
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            int col = (w * 32 + l) * 8;
            float s = 0.0f;
            if (col < dim)
                for (int i = 0; i < 8; ++i) s = fmaf(r[col + i], r[col + i], s);
            lane[l] = s;
        }
        for (int off = 16; off >= 1; off >>= 1) {
            float nxt[32];
            for (int l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ off];
            memcpy(lane, nxt, sizeof(lane));
        }
        tot = (w == 0) ? lane[0] : tot + lane[0];
    }
    return tot;
}

/* ------------------------------------------------------------------ fused norm family
 * Covers rms_norm_fp8 (norm.cu:286-343), ada_rms_norm_style (norm.cu:345-389),
 * ada_rms_norm_style_fp8 (norm.cu:392-442), residual_add_rms_norm_fp8
 * (norm.cu:445-495), residual_add_rms_norm (norm.cu:498-539) and
 * gate_residual_ada_norm_fp8 (fusion.cu:15-81).
 *
 * residual: (rows, dim) bf16 in/out (updated only when x != NULL)
 * x, gate_in: optional; gate_in row r at gate_in + r*gate_in_stride
 * weight: (dim,) or NULL = ones
 * style: optional rows [scale|shift|gate] of 3*dim at style + r*style_stride
 * out_fp8 / out_bf16: exactly one non-NULL; scale used only for fp8
 * gate_out: optional (rows, dim) copy of the style gate chunk
 */
void orc_norm(uint16_t* residual, const uint16_t* x, const uint16_t* gate_in, long long gate_in_stride,
              const uint16_t* weight, const uint16_t* style, long long style_stride, uint8_t* out_fp8,
              uint16_t* out_bf16, uint16_t* gate_out, int rows, int dim, float eps, float scale) {
    float inv_scale = 1.0f / scale;
    float rbuf[16384];
    for (int row = 0; row < rows; ++row) {
        uint16_t* res = residual + (size_t)row * dim;
        float ssq_in[16384];
        for (int c = 0; c < dim; ++c) {
            float r = bf16_to_f32(res[c]);
            if (x) {
                float xv = bf16_to_f32(x[(size_t)row * dim + c]);
                if (gate_in) {
                    float g = bf16_to_f32(gate_in[(size_t)row * gate_in_stride + c]);
                    r = fmaf(xv, g, r);
                } else {
                    r = r + xv;
                }
                ssq_in[c] = r;              /* unrounded feeds the sum */
                res[c] = f32_to_bf16(r);    /* stored rounded */
                rbuf[c] = bf16_to_f32(res[c]); /* rounded feeds the norm */
            } else {
                ssq_in[c] = r;
                rbuf[c] = r;
            }
        }
        float tot = row_ssq_tree(ssq_in, dim);
        float var = tot / (float)dim + eps;
        float rms = 1.0f / sqrtf(var);
        const uint16_t* srow = style ? style + (size_t)row * style_stride : 0;
        for (int c = 0; c < dim; ++c) {
            float w = weight ? bf16_to_f32(weight[c]) : 1.0f;
            float n = (rbuf[c] * rms) * w;
            if (srow) {
                float sc = bf16_to_f32(srow[c]);
                float sh = bf16_to_f32(srow[dim + c]);
                n = fmaf(n, 1.0f + sc, sh);
                if (gate_out) gate_out[(size_t)row * dim + c] = srow[2 * (size_t)dim + c];
            }
            if (out_fp8) out_fp8[(size_t)row * dim + c] = f32_to_e4m3(clamp448(n * inv_scale));
            else out_bf16[(size_t)row * dim + c] = f32_to_bf16(n);
        }
    }
}

/* ------------------------------------------------------------------ GeGLU
 * gate_silu_mul_merged_fp8, csrc/kernels/activation.cu:249-266 */
void orc_geglu_fp8(const uint16_t* merged, uint8_t* out, int rows, int H, float scale) {
    float inv_scale = 1.0f / scale;
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < H; ++c) {
            float g = bf16_to_f32(merged[(size_t)r * 2 * H + c]);
            float u = bf16_to_f32(merged[(size_t)r * 2 * H + H + c]);
            float v = (det_gelu_tanh(g) * u) * inv_scale;
            out[(size_t)r * H + c] = f32_to_e4m3(clamp448(v));
        }
}
/* SiLU gate (SwiGLU): silu_mul_split_fp8_kernel, csrc/kernels/activation.cu:291-306, on the merged [gate | up] layout */
static float det_silu(float g) { return g / (1.0f + det_expf(-g)); }
void orc_swiglu_fp8(const uint16_t* merged, uint8_t* out, int rows, int H, float scale) {
    float inv_scale = 1.0f / scale;
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < H; ++c) {
            float g = bf16_to_f32(merged[(size_t)r * 2 * H + c]);
            float u = bf16_to_f32(merged[(size_t)r * 2 * H + H + c]);
            float v = (det_silu(g) * u) * inv_scale;
            out[(size_t)r * H + c] = f32_to_e4m3(clamp448(v));
        }
}
void orc_swiglu_bf16(const uint16_t* merged, uint16_t* out, int rows, int H) {
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < H; ++c) {
            float g = bf16_to_f32(merged[(size_t)r * 2 * H + c]);
            float u = bf16_to_f32(merged[(size_t)r * 2 * H + H + c]);
            out[(size_t)r * H + c] = f32_to_bf16(det_silu(g) * u);
        }
}
void orc_geglu_bf16(const uint16_t* merged, uint16_t* out, int rows, int H) {
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < H; ++c) {
            float g = bf16_to_f32(merged[(size_t)r * 2 * H + c]);
            float u = bf16_to_f32(merged[(size_t)r * 2 * H + H + c]);
            out[(size_t)r * H + c] = f32_to_bf16(det_gelu_tanh(g) * u);
        }
}

/* ------------------------------------------------------------------ quantise
 * quantize_fp8_kernel_generic, csrc/kernels/quantize.cu:61-75 */
void orc_quantize_fp8_static(const uint16_t* in, uint8_t* out, long long n, float scale) {
    float inv_scale = 1.0f / scale;
    for (long long i = 0; i < n; ++i) out[i] = f32_to_e4m3(clamp448(bf16_to_f32(in[i]) * inv_scale));
}
/* absmax + compute_scale_kernel, csrc/kernels/quantize.cu:131-136 */
float orc_amax_scale(const uint16_t* in, long long n) {
    float m = 0.0f;
    for (long long i = 0; i < n; ++i) {
        float a = fabsf(bf16_to_f32(in[i]));
        if (a > m) m = a;
    }
    float s = m / 448.0f;
    return s < 1e-12f ? 1e-12f : s;
}
void orc_dequantize_fp8(const uint8_t* in, float* out, long long n, float scale) {
    for (long long i = 0; i < n; ++i) out[i] = e4m3_to_f32(in[i]) * scale;
}

/* ------------------------------------------------------------------ adds
 * residual_add (elementwise.cu:302), bias_residual (elementwise.cu:207),
 * gate_mul_residual (elementwise.cu:34).  mode 0: r+x, 1: (r+x)+bias[c], 2: fma(x,gate,r) */
void orc_add(uint16_t* res, const uint16_t* x, const uint16_t* aux, long long aux_stride, int rows, int dim,
             int mode) {
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < dim; ++c) {
            size_t i = (size_t)r * dim + c;
            float a = bf16_to_f32(res[i]), b = bf16_to_f32(x[i]);
            float o;
            if (mode == 0) o = a + b;
            else if (mode == 1) o = (a + b) + bf16_to_f32(aux[c]);
            else o = fmaf(b, bf16_to_f32(aux[(size_t)r * aux_stride + c]), a);
            res[i] = f32_to_bf16(o);
        }
}

/* ------------------------------------------------------------------ RoPE + split
 * qkv_split_rope_kernel / _devpos, csrc/kernels/rope.cu:135-264.
 * Adjacent-pair rotation, table row [cos0,sin0,cos1,sin1,...]; K,V rows written at pos+t. */
void orc_qkv_split_rope(const uint16_t* qkv, const uint16_t* rope, uint16_t* Q, uint16_t* K, uint16_t* V, int pos,
                        int seq, int q_dim, int k_dim, int v_dim, int head_dim) {
    int W = q_dim + k_dim + v_dim;
    for (int t = 0; t < seq; ++t) {
        const uint16_t* row = qkv + (size_t)t * W;
        const uint16_t* tab = rope + (size_t)t * head_dim;
        for (int c = 0; c < q_dim + k_dim; c += 2) {
            int cc = c < q_dim ? c : c - q_dim;
            int d = cc % head_dim;
            float x0 = bf16_to_f32(row[c]), x1 = bf16_to_f32(row[c + 1]);
            float cs = bf16_to_f32(tab[d]), sn = bf16_to_f32(tab[d + 1]);
            float o0 = fmaf(x0, cs, -(x1 * sn));
            float o1 = fmaf(x1, cs, x0 * sn);
            uint16_t* dst = c < q_dim ? Q + (size_t)t * q_dim + cc : K + (size_t)(pos + t) * k_dim + cc;
            dst[0] = f32_to_bf16(o0);
            dst[1] = f32_to_bf16(o1);
        }
        memcpy(V + (size_t)(pos + t) * v_dim, row + q_dim + k_dim, (size_t)v_dim * 2);
    }
}

/* ------------------------------------------------------------------ FP8 GEMM (fp64 accumulate)
 * D(M,N) bf16 = (sa*sb) * A_e4m3(M,K) . B   with B given (N,K) row-major when b_is_nk, else (K,N).
 * GemmRunner::fp8_nn_dev, csrc/gemm/gemm_runner.cu:67-76,263-272 (math only: fp32-or-better
 * accumulate, product of the two scales applied to the accumulator, bf16 result). */
void orc_gemm_fp8(const uint8_t* A, const uint8_t* B, uint16_t* D, float* Df, int M, int N, int K, float sa,
                  float sb, int b_is_nk) {
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = e4m3_to_f32((uint8_t)i);
    float alpha = sa * sb;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            double acc = 0.0;
            if (b_is_nk)
                for (int k = 0; k < K; ++k) acc += (double)lut[A[(size_t)m * K + k]] * (double)lut[B[(size_t)n * K + k]];
            else
                for (int k = 0; k < K; ++k) acc += (double)lut[A[(size_t)m * K + k]] * (double)lut[B[(size_t)k * N + n]];
            float v = (float)acc * alpha;
            if (D) D[(size_t)m * N + n] = f32_to_bf16(v);
            if (Df) Df[(size_t)m * N + n] = v;
        }
}

/* ------------------------------------------------------------------ video-DiT (Wan-shape) producers */
/* block-wide sum as the kernels do it: threads own 8 consecutive elements, xor-butterfly per 32 threads,
 * warp totals added in order.  part[] holds the per-thread partial sums. */
static float tree_sum_threads(const float* part, int nthreads) {
    float tot = 0.0f;
    for (int w = 0; w < nthreads / 32; ++w) {
        float lane[32], nxt[32];
        memcpy(lane, part + w * 32, sizeof(lane));
        for (int off = 16; off >= 1; off >>= 1) {
            for (int l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ off];
            memcpy(lane, nxt, sizeof(lane));
        }
        tot = (w == 0) ? lane[0] : tot + lane[0];
    }
    return tot;
}

/* 0.5 x (1 + tanh(0.7978845608 (x + 0.044715 x^3))), tanh(u) = 1 - 2 / (1 + e^{2u})
 * csrc/quantize/bias_gelu_quantize_fp8.cu:18-23 */
static inline float det_gelu_tanh_form(float x) {
    float x3 = (x * x) * x;
    float u = 0.7978845608f * fmaf(0.044715f, x3, x);
    float e = det_expf(2.0f * u);
    float th = 1.0f - 2.0f / (1.0f + e);
    return (0.5f * x) * (1.0f + th);
}
float orc_det_gelu_tanh_form(float x) { return det_gelu_tanh_form(x); }

/* ada_layer_norm_fp8 (csrc/quantize/ada_layer_norm_fp8.cu:58-147), ada_layer_norm_bf16[_per_token]
 * (csrc/kernels/dit_bf16.cu:151-278), layer_norm (csrc/kernels/norm.cu:113-162).
 * Two-pass statistics (mean, then mean of squared deviations), modulated value rounded through bf16 before FP8. */
void orc_layer_norm(const uint16_t* x, const uint16_t* weight, const uint16_t* bias, const uint16_t* scale,
                    const uint16_t* shift, long long mod_stride, uint8_t* out_fp8, uint16_t* out_bf16, int rows,
                    int dim, float eps, float qscale) {
    int nthreads = ((dim / 8 + 31) / 32) * 32;
    float inv_a = 1.0f / qscale;
    static float part[1024], v[8192];
    for (int r = 0; r < rows; ++r) {
        const uint16_t* xr = x + (size_t)r * dim;
        for (int t = 0; t < nthreads; ++t) {
            float s = 0.0f;
            for (int i = 0; i < 8; ++i) {
                int c = t * 8 + i;
                if (c < dim) { v[c] = bf16_to_f32(xr[c]); s = s + v[c]; }
            }
            part[t] = s;
        }
        float mean = tree_sum_threads(part, nthreads) / (float)dim;
        for (int t = 0; t < nthreads; ++t) {
            float q = 0.0f;
            for (int i = 0; i < 8; ++i) {
                int c = t * 8 + i;
                if (c < dim) { v[c] = v[c] - mean; q = fmaf(v[c], v[c], q); }
            }
            part[t] = q;
        }
        float var = tree_sum_threads(part, nthreads) / (float)dim + eps;
        float inv_std = 1.0f / sqrtf(var);
        for (int c = 0; c < dim; ++c) {
            float n = v[c] * inv_std;
            if (weight) n = fmaf(n, bf16_to_f32(weight[c]), bias ? bf16_to_f32(bias[c]) : 0.0f);
            if (scale) n = fmaf(n, 1.0f + bf16_to_f32(scale[(size_t)r * mod_stride + c]),
                                bf16_to_f32(shift[(size_t)r * mod_stride + c]));
            uint16_t b16 = f32_to_bf16(n);
            if (out_bf16) out_bf16[(size_t)r * dim + c] = b16;
            else out_fp8[(size_t)r * dim + c] = f32_to_e4m3(clamp448(bf16_to_f32(b16) * inv_a));
        }
    }
}

/* qkv_split_norm_rope_bf16, csrc/quantize/qkv_split_norm_rope_bf16.cu:16-140 */
void orc_qkv_split_norm_rope(const uint16_t* packed, const uint16_t* wq, const uint16_t* wk, const float* fre,
                             const float* fim, uint16_t* q_out, uint16_t* k_out, int B, int L, int N, int D_h,
                             int seq_len, float eps) {
    int dim = N * D_h;
    int nthreads = ((dim / 8 + 31) / 32) * 32;
    static float pq[1024], pk[1024];
    for (int row = 0; row < B * L; ++row) {
        int t = row % L;
        const uint16_t* q = packed + (size_t)row * 3 * dim;
        const uint16_t* k = q + dim;
        for (int th = 0; th < nthreads; ++th) {
            float sq = 0.0f, sk = 0.0f;
            for (int i = 0; i < 8; ++i) {
                int c = th * 8 + i;
                if (c < dim) {
                    float a = bf16_to_f32(q[c]), b = bf16_to_f32(k[c]);
                    sq = fmaf(a, a, sq);
                    sk = fmaf(b, b, sk);
                }
            }
            pq[th] = sq;
            pk[th] = sk;
        }
        float inv_q = 1.0f / sqrtf(tree_sum_threads(pq, nthreads) / (float)dim + eps);
        float inv_k = 1.0f / sqrtf(tree_sum_threads(pk, nthreads) / (float)dim + eps);
        for (int c = 0; c < dim; c += 2) {
            int cp = (c % D_h) >> 1;
            float qre = (bf16_to_f32(q[c]) * inv_q) * bf16_to_f32(wq[c]);
            float qim = (bf16_to_f32(q[c + 1]) * inv_q) * bf16_to_f32(wq[c + 1]);
            float kre = (bf16_to_f32(k[c]) * inv_k) * bf16_to_f32(wk[c]);
            float kim = (bf16_to_f32(k[c + 1]) * inv_k) * bf16_to_f32(wk[c + 1]);
            uint16_t* qo = q_out + (size_t)row * dim + c;
            uint16_t* ko = k_out + (size_t)row * dim + c;
            if (t < seq_len) {
                float fr = fre[(size_t)t * (D_h / 2) + cp], fi = fim[(size_t)t * (D_h / 2) + cp];
                qo[0] = f32_to_bf16(fmaf(qre, fr, -(qim * fi)));
                qo[1] = f32_to_bf16(fmaf(qre, fi, qim * fr));
                ko[0] = f32_to_bf16(fmaf(kre, fr, -(kim * fi)));
                ko[1] = f32_to_bf16(fmaf(kre, fi, kim * fr));
            } else {
                qo[0] = f32_to_bf16(qre); qo[1] = f32_to_bf16(qim);
                ko[0] = f32_to_bf16(kre); ko[1] = f32_to_bf16(kim);
            }
        }
    }
}

/* bias_gelu_quantize_fp8_static_bf16, csrc/quantize/bias_gelu_quantize_fp8.cu:24-49 */
void orc_bias_gelu_quantize_fp8(const uint16_t* in, const uint16_t* bias, uint8_t* out, long long M, int N,
                                float scale) {
    float inv_s = 1.0f / scale;
    for (long long i = 0; i < M * N; ++i) {
        float v = bf16_to_f32(in[i]);
        if (bias) v = v + bf16_to_f32(bias[i % N]);
        out[i] = f32_to_e4m3(clamp448(det_gelu_tanh_form(v) * inv_s));
    }
}

/* bias_gate_mul_residual_bf16 (csrc/kernels/elementwise.cu:1648-1683): r += (x + bias) * gate;
 * add_bias_bf16: x += bias (gate == NULL) */
void orc_bias_gate_mul_residual(uint16_t* res, const uint16_t* x, const uint16_t* bias, const uint16_t* gate,
                                long long gate_stride, long long rows, int dim) {
    for (long long r = 0; r < rows; ++r)
        for (int c = 0; c < dim; ++c) {
            size_t i = (size_t)r * dim + c;
            float b = bias ? bf16_to_f32(bias[c]) : 0.0f;
            float o;
            if (gate) o = fmaf(bf16_to_f32(x[i]) + b, bf16_to_f32(gate[(size_t)r * gate_stride + c]), bf16_to_f32(res[i]));
            else o = bf16_to_f32(res[i]) + b;
            res[i] = f32_to_bf16(o);
        }
}

/* adaln_modulation6_bf16, csrc/kernels/elementwise.cu:603-645 */
void orc_adaln_modulation6(const float* params, const float* layer_mod, uint16_t* out6, long long BS, int D) {
    for (long long bs = 0; bs < BS; ++bs)
        for (int j = 0; j < 6; ++j)
            for (int d = 0; d < D; ++d)
                out6[((size_t)j * BS + bs) * D + d] = f32_to_bf16(params[(bs * 6 + j) * D + d] + layer_mod[(size_t)j * D + d]);
}

/* ================================================================== NVFP4
 * e2m1 elements (+-{0, .5, 1, 1.5, 2, 3, 4, 6}), 16-element blocks, one unsigned E4M3 scale per block,
 * scale bytes in the 128-row x 4-block atoms of the block-scaled GEMM.  Two quantiser conventions exist
 * in the reference and both are restated here:
 *   family 0 ("A", flash_rt_kernels: quantize_bf16_to_nvfp4[_swizzled], csrc/kernels/quantize.cu:375-526,
 *             conversions csrc/kernels/nvfp4_convert.cuh:31-105): scale = ceil_UE4M3(amax / 6) (rounded up,
 *             top code 0xFE, zero block -> 0), inv = scale > 0 ? 1 / scale : 0, thresholds compared with '<'
 *             (a tie goes to the larger magnitude);
 *   family 1 ("B", flash_rt_fp4: quantize_fp4_dynamic_sfa_*, csrc/quantize/quantize_fp4_sfa.cu:31-109 and the
 *             fused producers csrc/fused_fp4/norm_silu_fp4_sfa.cu:64-147, silu_mul_fp4_sfa_vec.cu:33-107):
 *             scale = RN-even E4M3 of max(amax / 6, 1e-12), inv = 1 / scale (IEEE: a zero scale gives inf and
 *             0 * inf = NaN, which falls through every '<=' test to code 7), thresholds compared with '<='
 *             (a tie goes to the smaller magnitude).
 * Family 1 is pinned bit for bit against the reference's own torch NVFP4 reference (golden vectors generated by
 * tests/golden/make_nvfp4_golden.py from its tests/test_fp4_integration_meta.py:31-57); family 0 has no CPU statement
 * in the reference and is restated from the source text only.
 * Low nibble = even element.  An optional FP32 global scale g divides the input first (x * (1 / g)); the
 * reference's quantisers carry none (g = 1).  Divisions are IEEE here; the reference builds with fast-math. */

static inline float ue4m3_to_f32(uint8_t c) {
    int e = (c >> 3) & 0xF, m = c & 7;
    if (e == 0) return ldexpf((float)m * 0.125f, -6);
    return ldexpf(1.0f + (float)m * 0.125f, e - 7);
}
float orc_ue4m3_to_f32(uint8_t c) { return ue4m3_to_f32(c); }

/* smallest unsigned-E4M3 value >= v (top code 0xFE above 240, as the reference) */
static inline uint8_t ue4m3_ceil(float v) {
    if (!(v > 0.0f)) return 0;
    if (v > 240.0f) return 0xFE;
    if (v < 0.015625f) {                       /* below 2^-6: subnormal step 2^-9 */
        int m = (int)ceilf(v * 512.0f);
        if (m > 7) return 0x08;                /* smallest normal */
        return (uint8_t)(m < 1 ? 1 : m);
    }
    int e;
    float f = frexpf(v, &e);                   /* v = f * 2^e, f in [0.5, 1) */
    float t = (f * 2.0f - 1.0f) * 8.0f;        /* exact: mantissa steps of 1/8 above 2^(e-1) */
    int m = (int)ceilf(t);
    int ex = e - 1 + 7;
    if (m >= 8) { m = 0; ex += 1; }
    if (ex >= 15) return 0xFE;
    return (uint8_t)((ex << 3) | m);
}
uint8_t orc_ue4m3_ceil(float v) { return ue4m3_ceil(v); }

static inline uint8_t e2m1_code(float v, int family) {
    static const float th[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    uint8_t sign = (v < 0.0f) ? 8u : 0u;
    float a = fabsf(v);
    int below = 0;                             /* thresholds the magnitude stays under; NaN stays under none */
    for (int i = 0; i < 7; ++i) below += family ? (a <= th[i]) : (a < th[i]);
    return (uint8_t)(sign | (7 - below));
}
static inline float e2m1_to_f32(uint8_t c) {
    static const float lut[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float m = lut[c & 7];
    return (c & 8) ? -m : m;
}

/* byte offset of the scale of (row, 16-element block blk) for a row length of K elements */
long long orc_nvfp4_sf_offset(long long row, int blk, int K) {
    long long katoms = (K + 63) / 64;
    return ((row / 128) * katoms + blk / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + blk % 4;
}
long long orc_nvfp4_sf_size(long long rows, int K) {
    return ((rows + 127) / 128) * (long long)((K + 63) / 64) * 512;
}

/* quantise one block of 16 fp32 values; returns the scale byte */
static uint8_t nvfp4_block(const float* v, uint8_t* packed8, int family) {
    float amax = 0.0f;
    for (int i = 0; i < 16; ++i) { float a = fabsf(v[i]); if (a > amax) amax = a; }
    uint8_t sb;
    float inv;
    if (family == 0) {
        sb = ue4m3_ceil(amax / 6.0f);
        float s = ue4m3_to_f32(sb);
        inv = s > 0.0f ? 1.0f / s : 0.0f;
    } else {
        float d = amax / 6.0f;
        if (d < 1e-12f) d = 1e-12f;
        sb = f32_to_e4m3(d);
        inv = 1.0f / e4m3_to_f32(sb);
    }
    for (int p = 0; p < 8; ++p) {
        uint8_t lo = e2m1_code(v[2 * p] * inv, family);
        uint8_t hi = e2m1_code(v[2 * p + 1] * inv, family);
        packed8[p] = (uint8_t)(lo | (hi << 4));
    }
    return sb;
}

/* in: fp32 (rows, D), D % 16 == 0.  packed (rows, D/2); sf: orc_nvfp4_sf_size(rows, D) bytes, zeroed by the caller */
void orc_nvfp4_quantize_f32(const float* in, uint8_t* packed, uint8_t* sf, long long rows, int D, int family,
                            float global_scale) {
    float inv_g = 1.0f / global_scale;
    for (long long r = 0; r < rows; ++r)
        for (int b = 0; b < D / 16; ++b) {
            float v[16];
            for (int i = 0; i < 16; ++i) {
                float x = in[r * D + b * 16 + i];
                v[i] = (global_scale == 1.0f) ? x : x * inv_g;
            }
            sf[orc_nvfp4_sf_offset(r, b, D)] = nvfp4_block(v, packed + r * (D / 2) + b * 8, family);
        }
}
void orc_nvfp4_quantize_bf16(const uint16_t* in, uint8_t* packed, uint8_t* sf, long long rows, int D, int family,
                             float global_scale) {
    float* tmp = (float*)malloc(sizeof(float) * (size_t)rows * D);
    for (long long i = 0; i < rows * D; ++i) tmp[i] = bf16_to_f32(in[i]);
    orc_nvfp4_quantize_f32(tmp, packed, sf, rows, D, family, global_scale);
    free(tmp);
}
/* out fp32 (rows, D) = e2m1 * block scale * global_scale */
void orc_nvfp4_dequantize(const uint8_t* packed, const uint8_t* sf, float* out, long long rows, int D,
                          float global_scale) {
    for (long long r = 0; r < rows; ++r)
        for (int c = 0; c < D; ++c) {
            uint8_t byte = packed[r * (D / 2) + c / 2];
            uint8_t code = (c & 1) ? (byte >> 4) : (byte & 15);
            float s = ue4m3_to_f32(sf[orc_nvfp4_sf_offset(r, c / 16, D)] & 0x7F);
            out[r * D + c] = e2m1_to_f32(code) * s * global_scale;
        }
}
/* GeGLU straight to NVFP4 (gate_geglu_fp4_sfa_vec, csrc/fused_fp4/silu_mul_fp4_sfa_vec.cu:50-107): the fp32
 * product gelu(gate) * up is quantised without an intermediate 16-bit rounding. */
void orc_geglu_nvfp4(const uint16_t* merged, uint8_t* packed, uint8_t* sf, int rows, int H, int family) {
    float* tmp = (float*)malloc(sizeof(float) * (size_t)rows * H);
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < H; ++c) {
            float g = bf16_to_f32(merged[(size_t)r * 2 * H + c]);
            float u = bf16_to_f32(merged[(size_t)r * 2 * H + H + c]);
            tmp[(size_t)r * H + c] = det_gelu_tanh(g) * u;
        }
    orc_nvfp4_quantize_f32(tmp, packed, sf, rows, H, family, 1.0f);
    free(tmp);
}

/* ------------------------------------------------------------------ classifier-free guidance combine
 * cfg_combine_kernel, csrc/kernels/elementwise.cu:2299-2324: residual += v_uncond + beta * (v_cond - v_uncond) */
void orc_cfg_combine_bf16(uint16_t* residual, const uint16_t* vc, const uint16_t* vu, float beta, long long n) {
    for (long long i = 0; i < n; ++i) {
        float c = bf16_to_f32(vc[i]), u = bf16_to_f32(vu[i]);
        residual[i] = f32_to_bf16(bf16_to_f32(residual[i]) + fmaf(beta, c - u, u));
    }
}
void orc_cfg_combine_f32(float* residual, const float* vc, const float* vu, float beta, long long n) {
    for (long long i = 0; i < n; ++i) residual[i] = residual[i] + fmaf(beta, vc[i] - vu[i], vu[i]);
}
