// Fused producers of the Wan-shape video-DiT block for sm_100a: adaLN (affine-free LayerNorm +
// modulation) -> FP8 / bf16, affine LayerNorm, packed-QKV split + full-width q/k RMSNorm + 3-D RoPE,
// bias + GELU(tanh) -> FP8, bias / gate residual updates, 6-way modulation table.
//
// Replaces, for sm_100a, the reference kernels
//   ada_layer_norm_fp8                 csrc/bindings.cpp:3482-3495 -> csrc/quantize/ada_layer_norm_fp8.cu:58-147
//   ada_layer_norm_bf16[_per_token]    csrc/bindings.cpp:2802-2816 -> csrc/kernels/dit_bf16.cu:151-278
//   layer_norm                         csrc/bindings.cpp:879-885   -> csrc/kernels/norm.cu:113-162
//   qkv_split_norm_rope_bf16           csrc/bindings.cpp:3574      -> csrc/quantize/qkv_split_norm_rope_bf16.cu:16-140
//   bias_gelu_quantize_fp8_static_bf16 csrc/bindings.cpp:3427-3440 -> csrc/quantize/bias_gelu_quantize_fp8.cu:24-49
//   bias_gate_mul_residual_bf16        csrc/bindings.cpp:1122-1131 -> csrc/kernels/elementwise.cu:1648-1683
//   add_bias_bf16                      csrc/bindings.cpp:2818-2826
//   adaln_modulation6_bf16             csrc/bindings.cpp:3705-3726 -> csrc/kernels/elementwise.cu:603-645
//
// Same arithmetic policy as the other fused kernels: explicitly rounded fp32 operations in a fixed order
// that the C oracle repeats, so FP8 codes and bf16 bits are compared for equality.  Rounding points kept
// from the reference: the modulated adaLN value is rounded through bf16 before the FP8 conversion; q/k
// norms are taken over the full model width; rotation multiplies complex pairs (2c, 2c+1) by fp32 freqs;
// rows t >= seq_len pass through un-rotated.
//
// One CTA per row, one 16-byte vector (8 bf16) per thread, row held in registers (single trip to HBM).
#include "common.cuh"

namespace frt {

// block-wide sum with the fixed tree: butterfly per warp, then warp totals in order (all threads get it)
__device__ __forceinline__ float block_sum_fixed(float v, float* warp_tot) {
    v = warp_sum_butterfly(v);
    const int nwarps = blockDim.x >> 5;
    __syncthreads();                              // protects warp_tot against the previous use
    if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = warp_tot[0];
    for (int w = 1; w < nwarps; ++w) tot = __fadd_rn(tot, warp_tot[w]);
    return tot;
}

// tanh-form GELU: 0.5 x (1 + tanh(0.7978845608 (x + 0.044715 x^3))), tanh(u) = 1 - 2 / (1 + e^{2u})
__device__ __forceinline__ float det_gelu_tanh_form(float x) {
    const float x3 = __fmul_rn(__fmul_rn(x, x), x);
    const float u = __fmul_rn(0.7978845608f, __fmaf_rn(0.044715f, x3, x));
    const float e = det_expf(__fmul_rn(2.0f, u));
    const float th = __fsub_rn(1.0f, __fdiv_rn(2.0f, __fadd_rn(1.0f, e)));
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, th));
}

// ------------------------------------------------------------------ LayerNorm family
// y = (x - mean) * inv_std [* w + b] [* (1 + scale) + shift]; out = fp8(clamp(bf16(y) / s)) or bf16(y)
template <bool OUT_FP8>
__global__ void __launch_bounds__(1024)
layer_norm_row_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ weight,
                      const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ scale,
                      const __nv_bfloat16* __restrict__ shift, long long mod_stride, void* __restrict__ out,
                      const float* __restrict__ d_scale, int dim, float eps) {
    __shared__ float warp_tot[32];
    const int row = blockIdx.x;
    const int col = threadIdx.x * 8;
    const bool active = col < dim;
    const size_t roff = (size_t)row * dim + col;
    uint4 wv = make_uint4(0, 0, 0, 0), bv = wv, sc = wv, sh = wv;
    if (active) {
        if (weight) wv = ld_global_v4(weight + col);
        if (bias) bv = ld_global_v4(bias + col);
        if (scale) sc = ld_global_v4(scale + (size_t)row * mod_stride + col);
        if (shift) sh = ld_global_v4(shift + (size_t)row * mod_stride + col);
    }
    float inv_a = 1.0f;
    if (OUT_FP8) inv_a = __fdiv_rn(1.0f, *d_scale);
    pdl_wait();
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    float s = 0.0f;
    if (active) {
        uint4 xv = ld_stream_v4(x + roff);
        const uint32_t* xw = &xv.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            unpack_bf16x2(xw[i], v[2 * i], v[2 * i + 1]);
            s = __fadd_rn(s, v[2 * i]);
            s = __fadd_rn(s, v[2 * i + 1]);
        }
    }
    pdl_launch_dependents();
    const float mean = __fdiv_rn(block_sum_fixed(s, warp_tot), (float)dim);
    float q = 0.0f;
    if (active) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = __fsub_rn(v[i], mean);
            q = __fmaf_rn(v[i], v[i], q);
        }
    }
    const float var = __fadd_rn(__fdiv_rn(block_sum_fixed(q, warp_tot), (float)dim), eps);
    const float inv_std = __fdiv_rn(1.0f, __fsqrt_rn(var));
    if (!active) return;
    const uint32_t* ww = &wv.x;
    const uint32_t* bw = &bv.x;
    const uint32_t* scw = &sc.x;
    const uint32_t* shw = &sh.x;
    float y[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float n0 = __fmul_rn(v[2 * i], inv_std), n1 = __fmul_rn(v[2 * i + 1], inv_std);
        if (weight) {
            float w0, w1, b0 = 0.0f, b1 = 0.0f;
            unpack_bf16x2(ww[i], w0, w1);
            if (bias) unpack_bf16x2(bw[i], b0, b1);
            n0 = __fmaf_rn(n0, w0, b0);
            n1 = __fmaf_rn(n1, w1, b1);
        }
        if (scale) {
            float s0, s1, h0, h1;
            unpack_bf16x2(scw[i], s0, s1);
            unpack_bf16x2(shw[i], h0, h1);
            n0 = __fmaf_rn(n0, __fadd_rn(1.0f, s0), h0);
            n1 = __fmaf_rn(n1, __fadd_rn(1.0f, s1), h1);
        }
        y[2 * i] = n0;
        y[2 * i + 1] = n1;
    }
    uint4 o16;
    o16.x = pack_bf16x2(y[0], y[1]);
    o16.y = pack_bf16x2(y[2], y[3]);
    o16.z = pack_bf16x2(y[4], y[5]);
    o16.w = pack_bf16x2(y[6], y[7]);
    if (!OUT_FP8) {
        st_global_v4(reinterpret_cast<__nv_bfloat16*>(out) + roff, o16);
    } else {
        float r[8];                                      // quantise the bf16-rounded value
        unpack_bf16x2(o16.x, r[0], r[1]);
        unpack_bf16x2(o16.y, r[2], r[3]);
        unpack_bf16x2(o16.z, r[4], r[5]);
        unpack_bf16x2(o16.w, r[6], r[7]);
        uint2 o8;
        o8.x = f32x4_to_e4m3x4(clamp448(__fmul_rn(r[0], inv_a)), clamp448(__fmul_rn(r[1], inv_a)),
                               clamp448(__fmul_rn(r[2], inv_a)), clamp448(__fmul_rn(r[3], inv_a)));
        o8.y = f32x4_to_e4m3x4(clamp448(__fmul_rn(r[4], inv_a)), clamp448(__fmul_rn(r[5], inv_a)),
                               clamp448(__fmul_rn(r[6], inv_a)), clamp448(__fmul_rn(r[7], inv_a)));
        st_global_v2(reinterpret_cast<uint8_t*>(out) + roff, o8);
    }
}

// ------------------------------------------------------------------ QKV split + q/k RMSNorm + 3-D RoPE
// packed (rows, 3*dim) bf16 = [q | k | v]; q_out / k_out (rows, dim); row = b * L + t
__global__ void __launch_bounds__(1024)
qkv_split_norm_rope_kernel(const __nv_bfloat16* __restrict__ packed, const __nv_bfloat16* __restrict__ wq,
                           const __nv_bfloat16* __restrict__ wk, const float* __restrict__ fre,
                           const float* __restrict__ fim, __nv_bfloat16* __restrict__ q_out,
                           __nv_bfloat16* __restrict__ k_out, int L, int dim, int D_h, int seq_len, float eps,
                           const float* __restrict__ ext_ssq_q, const float* __restrict__ ext_ssq_k, int full_dim) {
    __shared__ float warp_tot[32];
    const int row = blockIdx.x;
    const int t = row % L;
    const int col = threadIdx.x * 8;
    const bool active = col < dim;
    uint4 wqv = make_uint4(0, 0, 0, 0), wkv = wqv;
    float fr[4] = {1.f, 1.f, 1.f, 1.f}, fi[4] = {0.f, 0.f, 0.f, 0.f};
    const bool rope = t < seq_len;
    if (active) {
        wqv = ld_global_v4(wq + col);
        wkv = ld_global_v4(wk + col);
        if (rope) {
            const int cp = (col % D_h) >> 1;              // first complex pair of this vector inside its head
            const float4 a = *reinterpret_cast<const float4*>(fre + (size_t)t * (D_h >> 1) + cp);
            const float4 b = *reinterpret_cast<const float4*>(fim + (size_t)t * (D_h >> 1) + cp);
            fr[0] = a.x; fr[1] = a.y; fr[2] = a.z; fr[3] = a.w;
            fi[0] = b.x; fi[1] = b.y; fi[2] = b.z; fi[3] = b.w;
        }
    }
    pdl_wait();
    float q[8], k[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = k[i] = 0.0f;
    float sq = 0.0f, sk = 0.0f;
    if (active) {
        const __nv_bfloat16* base = packed + (size_t)row * 3 * dim + col;
        uint4 qv = ld_stream_v4(base), kv = ld_stream_v4(base + dim);
        const uint32_t* qw = &qv.x;
        const uint32_t* kw = &kv.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            unpack_bf16x2(qw[i], q[2 * i], q[2 * i + 1]);
            unpack_bf16x2(kw[i], k[2 * i], k[2 * i + 1]);
            sq = __fmaf_rn(q[2 * i], q[2 * i], sq);
            sq = __fmaf_rn(q[2 * i + 1], q[2 * i + 1], sq);
            sk = __fmaf_rn(k[2 * i], k[2 * i], sk);
            sk = __fmaf_rn(k[2 * i + 1], k[2 * i + 1], sk);
        }
    }
    pdl_launch_dependents();
    // tensor-parallel use: this CTA only sees its heads' slice of the row; the sums over the full width come in
    float tq, tk;
    if (ext_ssq_q) {
        tq = ext_ssq_q[row];
        tk = ext_ssq_k[row];
    } else {
        tq = block_sum_fixed(sq, warp_tot);
        tk = block_sum_fixed(sk, warp_tot);
    }
    const float inv_q = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tq, (float)full_dim), eps)));
    const float inv_k = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tk, (float)full_dim), eps)));
    if (!active) return;
    const uint32_t* wqw = &wqv.x;
    const uint32_t* wkw = &wkv.x;
    uint4 oq, ok;
    uint32_t* oqw = &oq.x;
    uint32_t* okw = &ok.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float a0, a1, b0, b1;
        unpack_bf16x2(wqw[i], a0, a1);
        unpack_bf16x2(wkw[i], b0, b1);
        const float qre = __fmul_rn(__fmul_rn(q[2 * i], inv_q), a0), qim = __fmul_rn(__fmul_rn(q[2 * i + 1], inv_q), a1);
        const float kre = __fmul_rn(__fmul_rn(k[2 * i], inv_k), b0), kim = __fmul_rn(__fmul_rn(k[2 * i + 1], inv_k), b1);
        if (rope) {
            oqw[i] = pack_bf16x2(__fmaf_rn(qre, fr[i], -__fmul_rn(qim, fi[i])), __fmaf_rn(qre, fi[i], __fmul_rn(qim, fr[i])));
            okw[i] = pack_bf16x2(__fmaf_rn(kre, fr[i], -__fmul_rn(kim, fi[i])), __fmaf_rn(kre, fi[i], __fmul_rn(kim, fr[i])));
        } else {
            oqw[i] = pack_bf16x2(qre, qim);
            okw[i] = pack_bf16x2(kre, kim);
        }
    }
    st_global_v4(q_out + (size_t)row * dim + col, oq);
    st_global_v4(k_out + (size_t)row * dim + col, ok);
}

// ------------------------------------------------------------------ bias + GELU(tanh) -> FP8
__global__ void __launch_bounds__(256)
bias_gelu_fp8_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ bias,
                     uint8_t* __restrict__ out, const float* __restrict__ d_scale, long long rows, int N) {
    const float inv_s = __fdiv_rn(1.0f, *d_scale);
    pdl_wait();
    const int vec_per_row = N >> 3;
    const long long total = rows * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int col = (int)(i % vec_per_row) << 3;
        uint4 xv = ld_stream_v4(in + i * 8);
        uint4 bv = bias ? ld_global_v4(bias + col) : make_uint4(0, 0, 0, 0);
        const uint32_t* xw = &xv.x;
        const uint32_t* bw = &bv.x;
        float o[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float x0, x1, b0, b1;
            unpack_bf16x2(xw[k], x0, x1);
            unpack_bf16x2(bw[k], b0, b1);
            if (bias) { x0 = __fadd_rn(x0, b0); x1 = __fadd_rn(x1, b1); }
            o[2 * k] = clamp448(__fmul_rn(det_gelu_tanh_form(x0), inv_s));
            o[2 * k + 1] = clamp448(__fmul_rn(det_gelu_tanh_form(x1), inv_s));
        }
        uint2 ov;
        ov.x = f32x4_to_e4m3x4(o[0], o[1], o[2], o[3]);
        ov.y = f32x4_to_e4m3x4(o[4], o[5], o[6], o[7]);
        st_global_v2(out + i * 8, ov);
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------ residual <- residual + (x + bias) * gate   (gate per row or shared)
// MODE 0: res += (x + bias) * gate     MODE 1: x += bias (in place, res == x)
template <int MODE>
__global__ void __launch_bounds__(256)
bias_gate_res_kernel(__nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ gate,
                     long long gate_stride, long long rows, int dim) {
    pdl_wait();
    const int vec_per_row = dim >> 3;
    const long long total = rows * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / vec_per_row;
        const int col = (int)(i - row * vec_per_row) << 3;
        uint4 rv = ld_global_v4(res + i * 8);
        uint4 bv = bias ? ld_global_v4(bias + col) : make_uint4(0, 0, 0, 0);
        uint4 xv = make_uint4(0, 0, 0, 0), gv = xv;
        if (MODE == 0) {
            xv = ld_stream_v4(x + i * 8);
            gv = ld_global_v4(gate + row * gate_stride + col);
        }
        const uint32_t* rw = &rv.x;
        const uint32_t* xw = &xv.x;
        const uint32_t* bw = &bv.x;
        const uint32_t* gw = &gv.x;
        uint4 ov;
        uint32_t* ow = &ov.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float r0, r1, x0, x1, b0, b1, g0, g1;
            unpack_bf16x2(rw[k], r0, r1);
            unpack_bf16x2(xw[k], x0, x1);
            unpack_bf16x2(bw[k], b0, b1);
            unpack_bf16x2(gw[k], g0, g1);
            if (MODE == 0) {
                r0 = __fmaf_rn(__fadd_rn(x0, b0), g0, r0);
                r1 = __fmaf_rn(__fadd_rn(x1, b1), g1, r1);
            } else {
                r0 = __fadd_rn(r0, b0);
                r1 = __fadd_rn(r1, b1);
            }
            ow[k] = pack_bf16x2(r0, r1);
        }
        st_global_v4(res + i * 8, ov);
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------ six modulation tensors
// out_j[b, s, :] = bf16(adaln_params[b, s, j, :] + layer_modulation[j, :]), fp32 inputs
__global__ void __launch_bounds__(256)
modulation6_kernel(const float* __restrict__ params, const float* __restrict__ layer_mod,
                   __nv_bfloat16* o0, __nv_bfloat16* o1, __nv_bfloat16* o2, __nv_bfloat16* o3, __nv_bfloat16* o4,
                   __nv_bfloat16* o5, int D, long long n) {
    pdl_wait();
    __nv_bfloat16* outs[6] = {o0, o1, o2, o3, o4, o5};
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const int d = (int)(idx % D);
        const long long base = (idx / D) * 6LL * D + d;
#pragma unroll
        for (int j = 0; j < 6; ++j)
            outs[j][idx] = __float2bfloat16_rn(__fadd_rn(params[base + (long long)j * D], layer_mod[(long long)j * D + d]));
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------ tensor-parallel helpers for full-width norms
// out[r] (+)= sum over `ncols` columns of x[r, col0 + c]^2   (one warp per row, fp32)
__global__ void __launch_bounds__(256)
row_sumsq_kernel(const __nv_bfloat16* __restrict__ x, long long row_stride, int col0, int ncols,
                 float* __restrict__ out, long long rows) {
    pdl_wait();
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const __nv_bfloat16* xr = x + row * row_stride + col0;
    float s = 0.0f;
    for (int c = lane * 8; c < ncols; c += 256) {
        uint4 v = ld_global_v4(xr + c);
        const uint32_t* w = &v.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float a, b;
            unpack_bf16x2(w[i], a, b);
            s = __fmaf_rn(a, a, s);
            s = __fmaf_rn(b, b, s);
        }
    }
    s = warp_sum_butterfly(s);
    if (lane == 0) out[row] = s;
}

// y[r, :] = bf16(x[r, :] * rsqrt(ssq[r] / full_dim + eps) * w[:]) on a column slice of width `dim`
__global__ void __launch_bounds__(256)
rms_norm_ext_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, const __nv_bfloat16* __restrict__ w,
                    const float* __restrict__ ssq, __nv_bfloat16* __restrict__ out, long long out_stride,
                    long long rows, int dim, int full_dim, float eps) {
    pdl_wait();
    const int vec_per_row = dim >> 3;
    const long long total = rows * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / vec_per_row;
        const int col = (int)(i - row * vec_per_row) << 3;
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ssq[row], (float)full_dim), eps)));
        uint4 xv = ld_global_v4(x + row * x_stride + col);
        uint4 wv = ld_global_v4(w + col);
        const uint32_t* xw = &xv.x;
        const uint32_t* ww = &wv.x;
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float a, b, w0, w1;
            unpack_bf16x2(xw[k], a, b);
            unpack_bf16x2(ww[k], w0, w1);
            ow[k] = pack_bf16x2(__fmul_rn(__fmul_rn(a, inv), w0), __fmul_rn(__fmul_rn(b, inv), w1));
        }
        st_global_v4(out + row * out_stride + col, o);
    }
}

template <typename K, typename... Args>
static int launch_k(K kernel, unsigned grid, unsigned block, cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}
static inline bool mis(const void* p, int a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }
static inline unsigned cap_grid(long long items, int threads) {
    long long need = (items + threads - 1) / threads;
    long long cap = 148LL * 8;
    return (unsigned)(need < 1 ? 1 : (need < cap ? need : cap));
}

}  // namespace frt

using namespace frt;

extern "C" {

// LayerNorm over `dim` per row: y = (x - mean) * inv_std, then optional affine (weight, bias (dim,)), then optional
// modulation y * (1 + scale) + shift with scale / shift rows at + r * mod_stride (0 = one shared (dim,) row).
// out_fp8 != NULL: e4m3(clamp(bf16(y) * (1 / *d_scale))); else out_bf16 = bf16(y).
int frt_b200_layer_norm(const void* x, const void* weight, const void* bias, const void* scale, const void* shift,
                        long long mod_stride, void* out_fp8, void* out_bf16, const float* d_scale, int rows, int dim,
                        float eps, int flags, void* stream) {
    if (!x || (!out_fp8 && !out_bf16) || (out_fp8 && out_bf16) || rows < 0 || dim <= 0) return FRT_ERR_INVALID;
    if (out_fp8 && !d_scale) return FRT_ERR_INVALID;
    if ((scale == nullptr) != (shift == nullptr) || (bias && !weight)) return FRT_ERR_INVALID;
    if ((dim & 7) || dim > 8192 || (mod_stride & 7)) return FRT_ERR_UNSUPPORTED;
    if (mis(x, 16) || mis(weight, 16) || mis(bias, 16) || mis(scale, 16) || mis(shift, 16) || mis(out_bf16, 16) ||
        mis(out_fp8, 8))
        return FRT_ERR_INVALID;
    if (rows == 0) return FRT_OK;
    const unsigned threads = ((dim / 8 + 31) / 32) * 32;
    auto X = (const __nv_bfloat16*)x;
    auto W = (const __nv_bfloat16*)weight;
    auto B = (const __nv_bfloat16*)bias;
    auto SC = (const __nv_bfloat16*)scale;
    auto SH = (const __nv_bfloat16*)shift;
    if (out_fp8)
        return launch_k(layer_norm_row_kernel<true>, rows, threads, (cudaStream_t)stream, flags & 1, X, W, B, SC, SH,
                        mod_stride, out_fp8, d_scale, dim, eps);
    return launch_k(layer_norm_row_kernel<false>, rows, threads, (cudaStream_t)stream, flags & 1, X, W, B, SC, SH,
                    mod_stride, out_bf16, d_scale, dim, eps);
}

// packed_qkv (B*L, 3*dim) bf16, dim = N * D_h; q_out / k_out (B*L, dim); freqs (seq_len.., D_h/2) fp32.
int frt_b200_qkv_split_norm_rope(const void* packed_qkv, const void* norm_q_w, const void* norm_k_w,
                                 const float* freqs_re, const float* freqs_im, void* q_out, void* k_out, int B, int L,
                                 int N, int D_h, int seq_len, float eps, const float* ext_ssq_q,
                                 const float* ext_ssq_k, int full_dim, int flags, void* stream) {
    if (!packed_qkv || !norm_q_w || !norm_k_w || !freqs_re || !freqs_im || !q_out || !k_out) return FRT_ERR_INVALID;
    if (B < 0 || L <= 0 || N <= 0 || D_h <= 0) return FRT_ERR_INVALID;
    const long long dim = (long long)N * D_h;
    if ((D_h & 7) || dim > 8192) return FRT_ERR_UNSUPPORTED;
    if (mis(packed_qkv, 16) || mis(norm_q_w, 16) || mis(norm_k_w, 16) || mis(freqs_re, 16) || mis(freqs_im, 16) ||
        mis(q_out, 16) || mis(k_out, 16))
        return FRT_ERR_INVALID;
    if (B == 0) return FRT_OK;
    const unsigned threads = (unsigned)(((dim / 8 + 31) / 32) * 32);
    return launch_k(qkv_split_norm_rope_kernel, (unsigned)(B * L), threads, (cudaStream_t)stream, flags & 1,
                    (const __nv_bfloat16*)packed_qkv, (const __nv_bfloat16*)norm_q_w, (const __nv_bfloat16*)norm_k_w,
                    freqs_re, freqs_im, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_out, L, (int)dim, D_h, seq_len, eps,
                    (ext_ssq_q && ext_ssq_k) ? ext_ssq_q : (const float*)nullptr,
                    (ext_ssq_q && ext_ssq_k) ? ext_ssq_k : (const float*)nullptr,
                    (ext_ssq_q && ext_ssq_k && full_dim > 0) ? full_dim : (int)dim);
}

// out[r] = sum_c x[r, col0 + c]^2 over ncols columns (fp32); x rows are row_stride elements apart.  ncols % 8 == 0.
int frt_b200_row_sumsq(const void* x, long long row_stride, int col0, int ncols, float* out, long long rows, int flags,
                       void* stream) {
    if (!x || !out || rows < 0 || ncols <= 0 || col0 < 0) return FRT_ERR_INVALID;
    if ((ncols & 7) || (col0 & 7) || (row_stride & 7) || mis(x, 16)) return FRT_ERR_UNSUPPORTED;
    if (rows == 0) return FRT_OK;
    return launch_k(row_sumsq_kernel, (unsigned)((rows + 7) / 8), 256, (cudaStream_t)stream, flags & 1,
                    (const __nv_bfloat16*)x, row_stride, col0, ncols, out, rows);
}

// out[r, 0:dim] = bf16(x[r, 0:dim] * rsqrt(ssq[r] / full_dim + eps) * weight[0:dim]); row pitches in elements.
int frt_b200_rms_norm_ext(const void* x, long long x_stride, const void* weight, const float* ssq, void* out,
                          long long out_stride, long long rows, int dim, int full_dim, float eps, int flags,
                          void* stream) {
    if (!x || !weight || !ssq || !out || rows < 0 || dim <= 0 || full_dim <= 0) return FRT_ERR_INVALID;
    if ((dim & 7) || (x_stride & 7) || (out_stride & 7) || mis(x, 16) || mis(weight, 16) || mis(out, 16))
        return FRT_ERR_UNSUPPORTED;
    if (rows == 0) return FRT_OK;
    return launch_k(rms_norm_ext_kernel, cap_grid(rows * (dim >> 3), 256), 256, (cudaStream_t)stream, flags & 1,
                    (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)weight, ssq, (__nv_bfloat16*)out,
                    out_stride, rows, dim, full_dim, eps);
}

// out (M, N) e4m3 = clamp(gelu_tanh(in + bias) * (1 / *d_scale)); bias (N,) or NULL.
int frt_b200_bias_gelu_quantize_fp8(const void* in_bf16, const void* bias, void* out_fp8, const float* d_scale,
                                    long long M, int N, int flags, void* stream) {
    if (!in_bf16 || !out_fp8 || !d_scale || M < 0 || N <= 0) return FRT_ERR_INVALID;
    if ((N & 7) || mis(in_bf16, 16) || mis(bias, 16) || mis(out_fp8, 8)) return FRT_ERR_UNSUPPORTED;
    if (M == 0) return FRT_OK;
    return launch_k(bias_gelu_fp8_kernel, cap_grid(M * (N >> 3), 256), 256, (cudaStream_t)stream, flags & 1,
                    (const __nv_bfloat16*)in_bf16, (const __nv_bfloat16*)bias, (uint8_t*)out_fp8, d_scale, M, N);
}

// residual (rows, dim) += (x + bias) * gate; gate rows at + r * gate_stride (0 = shared row); bias (dim,) or NULL.
int frt_b200_bias_gate_mul_residual(void* residual, const void* x, const void* bias, const void* gate,
                                    long long gate_stride, long long rows, int dim, int flags, void* stream) {
    if (!residual || !x || !gate || rows < 0 || dim <= 0) return FRT_ERR_INVALID;
    if ((dim & 7) || (gate_stride & 7) || mis(residual, 16) || mis(x, 16) || mis(bias, 16) || mis(gate, 16))
        return FRT_ERR_UNSUPPORTED;
    if (rows == 0) return FRT_OK;
    return launch_k(bias_gate_res_kernel<0>, cap_grid(rows * (dim >> 3), 256), 256, (cudaStream_t)stream, flags & 1,
                    (__nv_bfloat16*)residual, (const __nv_bfloat16*)x, (const __nv_bfloat16*)bias,
                    (const __nv_bfloat16*)gate, gate_stride, rows, dim);
}

// x (rows, dim) += bias (dim,)
int frt_b200_add_bias(void* x, const void* bias, long long rows, int dim, int flags, void* stream) {
    if (!x || !bias || rows < 0 || dim <= 0) return FRT_ERR_INVALID;
    if ((dim & 7) || mis(x, 16) || mis(bias, 16)) return FRT_ERR_UNSUPPORTED;
    if (rows == 0) return FRT_OK;
    return launch_k(bias_gate_res_kernel<1>, cap_grid(rows * (dim >> 3), 256), 256, (cudaStream_t)stream, flags & 1,
                    (__nv_bfloat16*)x, (const __nv_bfloat16*)nullptr, (const __nv_bfloat16*)bias,
                    (const __nv_bfloat16*)nullptr, 0LL, rows, dim);
}

// out_j (B, S, D) bf16 = adaln_params (B, S, 6, D) fp32 [:, :, j] + layer_modulation (6, D) fp32 [j]
int frt_b200_adaln_modulation6(const float* adaln_params, const float* layer_modulation, void* out0, void* out1,
                               void* out2, void* out3, void* out4, void* out5, int B, int S, int D, int flags,
                               void* stream) {
    if (!adaln_params || !layer_modulation || !out0 || !out1 || !out2 || !out3 || !out4 || !out5) return FRT_ERR_INVALID;
    if (B < 0 || S < 0 || D <= 0) return FRT_ERR_INVALID;
    const long long n = (long long)B * S * D;
    if (n == 0) return FRT_OK;
    return launch_k(modulation6_kernel, cap_grid(n, 256), 256, (cudaStream_t)stream, flags & 1, adaln_params,
                    layer_modulation, (__nv_bfloat16*)out0, (__nv_bfloat16*)out1, (__nv_bfloat16*)out2,
                    (__nv_bfloat16*)out3, (__nv_bfloat16*)out4, (__nv_bfloat16*)out5, D, n);
}

}  // extern "C"
