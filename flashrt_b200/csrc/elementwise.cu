// Elementwise kernels of the denoise path: GeGLU -> FP8, bf16 -> FP8 quantise
// (static / device-computed scale), scale max-accumulate, residual / bias /
// gated adds, fused RoPE + QKV split with KV-cache append.
//
// Replaces, for sm_100a, the reference kernels
//   gate_silu_mul_merged_fp8     csrc/kernels/activation.cu:249-279   (binding gate_geglu_merged_fp8)
//   quantize_fp8_static/_device  csrc/kernels/quantize.cu:61-75,131-156,297-311
//   fp8_accumulate_scale_max     csrc/kernels/quantize.cu:137-146
//   residual_add / bias_residual / gate_mul_residual   csrc/kernels/elementwise.cu:34,207,302
//   qkv_split_rope[_devpos]      csrc/kernels/rope.cu:135-277
//   cfg_combine_into_residual    csrc/kernels/elementwise.cu:2299-2338
//
// All kernels move 16 bytes per thread per access, fully coalesced, and use a
// grid-stride loop over a grid capped at a multiple of the SM count.
#include "common.cuh"

namespace frt {

static int g_sm_count = 0;
static int sm_count() {
    if (g_sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}
static inline unsigned grid_for(long long work_items, int threads, int ctas_per_sm) {
    long long need = (work_items + threads - 1) / threads;
    long long cap = (long long)sm_count() * ctas_per_sm;
    if (need < 1) need = 1;
    return (unsigned)(need < cap ? need : cap);
}

template <typename K, typename... Args>
static int launch(K kernel, unsigned grid, unsigned block, cudaStream_t stream, bool pdl, Args... args) {
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

// ------------------------------------------------------------------ GeGLU -> FP8
// merged row = [gate(0..H) | up(H..2H)] bf16; out (rows, H) fp8.
template <int ACT>
__global__ void __launch_bounds__(256)
geglu_fp8_kernel(const __nv_bfloat16* __restrict__ merged, uint8_t* __restrict__ out, int rows, int H,
                 const float* __restrict__ d_scale) {
    const float inv_scale = __fdiv_rn(1.0f, *d_scale);
    pdl_wait();
    const int vec_per_row = H >> 3;
    const long long total = (long long)rows * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / vec_per_row;
        const int col = (int)(i - row * vec_per_row) << 3;
        const __nv_bfloat16* g = merged + row * 2 * H + col;
        uint4 gv = ld_stream_v4(g);
        uint4 uv = ld_stream_v4(g + H);
        const uint32_t* gw = &gv.x;
        const uint32_t* uw = &uv.x;
        float o[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float g0, g1, u0, u1;
            unpack_bf16x2(gw[k], g0, g1);
            unpack_bf16x2(uw[k], u0, u1);
            o[2 * k] = clamp448(__fmul_rn(__fmul_rn(det_gate_act<ACT>(g0), u0), inv_scale));
            o[2 * k + 1] = clamp448(__fmul_rn(__fmul_rn(det_gate_act<ACT>(g1), u1), inv_scale));
        }
        uint2 ov;
        ov.x = f32x4_to_e4m3x4(o[0], o[1], o[2], o[3]);
        ov.y = f32x4_to_e4m3x4(o[4], o[5], o[6], o[7]);
        st_global_v2(out + row * H + col, ov);
    }
    pdl_launch_dependents();
}

// merged -> bf16 (non-quantised sibling, reference gate_geglu_merged)
template <int ACT>
__global__ void __launch_bounds__(256)
geglu_bf16_kernel(const __nv_bfloat16* __restrict__ merged, __nv_bfloat16* __restrict__ out, int rows, int H) {
    pdl_wait();
    const int vec_per_row = H >> 3;
    const long long total = (long long)rows * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / vec_per_row;
        const int col = (int)(i - row * vec_per_row) << 3;
        const __nv_bfloat16* g = merged + row * 2 * H + col;
        uint4 gv = ld_stream_v4(g);
        uint4 uv = ld_stream_v4(g + H);
        const uint32_t* gw = &gv.x;
        const uint32_t* uw = &uv.x;
        uint4 ov;
        uint32_t* ow = &ov.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float g0, g1, u0, u1;
            unpack_bf16x2(gw[k], g0, g1);
            unpack_bf16x2(uw[k], u0, u1);
            ow[k] = pack_bf16x2(__fmul_rn(det_gate_act<ACT>(g0), u0), __fmul_rn(det_gate_act<ACT>(g1), u1));
        }
        st_global_v4(out + row * H + col, ov);
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------ bf16 -> FP8, given scale
__global__ void __launch_bounds__(256)
quantize_fp8_kernel(const __nv_bfloat16* __restrict__ in, uint8_t* __restrict__ out, long long n,
                    const float* __restrict__ d_scale) {
    const float inv_scale = __fdiv_rn(1.0f, *d_scale);
    pdl_wait();
    const long long nvec = n >> 3;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        uint4 v = ld_stream_v4(in + i * 8);
        const uint32_t* w = &v.x;
        float f[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            unpack_bf16x2(w[k], f[2 * k], f[2 * k + 1]);
            f[2 * k] = clamp448(__fmul_rn(f[2 * k], inv_scale));
            f[2 * k + 1] = clamp448(__fmul_rn(f[2 * k + 1], inv_scale));
        }
        uint2 ov;
        ov.x = f32x4_to_e4m3x4(f[0], f[1], f[2], f[3]);
        ov.y = f32x4_to_e4m3x4(f[4], f[5], f[6], f[7]);
        st_global_v2(out + i * 8, ov);
    }
    // ragged tail (n not a multiple of 8): one thread, scalar
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        for (long long j = nvec << 3; j < n; ++j) {
            float f = clamp448(__fmul_rn(__bfloat162float(in[j]), inv_scale));
            out[j] = (uint8_t)(f32x2_to_e4m3x2(f, 0.0f) & 0xff);
        }
    }
    pdl_launch_dependents();
}

// absmax into *d_amax (float, non-negative: ordered as int)
__global__ void __launch_bounds__(256)
absmax_kernel(const __nv_bfloat16* __restrict__ in, long long n, float* d_amax) {
    float m = 0.0f;
    const long long nvec = n >> 3;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
         i += (long long)gridDim.x * blockDim.x) {
        uint4 v = ld_global_v4(in + i * 8);
        const uint32_t* w = &v.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float a, b;
            unpack_bf16x2(w[k], a, b);
            m = fmaxf(m, fmaxf(fabsf(a), fabsf(b)));
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (long long j = nvec << 3; j < n; ++j) m = fmaxf(m, fabsf(__bfloat162float(in[j])));
    m = warp_max_butterfly(m);
    if ((threadIdx.x & 31) == 0) atomicMax(reinterpret_cast<int*>(d_amax), __float_as_int(m));
}

// scale = max(amax / 448, 1e-12), in place
__global__ void amax_to_scale_kernel(float* d_scale) {
    float s = __fdiv_rn(*d_scale, 448.0f);
    *d_scale = s < 1e-12f ? 1e-12f : s;
}

__global__ void accumulate_scale_max_kernel(const float* src, float* dst) {
    atomicMax(reinterpret_cast<int*>(dst), __float_as_int(*src));
}

// ------------------------------------------------------------------ residual-style adds
// MODE 0: res += x            MODE 1: res += x + bias[col]      MODE 2: res += x * gate
template <int MODE>
__global__ void __launch_bounds__(256)
add_kernel(__nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ x,
           const __nv_bfloat16* __restrict__ aux, long long aux_stride, long long rows, int dim) {
    pdl_wait();
    const int vec_per_row = dim >> 3;
    const long long total = rows * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / vec_per_row;
        const int col = (int)(i - row * vec_per_row) << 3;
        uint4 rv = ld_global_v4(res + i * 8);
        uint4 xv = ld_stream_v4(x + i * 8);
        uint4 av = make_uint4(0, 0, 0, 0);
        if (MODE == 1) av = ld_global_v4(aux + col);
        if (MODE == 2) av = ld_global_v4(aux + row * aux_stride + col);
        const uint32_t* rw = &rv.x;
        const uint32_t* xw = &xv.x;
        const uint32_t* aw = &av.x;
        uint4 ov;
        uint32_t* ow = &ov.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float r0, r1, x0, x1, a0, a1;
            unpack_bf16x2(rw[k], r0, r1);
            unpack_bf16x2(xw[k], x0, x1);
            unpack_bf16x2(aw[k], a0, a1);
            if (MODE == 0) {
                r0 = __fadd_rn(r0, x0);
                r1 = __fadd_rn(r1, x1);
            } else if (MODE == 1) {
                r0 = __fadd_rn(__fadd_rn(r0, x0), a0);
                r1 = __fadd_rn(__fadd_rn(r1, x1), a1);
            } else {
                r0 = __fmaf_rn(x0, a0, r0);
                r1 = __fmaf_rn(x1, a1, r1);
            }
            ow[k] = pack_bf16x2(r0, r1);
        }
        st_global_v4(res + i * 8, ov);
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------ RoPE + QKV split + KV append
// qkv row = [q (q_dim) | k (k_dim) | v (v_dim)] bf16.  Rotation acts on adjacent
// pairs (2i, 2i+1) with table row [cos0, sin0, cos1, sin1, ...] (head_dim bf16).
// Q goes to (seq, q_dim); K and V rows land at row (pos + t) of their caches,
// pos = *devpos when devpos is given, else 0 (the caller pre-offsets K/V).
__global__ void __launch_bounds__(256)
qkv_split_rope_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ rope,
                      __nv_bfloat16* __restrict__ Q, __nv_bfloat16* __restrict__ K,
                      __nv_bfloat16* __restrict__ V, const int* __restrict__ devpos, int seq, int q_dim,
                      int k_dim, int v_dim, int head_dim) {
    const int pos = devpos ? *devpos : 0;
    pdl_wait();
    const int row_w = q_dim + k_dim + v_dim;
    const int vec_per_row = row_w >> 3;
    const long long total = (long long)seq * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / vec_per_row);
        const int col = (int)(i - (long long)row * vec_per_row) << 3;
        uint4 v = ld_stream_v4(qkv + (long long)row * row_w + col);
        if (col >= q_dim + k_dim) {
            st_global_v4(V + (long long)(pos + row) * v_dim + (col - q_dim - k_dim), v);
            continue;
        }
        const bool is_q = col < q_dim;
        const int c = is_q ? col : col - q_dim;
        const int d = c % head_dim;                       // offset inside the head, multiple of 8
        uint4 t = ld_global_v4(rope + (long long)row * head_dim + d);
        const uint32_t* xw = &v.x;
        const uint32_t* tw = &t.x;
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float x0, x1, cs, sn;
            unpack_bf16x2(xw[k], x0, x1);
            unpack_bf16x2(tw[k], cs, sn);
            float o0 = __fmaf_rn(x0, cs, -__fmul_rn(x1, sn));
            float o1 = __fmaf_rn(x1, cs, __fmul_rn(x0, sn));
            ow[k] = pack_bf16x2(o0, o1);
        }
        if (is_q) st_global_v4(Q + (long long)row * q_dim + c, o);
        else st_global_v4(K + (long long)(pos + row) * k_dim + c, o);
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------ classifier-free guidance combine
// residual[i] += v_uncond[i] + beta * (v_cond[i] - v_uncond[i])   (one fma for the guided velocity, one add)
template <typename T>
__global__ void __launch_bounds__(256)
cfg_combine_kernel(T* __restrict__ residual, const T* __restrict__ v_cond, const T* __restrict__ v_uncond,
                   float beta, long long n) {
    pdl_wait();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float r, vc, vu;
        if constexpr (sizeof(T) == 4) {
            r = residual[i]; vc = v_cond[i]; vu = v_uncond[i];
        } else {
            r = __bfloat162float(residual[i]); vc = __bfloat162float(v_cond[i]); vu = __bfloat162float(v_uncond[i]);
        }
        const float out = __fadd_rn(r, __fmaf_rn(beta, __fsub_rn(vc, vu), vu));
        if constexpr (sizeof(T) == 4) residual[i] = out; else residual[i] = __float2bfloat16_rn(out);
    }
    pdl_launch_dependents();
}

// the three status words of the tensor-core kernels into one array (and optionally cleared), in stream order
__global__ void status_gather_kernel(int* gemm, int* attn, int* loop, int* out, int reset) {
    pdl_wait();
    if (threadIdx.x == 0) {
        out[0] = *gemm;
        out[1] = *attn;
        out[2] = *loop;
        if (reset) { *gemm = 0; *attn = 0; *loop = 0; }
    }
}

}  // namespace frt

using namespace frt;
static inline bool mis16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

extern "C" {

int frt_b200_geglu_fp8(const void* merged, void* out_fp8, int rows, int half_dim, const float* d_scale,
                       int flags, void* stream) {
    if (!merged || !out_fp8 || !d_scale || rows < 0 || half_dim <= 0) return FRT_ERR_INVALID;
    if ((half_dim & 7) || mis16(merged) || (reinterpret_cast<uintptr_t>(out_fp8) & 7)) return FRT_ERR_UNSUPPORTED;
    if (rows == 0) return FRT_OK;
    long long items = (long long)rows * (half_dim >> 3);
    if (flags & 2)      // SiLU gate (SwiGLU)
        return launch(geglu_fp8_kernel<1>, grid_for(items, 256, 8), 256, (cudaStream_t)stream, flags & 1,
                      (const __nv_bfloat16*)merged, (uint8_t*)out_fp8, rows, half_dim, d_scale);
    return launch(geglu_fp8_kernel<0>, grid_for(items, 256, 8), 256, (cudaStream_t)stream, flags & 1,
                  (const __nv_bfloat16*)merged, (uint8_t*)out_fp8, rows, half_dim, d_scale);
}

int frt_b200_geglu_bf16(const void* merged, void* out_bf16, int rows, int half_dim, int flags, void* stream) {
    if (!merged || !out_bf16 || rows < 0 || half_dim <= 0) return FRT_ERR_INVALID;
    if ((half_dim & 7) || mis16(merged) || mis16(out_bf16)) return FRT_ERR_UNSUPPORTED;
    if (rows == 0) return FRT_OK;
    long long items = (long long)rows * (half_dim >> 3);
    if (flags & 2)
        return launch(geglu_bf16_kernel<1>, grid_for(items, 256, 8), 256, (cudaStream_t)stream, flags & 1,
                      (const __nv_bfloat16*)merged, (__nv_bfloat16*)out_bf16, rows, half_dim);
    return launch(geglu_bf16_kernel<0>, grid_for(items, 256, 8), 256, (cudaStream_t)stream, flags & 1,
                  (const __nv_bfloat16*)merged, (__nv_bfloat16*)out_bf16, rows, half_dim);
}

int frt_b200_quantize_fp8_static(const void* in_bf16, void* out_fp8, const float* d_scale, long long n,
                                 int flags, void* stream) {
    if (!in_bf16 || !out_fp8 || !d_scale || n < 0) return FRT_ERR_INVALID;
    if (mis16(in_bf16) || (reinterpret_cast<uintptr_t>(out_fp8) & 7)) return FRT_ERR_UNSUPPORTED;
    if (n == 0) return FRT_OK;
    return launch(quantize_fp8_kernel, grid_for((n + 7) >> 3, 256, 8), 256, (cudaStream_t)stream, flags & 1,
                  (const __nv_bfloat16*)in_bf16, (uint8_t*)out_fp8, n, d_scale);
}

// scale = max(absmax(in)/448, 1e-12) written to *d_scale, then quantise with it.
int frt_b200_quantize_fp8_device(const void* in_bf16, void* out_fp8, float* d_scale, long long n, void* stream) {
    if (!in_bf16 || !out_fp8 || !d_scale || n < 0) return FRT_ERR_INVALID;
    if (mis16(in_bf16) || (reinterpret_cast<uintptr_t>(out_fp8) & 7)) return FRT_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(d_scale, 0, sizeof(float), s);
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    if (n > 0) {
        absmax_kernel<<<grid_for((n + 7) >> 3, 256, 4), 256, 0, s>>>((const __nv_bfloat16*)in_bf16, n, d_scale);
        FRT_CHECK_LAUNCH();
    }
    amax_to_scale_kernel<<<1, 1, 0, s>>>(d_scale);
    FRT_CHECK_LAUNCH();
    if (n == 0) return FRT_OK;
    return frt_b200_quantize_fp8_static(in_bf16, out_fp8, d_scale, n, 0, stream);
}

int frt_b200_fp8_accumulate_scale_max(const float* src_scale, float* dst_scale, void* stream) {
    if (!src_scale || !dst_scale) return FRT_ERR_INVALID;
    accumulate_scale_max_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(src_scale, dst_scale);
    FRT_CHECK_LAUNCH();
    return FRT_OK;
}

int frt_b200_residual_add(void* residual, const void* x, long long n, int flags, void* stream) {
    if (!residual || !x || n < 0) return FRT_ERR_INVALID;
    if ((n & 7) || mis16(residual) || mis16(x)) return FRT_ERR_UNSUPPORTED;
    if (n == 0) return FRT_OK;
    return launch(add_kernel<0>, grid_for(n >> 3, 256, 8), 256, (cudaStream_t)stream, flags & 1,
                  (__nv_bfloat16*)residual, (const __nv_bfloat16*)x, (const __nv_bfloat16*)nullptr, 0LL,
                  (long long)1, (int)n);
}

int frt_b200_bias_residual(void* residual, const void* x, const void* bias, int rows, int dim, int flags,
                           void* stream) {
    if (!residual || !x || !bias || rows < 0 || dim <= 0) return FRT_ERR_INVALID;
    if ((dim & 7) || mis16(residual) || mis16(x) || mis16(bias)) return FRT_ERR_UNSUPPORTED;
    if (rows == 0) return FRT_OK;
    return launch(add_kernel<1>, grid_for((long long)rows * (dim >> 3), 256, 8), 256, (cudaStream_t)stream,
                  flags & 1, (__nv_bfloat16*)residual, (const __nv_bfloat16*)x, (const __nv_bfloat16*)bias, 0LL,
                  (long long)rows, dim);
}

int frt_b200_gate_mul_residual(void* residual, const void* x, const void* gate, long long gate_stride, int rows,
                               int dim, int flags, void* stream) {
    if (!residual || !x || !gate || rows < 0 || dim <= 0) return FRT_ERR_INVALID;
    if ((dim & 7) || (gate_stride & 7) || mis16(residual) || mis16(x) || mis16(gate)) return FRT_ERR_UNSUPPORTED;
    if (rows == 0) return FRT_OK;
    return launch(add_kernel<2>, grid_for((long long)rows * (dim >> 3), 256, 8), 256, (cudaStream_t)stream,
                  flags & 1, (__nv_bfloat16*)residual, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gate,
                  gate_stride, (long long)rows, dim);
}

int frt_b200_qkv_split_rope(const void* qkv, const void* rope, void* Q, void* K, void* V, const int* devpos,
                            int seq, int q_dim, int k_dim, int v_dim, int head_dim, int flags, void* stream) {
    if (!qkv || !rope || !Q || !K || !V || seq < 0) return FRT_ERR_INVALID;
    if (q_dim <= 0 || k_dim <= 0 || v_dim <= 0 || head_dim <= 0) return FRT_ERR_INVALID;
    if ((q_dim & 7) || (k_dim & 7) || (v_dim & 7) || (head_dim & 7) || (q_dim % head_dim) || (k_dim % head_dim))
        return FRT_ERR_UNSUPPORTED;
    if (mis16(qkv) || mis16(rope) || mis16(Q) || mis16(K) || mis16(V)) return FRT_ERR_UNSUPPORTED;
    if (seq == 0) return FRT_OK;
    long long items = (long long)seq * ((q_dim + k_dim + v_dim) >> 3);
    return launch(qkv_split_rope_kernel, grid_for(items, 256, 8), 256, (cudaStream_t)stream, flags & 1,
                  (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)rope, (__nv_bfloat16*)Q, (__nv_bfloat16*)K,
                  (__nv_bfloat16*)V, devpos, seq, q_dim, k_dim, v_dim, head_dim);
}

// residual <- residual + (v_uncond + beta * (v_cond - v_uncond)), n elements; F32 = 1: all three arrays fp32 (the
// Euler state of this library), else bf16 as in the reference.  n % 2 == 0 as there.
int frt_b200_cfg_combine_into_residual(void* residual, const void* v_cond, const void* v_uncond, float beta,
                                       long long n, int f32, int flags, void* stream) {
    if (!residual || !v_cond || !v_uncond || n < 0) return FRT_ERR_INVALID;
    if (n & 1) return FRT_ERR_UNSUPPORTED;
    if (n == 0) return FRT_OK;
    if (f32)
        return launch(cfg_combine_kernel<float>, grid_for(n, 256, 8), 256, (cudaStream_t)stream, flags & 1,
                      (float*)residual, (const float*)v_cond, (const float*)v_uncond, beta, n);
    return launch(cfg_combine_kernel<__nv_bfloat16>, grid_for(n, 256, 8), 256, (cudaStream_t)stream, flags & 1,
                  (__nv_bfloat16*)residual, (const __nv_bfloat16*)v_cond, (const __nv_bfloat16*)v_uncond, beta, n);
}

// Status words of the GEMM, attention and one-launch loop kernels -> out3[0..2] (device ints), as a kernel in stream
// order: capturable, so a graph can hand the words back together with its results and the host needs no blocking
// status call after every replay.  reset != 0 clears the words after copying them.
int frt_b200_status_words_async(int* out3, int reset, int flags, void* stream) {
    if (!out3) return FRT_ERR_INVALID;
    static int* ptrs[64][3] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    if (dev < 0 || dev >= 64) return FRT_ERR_UNSUPPORTED;
    if (!ptrs[dev][2]) {       // idempotent: concurrent first calls write the same addresses
        int* a = gemm_status_device_ptr();
        int* b = attention_status_device_ptr();
        int* c = expert_loop_status_device_ptr();
        if (!a || !b || !c) return FRT_ERR_INVALID;
        ptrs[dev][0] = a; ptrs[dev][1] = b; ptrs[dev][2] = c;
    }
    return launch(status_gather_kernel, 1, 32, (cudaStream_t)stream, flags & 1, ptrs[dev][0], ptrs[dev][1], ptrs[dev][2],
                  out3, reset);
}

int frt_b200_device_sm_count(void) { return sm_count(); }

}  // extern "C"
