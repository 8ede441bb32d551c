// Small helpers of the denoise path that are not bandwidth- or tensor-bound:
// the 32 <-> 1024 action projections (bf16, K or N = 32), device copies, device
// queries.
//
// Replaces, for sm_100a, the reference entry points
//   GemmRunner::bf16_nn          csrc/bindings.cpp:662-667 (cuBLASLt) for the action in/out projections
//   gpu_copy                     csrc/bindings.cpp:2533-2537
//   get_sm_version               csrc/bindings.cpp:2447-2453
#include "common.cuh"

namespace frt {

// D(M,N) bf16 = A(M,K) . B(K,N) (+ bias(N)) (+ D when accumulate), bf16 operands, fp32 accumulate.
// Block: 32 output columns x 16 K-slices, 2 output rows.  The projections this
// serves move < 100 KB; the shape of the grid only has to cover the machine.
constexpr int SG_COLS = 32, SG_KS = 16, SG_ROWS = 2, SG_KCHUNK = 1024;

template <bool A_F32, bool D_F32>
__global__ void __launch_bounds__(SG_COLS * SG_KS)
small_gemm_bf16_kernel(const void* __restrict__ Av, const __nv_bfloat16* __restrict__ B,
                       void* __restrict__ Dv, const __nv_bfloat16* __restrict__ bias, int M, int N, int K,
                       int accumulate) {
    const __nv_bfloat16* A = reinterpret_cast<const __nv_bfloat16*>(Av);
    const float* Af = reinterpret_cast<const float*>(Av);
    __nv_bfloat16* D = reinterpret_cast<__nv_bfloat16*>(Dv);
    float* Df = reinterpret_cast<float*>(Dv);
    __shared__ float a_s[SG_ROWS][SG_KCHUNK];
    __shared__ float part[SG_KS][SG_ROWS][SG_COLS];
    const int tx = threadIdx.x % SG_COLS;
    const int ks = threadIdx.x / SG_COLS;
    const int n = blockIdx.x * SG_COLS + tx;
    const int m0 = blockIdx.y * SG_ROWS;
    pdl_launch_dependents();     // the dependent kernel still waits for this grid to complete
    pdl_wait();
    float acc[SG_ROWS] = {};
    for (int k0 = 0; k0 < K; k0 += SG_KCHUNK) {
        const int kc = K - k0 < SG_KCHUNK ? K - k0 : SG_KCHUNK;
        __syncthreads();
        for (int i = threadIdx.x; i < SG_ROWS * kc; i += blockDim.x) {
            const int r = i / kc, k = i - r * kc;
            const size_t ai = (size_t)(m0 + r) * K + k0 + k;
            // an fp32 operand is rounded to bf16 first: the projection multiplies bf16 by bf16
            a_s[r][k] = (m0 + r < M) ? (A_F32 ? __bfloat162float(__float2bfloat16_rn(Af[ai])) : __bfloat162float(A[ai]))
                                     : 0.0f;
        }
        __syncthreads();
        if (n < N) {
            // the loads of B do not depend on one another: keep 16 of them in flight per thread
#pragma unroll 16
            for (int k = ks; k < kc; k += SG_KS) {
                const float b = __bfloat162float(B[(size_t)(k0 + k) * N + n]);
#pragma unroll
                for (int r = 0; r < SG_ROWS; ++r) acc[r] = fmaf(a_s[r][k], b, acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < SG_ROWS; ++r) part[ks][r][tx] = acc[r];
    __syncthreads();
    if (ks < SG_ROWS && n < N && m0 + ks < M) {
        const int r = ks;
        float s = 0.0f;
#pragma unroll
        for (int q = 0; q < SG_KS; ++q) s += part[q][r][tx];
        if (bias) s += __bfloat162float(bias[n]);
        const size_t o = (size_t)(m0 + r) * N + n;
        if (D_F32) {
            if (accumulate) s += Df[o];
            Df[o] = s;
        } else {
            if (accumulate) s += __bfloat162float(D[o]);
            D[o] = __float2bfloat16_rn(s);
        }
    }
}

// ------------------------------------------------------------------ boundary between two Euler steps, one launch
// Per token (one CTA, dim / 8 threads, 8 features each -- the layout of norm_row_kernel):
//   [has_prev]  xn = bf16(adaRMS(x; style_prev))                      final norm of the step that ends
//               noise += xn . W_out + b_out                            action out-projection (pre-scaled by dt) + Euler
//   [has_next]  x = bf16(bf16(noise) . W_in + b_in)                    action in-projection of the step that begins
//               act8 = e4m3(adaRMS(x; style_next) / *scale)            first norm of layer 0
// Every sum is formed in the order of the kernels this replaces (norm_row_kernel: 8-element fma chain, xor butterfly,
// warp totals in order; small_gemm_bf16_kernel: 16 interleaved K-slices, partials added in slice order, then bias, then
// the old value), so the results are theirs bit for bit.  ACTION = 32 columns of the action space.
constexpr int SB_ACTION = 32;

__device__ __forceinline__ float sb_block_rms(float ssq, float* warp_tot, int dim, float eps) {
    ssq = warp_sum_butterfly(ssq);
    const int nwarps = blockDim.x >> 5;
    __syncthreads();                                    // warp_tot may still be read from the previous use
    if ((threadIdx.x & 31) == 0) warp_tot[threadIdx.x >> 5] = ssq;
    __syncthreads();
    float tot = warp_tot[0];
    for (int w = 1; w < nwarps; ++w) tot = __fadd_rn(tot, warp_tot[w]);
    const float var = __fadd_rn(__fdiv_rn(tot, (float)dim), eps);
    return __fdiv_rn(1.0f, __fsqrt_rn(var));
}

__global__ void __launch_bounds__(256)
step_boundary_kernel(__nv_bfloat16* __restrict__ x, float* __restrict__ noise, const __nv_bfloat16* __restrict__ style_prev,
                     const __nv_bfloat16* __restrict__ w_out, const __nv_bfloat16* __restrict__ b_out,
                     const __nv_bfloat16* __restrict__ w_in, const __nv_bfloat16* __restrict__ b_in,
                     const __nv_bfloat16* __restrict__ style_next, uint8_t* __restrict__ act8,
                     const float* __restrict__ d_scale, int dim, float eps) {
    extern __shared__ float sb_smem[];
    float* a_s = sb_smem;                               // [dim] normalised row (bf16 values)
    float* part = a_s + dim;                            // [16][32] K-slice partials of the out-projection
    float* nz = part + 16 * SB_ACTION;                  // [32] action row, fp32
    float* warp_tot = nz + SB_ACTION;                   // [32]
    __nv_bfloat16* w_s = reinterpret_cast<__nv_bfloat16*>(warp_tot + 32);   // [dim][32] out-projection weights
    const int t = blockIdx.x, tid = threadIdx.x, col = tid * 8;
    const size_t roff = (size_t)t * dim + col;
    pdl_launch_dependents();
    if (style_prev) {
        // the out-projection weights do not depend on the kernel in front: all 16-byte loads in flight, into shared memory
        const uint4* src = reinterpret_cast<const uint4*>(w_out);
        uint4* dst = reinterpret_cast<uint4*>(w_s);
        for (int i = tid; i < dim * SB_ACTION / 8; i += blockDim.x) dst[i] = src[i];
    }
    // so do this thread's 8 columns of the in-projection weights (32 rows), held in registers across the first half
    uint4 wrow[SB_ACTION];
    if (style_next) {
#pragma unroll
        for (int k = 0; k < SB_ACTION; ++k) wrow[k] = ld_global_v4(w_in + (size_t)k * dim + col);
    }
    pdl_wait();
    if (style_prev) {
        const uint4 rv = ld_global_v4(x + roff);
        const uint4 sc = ld_global_v4(style_prev + col), sh = ld_global_v4(style_prev + dim + col);
        const uint32_t* rw = &rv.x;
        float r[8], ssq = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            unpack_bf16x2(rw[i], r[2 * i], r[2 * i + 1]);
            ssq = __fmaf_rn(r[2 * i], r[2 * i], ssq);
            ssq = __fmaf_rn(r[2 * i + 1], r[2 * i + 1], ssq);
        }
        const float rms = sb_block_rms(ssq, warp_tot, dim, eps);
        const uint32_t* scw = &sc.x;
        const uint32_t* shw = &sh.x;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float s0, s1, h0, h1;
            unpack_bf16x2(scw[i], s0, s1);
            unpack_bf16x2(shw[i], h0, h1);
            const float n0 = __fmaf_rn(__fmul_rn(__fmul_rn(r[2 * i], rms), 1.0f), __fadd_rn(1.0f, s0), h0);
            const float n1 = __fmaf_rn(__fmul_rn(__fmul_rn(r[2 * i + 1], rms), 1.0f), __fadd_rn(1.0f, s1), h1);
            a_s[col + 2 * i] = __bfloat162float(__float2bfloat16_rn(n0));
            a_s[col + 2 * i + 1] = __bfloat162float(__float2bfloat16_rn(n1));
        }
        __syncthreads();
        // out-projection: column n, K-slices ks = k mod 16; thread (n, g) forms the slices g, g + groups, ...
        const int n = tid % SB_ACTION, g = tid / SB_ACTION, groups = blockDim.x / SB_ACTION;
        for (int ks = g; ks < 16; ks += groups) {
            float acc = 0.0f;
#pragma unroll 8
            for (int k = ks; k < dim; k += 16) acc = fmaf(a_s[k], __bfloat162float(w_s[k * SB_ACTION + n]), acc);
            part[ks * SB_ACTION + n] = acc;
        }
        __syncthreads();
        if (tid < SB_ACTION) {
            float s = 0.0f;
#pragma unroll
            for (int q = 0; q < 16; ++q) s += part[q * SB_ACTION + tid];
            if (b_out) s += __bfloat162float(b_out[tid]);
            s += noise[(size_t)t * SB_ACTION + tid];
            noise[(size_t)t * SB_ACTION + tid] = s;
            nz[tid] = s;
        }
    } else if (tid < SB_ACTION) {
        nz[tid] = noise[(size_t)t * SB_ACTION + tid];
    }
    if (!style_next) return;
    __syncthreads();
    // in-projection: a = bf16(noise); 16 slices of two terms each, partials added in slice order, then the bias
    float xb[8], ssq = 0.0f;
    {
        float a[SB_ACTION];
#pragma unroll
        for (int k = 0; k < SB_ACTION; ++k) a[k] = __bfloat162float(__float2bfloat16_rn(nz[k]));
        const uint4 bv = b_in ? ld_global_v4(b_in + col) : make_uint4(0, 0, 0, 0);
        const uint32_t* bw = &bv.x;
        uint4 ov;
        uint32_t* ow = &ov.x;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float s = 0.0f;
#pragma unroll
            for (int q = 0; q < 16; ++q) {
                const uint32_t w0 = (&wrow[q].x)[j >> 1], w1 = (&wrow[q + 16].x)[j >> 1];
                float acc = fmaf(a[q], bf16_bits_to_f32((w0 >> ((j & 1) * 16)) & 0xffffu), 0.0f);
                acc = fmaf(a[q + 16], bf16_bits_to_f32((w1 >> ((j & 1) * 16)) & 0xffffu), acc);
                s += acc;
            }
            if (b_in) s += bf16_bits_to_f32((bw[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
            xb[j] = __bfloat162float(__float2bfloat16_rn(s));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            ow[i] = pack_bf16x2(xb[2 * i], xb[2 * i + 1]);
            ssq = __fmaf_rn(xb[2 * i], xb[2 * i], ssq);
            ssq = __fmaf_rn(xb[2 * i + 1], xb[2 * i + 1], ssq);
        }
        st_global_v4(x + roff, ov);
    }
    const float rms = sb_block_rms(ssq, warp_tot, dim, eps);
    const float inv_scale = __fdiv_rn(1.0f, *d_scale);
    const uint4 sc = ld_global_v4(style_next + col), sh = ld_global_v4(style_next + dim + col);
    const uint32_t* scw = &sc.x;
    const uint32_t* shw = &sh.x;
    float v[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float s0, s1, h0, h1;
        unpack_bf16x2(scw[i], s0, s1);
        unpack_bf16x2(shw[i], h0, h1);
        v[2 * i] = __fmaf_rn(__fmul_rn(__fmul_rn(xb[2 * i], rms), 1.0f), __fadd_rn(1.0f, s0), h0);
        v[2 * i + 1] = __fmaf_rn(__fmul_rn(__fmul_rn(xb[2 * i + 1], rms), 1.0f), __fadd_rn(1.0f, s1), h1);
    }
    uint2 o;
    o.x = f32x4_to_e4m3x4(clamp448(__fmul_rn(v[0], inv_scale)), clamp448(__fmul_rn(v[1], inv_scale)),
                          clamp448(__fmul_rn(v[2], inv_scale)), clamp448(__fmul_rn(v[3], inv_scale)));
    o.y = f32x4_to_e4m3x4(clamp448(__fmul_rn(v[4], inv_scale)), clamp448(__fmul_rn(v[5], inv_scale)),
                          clamp448(__fmul_rn(v[6], inv_scale)), clamp448(__fmul_rn(v[7], inv_scale)));
    st_global_v2(act8 + roff, o);
}

}  // namespace frt

using namespace frt;

extern "C" {

// io: bit0 = A is fp32 (rounded to bf16 on load), bit1 = D is fp32
int frt_b200_gemm_bf16_nn_small(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                                int accumulate, int io, int flags, void* stream) {
    if (!A || !B || !D || M < 0 || N <= 0 || K <= 0) return FRT_ERR_INVALID;
    if (M == 0) return FRT_OK;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + SG_COLS - 1) / SG_COLS, (M + SG_ROWS - 1) / SG_ROWS);
    cfg.blockDim = dim3(SG_COLS * SG_KS);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & 1) ? 1 : 0;
    const __nv_bfloat16* Bp = (const __nv_bfloat16*)B;
    const __nv_bfloat16* bp = (const __nv_bfloat16*)bias;
    cudaError_t e;
    switch (io & 3) {
        case 0: e = cudaLaunchKernelEx(&cfg, small_gemm_bf16_kernel<false, false>, A, Bp, D, bp, M, N, K, accumulate); break;
        case 1: e = cudaLaunchKernelEx(&cfg, small_gemm_bf16_kernel<true, false>, A, Bp, D, bp, M, N, K, accumulate); break;
        case 2: e = cudaLaunchKernelEx(&cfg, small_gemm_bf16_kernel<false, true>, A, Bp, D, bp, M, N, K, accumulate); break;
        default: e = cudaLaunchKernelEx(&cfg, small_gemm_bf16_kernel<true, true>, A, Bp, D, bp, M, N, K, accumulate); break;
    }
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}

// The launches between two Euler steps of the action-expert loop as one (per token: final adaRMS of the step that ends,
// action out-projection accumulated into the fp32 noise, action in-projection of the step that begins, first adaRMS ->
// FP8 of layer 0): Pi05Pipeline.transformer_decoder, flash_rt/models/pi05/pipeline_rtx.py:1451-1504 (C8 of one step and
// C0 / C1 of the next).  style_prev NULL: only the second half (first step); style_next NULL: only the first half (last
// step).  Bit for bit what frt_b200_norm_bf16 -> frt_b200_gemm_bf16_nn_small (accumulate, fp32 D) ->
// frt_b200_gemm_bf16_nn_small (fp32 A) -> frt_b200_norm_fp8 give.  action_dim == 32, dim % 256 == 0, dim <= 2048.
int frt_b200_step_boundary(void* x, float* noise, const void* style_prev, const void* w_out, const void* b_out,
                           const void* w_in, const void* b_in, const void* style_next, void* act8,
                           const float* d_act_scale, int rows, int dim, int action_dim, float eps, int flags,
                           void* stream) {
    if (!x || !noise || rows < 0 || (!style_prev && !style_next)) return FRT_ERR_INVALID;
    if (style_prev && !w_out) return FRT_ERR_INVALID;
    if (style_next && (!w_in || !act8 || !d_act_scale)) return FRT_ERR_INVALID;
    if (action_dim != SB_ACTION || dim <= 0 || (dim % 256) || dim > 2048) return FRT_ERR_UNSUPPORTED;
    const void* ptrs[] = {x, style_prev, w_in, b_in, style_next};
    for (const void* q : ptrs)
        if (reinterpret_cast<uintptr_t>(q) & 15) return FRT_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(w_out) & 15) return FRT_ERR_INVALID;
    if (reinterpret_cast<uintptr_t>(act8) & 7) return FRT_ERR_INVALID;
    if (rows == 0) return FRT_OK;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rows);
    cfg.blockDim = dim3(dim / 8);
    const size_t smem = (size_t)(dim + 16 * SB_ACTION + 2 * SB_ACTION) * sizeof(float) + (size_t)dim * SB_ACTION * 2;
    static PerDeviceOnce attr_once;
    int attr_dev = 0;
    if (attr_once.need(attr_dev)) {
        cudaError_t ea = cudaFuncSetAttribute(step_boundary_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)((2048 + 16 * SB_ACTION + 2 * SB_ACTION) * sizeof(float) + 2048 * SB_ACTION * 2));
        if (ea != cudaSuccess) return FRT_CUDA_ERR(ea);
        attr_once.set(attr_dev);
    }
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & 1) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, step_boundary_kernel, (__nv_bfloat16*)x, noise,
                                       (const __nv_bfloat16*)style_prev, (const __nv_bfloat16*)w_out,
                                       (const __nv_bfloat16*)b_out, (const __nv_bfloat16*)w_in,
                                       (const __nv_bfloat16*)b_in, (const __nv_bfloat16*)style_next, (uint8_t*)act8,
                                       d_act_scale, dim, eps);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}

int frt_b200_copy(void* dst, const void* src, long long nbytes, void* stream) {
    if (!dst || !src || nbytes < 0) return FRT_ERR_INVALID;
    if (nbytes == 0) return FRT_OK;
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)nbytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}

// compute capability as major*10 + minor (100 on B200), or a negative status
int frt_b200_sm_version(void) {
    int dev = 0, major = 0, minor = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    return major * 10 + minor;
}

}  // extern "C"
