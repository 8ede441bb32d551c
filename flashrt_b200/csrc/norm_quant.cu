// Fused (gated-)residual + RMSNorm / adaRMS modulation + FP8 E4M3 (or bf16) output.
//
// Replaces, for sm_100a, the reference kernels
//   rms_norm_fp8                 csrc/kernels/norm.cu:286-343
//   ada_rms_norm_style           csrc/kernels/norm.cu:345-389
//   ada_rms_norm_style_fp8       csrc/kernels/norm.cu:392-442
//   residual_add_rms_norm_fp8    csrc/kernels/norm.cu:445-495
//   residual_add_rms_norm        csrc/kernels/norm.cu:498-539
//   gate_residual_ada_norm_fp8   csrc/kernels/fusion.cu:15-81
//
// Design: one CTA per row, one 16-byte vector (8 bf16) per thread, so a row of
// `dim` elements uses dim/8 threads (rounded up to whole warps).  The row is
// read once and kept in registers: the residual update, its bf16 rounding, the
// sum of squares and the normalisation all happen without a second trip to
// memory.  All loads are 16-byte and coalesced; the FP8 result leaves as one
// 8-byte store per thread, the updated residual as one 16-byte store.
//
// Rounding points kept from the reference: the residual update is computed in
// fp32 and stored as bf16; the sum of squares uses the unrounded fp32 value;
// the normalisation reads the rounded bf16 value; the modulated value is not
// rounded to bf16 before the FP8 conversion; quantisation multiplies by the
// fp32 reciprocal of the scale, clamps to +-448 and converts RN-even.
//
// Reduction tree (fixed, mirrored by the C oracle): per thread a sequential
// fma chain over its 8 elements; xor-butterfly over the 32 lanes; warp totals
// summed in warp order by every thread.
#include "nvfp4.cuh"

namespace frt {

enum { OUT_BF16 = 0, OUT_E4M3 = 1, OUT_NVFP4_A = 2, OUT_NVFP4_B = 3 };

struct NormArgs {
    __nv_bfloat16* residual;       // in/out row-major (rows, dim); or input x when !HAS_X
    const __nv_bfloat16* x;        // sub-layer output to add (HAS_X)
    const __nv_bfloat16* gate_in;  // multiplies x before the add (HAS_GATE)
    long long gate_in_stride;      // elements between gate rows (0 = one shared row)
    const __nv_bfloat16* weight;   // (dim,) or null (= ones)
    const __nv_bfloat16* style;    // rows of [scale | shift | gate], 3*dim each (HAS_STYLE)
    long long style_stride;        // elements between style rows (0 = one shared row)
    void* out;                     // fp8 (rows, dim), bf16 (rows, dim) or packed e2m1 (rows, dim / 2)
    uint8_t* sf_out;               // NVFP4 block scales in the GEMM's scale-factor atoms
    __nv_bfloat16* gate_out;       // copy of the style gate chunk, or null
    const float* d_scale;          // device scalar: quantisation scale (OUT_FP8)
    int rows;
    int dim;
    float eps;
};

template <bool HAS_X, bool HAS_GATE, bool HAS_STYLE, int OUT>
__global__ void __launch_bounds__(1024)
norm_row_kernel(NormArgs a) {
    constexpr bool OUT_FP8 = OUT == OUT_E4M3;
    constexpr bool OUT_FP4 = OUT == OUT_NVFP4_A || OUT == OUT_NVFP4_B;
    __shared__ float warp_tot[32];
    const int row = blockIdx.x;
    const int tid = threadIdx.x;
    const int col = tid * 8;
    const bool active = col < a.dim;
    const size_t roff = (size_t)row * a.dim + col;

    float r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = 0.0f;
    uint4 wv = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u);
    uint4 sc = make_uint4(0, 0, 0, 0), sh = sc, gt = sc;

    // The next kernel in the stream may start its own input-independent prologue right away (it still waits for
    // this grid to finish before it touches anything this grid writes).
    pdl_launch_dependents();
    // Everything that does not depend on the producer kernel is fetched first.
    if (active) {
        if (a.weight) wv = ld_global_v4(a.weight + col);
        if (HAS_STYLE) {
            const __nv_bfloat16* srow = a.style + (size_t)row * a.style_stride;
            sc = ld_global_v4(srow + col);
            sh = ld_global_v4(srow + a.dim + col);
            if (a.gate_out) gt = ld_global_v4(srow + 2 * (size_t)a.dim + col);
        }
    }
    float inv_scale = 1.0f;
    if (OUT_FP8) inv_scale = __fdiv_rn(1.0f, *a.d_scale);

    pdl_wait();

    float ssq = 0.0f;
    uint4 rbits = make_uint4(0, 0, 0, 0);
    if (active) {
        uint4 rv = ld_global_v4(a.residual + roff);
        const uint32_t* rw = &rv.x;
        if (HAS_X) {
            uint4 xv = ld_stream_v4(a.x + roff);
            const uint32_t* xw = &xv.x;
            uint4 gv = make_uint4(0, 0, 0, 0);
            if (HAS_GATE) gv = ld_global_v4(a.gate_in + (size_t)row * a.gate_in_stride + col);
            const uint32_t* gw = &gv.x;
            uint32_t* ow = &rbits.x;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float r0, r1, x0, x1;
                unpack_bf16x2(rw[i], r0, r1);
                unpack_bf16x2(xw[i], x0, x1);
                if (HAS_GATE) {
                    float g0, g1;
                    unpack_bf16x2(gw[i], g0, g1);
                    r0 = __fmaf_rn(x0, g0, r0);
                    r1 = __fmaf_rn(x1, g1, r1);
                } else {
                    r0 = __fadd_rn(r0, x0);
                    r1 = __fadd_rn(r1, x1);
                }
                ssq = __fmaf_rn(r0, r0, ssq);
                ssq = __fmaf_rn(r1, r1, ssq);
                ow[i] = pack_bf16x2(r0, r1);
                unpack_bf16x2(ow[i], r[2 * i], r[2 * i + 1]);   // rounded value feeds the norm
            }
            st_global_v4(a.residual + roff, rbits);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                unpack_bf16x2(rw[i], r[2 * i], r[2 * i + 1]);
                ssq = __fmaf_rn(r[2 * i], r[2 * i], ssq);
                ssq = __fmaf_rn(r[2 * i + 1], r[2 * i + 1], ssq);
            }
        }
    }
    ssq = warp_sum_butterfly(ssq);
    const int nwarps = blockDim.x >> 5;
    if ((tid & 31) == 0) warp_tot[tid >> 5] = ssq;
    __syncthreads();
    float tot = warp_tot[0];
    for (int w = 1; w < nwarps; ++w) tot = __fadd_rn(tot, warp_tot[w]);
    const float var = __fadd_rn(__fdiv_rn(tot, (float)a.dim), a.eps);
    const float rms = __fdiv_rn(1.0f, __fsqrt_rn(var));

    if (!OUT_FP4 && !active) return;   // the NVFP4 path shuffles between lane pairs: every lane stays

    float v[8];
    const uint32_t* ww = &wv.x;
    const uint32_t* scw = &sc.x;
    const uint32_t* shw = &sh.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float w0, w1;
        unpack_bf16x2(ww[i], w0, w1);
        float n0 = __fmul_rn(__fmul_rn(r[2 * i], rms), w0);
        float n1 = __fmul_rn(__fmul_rn(r[2 * i + 1], rms), w1);
        if (HAS_STYLE) {
            float s0, s1, h0, h1;
            unpack_bf16x2(scw[i], s0, s1);
            unpack_bf16x2(shw[i], h0, h1);
            n0 = __fmaf_rn(n0, __fadd_rn(1.0f, s0), h0);
            n1 = __fmaf_rn(n1, __fadd_rn(1.0f, s1), h1);
        }
        v[2 * i] = n0;
        v[2 * i + 1] = n1;
    }
    if (OUT_FP4) {
        // The modulated value is rounded to bf16 (what the bf16-output kernel stores) and then quantised in
        // blocks of 16 = this thread's 8 values and its lane neighbour's; the even lane writes the scale byte.
        constexpr int FAM = OUT == OUT_NVFP4_A ? 0 : 1;
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
            amax = fmaxf(amax, fabsf(v[i]));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        float inv;
        const uint32_t sb = nvfp4::block_scale<FAM>(amax, inv);
        if (active) {
            *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(a.out) + (roff >> 1)) = nvfp4::pack8<FAM>(v, inv);
            if ((tid & 1) == 0) a.sf_out[nvfp4::sf_offset(row, col >> 4, (a.dim + 63) >> 6)] = (uint8_t)sb;
            if (HAS_STYLE && a.gate_out) st_global_v4(a.gate_out + roff, gt);
        }
        return;
    }
    if (OUT_FP8) {
        uint2 o;
        o.x = f32x4_to_e4m3x4(clamp448(__fmul_rn(v[0], inv_scale)), clamp448(__fmul_rn(v[1], inv_scale)),
                              clamp448(__fmul_rn(v[2], inv_scale)), clamp448(__fmul_rn(v[3], inv_scale)));
        o.y = f32x4_to_e4m3x4(clamp448(__fmul_rn(v[4], inv_scale)), clamp448(__fmul_rn(v[5], inv_scale)),
                              clamp448(__fmul_rn(v[6], inv_scale)), clamp448(__fmul_rn(v[7], inv_scale)));
        st_global_v2(reinterpret_cast<uint8_t*>(a.out) + roff, o);
    } else {
        uint4 o;
        o.x = pack_bf16x2(v[0], v[1]);
        o.y = pack_bf16x2(v[2], v[3]);
        o.z = pack_bf16x2(v[4], v[5]);
        o.w = pack_bf16x2(v[6], v[7]);
        st_global_v4(reinterpret_cast<__nv_bfloat16*>(a.out) + roff, o);
    }
    if (HAS_STYLE && a.gate_out) st_global_v4(a.gate_out + roff, gt);
}

template <bool HAS_X, bool HAS_GATE, bool HAS_STYLE, int OUT>
static int launch_norm(const NormArgs& a, cudaStream_t stream, bool pdl) {
    if (a.rows < 0 || a.dim <= 0 || (a.dim & 7) || a.dim > 8192) return FRT_ERR_UNSUPPORTED;
    if (a.rows == 0) return FRT_OK;
    int threads = ((a.dim / 8 + 31) / 32) * 32;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.rows);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, norm_row_kernel<HAS_X, HAS_GATE, HAS_STYLE, OUT>, a);
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    return FRT_OK;
}

}  // namespace frt

using namespace frt;

template <int OUT>
static int dispatch_norm_nvfp4(const NormArgs& a, bool has_x, bool has_gate, bool has_style, cudaStream_t s, bool pdl) {
    if (has_x) {
        if (has_gate) {
            if (has_style) return launch_norm<true, true, true, OUT>(a, s, pdl);
            return launch_norm<true, true, false, OUT>(a, s, pdl);
        }
        if (has_style) return launch_norm<true, false, true, OUT>(a, s, pdl);
        return launch_norm<true, false, false, OUT>(a, s, pdl);
    }
    if (has_style) return launch_norm<false, false, true, OUT>(a, s, pdl);
    return launch_norm<false, false, false, OUT>(a, s, pdl);
}

static inline bool misaligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

extern "C" {

// flags: bit0 = launch with programmatic stream serialization (PDL)
int frt_b200_norm_fp8(void* residual, const void* x, const void* gate_in, long long gate_in_stride,
                      const void* weight, const void* style, long long style_stride, void* out_fp8,
                      void* gate_out, int rows, int dim, float eps, const float* d_scale, int flags,
                      void* stream) {
    if (!residual || !out_fp8 || !d_scale) return FRT_ERR_INVALID;
    if (gate_in && !x) return FRT_ERR_INVALID;
    if (misaligned16(residual) || misaligned16(x) || misaligned16(gate_in) || misaligned16(weight) ||
        misaligned16(style) || misaligned16(gate_out) || (reinterpret_cast<uintptr_t>(out_fp8) & 7))
        return FRT_ERR_INVALID;
    if ((gate_in_stride & 7) || (style_stride & 7)) return FRT_ERR_INVALID;
    NormArgs a;
    a.residual = (__nv_bfloat16*)residual;
    a.x = (const __nv_bfloat16*)x;
    a.gate_in = (const __nv_bfloat16*)gate_in;
    a.gate_in_stride = gate_in_stride;
    a.weight = (const __nv_bfloat16*)weight;
    a.style = (const __nv_bfloat16*)style;
    a.style_stride = style_stride;
    a.out = out_fp8;
    a.sf_out = nullptr;
    a.gate_out = (__nv_bfloat16*)gate_out;
    a.d_scale = d_scale;
    a.rows = rows;
    a.dim = dim;
    a.eps = eps;
    cudaStream_t s = (cudaStream_t)stream;
    bool pdl = flags & 1;
    if (x) {
        if (gate_in) {
            if (style) return launch_norm<true, true, true, OUT_E4M3>(a, s, pdl);
            return launch_norm<true, true, false, OUT_E4M3>(a, s, pdl);
        }
        if (style) return launch_norm<true, false, true, OUT_E4M3>(a, s, pdl);
        return launch_norm<true, false, false, OUT_E4M3>(a, s, pdl);
    }
    if (style) return launch_norm<false, false, true, OUT_E4M3>(a, s, pdl);
    return launch_norm<false, false, false, OUT_E4M3>(a, s, pdl);
}

int frt_b200_norm_bf16(void* residual, const void* x, const void* gate_in, long long gate_in_stride,
                       const void* weight, const void* style, long long style_stride, void* out_bf16,
                       void* gate_out, int rows, int dim, float eps, int flags, void* stream) {
    if (!residual || !out_bf16) return FRT_ERR_INVALID;
    if (gate_in && !x) return FRT_ERR_INVALID;
    if (misaligned16(residual) || misaligned16(x) || misaligned16(gate_in) || misaligned16(weight) ||
        misaligned16(style) || misaligned16(gate_out) || misaligned16(out_bf16))
        return FRT_ERR_INVALID;
    if ((gate_in_stride & 7) || (style_stride & 7)) return FRT_ERR_INVALID;
    NormArgs a;
    a.residual = (__nv_bfloat16*)residual;
    a.x = (const __nv_bfloat16*)x;
    a.gate_in = (const __nv_bfloat16*)gate_in;
    a.gate_in_stride = gate_in_stride;
    a.weight = (const __nv_bfloat16*)weight;
    a.style = (const __nv_bfloat16*)style;
    a.style_stride = style_stride;
    a.out = out_bf16;
    a.sf_out = nullptr;
    a.gate_out = (__nv_bfloat16*)gate_out;
    a.d_scale = nullptr;
    a.rows = rows;
    a.dim = dim;
    a.eps = eps;
    cudaStream_t s = (cudaStream_t)stream;
    bool pdl = flags & 1;
    if (x) {
        if (gate_in) {
            if (style) return launch_norm<true, true, true, OUT_BF16>(a, s, pdl);
            return launch_norm<true, true, false, OUT_BF16>(a, s, pdl);
        }
        if (style) return launch_norm<true, false, true, OUT_BF16>(a, s, pdl);
        return launch_norm<true, false, false, OUT_BF16>(a, s, pdl);
    }
    if (style) return launch_norm<false, false, true, OUT_BF16>(a, s, pdl);
    return launch_norm<false, false, false, OUT_BF16>(a, s, pdl);
}

// Same fused norm with an NVFP4 result: packed e2m1 (rows, dim / 2) and block scales in the GEMM's scale-factor
// atoms (zero-filled by the caller once).  The modulated value is rounded to bf16 first, so the result equals
// frt_b200_norm_bf16 followed by frt_b200_quantize_nvfp4 byte for byte.  dim % 16 == 0.  family: 0 / 1.
int frt_b200_norm_nvfp4(void* residual, const void* x, const void* gate_in, long long gate_in_stride,
                        const void* weight, const void* style, long long style_stride, void* out_packed,
                        void* out_sf, void* gate_out, int rows, int dim, float eps, int family, int flags,
                        void* stream) {
    if (!residual || !out_packed || !out_sf) return FRT_ERR_INVALID;
    if (gate_in && !x) return FRT_ERR_INVALID;
    if (family != 0 && family != 1) return FRT_ERR_INVALID;
    if (dim % 16) return FRT_ERR_UNSUPPORTED;
    if (misaligned16(residual) || misaligned16(x) || misaligned16(gate_in) || misaligned16(weight) ||
        misaligned16(style) || misaligned16(gate_out) || (reinterpret_cast<uintptr_t>(out_packed) & 3))
        return FRT_ERR_INVALID;
    if ((gate_in_stride & 7) || (style_stride & 7)) return FRT_ERR_INVALID;
    NormArgs a;
    a.residual = (__nv_bfloat16*)residual;
    a.x = (const __nv_bfloat16*)x;
    a.gate_in = (const __nv_bfloat16*)gate_in;
    a.gate_in_stride = gate_in_stride;
    a.weight = (const __nv_bfloat16*)weight;
    a.style = (const __nv_bfloat16*)style;
    a.style_stride = style_stride;
    a.out = out_packed;
    a.sf_out = (uint8_t*)out_sf;
    a.gate_out = (__nv_bfloat16*)gate_out;
    a.d_scale = nullptr;
    a.rows = rows;
    a.dim = dim;
    a.eps = eps;
    cudaStream_t s = (cudaStream_t)stream;
    if (family == 0) return dispatch_norm_nvfp4<OUT_NVFP4_A>(a, x != nullptr, gate_in != nullptr, style != nullptr, s, flags & 1);
    return dispatch_norm_nvfp4<OUT_NVFP4_B>(a, x != nullptr, gate_in != nullptr, style != nullptr, s, flags & 1);
}

}  // extern "C"
