// NVFP4 producers for sm_100a: bf16 -> packed e2m1 + unsigned-E4M3 block scales written straight
// into the block-scaled GEMM's scale-factor atoms, and GeGLU -> NVFP4.
//
// Replaces, for sm_100a, the reference entry points
//   quantize_bf16_to_nvfp4_swizzled           csrc/bindings.cpp:1277-1285 -> csrc/kernels/quantize.cu:450-526  (family 0)
//   quantize_fp4_dynamic_sfa_bf16_vec         csrc/fp4_bindings.cpp:1124-1137 -> csrc/quantize/quantize_fp4_sfa_bf16.cu
//   quantize_fp4_dynamic_sfa_fp16[_vec]       csrc/fp4_bindings.cpp:299-333 -> csrc/quantize/quantize_fp4_sfa.cu:63-109 (family 1;
//                                             16-bit input is bf16 here, the residual stream of this library)
//   gate_geglu_fp4_sfa[_v2,_vec]_fp16         csrc/fp4_bindings.cpp:711-753 -> csrc/fused_fp4/silu_mul_fp4_sfa_vec.cu:50-107
//   sfa_size_bytes                            csrc/fp4_bindings.cpp:349-352
//
// One thread owns one 16-element block: two 16-byte loads, one 8-byte packed store, one scale byte.
// Consecutive threads own consecutive blocks of a row, so loads and packed stores are fully coalesced.
#include "nvfp4.cuh"

namespace frt {

template <int FAMILY>
__global__ void __launch_bounds__(256)
quantize_nvfp4_kernel(const __nv_bfloat16* __restrict__ in, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf,
                      long long rows, int D, const float* __restrict__ d_global) {
    const int nblk = D >> 4;
    const int katoms = (D + 63) >> 6;
    const long long total = rows * nblk;
    float inv_g = 1.0f;
    const bool has_g = d_global != nullptr;
    if (has_g) inv_g = __fdiv_rn(1.0f, *d_global);
    pdl_launch_dependents();
    pdl_wait();
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / nblk;
        const int blk = (int)(idx - row * nblk);
        const __nv_bfloat16* src = in + row * D + blk * 16;
        const uint4 a = ld_stream_v4(src), b = ld_stream_v4(src + 8);
        float v[16];
        unpack_bf16x2(a.x, v[0], v[1]);
        unpack_bf16x2(a.y, v[2], v[3]);
        unpack_bf16x2(a.z, v[4], v[5]);
        unpack_bf16x2(a.w, v[6], v[7]);
        unpack_bf16x2(b.x, v[8], v[9]);
        unpack_bf16x2(b.y, v[10], v[11]);
        unpack_bf16x2(b.z, v[12], v[13]);
        unpack_bf16x2(b.w, v[14], v[15]);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (has_g) v[i] = __fmul_rn(v[i], inv_g);
            amax = fmaxf(amax, fabsf(v[i]));
        }
        float inv;
        const uint32_t sb = nvfp4::block_scale<FAMILY>(amax, inv);
        uint2 o;
        o.x = nvfp4::pack8<FAMILY>(v, inv);
        o.y = nvfp4::pack8<FAMILY>(v + 8, inv);
        st_global_v2(packed + row * (D >> 1) + blk * 8, o);
        sf[nvfp4::sf_offset(row, blk, katoms)] = (uint8_t)sb;
    }
}

template <int FAMILY>
__global__ void __launch_bounds__(256)
geglu_nvfp4_kernel(const __nv_bfloat16* __restrict__ merged, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf,
                   int rows, int H) {
    const int nblk = H >> 4;
    const int katoms = (H + 63) >> 6;
    const long long total = (long long)rows * nblk;
    pdl_launch_dependents();
    pdl_wait();
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / nblk;
        const int blk = (int)(idx - row * nblk);
        const __nv_bfloat16* g = merged + row * 2 * H + blk * 16;
        const uint4 g0 = ld_stream_v4(g), g1 = ld_stream_v4(g + 8);
        const uint4 u0 = ld_stream_v4(g + H), u1 = ld_stream_v4(g + H + 8);
        const uint32_t gw[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const uint32_t uw[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        float v[16];
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float ga, gb, ua, ub;
            unpack_bf16x2(gw[i], ga, gb);
            unpack_bf16x2(uw[i], ua, ub);
            v[2 * i] = __fmul_rn(det_gelu_tanh(ga), ua);
            v[2 * i + 1] = __fmul_rn(det_gelu_tanh(gb), ub);
            amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
        }
        float inv;
        const uint32_t sb = nvfp4::block_scale<FAMILY>(amax, inv);
        uint2 o;
        o.x = nvfp4::pack8<FAMILY>(v, inv);
        o.y = nvfp4::pack8<FAMILY>(v + 8, inv);
        st_global_v2(packed + row * (H >> 1) + blk * 8, o);
        sf[nvfp4::sf_offset(row, blk, katoms)] = (uint8_t)sb;
    }
}

template <typename K, typename... Args>
static int launch_1d(K kernel, long long work, bool pdl, cudaStream_t stream, Args... args) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long blocks = (work + 255) / 256;
    const long long cap = (long long)sms * 8;
    if (blocks > cap) blocks = cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}

}  // namespace frt

using namespace frt;

extern "C" {

// bytes of the scale-factor buffer of a (rows, K) NVFP4 matrix: ceil(rows / 128) * ceil(K / 64) * 512.
// The buffer must be zero-filled once before first use: padding rows / blocks are never written.
int frt_b200_nvfp4_sf_bytes(long long rows, int K, long long* out_bytes) {
    if (rows < 0 || K <= 0 || !out_bytes) return FRT_ERR_INVALID;
    *out_bytes = ((rows + 127) / 128) * (long long)((K + 63) / 64) * 512;
    return FRT_OK;
}

// in (rows, D) bf16 -> packed (rows, D/2) + sf.  family 0 / 1: see nvfp4.cuh.  d_global_scale: optional device
// float g (NULL = 1): the input is multiplied by 1 / g first and g belongs in the GEMM's alpha.
// flags: bit0 = programmatic dependent launch.  D % 16 == 0; in 16-byte, packed 8-byte aligned.
int frt_b200_quantize_nvfp4(const void* in, void* packed, void* sf, long long rows, int D, int family,
                            const float* d_global_scale, int flags, void* stream) {
    if (!in || !packed || !sf || rows < 0 || D <= 0) return FRT_ERR_INVALID;
    if (D % 16) return FRT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(packed) & 7)) return FRT_ERR_INVALID;
    if (family != 0 && family != 1) return FRT_ERR_INVALID;
    if (rows == 0) return FRT_OK;
    const long long work = rows * (D / 16);
    if (family == 0)
        return launch_1d(quantize_nvfp4_kernel<0>, work, flags & 1, (cudaStream_t)stream, (const __nv_bfloat16*)in,
                         (uint8_t*)packed, (uint8_t*)sf, rows, D, d_global_scale);
    return launch_1d(quantize_nvfp4_kernel<1>, work, flags & 1, (cudaStream_t)stream, (const __nv_bfloat16*)in,
                     (uint8_t*)packed, (uint8_t*)sf, rows, D, d_global_scale);
}

// merged (rows, 2H) bf16 = [gate | up] -> NVFP4 of gelu_tanh(gate) * up (fp32 product, no 16-bit rounding).
int frt_b200_geglu_nvfp4(const void* merged, void* packed, void* sf, int rows, int H, int family, int flags,
                         void* stream) {
    if (!merged || !packed || !sf || rows < 0 || H <= 0) return FRT_ERR_INVALID;
    if (H % 16) return FRT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(merged) & 15) || (reinterpret_cast<uintptr_t>(packed) & 7)) return FRT_ERR_INVALID;
    if (family != 0 && family != 1) return FRT_ERR_INVALID;
    if (rows == 0) return FRT_OK;
    const long long work = (long long)rows * (H / 16);
    if (family == 0)
        return launch_1d(geglu_nvfp4_kernel<0>, work, flags & 1, (cudaStream_t)stream, (const __nv_bfloat16*)merged,
                         (uint8_t*)packed, (uint8_t*)sf, rows, H);
    return launch_1d(geglu_nvfp4_kernel<1>, work, flags & 1, (cudaStream_t)stream, (const __nv_bfloat16*)merged,
                     (uint8_t*)packed, (uint8_t*)sf, rows, H);
}

}  // extern "C"
