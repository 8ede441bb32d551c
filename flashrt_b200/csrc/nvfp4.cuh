// NVFP4 device helpers: e2m1 element codes, unsigned-E4M3 block scales and the
// scale-factor layout of the block-scaled GEMM.
//
// Format: values +-{0, .5, 1, 1.5, 2, 3, 4, 6} (4 bits, low nibble = even element),
// one unsigned E4M3 scale per 16 consecutive elements of a row.  Scale bytes live in
// 512-byte atoms of 128 rows x 4 blocks, byte (r % 32) * 16 + ((r % 128) / 32) * 4 + (blk % 4),
// atoms ordered K-fastest: atom = (r / 128) * ceil(K / 64) + blk / 4.  This is the layout
// tcgen05.cp (32x128b.warpx4) moves into tensor memory unchanged, and the one the
// reference writes (csrc/kernels/quantize.cu:476-486; CUTLASS Sm1xxBlockScaledConfig<16>
// at csrc/quantize/quantize_fp4_sfa.cu:191-206).
//
// Two quantiser conventions of the reference are kept, selected by `family`:
//   0: scale = smallest UE4M3 >= amax / 6 (csrc/kernels/nvfp4_convert.cuh:78-105), zero block -> scale 0
//      and inverse 0, element thresholds compared with '<'   (nvfp4_convert.cuh:31-45)
//   1: scale = RN-even E4M3 of max(amax / 6, 1e-12), inverse = 1 / scale, thresholds compared with '<='
//      (csrc/quantize/quantize_fp4_sfa.cu:31-50, 89-108)
// All arithmetic is explicitly rounded IEEE fp32, mirrored by the C oracle.
#pragma once
#include "common.cuh"

namespace frt {
namespace nvfp4 {

__device__ __forceinline__ long long sf_offset(long long row, int blk, int katoms) {
    return ((row >> 7) * katoms + (blk >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (blk & 3);
}

__device__ __forceinline__ float ue4m3_to_f32(uint32_t c) {
    const int e = (c >> 3) & 0xF, m = c & 7;
    // (1 + m/8) * 2^(e-7) for normals, (m/8) * 2^-6 for e == 0; both exact in fp32
    const float mant = e ? __fadd_rn(1.0f, (float)m * 0.125f) : (float)m * 0.125f;
    return __fmul_rn(mant, __int_as_float((127 + (e ? e - 7 : -6)) << 23));
}

// smallest unsigned-E4M3 value >= v; codes above 240 collapse to 0xFE as in the reference
__device__ __forceinline__ uint32_t ue4m3_ceil(float v) {
    if (!(v > 0.0f)) return 0u;
    if (v > 240.0f) return 0xFEu;
    if (v < 0.015625f) {
        const int m = (int)ceilf(__fmul_rn(v, 512.0f));
        if (m > 7) return 0x08u;
        return (uint32_t)(m < 1 ? 1 : m);
    }
    const uint32_t bits = __float_as_uint(v);
    int ex = (int)((bits >> 23) & 0xFF) - 127 + 7;
    const uint32_t frac = bits & 0x7FFFFFu;
    uint32_t m = frac >> 20;
    if (frac & 0xFFFFFu) ++m;
    if (m >= 8) { m = 0; ++ex; }
    if (ex >= 15) return 0xFEu;
    return ((uint32_t)ex << 3) | m;
}

// RN-even E4M3 (saturating finite) of a non-negative value, and back
__device__ __forceinline__ uint32_t e4m3_rn(float v) {
    return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

template <int FAMILY>
__device__ __forceinline__ uint32_t e2m1_code(float v) {
    const float a = fabsf(v);
    int below;   // thresholds the magnitude stays under (NaN stays under none -> code 7)
    if (FAMILY == 0)
        below = (a < 0.25f) + (a < 0.75f) + (a < 1.25f) + (a < 1.75f) + (a < 2.5f) + (a < 3.5f) + (a < 5.0f);
    else
        below = (a <= 0.25f) + (a <= 0.75f) + (a <= 1.25f) + (a <= 1.75f) + (a <= 2.5f) + (a <= 3.5f) + (a <= 5.0f);
    return ((v < 0.0f) ? 8u : 0u) | (uint32_t)(7 - below);
}

// scale byte and the multiplier applied to the elements, from the block's largest magnitude
template <int FAMILY>
__device__ __forceinline__ uint32_t block_scale(float amax, float& inv) {
    uint32_t sb;
    if (FAMILY == 0) {
        sb = ue4m3_ceil(__fdiv_rn(amax, 6.0f));
        const float s = ue4m3_to_f32(sb);
        inv = s > 0.0f ? __fdiv_rn(1.0f, s) : 0.0f;
    } else {
        sb = e4m3_rn(fmaxf(__fdiv_rn(amax, 6.0f), 1e-12f));
        inv = __fdiv_rn(1.0f, ue4m3_to_f32(sb));
    }
    return sb;
}

// eight values -> four bytes (element 0 in the low nibble of byte 0)
template <int FAMILY>
__device__ __forceinline__ uint32_t pack8(const float* v, float inv) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) w |= e2m1_code<FAMILY>(__fmul_rn(v[i], inv)) << (4 * i);
    return w;
}

}  // namespace nvfp4
}  // namespace frt
