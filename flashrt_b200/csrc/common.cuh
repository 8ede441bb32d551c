// Shared device helpers for the sm_100a denoise-path kernels.
//
// Arithmetic policy: every fused norm / quantise / activation kernel in this
// library computes with explicitly rounded IEEE-754 fp32 operations
// (__fmul_rn, __fadd_rn, __fmaf_rn, __fdiv_rn, __fsqrt_rn) in a fixed order,
// so that a plain-C restatement of the same sequence reproduces every output
// byte.  No fast-math, no approximate reciprocal / rsqrt / exp in those
// kernels.  (GEMM and attention kernels are floating-point kernels with a
// stated tolerance and may use approximate exp2.)
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FRT_OK 0
#define FRT_ERR_INVALID (-1)
#define FRT_ERR_UNSUPPORTED (-2)
#define FRT_ERR_TIMEOUT (-3)
#define FRT_CUDA_ERR(e) (-(1000 + (int)(e)))

#define FRT_CHECK_LAUNCH()                                  \
    do {                                                    \
        cudaError_t _e = cudaGetLastError();                \
        if (_e != cudaSuccess) return FRT_CUDA_ERR(_e);     \
    } while (0)

namespace frt {

// ---------------------------------------------------------------- bf16 <-> f32
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) {
    return __uint_as_float(b16 << 16);
}
__device__ __forceinline__ void unpack_bf16x2(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
}
// round-to-nearest-even fp32 -> bf16, returned in the low 16 bits
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
}

// ---------------------------------------------------------------- fp8 e4m3
// clamp to +-448 (fmaxf/fminf return the non-NaN operand, so NaN -> -448),
// then round-to-nearest-even, saturating-finite.
__device__ __forceinline__ float clamp448(float v) {
    return fminf(fmaxf(v, -448.0f), 448.0f);
}
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
    // low byte = lo, high byte = hi
    return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
    return f32x2_to_e4m3x2(a, b) | (f32x2_to_e4m3x2(c, d) << 16);
}

// ---------------------------------------------------------------- exp
// e^x from correctly rounded fp32 operations only (Cody-Waite reduction by
// ln2 in two pieces, degree-7 Taylor/Horner on |r| <= ln2/2, exact scaling by
// 2^n).  The C oracle carries the identical sequence.
__device__ __forceinline__ float det_expf(float x) {
    x = fminf(fmaxf(x, -87.0f), 88.0f);
    float n = rintf(__fmul_rn(x, 1.4426950408889634f));
    float r = __fmaf_rn(n, -0.693145751953125f, x);            // ln2 high part (exact in 12 bits)
    r = __fmaf_rn(n, -1.4286068203094173e-06f, r);             // ln2 low part
    float p = 1.9841269841269841e-04f;                         // 1/5040
    p = __fmaf_rn(p, r, 1.3888888888888889e-03f);              // 1/720
    p = __fmaf_rn(p, r, 8.3333333333333332e-03f);              // 1/120
    p = __fmaf_rn(p, r, 4.1666666666666664e-02f);              // 1/24
    p = __fmaf_rn(p, r, 1.6666666666666666e-01f);              // 1/6
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    float s = __int_as_float(((int)n + 127) << 23);            // 2^n, n in [-126,127]
    return __fmul_rn(p, s);
}

// tanh-approximated GELU written as x * sigmoid(2u), u = 0.79788456*(x + 0.044715 x^3)
//   gelu(g) = g / (1 + exp(-1.5957691216057308 * g * (1 + 0.044715 g^2)))
__device__ __forceinline__ float det_gelu_tanh(float g) {
    float inner = __fmaf_rn(__fmul_rn(0.044715f, g), g, 1.0f);
    float arg = __fmul_rn(__fmul_rn(-1.5957691216057308f, g), inner);
    float e = det_expf(arg);
    return __fdiv_rn(g, __fadd_rn(1.0f, e));
}

// SiLU: g * sigmoid(g) = g / (1 + exp(-g))  (silu_mul_split_fp8_kernel, csrc/kernels/activation.cu:291-306)
__device__ __forceinline__ float det_silu(float g) {
    return __fdiv_rn(g, __fadd_rn(1.0f, det_expf(-g)));
}
// GELU(tanh) with the hardware tanh (tanh.approx.f32, relative error 2^-11): 0.5 g (1 + tanh(0.79788456 g (1 + 0.044715 g^2))).
// Six instructions instead of about thirty; not reproducible bit for bit on a CPU, hence an option beside det_gelu_tanh.
// (The reference's kernel is itself built on the fast __expf: csrc/kernels/activation.cu:249-266.)
__device__ __forceinline__ float fast_gelu_tanh(float g) {
    const float u = __fmul_rn(__fmul_rn(0.7978845608028654f, g), __fmaf_rn(__fmul_rn(0.044715f, g), g, 1.0f));
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    return __fmul_rn(__fmul_rn(0.5f, g), __fadd_rn(1.0f, t));
}

// gate activation of the gated FFN epilogues: 0 = GELU(tanh) (GeGLU), 1 = SiLU (SwiGLU)
template <int ACT>
__device__ __forceinline__ float det_gate_act(float g) {
    return ACT == 1 ? det_silu(g) : det_gelu_tanh(g);
}

// ---------------------------------------------------------------- reductions
// xor-butterfly: every lane ends with the same value; tree order is fixed.
__device__ __forceinline__ float warp_sum_butterfly(float v) {
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 16));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 8));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
    v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return v;
}
__device__ __forceinline__ float warp_max_butterfly(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return v;
}

// Element of every bf16 GEMM epilogue: alpha * acc, or alpha * acc + bias with ONE rounding.  Written out so that every
// kernel that can serve a shape produces the same bits (the compiler is otherwise free to fuse or not, site by site).
__device__ __forceinline__ float scale_bias(float acc, float alpha, float bias, bool has_bias) {
    return has_bias ? __fmaf_rn(acc, alpha, bias) : __fmul_rn(acc, alpha);
}

// Device addresses of the three status words (each lives in the translation unit of its kernels); nullptr on error.
int* gemm_status_device_ptr();
int* attention_status_device_ptr();
int* expert_loop_status_device_ptr();

// ---------------------------------------------------------------- 16-byte I/O
__device__ __forceinline__ uint4 ld_global_v4(const void* p) {
    return *reinterpret_cast<const uint4*>(p);
}
// streaming (read-once) 16-byte load that does not allocate in L1
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ float4 ld_global_f4(const float* p) {
    return *reinterpret_cast<const float4*>(p);
}
__device__ __forceinline__ void st_global_v4(void* p, uint4 v) {
    *reinterpret_cast<uint4*>(p) = v;
}
__device__ __forceinline__ void st_global_v2(void* p, uint2 v) {
    *reinterpret_cast<uint2*>(p) = v;
}

// programmatic dependent launch: wait for the producer grid's memory, and
// let the dependent grid start its prologue early.
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- host: per-device launch set-up
// Function attributes (dynamic shared memory size, non-portable cluster size) and the SM count belong to a device,
// not to the process: a launcher sets them once per device ordinal.
struct PerDeviceOnce {
    bool done[64] = {};
    bool need(int& dev) {
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { dev = -1; return true; }
        return !done[dev];
    }
    void set(int dev) { if (dev >= 0 && dev < 64) done[dev] = true; }
};
inline int device_sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev] > 0 ? sms[dev] : 148;
}

}  // namespace frt
