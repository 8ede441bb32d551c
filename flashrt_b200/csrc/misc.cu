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
