// Large-M FP8 GEMM with one 256 x 256 output tile per CTA PAIR (tcgen05 cta_group::2), persistent.
//
// Included by gemm_fp8.cu inside namespace frt (GemmParams, tensor-map cache, status word, gemm_persistent.cuh).
//
// Why: with one CTA per 128 x 256 tile every MMA of 128 x 256 x 32 reads 4 KB of A and 8 KB of B from that CTA's
// shared memory -- 96 bytes per clock of the 128 the SM can deliver, and the K = 1024 shapes stall on it.  A pair
// of CTAs (a cluster of two) computes 256 x 256: each CTA stages ITS 128 rows of A and ITS 128 of the 256 weight
// rows (16 KB + 16 KB per k-block instead of 16 + 32), the leader CTA issues one tcgen05.mma.cta_group::2 that
// reads both CTAs' shared memory, and each CTA receives its 128 rows x 256 columns of the result in its own
// tensor memory.  Same bytes from L2 per flop as two independent 128 x 256 tiles sharing a weight tile, but two
// thirds of the shared-memory operand traffic per SM.
//
// Protocol (rank 0 = leader):
//   * both producers wait for their own empty[s], the leader posts the byte count of BOTH CTAs on its full[s], both
//     issue their TMA loads (cta_group::2 form, no multi-destination copy) signalling the LEADER's full[s];
//   * the leader's MMA thread waits for full[s], issues four MMAs (K = 32 each) and commits twice: to its own
//     empty[s] and to the peer's (a tcgen05.commit addressed at the peer's barrier), likewise for acc_full[buf];
//   * eight epilogue warps per CTA drain that CTA's accumulator and arrive on the leader's acc_empty[buf]
//     (512 arrivals), which the leader's MMA thread waits for before it reuses the buffer.
// Tensor memory is allocated and freed with the cta_group::2 forms by the same warp of both CTAs.  Every wait is
// bounded by the kernel deadline; the CTAs meet at a cluster barrier before either leaves.
#pragma once

struct PairCfg {
    static constexpr int BN = 256;                       // columns of the pair's tile (128 weight rows per CTA)
    static constexpr int A_BYTES = 128 * 128;
    static constexpr int B_BYTES = 128 * 128;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // per CTA
    static constexpr int STAGES = 6;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
    static constexpr int TMEM_COLS = 512;                // two accumulators of 256 columns
    static constexpr int EPI_THREADS = 256;
};

namespace tc {
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {   // same warp of both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// tiled load whose completion bytes are posted on a barrier given as a shared::cluster address (the leader's)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                 int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(m), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
// D[tmem of both CTAs] (+)= A[both CTAs' smem] . B[both CTAs' smem]; issued by one thread of the leader CTA
__device__ __forceinline__ void mma_f8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    const uint32_t z = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(z)
        : "memory");
}
// all MMAs issued so far by this thread -> one arrival on the barrier at a shared::cluster address
__device__ __forceinline__ void mma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
}  // namespace tc

__global__ void __launch_bounds__(320, 1)
gemm_fp8_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, GemmParams p) {
    using Cfg = PairCfg;
    constexpr int STAGES = Cfg::STAGES, BN = Cfg::BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);   // used in the leader only
    uint64_t* empty = full + STAGES;          // one per CTA: the leader's commits arrive on both
    uint64_t* acc_full = empty + STAGES;      // [2] one per CTA
    uint64_t* acc_empty = acc_full + 2;       // [2] used in the leader only: 512 arrivals
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint64_t deadline = tc::global_timer_ns() + FRT_KERNEL_DEADLINE_NS;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();          // 0 = leader
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int m_tiles = (p.M + 255) / 256;
    const int n_tiles = (p.N + BN - 1) / BN;
    const int total = m_tiles * n_tiles;
    const int kbt = p.kb_total;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(&acc_full[i], 1);
            tc::mbar_init(&acc_empty[i], 2 * Cfg::EPI_THREADS);
        }
        *abort_flag = 0;
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&tmA);
        tc::tma_prefetch_desc(&tmW);
    }
    if (warp == 1) {
        tc::tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
        tc::tmem_relinquish_pair();
    }
    tc::tc_fence_before_sync();
    tc::cluster_sync_all();                    // both CTAs' barriers exist before anything signals across
    tc::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer (both CTAs): its half of A and of the weight rows, bytes posted at the leader
        pdl_wait();
        long long kc = 0;
        for (int t = pair; t < total && !*abort_flag; t += npairs) {
            const int m0 = (t % m_tiles) * 256 + (int)rank * 128, n0 = (t / m_tiles) * BN + (int)rank * 128;
            for (int kb = 0; kb < kbt; ++kb, ++kc) {
                const int s = (int)(kc % STAGES);
                if (kc >= STAGES &&
                    !tc::mbar_wait_until(&empty[s], (uint32_t)(((kc / STAGES) - 1) & 1), deadline, abort_flag)) {
                    if (!*abort_flag) atomicCAS(&g_gemm_status, 0, ERR_PRODUCER | (blockIdx.x << 8));
                    *abort_flag = 1;
                    break;
                }
                uint8_t* dst = smem + s * Cfg::STAGE_BYTES;
                if (rank == 0) tc::mbar_arrive_expect_tx(&full[s], 2 * Cfg::STAGE_BYTES);
                const uint32_t bar = tc::dsmem_map(tc::smem_u32(&full[s]), 0);
                tc::tma_load_2d_pair(dst, &tmA, bar, kb * 128, m0);
                tc::tma_load_2d_pair(dst + Cfg::A_BYTES, &tmW, bar, kb * 128, n0);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---------------- MMA issuer (leader only): accumulator i & 1 for the pair's i-th tile
        constexpr uint32_t idesc = tc::make_idesc(0, 0, 0, 0, 256, BN);
        const uint64_t dA0 = tc::make_desc_kmajor_sw128(tc::smem_u32(smem));
        const uint64_t dB0 = tc::make_desc_kmajor_sw128(tc::smem_u32(smem + Cfg::A_BYTES));
        long long kc = 0;
        int i = 0;
        for (int t = pair; t < total && !*abort_flag; t += npairs, ++i) {
            const int buf = i & 1;
            if (i >= 2 && !tc::mbar_wait_until(&acc_empty[buf], (uint32_t)(((i >> 1) - 1) & 1), deadline, abort_flag)) {
                if (!*abort_flag) atomicCAS(&g_gemm_status, 0, ERR_MMA | (blockIdx.x << 8));
                *abort_flag = 1;
                break;
            }
            tc::tc_fence_after_sync();
            const uint32_t d_tm = tmem + buf * BN;
            for (int kb = 0; kb < kbt; ++kb, ++kc) {
                const int s = (int)(kc % STAGES);
                if (!tc::mbar_wait_until(&full[s], (uint32_t)((kc / STAGES) & 1), deadline, abort_flag)) {
                    if (!*abort_flag) atomicCAS(&g_gemm_status, 0, ERR_MMA | (blockIdx.x << 8));
                    *abort_flag = 1;
                    break;
                }
                tc::tc_fence_after_sync();
                const uint64_t so = (uint64_t)(s * (Cfg::STAGE_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc::mma_f8_pair(d_tm, dA0 + so + 2 * k, dB0 + so + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                const uint32_t e_addr = tc::smem_u32(&empty[s]);
                tc::mma_commit_pair(tc::dsmem_map(e_addr, 0));
                tc::mma_commit_pair(tc::dsmem_map(e_addr, 1));
            }
            if (*abort_flag) break;
            const uint32_t f_addr = tc::smem_u32(&acc_full[buf]);
            tc::mma_commit_pair(tc::dsmem_map(f_addr, 0));
            tc::mma_commit_pair(tc::dsmem_map(f_addr, 1));
        }
    } else if (warp >= 2) {
        // ---------------- epilogue (both CTAs): this CTA's 128 rows x 256 columns
        pdl_wait();
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        float alpha = p.alpha_host;
        if (p.sa) alpha *= *p.sa;
        if (p.sb) alpha *= *p.sb;
        int i = 0;
        for (int t = pair; t < total; t += npairs, ++i) {
            const int buf = i & 1;
            const bool ok = tc::mbar_wait_until(&acc_full[buf], (uint32_t)((i >> 1) & 1), deadline, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) {
                if (!*abort_flag) atomicCAS(&g_gemm_status, 0, ERR_EPILOGUE | (blockIdx.x << 8));
                *abort_flag = 1;
                break;
            }
            tc::tc_fence_after_sync();
            const int m = (t % m_tiles) * 256 + (int)rank * 128 + q * 32 + lane;
            const int n0 = (t / m_tiles) * BN + half * (BN / 2);
            const uint32_t t_src = tmem + buf * BN + half * (BN / 2) + lane_off;
#pragma unroll 1
            for (int c = 0; c < BN / 2; c += 32) {
                uint32_t v[32];
                tc::tmem_ld32(t_src + c, v);
                tc::tmem_ld_wait();
                if (m < p.M) {
                    const int nb = n0 + c;
                    __nv_bfloat16* orow = p.out + (size_t)m * p.N + nb;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        if (nb + j + 8 <= p.N && ((reinterpret_cast<uintptr_t>(orow + j) & 15) == 0)) {
                            float f[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                f[e] = scale_bias(__uint_as_float(v[j + e]), alpha,
                                                  p.bias ? __bfloat162float(p.bias[nb + j + e]) : 0.0f, p.bias != nullptr);
                            }
                            uint4 o;
                            o.x = pack_bf16x2(f[0], f[1]);
                            o.y = pack_bf16x2(f[2], f[3]);
                            o.z = pack_bf16x2(f[4], f[5]);
                            o.w = pack_bf16x2(f[6], f[7]);
                            st_global_v4(orow + j, o);
                        } else {
                            for (int e = 0; e < 8; ++e)
                                if (nb + j + e < p.N) {
                                    const float f = scale_bias(__uint_as_float(v[j + e]), alpha,
                                                               p.bias ? __bfloat162float(p.bias[nb + j + e]) : 0.0f,
                                                               p.bias != nullptr);
                                    orow[j + e] = __float2bfloat16_rn(f);
                                }
                        }
                    }
                }
            }
            tc::tc_fence_before_sync();
            tc::mbar_arrive_cluster(tc::dsmem_map(tc::smem_u32(&acc_empty[buf]), 0));
        }
    }
    __syncwarp();
    tc::tc_fence_before_sync();
    tc::cluster_sync_all();                    // the leader's MMAs read the peer's shared memory until the end
    if (warp == 1) tc::tmem_dealloc_pair(tmem, Cfg::TMEM_COLS);
}

static int launch_gemm_pair(const void* A, const void* W, GemmParams p, int K, bool pdl, cudaStream_t stream) {
    using Cfg = PairCfg;
    static PerDeviceOnce attr_once;
    int attr_dev = 0;
    const int sms = device_sm_count();
    if (attr_once.need(attr_dev)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_fp8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        attr_once.set(attr_dev);
    }
    CUtensorMap tmA, tmW;
    int rc = get_tmap_2d_u8(&tmA, A, (uint64_t)p.M, (uint64_t)K, (uint64_t)K, 128);
    if (rc) return rc;
    rc = get_tmap_2d_u8(&tmW, W, (uint64_t)p.N, (uint64_t)K, (uint64_t)K, 128);
    if (rc) return rc;
    const int total = ((p.M + 255) / 256) * ((p.N + Cfg::BN - 1) / Cfg::BN);
    const int pairs = total < sms / 2 ? total : sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(320);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 2;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_fp8_pair_kernel, tmA, tmW, p);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}
