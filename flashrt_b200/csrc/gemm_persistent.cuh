// Large-M FP8 GEMM as a persistent kernel: one CTA per SM walks a static list of 128 x BN output tiles.
//
// Included by gemm_fp8.cu inside namespace frt (GemmParams, tensor-map cache, status word).
//
// Why: with one tile per CTA the prologue (barriers, TMEM allocation, first TMA round trip) and the epilogue
// (TMEM -> registers -> global) of every tile are exposed; at K = 1024 they cost more than the MMAs.  Here
//   * the TMA producer runs ahead across tile boundaries (the shared-memory ring never drains),
//   * two accumulators live in TMEM (2 x BN columns): the MMA warp fills one while eight epilogue warps drain
//     the other, so the epilogue -- including the bias + GELU + FP8 form -- hides behind the next mainloop,
//   * consecutive tiles of the list share their weight columns (tile = n_tile * m_tiles + m_tile), so the CTAs
//     of one wave read the same BN weight rows from L2.
// Warps: 0 TMA producer, 1 MMA issuer (+ TMEM owner), 2..9 epilogue (lane quadrant = warp % 4, column half =
// (warp - 2) / 4).  Every wait is bounded by the kernel deadline; on expiry the status word is set and all roles
// leave their loops.
#pragma once

// EPI_P_BIAS_GELU_FAST_FP8: the same epilogue with the GELU through the hardware tanh -- a template value, not a run-time
// flag: a select inside the unrolled loop over a thread's values costs as much as the arithmetic it chooses between
enum { EPI_P_BF16 = 0, EPI_P_BIAS_GELU_FP8 = 1, EPI_P_BIAS_GELU_FAST_FP8 = 2 };

// tanh-form GELU with explicitly rounded fp32 operations, the same sequence as bias_gelu_fp8_kernel
// (csrc/quantize/bias_gelu_quantize_fp8.cu:24-49 in the reference)
__device__ __forceinline__ float gelu_tanh_form_rn(float x) {
    const float x3 = __fmul_rn(__fmul_rn(x, x), x);
    const float u = __fmul_rn(0.7978845608f, __fmaf_rn(0.044715f, x3, x));
    const float e = det_expf(__fmul_rn(2.0f, u));
    const float th = __fsub_rn(1.0f, __fdiv_rn(2.0f, __fadd_rn(1.0f, e)));
    return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, th));
}

template <int BN, bool FP4 = false>
struct PGemmCfg {
    static_assert(!FP4 || BN == 128, "NVFP4: two 128-column accumulators plus the scale columns fill tensor memory");
    static constexpr int L_BYTES = 128 * 128;
    static constexpr int C_BYTES = BN * 128;
    static constexpr int SF_BYTES = FP4 ? 2048 : 0;    // four 512-byte scale atoms (one per K = 64 step) per operand
    static constexpr int STAGE_BYTES = L_BYTES + C_BYTES + 2 * SF_BYTES;
    static constexpr int MAX_STAGES = (227 * 1024 - 2048) / STAGE_BYTES;
    static constexpr int STAGES = MAX_STAGES > 6 ? 6 : MAX_STAGES;
    // bf16 epilogue staging: every epilogue warp owns 32 rows x 128 bytes, through which its 32 x 64 block of results is
    // turned from "thread = row" (what tcgen05.ld gives) into "8 threads = one 128-byte line" for the global store
    static constexpr int EPI_STAGE_BYTES = FP4 ? 0 : 8 * 32 * 128;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + EPI_STAGE_BYTES;
    static constexpr int SF_COL = 2 * BN;             // NVFP4: 16 scale columns per operand behind the accumulators
    static constexpr int TMEM_COLS = FP4 ? 512 : 2 * BN;   // BN in {128, 256}
    static constexpr int EPI_THREADS = 256;
};

template <int BN, int EPI, bool FP4 = false>
__global__ void __launch_bounds__(320, 1)
gemm_fp8_persistent_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                           GemmParams p) {
    using Cfg = PGemmCfg<BN, FP4>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;      // [2]
    uint64_t* acc_empty = acc_full + 2;       // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint64_t deadline = tc::global_timer_ns() + FRT_KERNEL_DEADLINE_NS;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m_tiles = (p.M + 127) / 128;
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
            tc::mbar_init(&acc_empty[i], Cfg::EPI_THREADS);
        }
        *abort_flag = 0;
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&tmA);
        tc::tma_prefetch_desc(&tmW);
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer: runs ahead over tile boundaries
        pdl_wait();
        long long kc = 0;
        for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x) {
            const int m0 = (t % m_tiles) * 128, n0 = (t / m_tiles) * BN;
            for (int kb = 0; kb < kbt; ++kb, ++kc) {
                const int s = (int)(kc % STAGES);
                if (kc >= STAGES &&
                    !tc::mbar_wait_until(&empty[s], (uint32_t)(((kc / STAGES) - 1) & 1), deadline, abort_flag)) {
                    if (!*abort_flag) atomicCAS(&g_gemm_status, 0, ERR_PRODUCER | (blockIdx.x << 8));
                    *abort_flag = 1;
                    break;
                }
                uint8_t* dst = smem + s * Cfg::STAGE_BYTES;
                tc::mbar_arrive_expect_tx(&full[s], Cfg::STAGE_BYTES);
                tc::tma_load_2d(dst, &tmA, &full[s], kb * 128, m0);
                if (!FP4 && p.w_kn) {      // (K, N) weights: one 128 x 128-byte box per 128 output features
#pragma unroll
                    for (int j = 0; j < BN / 128; ++j)
                        tc::tma_load_2d(dst + Cfg::L_BYTES + j * 16384, &tmW, &full[s], n0 + j * 128, kb * 128);
                } else {
                    tc::tma_load_2d(dst + Cfg::L_BYTES, &tmW, &full[s], kb * 128, n0);
                }
                if (FP4) {      // activations are the lane operand here: sf_lane = SFA, sf_col = SFW
                    uint8_t* sf = dst + Cfg::L_BYTES + Cfg::C_BYTES;
                    tc::bulk_load(sf, p.sf_lane + ((size_t)(m0 / 128) * p.sf_katoms + (size_t)kb * 4) * 512, 2048,
                                  &full[s]);
                    tc::bulk_load(sf + 2048, p.sf_col + ((size_t)(n0 / 128) * p.sf_katoms + (size_t)kb * 4) * 512,
                                  2048, &full[s]);
                }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer: accumulator i & 1 for the CTA's i-th tile
        const bool w_kn = !FP4 && p.w_kn;
        const uint32_t idesc = FP4 ? tc::make_idesc_nvfp4(128, BN)
                                   : (tc::make_idesc(0, 0, 0, 0, 128, BN) | (w_kn ? (1u << 16) : 0u));
        const uint32_t sf_smem0 = tc::smem_u32(smem + Cfg::L_BYTES + Cfg::C_BYTES);
        const uint32_t tmem_sfa = tmem + Cfg::SF_COL, tmem_sfw = tmem + Cfg::SF_COL + 16;
        const uint64_t dL0 = tc::make_desc_kmajor_sw128(tc::smem_u32(smem));
        const uint64_t dC0 = w_kn ? tc::make_desc_mnmajor_sw128(tc::smem_u32(smem + Cfg::L_BYTES), 16384)
                                  : tc::make_desc_kmajor_sw128(tc::smem_u32(smem + Cfg::L_BYTES));
        const uint64_t cstep = w_kn ? (uint64_t)((32 * 128) >> 4) : 2u;
        long long kc = 0;
        int i = 0;
        for (int t = blockIdx.x; t < total && !*abort_flag; t += gridDim.x, ++i) {
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
                if (FP4) {
                    const uint32_t sf = sf_smem0 + (uint32_t)(s * Cfg::STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        tc::tmem_cp_sf_atom(tmem_sfa + 4 * k, sf + 512 * k);
                        tc::tmem_cp_sf_atom(tmem_sfw + 4 * k, sf + 2048 + 512 * k);
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc::mma_nvfp4(d_tm, dL0 + so + 2 * k, dC0 + so + 2 * k, idesc, tmem_sfa + 4 * k,
                                      tmem_sfw + 4 * k, (kb > 0 || k > 0) ? 1u : 0u);
                } else {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc::mma_f8(d_tm, dL0 + so + 2 * k, dC0 + so + cstep * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                tc::mma_commit(&empty[s]);
            }
            if (*abort_flag) break;
            tc::mma_commit(&acc_full[buf]);
        }
    } else if (warp >= 2) {
        // ---------------- epilogue: eight warps drain one accumulator while the other one fills
        pdl_wait();
        const int q = warp & 3;                         // TMEM lane quadrant this warp may access
        const int half = (warp - 2) >> 2;               // which half of the BN columns
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        float alpha = p.alpha_host;
        if (p.sa) alpha *= *p.sa;
        if (p.sb) alpha *= *p.sb;
        const float inv_os = (EPI != EPI_P_BF16) ? __fdiv_rn(1.0f, *p.out_scale) : 0.0f;
        // whole 128-byte lines per store instruction when rows and column blocks are 16-byte aligned
        const bool lines = EPI == EPI_P_BF16 && Cfg::EPI_STAGE_BYTES > 0 && (p.N % 8) == 0 &&
                           (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 &&
                           (!p.bias || (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0);
        uint8_t* stg = smem + STAGES * Cfg::STAGE_BYTES + 256 + (warp - 2) * (32 * 128);
        int i = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++i) {
            const int buf = i & 1;
            const bool ok = tc::mbar_wait_until(&acc_full[buf], (uint32_t)((i >> 1) & 1), deadline, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) {          // leave as a whole warp: tcgen05.ld is warp-collective
                if (!*abort_flag) atomicCAS(&g_gemm_status, 0, ERR_EPILOGUE | (blockIdx.x << 8));
                *abort_flag = 1;
                break;
            }
            tc::tc_fence_after_sync();
            const int m = (t % m_tiles) * 128 + q * 32 + lane;
            const int n0 = (t / m_tiles) * BN + half * (BN / 2);
            const uint32_t t_src = tmem + buf * BN + half * (BN / 2) + lane_off;
            if (lines) {
                const int m_base = (t % m_tiles) * 128 + q * 32;
#pragma unroll 1
                for (int c = 0; c < BN / 2; c += 64) {
                    uint32_t v[64];
                    tc::tmem_ld32(t_src + c, v);
                    tc::tmem_ld32(t_src + c + 32, v + 32);
                    tc::tmem_ld_wait();
                    const int nb = n0 + c;
                    // this thread's row: 64 results -> bf16 -> eight 16-byte chunks, chunk index xor (row & 7)
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        float f[8];
                        uint4 bv = make_uint4(0, 0, 0, 0);
                        const bool has_b = p.bias && nb + 8 * k + 8 <= p.N;
                        if (has_b) bv = ld_global_v4(p.bias + nb + 8 * k);
                        const uint32_t* bw = &bv.x;
#pragma unroll
                        for (int e = 0; e < 8; ++e) {           // the same expression as the direct path below
                            f[e] = scale_bias(__uint_as_float(v[8 * k + e]), alpha,
                                              bf16_bits_to_f32((bw[e >> 1] >> ((e & 1) * 16)) & 0xffffu), has_b);
                        }
                        uint4 o;
                        o.x = pack_bf16x2(f[0], f[1]);
                        o.y = pack_bf16x2(f[2], f[3]);
                        o.z = pack_bf16x2(f[4], f[5]);
                        o.w = pack_bf16x2(f[6], f[7]);
                        *reinterpret_cast<uint4*>(stg + lane * 128 + ((k ^ (lane & 7)) << 4)) = o;
                    }
                    __syncwarp();
                    // four rows x 128 bytes per instruction
                    const int ch = lane & 7;
#pragma unroll
                    for (int r4 = 0; r4 < 8; ++r4) {
                        const int row = r4 * 4 + (lane >> 3);
                        const uint4 o = *reinterpret_cast<const uint4*>(stg + row * 128 + ((ch ^ (row & 7)) << 4));
                        const int mm = m_base + row, nn = nb + ch * 8;
                        if (mm < p.M && nn + 8 <= p.N) st_global_v4(p.out + (size_t)mm * p.N + nn, o);
                    }
                    __syncwarp();
                }
                tc::tc_fence_before_sync();
                tc::mbar_arrive(&acc_empty[buf]);
                continue;
            }
#pragma unroll 1
            for (int c = 0; c < BN / 2; c += 32) {
                uint32_t v[32];
                tc::tmem_ld32(t_src + c, v);
                tc::tmem_ld_wait();
                if (m < p.M) {
                    const int nb = n0 + c;
                    if (EPI == EPI_P_BF16) {
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
                    } else {
                        // bf16(alpha * acc) + bias -> GELU -> e4m3: the rounding points of GEMM -> bias_gelu_quantize
                        uint8_t* orow = p.out8 + (size_t)m * p.N + nb;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            if (nb + j + 8 <= p.N) {
                                float g[8], bj[8];
                                // 8 bias values with one load when they are 16-byte aligned (nb + j is a multiple of 8)
                                if (p.bias && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) {
                                    const uint4 bv = ld_global_v4(p.bias + nb + j);
                                    unpack_bf16x2(bv.x, bj[0], bj[1]);
                                    unpack_bf16x2(bv.y, bj[2], bj[3]);
                                    unpack_bf16x2(bv.z, bj[4], bj[5]);
                                    unpack_bf16x2(bv.w, bj[6], bj[7]);
                                } else {
#pragma unroll
                                    for (int e = 0; e < 8; ++e) bj[e] = p.bias ? __bfloat162float(p.bias[nb + j + e]) : 0.0f;
                                }
                                const bool hb = p.bias != nullptr;
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    float x = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[j + e]) * alpha));
                                    if (hb) x = __fadd_rn(x, bj[e]);
                                    g[e] = clamp448(__fmul_rn(EPI == EPI_P_BIAS_GELU_FAST_FP8 ? fast_gelu_tanh(x) : gelu_tanh_form_rn(x),
                                                              inv_os));
                                }
                                uint2 o8;
                                o8.x = f32x4_to_e4m3x4(g[0], g[1], g[2], g[3]);
                                o8.y = f32x4_to_e4m3x4(g[4], g[5], g[6], g[7]);
                                st_global_v2(orow + j, o8);
                            }
                        }
                    }
                }
            }
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&acc_empty[buf]);
        }
    }
    __syncwarp();
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, Cfg::TMEM_COLS);
}

template <int BN, int EPI, bool FP4 = false>
static int launch_gemm_persistent(const void* A, const void* W, GemmParams p, int K, bool pdl, cudaStream_t stream) {
    using Cfg = PGemmCfg<BN, FP4>;
    static PerDeviceOnce attr_once;
    int attr_dev = 0;
    const int sms = device_sm_count();
    if (attr_once.need(attr_dev)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_fp8_persistent_kernel<BN, EPI, FP4>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        attr_once.set(attr_dev);
    }
    CUtensorMap tmA, tmW;
    const uint64_t row_bytes = FP4 ? (uint64_t)K / 2 : (uint64_t)K;
    if (FP4) p.sf_katoms = K / 64;
    int rc = get_tmap_2d_u8(&tmA, A, (uint64_t)p.M, row_bytes, row_bytes, 128);
    if (rc) return rc;
    rc = (!FP4 && p.w_kn) ? get_tmap_2d_u8(&tmW, W, (uint64_t)K, (uint64_t)p.N, (uint64_t)p.N, 128)
                          : get_tmap_2d_u8(&tmW, W, (uint64_t)p.N, row_bytes, row_bytes, BN);
    if (rc) return rc;
    const int total = ((p.M + 127) / 128) * ((p.N + BN - 1) / BN);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(total < sms ? total : sms);
    cfg.blockDim = dim3(320);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_fp8_persistent_kernel<BN, EPI, FP4>, tmA, tmW, p);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}
