// FP8 E4M3 x E4M3 -> bf16 GEMM for sm_100a: TMA-fed shared-memory pipeline,
// tcgen05.mma (kind::f8f6f4) issued by one thread, fp32 accumulator in TMEM,
// tcgen05.ld epilogue with the per-tensor scales (device pointers), optional
// bias, bf16 store.
//
// Replaces, for sm_100a, the reference entry points
//   GemmRunner::fp8_nn_dev / fp8_nt_dev     csrc/gemm/gemm_runner.cu:67-76 (cuBLASLt)
//   fp8_gemm_descale_bf16out               csrc/kernels/decoder_fused.cu:310-468
//   (+ fused epilogues standing in for qkv_split_rope, csrc/kernels/rope.cu:135-277, and
//      gate_silu_mul_merged_fp8, csrc/kernels/activation.cu:249-279, after the M <= 256 GEMM)
//   cutlass_fp8_{sq,t1,wide,plain}_bf16out csrc/gemm/cutlass_sm100.cu:75-125
//
// Math: D(M,N) = alpha * A(M,K) . W(N,K)^T (+ bias), alpha = sa * sb * alpha_host,
// products exact, fp32 accumulation, bf16 RN-even result.
//
// Both operands are K-major ("NT": activations (M,K) row-major, weights (N,K)
// row-major).  One CTA computes one 128 x BN accumulator tile; the 128 TMEM lanes
// are fed by the "lane operand", the BN columns by the "column operand":
//   * SWAP = true  (small M): lanes = 128 weight rows, columns = the (<= 256)
//     activation rows.  Every weight byte is streamed exactly once and the MMA
//     M-dimension is fully used even for M = 16 or 50.
//   * SWAP = false (large M): lanes = 128 activation rows, columns = BN weight rows.
// Split-K: the CTAs of one thread-block cluster (1 x 1 x S, S <= 16) each
// accumulate a slice of K, exchange fp32 partials through distributed shared
// memory and each reduces 1/S of the tile's columns in fixed order (split 0, 1, ...).
// There is no global-memory workspace and the result is deterministic.
//
// Each TMA copy lands in the issuing CTA's own shared memory.
#include "common.cuh"
#include "tc05.cuh"

#include <cstring>
#include <mutex>
#include <unordered_map>

namespace frt {

// ------------------------------------------------------------------ status word
__device__ int g_gemm_status = 0;   // 0 ok; otherwise first failure code | (blockIdx.x << 8)

// ------------------------------------------------------------------ tensor maps (host)
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_encodeTiled g_encode = nullptr;
static std::mutex g_mu;

static int ensure_encode() {
    if (g_encode) return FRT_OK;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_encode) return FRT_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return FRT_ERR_UNSUPPORTED;
    g_encode = (PFN_encodeTiled)fn;
    return FRT_OK;
}

// 2D byte matrix (rows x row_bytes, row pitch = pitch_bytes), box = 128 bytes x box_rows, 128-byte swizzle.
int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t pitch_bytes,
                    uint32_t box_rows) {
    int rc = ensure_encode();
    if (rc) return rc;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15) || box_rows == 0 || box_rows > 256)
        return FRT_ERR_INVALID;
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FRT_OK : FRT_ERR_INVALID;
}

// ------------------------------------------------------------------ kernel
struct GemmParams {
    __nv_bfloat16* out;        // (M, N) row-major
    const float* sa;           // device scalars (may be null = 1)
    const float* sb;
    float alpha_host;
    const __nv_bfloat16* bias; // (N,) or null
    int M, N;
    int kb_total;              // ceil(K / 128)
    int lane_rows;             // extent of the lane operand (N if SWAP else M)
    int col_rows;              // extent of the column operand (M if SWAP else N)
    int w_is_lane;             // which operand holds the weights (prefetched before the PDL wait)
    // fused epilogues (SWAP kernels only)
    const __nv_bfloat16* rope; // EPI_ROPE_SPLIT: (M, head_dim) rows [cos0, sin0, cos1, sin1, ...]
    __nv_bfloat16* outQ;       //   Q (M, q_dim); K, V rows written at (*devpos + m)
    __nv_bfloat16* outK;
    __nv_bfloat16* outV;
    const int* devpos;
    int q_dim, k_dim, v_dim, head_dim;
    uint8_t* out8;             // EPI_GEGLU_FP8: (M, half) e4m3 codes
    const float* out_scale;    //   device scalar: quantisation scale of the GeGLU result
    int half;                  //   hidden width; weight rows [0, half) = gate, [half, 2 half) = up
    int fast_act;              // bias + GELU + FP8 epilogue: GELU through the hardware tanh instead of the exact form
    // NVFP4 kernels: unsigned-E4M3 block scales of both operands in 512-byte atoms (128 rows x 4 blocks)
    const uint8_t* sf_lane;
    const uint8_t* sf_col;
    int sf_katoms;             //   atoms along K = K / 64
    int sf_col_rblocks;        //   128-row atom rows of the column operand's scale buffer
    // EPI_GATE_RES_NORM_FP8: residual (M, N) bf16 in/out, gate (N,), style rows [scale (N) | shift (N)], next site's
    // FP8 activations out8 (M, N) with out_scale; the cluster spans all N / 128 tiles so that the row statistics
    // can be exchanged through distributed shared memory
    __nv_bfloat16* resid;
    const __nv_bfloat16* gate;
    const __nv_bfloat16* style;
    float eps;
    int w_kn;                  // large-M persistent kernel: weights stored (K, N) row-major
};

enum { EPI_BF16 = 0, EPI_ROPE_SPLIT = 1, EPI_GEGLU_FP8 = 2, EPI_GATE_RES_NORM_FP8 = 3 };

template <int BN, bool FP4 = false>
struct GemmCfg {
    static constexpr int BK = 128;                       // bytes per k-block: 128 fp8 or 256 packed fp4 elements
    static constexpr int L_BYTES = 128 * BK;             // 16 KB
    static constexpr int C_BYTES = BN * BK;
    static constexpr int CB = (BN + 127) / 128;          // 128-row scale atoms spanned by the column operand
    static constexpr int SFL_BYTES = FP4 ? 4 * 512 : 0;  // 4 atoms (one per K = 64 step) of the lane operand
    static constexpr int SFC_BYTES = FP4 ? 4 * 512 * CB : 0;
    static constexpr int STAGE_BYTES = L_BYTES + C_BYTES + SFL_BYTES + SFC_BYTES;
    static constexpr int MAX_STAGES = (227 * 1024 - 2048) / STAGE_BYTES;
    static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
    static constexpr int RED_BYTES = 128 * BN * 4;
    static_assert(RED_BYTES <= STAGES * STAGE_BYTES, "split-K staging must fit in the pipeline buffers");
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
    static constexpr int ACC_COLS = BN < 32 ? 32 : BN;
    static constexpr int SF_COLS = FP4 ? 16 + 16 * CB : 0;   // 4 columns per atom, 4 K-steps, both operands
    static constexpr int NEED_COLS = ACC_COLS + SF_COLS;
    static constexpr int TMEM_COLS = NEED_COLS <= 32 ? 32 : NEED_COLS <= 64 ? 64 : NEED_COLS <= 128 ? 128
                                     : NEED_COLS <= 256 ? 256 : 512;   // power of two >= 32
};

enum { ERR_PRODUCER = 1, ERR_MMA = 2, ERR_EPILOGUE = 3 };

// one asm block = eight independent distributed-shared-memory loads in flight
__device__ __forceinline__ void dsmem_ld8(const uint32_t* a, float* v) {
    asm volatile(
        "ld.shared::cluster.f32 %0, [%8];\n\t"
        "ld.shared::cluster.f32 %1, [%9];\n\t"
        "ld.shared::cluster.f32 %2, [%10];\n\t"
        "ld.shared::cluster.f32 %3, [%11];\n\t"
        "ld.shared::cluster.f32 %4, [%12];\n\t"
        "ld.shared::cluster.f32 %5, [%13];\n\t"
        "ld.shared::cluster.f32 %6, [%14];\n\t"
        "ld.shared::cluster.f32 %7, [%15];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7])
        : "memory");
}

// Sum over the S cluster ranks (fixed order 0, 1, ...) of the staged partial at byte offset `off` inside
// every rank's staging buffer.  rank_base[s] = cluster address of rank s's buffer.
template <int MAXS>
__device__ __forceinline__ float reduce_ranks(const uint32_t* rank_base, uint32_t S, uint32_t off) {
    float acc = 0.0f;
#pragma unroll
    for (int g = 0; g < MAXS; g += 8) {
        if ((uint32_t)g >= S) break;
        uint32_t a[8];
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = rank_base[(uint32_t)(g + j) < S ? g + j : 0] + off;
        dsmem_ld8(a, v);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if ((uint32_t)(g + j) < S) acc += v[j];
    }
    return acc;
}

template <int BN, bool SWAP, int EPI, bool FP4 = false>
__global__ void __launch_bounds__(128, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmL, const __grid_constant__ CUtensorMap tmC, GemmParams p) {
    static_assert(EPI == EPI_BF16 || SWAP, "fused epilogues exist for the small-M (swapped) kernel only");
    static_assert(!FP4 || (BN >= 32 && EPI != EPI_GEGLU_FP8), "NVFP4: column tiles start on 32-row scale groups");
    using Cfg = GemmCfg<BN, FP4>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* accum_bar = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;
    volatile int* consumed = abort_flag + 2;

    const uint64_t deadline = tc::global_timer_ns() + FRT_KERNEL_DEADLINE_NS;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // first row of the lane operand; with the GeGLU epilogue a tile is 64 gate rows + the 64 matching up rows
    const int lane0 = (EPI == EPI_GEGLU_FP8) ? blockIdx.x * 64 : blockIdx.x * 128;
    const int col0 = blockIdx.y * BN;                // first row of the column operand
    // split-K ranks: the CTAs of a (1, 1, S) cluster, or -- with the fused norm -- the z extent of a (tiles, 1, S) one
    const uint32_t S = (EPI == EPI_GATE_RES_NORM_FP8) ? gridDim.z : tc::cluster_nctarank();
    const uint32_t rank = (EPI == EPI_GATE_RES_NORM_FP8) ? blockIdx.z : tc::cluster_ctarank();
    const int kb_begin = (int)((long long)p.kb_total * rank / S);
    const int kb_end = (int)((long long)p.kb_total * (rank + 1) / S);
    const int nkb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        tc::mbar_init(accum_bar, 1);
        *abort_flag = 0;
        *issued = 0;
        *consumed = 0;
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&tmL);
        tc::tma_prefetch_desc(&tmC);
    }
    if (warp == 2) {
        tc::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_d = *tmem_slot;

    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer
        const CUtensorMap* tmW = p.w_is_lane ? &tmL : &tmC;
        const CUtensorMap* tmX = p.w_is_lane ? &tmC : &tmL;
        const int w_off = p.w_is_lane ? 0 : Cfg::L_BYTES;
        const int x_off = p.w_is_lane ? Cfg::L_BYTES : 0;
        const int w_row = p.w_is_lane ? lane0 : col0;
        const int x_row = p.w_is_lane ? col0 : lane0;
        const int pre = nkb < STAGES ? nkb : STAGES;
        // weights do not depend on the producer grid: start streaming them now
        auto load_w = [&](int stage, int kb) {
            uint8_t* dst = stage_base + stage * Cfg::STAGE_BYTES + w_off;
            if (EPI == EPI_GEGLU_FP8) {   // tmL has a 64-row box here
                tc::tma_load_2d(dst, tmW, &full[stage], kb * 128, w_row);
                tc::tma_load_2d(dst + 64 * 128, tmW, &full[stage], kb * 128, p.half + w_row);
            } else {
                tc::tma_load_2d(dst, tmW, &full[stage], kb * 128, w_row);
            }
        };
        // NVFP4: the scale atoms of a k-block (4 K-steps) are 2048 contiguous bytes per 128-row group
        int c_atoms = Cfg::CB;
        if (FP4) {
            const int left = p.sf_col_rblocks - col0 / 128;
            c_atoms = left < Cfg::CB ? left : Cfg::CB;
        }
        const uint32_t stage_tx = Cfg::STAGE_BYTES - (FP4 ? (Cfg::CB - c_atoms) * 2048 : 0);
        auto load_sf_lane = [&](int stage, int kb) {
            uint8_t* dst = stage_base + stage * Cfg::STAGE_BYTES + Cfg::L_BYTES + Cfg::C_BYTES;
            tc::bulk_load(dst, p.sf_lane + ((size_t)(lane0 / 128) * p.sf_katoms + (size_t)kb * 4) * 512, 2048,
                          &full[stage]);
        };
        auto load_sf_col = [&](int stage, int kb) {
            uint8_t* dst = stage_base + stage * Cfg::STAGE_BYTES + Cfg::L_BYTES + Cfg::C_BYTES + Cfg::SFL_BYTES;
            for (int j = 0; j < c_atoms; ++j)
                tc::bulk_load(dst + j * 2048,
                              p.sf_col + ((size_t)(col0 / 128 + j) * p.sf_katoms + (size_t)kb * 4) * 512, 2048,
                              &full[stage]);
        };
        for (int i = 0; i < pre; ++i) {
            tc::mbar_arrive_expect_tx(&full[i], stage_tx);
            load_w(i, kb_begin + i);
            if (FP4) { if (p.w_is_lane) load_sf_lane(i, kb_begin + i); else load_sf_col(i, kb_begin + i); }
        }
        pdl_wait();
        for (int i = 0; i < pre; ++i) {
            tc::tma_load_2d(stage_base + i * Cfg::STAGE_BYTES + x_off, tmX, &full[i], (kb_begin + i) * 128, x_row);
            if (FP4) { if (p.w_is_lane) load_sf_col(i, kb_begin + i); else load_sf_lane(i, kb_begin + i); }
        }
        *issued = pre;
        for (int i = pre; i < nkb; ++i) {
            const int s = i % STAGES;
            const uint32_t ph = ((i / STAGES) - 1) & 1;
            const bool ok = tc::mbar_wait_until(&empty[s], ph, deadline, abort_flag);
            if (!ok) {
                *abort_flag = 1;
                atomicCAS(&g_gemm_status, 0, ERR_PRODUCER | (blockIdx.x << 8));
                break;
            }
            tc::mbar_arrive_expect_tx(&full[s], stage_tx);
            load_w(s, kb_begin + i);
            tc::tma_load_2d(stage_base + s * Cfg::STAGE_BYTES + x_off, tmX, &full[s], (kb_begin + i) * 128, x_row);
            if (FP4) {
                load_sf_lane(s, kb_begin + i);
                load_sf_col(s, kb_begin + i);
            }
            *issued = i + 1;
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        constexpr uint32_t idesc = FP4 ? tc::make_idesc_nvfp4(128, BN) : tc::make_idesc(0, 0, 0, 0, 128, BN);
        // NVFP4 scale factors in tensor memory, behind the accumulator: 4 columns per (operand atom, K-step)
        const uint32_t tmem_sfl = tmem_d + Cfg::ACC_COLS;
        const uint32_t tmem_sfc = tmem_sfl + 16;
        const uint32_t sfc_off = BN < 128 ? (uint32_t)((col0 & 127) >> 5) : 0u;   // 32-row group of this column tile
        bool failed = false;
        for (int i = 0; i < nkb; ++i) {
            const int s = i % STAGES;
            const uint32_t ph = (i / STAGES) & 1;
            const bool ok = tc::mbar_wait_until(&full[s], ph, deadline, abort_flag);
            if (!ok) {
                *abort_flag = 1;
                atomicCAS(&g_gemm_status, 0, ERR_MMA | (blockIdx.x << 8));
                failed = true;
                break;
            }
            tc::tc_fence_after_sync();
            const uint32_t sL = tc::smem_u32(stage_base + s * Cfg::STAGE_BYTES);
            const uint32_t sC = sL + Cfg::L_BYTES;
            const uint64_t dL = tc::make_desc_kmajor_sw128(sL);
            const uint64_t dC = tc::make_desc_kmajor_sw128(sC);
            if (FP4) {
                const uint32_t sSFL = sC + Cfg::C_BYTES;
                const uint32_t sSFC = sSFL + Cfg::SFL_BYTES;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    tc::tmem_cp_sf_atom(tmem_sfl + 4 * k, sSFL + 512 * k);
#pragma unroll
                    for (int j = 0; j < Cfg::CB; ++j)
                        tc::tmem_cp_sf_atom(tmem_sfc + k * 4 * Cfg::CB + 4 * j, sSFC + j * 2048 + 512 * k);
                }
#pragma unroll
                for (int k = 0; k < 4; ++k)   // 4 x (K = 64 e2m1 = 32 bytes) per 128-byte k-block
                    tc::mma_nvfp4(tmem_d, dL + 2 * k, dC + 2 * k, idesc, tmem_sfl + 4 * k,
                                  tmem_sfc + k * 4 * Cfg::CB + sfc_off, (i > 0 || k > 0) ? 1u : 0u);
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k)   // 4 x (K = 32) per 128-byte k-block; +32 bytes = +2 in the address field
                    tc::mma_f8(tmem_d, dL + 2 * k, dC + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            }
            tc::mma_commit(&empty[s]);
            *consumed = i + 1;
        }
        if (!failed) tc::mma_commit(accum_bar);
    }
    __syncwarp();

    // ---------------- epilogue: all four warps, warp w owns TMEM lanes 32w .. 32w+31
    pdl_wait();
    const bool acc_seen = tc::mbar_wait_until(accum_bar, 0, deadline, abort_flag);
    const bool have_acc = __all_sync(0xffffffffu, acc_seen);   // tcgen05.ld below is warp-collective
    if (!have_acc && !*abort_flag) {
        *abort_flag = 1;
        atomicCAS(&g_gemm_status, 0, ERR_EPILOGUE | (blockIdx.x << 8));
    }
    __syncwarp();
    tc::tc_fence_after_sync();

    float alpha = p.alpha_host;
    if (p.sa) alpha *= *p.sa;
    if (p.sb) alpha *= *p.sb;
    const int lrow = lane0 + warp * 32 + lane;                 // global row of the lane operand
    const uint32_t trow = tmem_d + ((uint32_t)(warp * 32) << 16);

    if (S == 1 && EPI == EPI_BF16 && !SWAP) {
        if (have_acc) {
            if (SWAP) {
                // lanes = output columns n, TMEM columns = output rows m
                const int n = lrow;
                const float b = (p.bias && n < p.N) ? __bfloat162float(p.bias[n]) : 0.0f;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t v[32];
                    if (BN >= 32) tc::tmem_ld32(trow + c, v); else tc::tmem_ld16(trow + c, v);
                    tc::tmem_ld_wait();
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < (BN >= 32 ? 32 : 16); ++j) {
                            const int m = col0 + c + j;
                            if (m < p.M)
                                p.out[(size_t)m * p.N + n] = __float2bfloat16_rn(scale_bias(__uint_as_float(v[j]), alpha, b, p.bias != nullptr));
                        }
                    }
                }
            } else {
                const int m = lrow;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t v[32];
                    if (BN >= 32) tc::tmem_ld32(trow + c, v); else tc::tmem_ld16(trow + c, v);
                    tc::tmem_ld_wait();
                    if (m < p.M) {
                        const int nb = col0 + c;
                        __nv_bfloat16* orow = p.out + (size_t)m * p.N + nb;
#pragma unroll
                        for (int j = 0; j < (BN >= 32 ? 32 : 16); j += 8) {
                            if (nb + j + 8 <= p.N && ((reinterpret_cast<uintptr_t>(orow + j) & 15) == 0)) {
                                float f[8];
#pragma unroll
                                for (int q = 0; q < 8; ++q) {
                                    f[q] = scale_bias(__uint_as_float(v[j + q]), alpha,
                                                      p.bias ? __bfloat162float(p.bias[nb + j + q]) : 0.0f, p.bias != nullptr);
                                }
                                uint4 o;
                                o.x = pack_bf16x2(f[0], f[1]);
                                o.y = pack_bf16x2(f[2], f[3]);
                                o.z = pack_bf16x2(f[4], f[5]);
                                o.w = pack_bf16x2(f[6], f[7]);
                                st_global_v4(orow + j, o);
                            } else {
                                for (int q = 0; q < 8; ++q)
                                    if (nb + j + q < p.N) {
                                        const float f = scale_bias(__uint_as_float(v[j + q]), alpha,
                                                                   p.bias ? __bfloat162float(p.bias[nb + j + q]) : 0.0f,
                                                                   p.bias != nullptr);
                                        orow[j + q] = __float2bfloat16_rn(f);
                                    }
                            }
                        }
                    }
                }
            }
        }
    } else {
        // ---------------- staged path: partials as red[col][lane] (fp32) in shared memory, then every rank of
        // the cluster finishes a slice of the columns, summing the ranks in fixed order through DSMEM.
        float* red = reinterpret_cast<float*>(stage_base);
        if (have_acc) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                if (BN >= 32) tc::tmem_ld32(trow + c, v); else tc::tmem_ld16(trow + c, v);
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < (BN >= 32 ? 32 : 16); ++j)
                    red[(c + j) * 128 + warp * 32 + lane] = __uint_as_float(v[j]);
            }
        }
        if (S > 1 || EPI == EPI_GATE_RES_NORM_FP8) tc::cluster_sync_all(); else __syncthreads();
        if constexpr (EPI == EPI_GATE_RES_NORM_FP8) {
            // ---- split-K sum, gated residual update, RMS statistics over the whole row (all tiles of the cluster),
            // adaRMS modulation and FP8 quantisation of the next GEMM's input.  Every thread reaches both barriers.
            // Cluster rank of CTA (tile x, split z) = x + gridDim.x * z.  S is 1 or 2.
            const uint32_t T = gridDim.x;                                  // tiles across the row = CTAs per split
            const uint32_t red_addr = tc::smem_u32(red);
            float* part = red + BN * 128;                                   // [token][16 groups] partial sums of squares
            float* tok_ssq = part + BN * 16;                                // [token] this tile's sum of squares
            const int cols_per = (BN + (int)S - 1) / (int)S;
            const int cbeg = (int)rank * cols_per;
            int cend = cbeg + cols_per < BN ? cbeg + cols_per : BN;
            if (col0 + cend > p.M) cend = p.M - col0;
            const int ntok = cend > cbeg ? cend - cbeg : 0;
            const int items = ntok * 16;
            const bool live = !*abort_flag;
            if (live) {
                const uint32_t other = S == 2 ? tc::dsmem_map(red_addr, blockIdx.x + T * (rank ^ 1u)) : red_addr;
#pragma unroll 2
                for (int it = threadIdx.x; it < items; it += 128) {
                    const int c = cbeg + it / 16, g = it % 16;
                    const int m = col0 + c, n = lane0 + g * 8;
                    float* mine = &red[c * 128 + g * 8];
                    float4 x0 = reinterpret_cast<const float4*>(mine)[0], x1 = reinterpret_cast<const float4*>(mine)[1];
                    if (S == 2) {
                        const float4 y0 = tc::dsmem_ld_f32x4(other + (uint32_t)(c * 128 + g * 8) * 4u);
                        const float4 y1 = tc::dsmem_ld_f32x4(other + (uint32_t)(c * 128 + g * 8) * 4u + 16u);
                        x0.x += y0.x; x0.y += y0.y; x0.z += y0.z; x0.w += y0.w;
                        x1.x += y1.x; x1.y += y1.y; x1.z += y1.z; x1.w += y1.w;
                    }
                    const float a[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                    const uint4 rv = ld_global_v4(p.resid + (size_t)m * p.N + n);
                    const uint4 gv = ld_global_v4(p.gate + n);
                    const uint32_t* rw = &rv.x;
                    const uint32_t* gw = &gv.x;
                    uint4 ob;
                    uint32_t* ow = &ob.x;
                    float ssq = 0.0f, rr[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float r0, r1, g0, g1;
                        unpack_bf16x2(rw[k], r0, r1);
                        unpack_bf16x2(gw[k], g0, g1);
                        // the GEMM result is rounded to bf16 as the separate kernel stores it, then x += o * gate
                        const float o0 = __bfloat162float(__float2bfloat16_rn(a[2 * k] * alpha));
                        const float o1 = __bfloat162float(__float2bfloat16_rn(a[2 * k + 1] * alpha));
                        r0 = __fmaf_rn(o0, g0, r0);
                        r1 = __fmaf_rn(o1, g1, r1);
                        ssq = __fmaf_rn(r0, r0, ssq);
                        ssq = __fmaf_rn(r1, r1, ssq);
                        ow[k] = pack_bf16x2(r0, r1);
                        unpack_bf16x2(ow[k], rr[2 * k], rr[2 * k + 1]);          // the rounded value feeds the norm
                    }
                    st_global_v4(p.resid + (size_t)m * p.N + n, ob);
                    reinterpret_cast<float4*>(mine)[0] = make_float4(rr[0], rr[1], rr[2], rr[3]);
                    reinterpret_cast<float4*>(mine)[1] = make_float4(rr[4], rr[5], rr[6], rr[7]);
                    part[(c - cbeg) * 16 + g] = ssq;
                }
            }
            __syncthreads();
            if (live && (int)threadIdx.x < ntok) {
                float t = 0.0f;
#pragma unroll
                for (int g = 0; g < 16; ++g) t = __fadd_rn(t, part[threadIdx.x * 16 + g]);
                tok_ssq[threadIdx.x] = t;
            }
            tc::cluster_sync_all();
            // one thread per token gathers the row total from the tiles (all remote loads in flight together; a
            // remote scalar round trip per work item would cost more than the separate norm kernel)
            float* tok_rms = tok_ssq + BN;
            if (live && (int)threadIdx.x < ntok) {
                const uint32_t ssq_addr = tc::smem_u32(tok_ssq) + 4u * threadIdx.x;
                float v[8];
#pragma unroll
                for (uint32_t x = 0; x < 8; ++x) v[x] = x < T ? tc::dsmem_ld_f32(tc::dsmem_map(ssq_addr, x + T * rank)) : 0.0f;
                float tot = 0.0f;
#pragma unroll
                for (uint32_t x = 0; x < 8; ++x) tot = __fadd_rn(tot, v[x]);          // tiles of the row in fixed order
                const float var = __fadd_rn(__fdiv_rn(tot, (float)p.N), p.eps);
                tok_rms[threadIdx.x] = __fdiv_rn(1.0f, __fsqrt_rn(var));
            }
            __syncthreads();
            if (live) {
                const float inv_os = __fdiv_rn(1.0f, *p.out_scale);
#pragma unroll 2
                for (int it = threadIdx.x; it < items; it += 128) {
                    const int c = cbeg + it / 16, g = it % 16;
                    const int m = col0 + c, n = lane0 + g * 8;
                    const float rms = tok_rms[c - cbeg];
                    const float* mine = &red[c * 128 + g * 8];
                    const uint4 sc = ld_global_v4(p.style + n), sh = ld_global_v4(p.style + p.N + n);
                    const uint32_t* scw = &sc.x;
                    const uint32_t* shw = &sh.x;
                    float q[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float s0, s1, h0, h1;
                        unpack_bf16x2(scw[k], s0, s1);
                        unpack_bf16x2(shw[k], h0, h1);
                        const float n0 = __fmaf_rn(__fmul_rn(mine[2 * k], rms), __fadd_rn(1.0f, s0), h0);
                        const float n1 = __fmaf_rn(__fmul_rn(mine[2 * k + 1], rms), __fadd_rn(1.0f, s1), h1);
                        q[2 * k] = clamp448(__fmul_rn(n0, inv_os));
                        q[2 * k + 1] = clamp448(__fmul_rn(n1, inv_os));
                    }
                    uint2 o8;
                    o8.x = f32x4_to_e4m3x4(q[0], q[1], q[2], q[3]);
                    o8.y = f32x4_to_e4m3x4(q[4], q[5], q[6], q[7]);
                    st_global_v2(p.out8 + (size_t)m * p.N + n, o8);
                }
            }
        } else if (!*abort_flag && SWAP) {
            // Work item = (column c of this rank's slice, group of 8 consecutive lanes): every remote read is a
            // 16-byte load, every global store a full 16-byte (bf16) or 8-byte (fp8) vector, and all loads of an
            // item are in flight together.  Ranks are summed in fixed order 0, 1, ...
            const uint32_t red_addr = tc::smem_u32(red);
            uint32_t rank_base[16];
#pragma unroll
            for (int r = 0; r < 16; ++r) rank_base[r] = tc::dsmem_map(red_addr, (uint32_t)r < S ? r : 0);
            const int cols_per = (BN + (int)S - 1) / (int)S;
            const int cbeg = (int)rank * cols_per;
            int cend = cbeg + cols_per < BN ? cbeg + cols_per : BN;
            if (col0 + cend > p.M) cend = p.M - col0;                       // columns are tokens
            constexpr int GROUPS = (EPI == EPI_GEGLU_FP8) ? 8 : 16;        // 8-lane groups per column that carry output
            const int items = (cend > cbeg ? cend - cbeg : 0) * GROUPS;
            const float inv_os = (EPI == EPI_GEGLU_FP8) ? __fdiv_rn(1.0f, *p.out_scale) : 0.0f;
            const int pos = (EPI == EPI_ROPE_SPLIT && p.devpos) ? *p.devpos : 0;
#pragma unroll 2
            for (int it = threadIdx.x; it < items; it += 128) {
                const int c = cbeg + it / GROUPS;
                const int g = it % GROUPS;
                const int m = col0 + c;
                const uint32_t off = (uint32_t)(c * 128 + g * 8) * 4u;
                float a[8], b[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) a[j] = b[j] = 0.0f;
                // lanes g*8 .. g*8+7 (and, for GeGLU, the matching up lanes 64 further on)
                if (S == 1) {
                    // single split: the partials are in this CTA's own shared memory -- ordinary loads, which the
                    // compiler is free to overlap across work items
                    const float4* src = reinterpret_cast<const float4*>(&red[c * 128 + g * 8]);
                    const float4 x0 = src[0], x1 = src[1];
                    a[0] = x0.x; a[1] = x0.y; a[2] = x0.z; a[3] = x0.w;
                    a[4] = x1.x; a[5] = x1.y; a[6] = x1.z; a[7] = x1.w;
                    if (EPI == EPI_GEGLU_FP8) {
                        const float4 y0 = src[16], y1 = src[17];
                        b[0] = y0.x; b[1] = y0.y; b[2] = y0.z; b[3] = y0.w;
                        b[4] = y1.x; b[5] = y1.y; b[6] = y1.z; b[7] = y1.w;
                    }
                }
#pragma unroll
                for (uint32_t r0 = 0; r0 < 16; r0 += 2) {
                    if (S == 1 || r0 >= S) break;
                    const uint32_t ra = rank_base[r0] + off;
                    const uint32_t rb = rank_base[r0 + 1 < S ? r0 + 1 : r0] + off;
                    float4 x0, x1, y0, y1;
                    asm volatile(
                        "ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%16];\n\t"
                        "ld.shared::cluster.v4.f32 {%4,%5,%6,%7}, [%17];\n\t"
                        "ld.shared::cluster.v4.f32 {%8,%9,%10,%11}, [%18];\n\t"
                        "ld.shared::cluster.v4.f32 {%12,%13,%14,%15}, [%19];"
                        : "=f"(x0.x), "=f"(x0.y), "=f"(x0.z), "=f"(x0.w), "=f"(x1.x), "=f"(x1.y), "=f"(x1.z), "=f"(x1.w),
                          "=f"(y0.x), "=f"(y0.y), "=f"(y0.z), "=f"(y0.w), "=f"(y1.x), "=f"(y1.y), "=f"(y1.z), "=f"(y1.w)
                        : "r"(ra), "r"(ra + 16u), "r"(rb), "r"(rb + 16u));
                    a[0] += x0.x; a[1] += x0.y; a[2] += x0.z; a[3] += x0.w;
                    a[4] += x1.x; a[5] += x1.y; a[6] += x1.z; a[7] += x1.w;
                    if (r0 + 1 < S) {
                        a[0] += y0.x; a[1] += y0.y; a[2] += y0.z; a[3] += y0.w;
                        a[4] += y1.x; a[5] += y1.y; a[6] += y1.z; a[7] += y1.w;
                    }
                    if (EPI == EPI_GEGLU_FP8) {
                        asm volatile(
                            "ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%16];\n\t"
                            "ld.shared::cluster.v4.f32 {%4,%5,%6,%7}, [%17];\n\t"
                            "ld.shared::cluster.v4.f32 {%8,%9,%10,%11}, [%18];\n\t"
                            "ld.shared::cluster.v4.f32 {%12,%13,%14,%15}, [%19];"
                            : "=f"(x0.x), "=f"(x0.y), "=f"(x0.z), "=f"(x0.w), "=f"(x1.x), "=f"(x1.y), "=f"(x1.z), "=f"(x1.w),
                              "=f"(y0.x), "=f"(y0.y), "=f"(y0.z), "=f"(y0.w), "=f"(y1.x), "=f"(y1.y), "=f"(y1.z), "=f"(y1.w)
                            : "r"(ra + 256u), "r"(ra + 272u), "r"(rb + 256u), "r"(rb + 272u));
                        b[0] += x0.x; b[1] += x0.y; b[2] += x0.z; b[3] += x0.w;
                        b[4] += x1.x; b[5] += x1.y; b[6] += x1.z; b[7] += x1.w;
                        if (r0 + 1 < S) {
                            b[0] += y0.x; b[1] += y0.y; b[2] += y0.z; b[3] += y0.w;
                            b[4] += y1.x; b[5] += y1.y; b[6] += y1.z; b[7] += y1.w;
                        }
                    }
                }
                if (EPI == EPI_BF16) {
                    const int n = lane0 + g * 8;
                    float f[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const bool hb = p.bias && n + j < p.N;
                        f[j] = scale_bias(a[j], alpha, hb ? __bfloat162float(p.bias[n + j]) : 0.0f, hb);
                    }
                    __nv_bfloat16* dst = p.out + (size_t)m * p.N + n;
                    if (n + 8 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                        uint4 o;
                        o.x = pack_bf16x2(f[0], f[1]);
                        o.y = pack_bf16x2(f[2], f[3]);
                        o.z = pack_bf16x2(f[4], f[5]);
                        o.w = pack_bf16x2(f[6], f[7]);
                        st_global_v4(dst, o);
                    } else {
                        for (int j = 0; j < 8; ++j)
                            if (n + j < p.N) dst[j] = __float2bfloat16_rn(f[j]);
                    }
                } else if (EPI == EPI_ROPE_SPLIT) {
                    // same rounding points as the separate kernels: bf16 GEMM result, fp32 rotation, bf16 store
                    const int n = lane0 + g * 8;                     // 8 features of the fused q|k|v row
                    if (n >= p.N) continue;
                    float v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(a[j] * alpha));
                    const bool is_q = n < p.q_dim;
                    const bool is_k = !is_q && n < p.q_dim + p.k_dim;
                    const int nr = is_q ? n : (is_k ? n - p.q_dim : n - p.q_dim - p.k_dim);
                    uint4 o;
                    if (is_q || is_k) {
                        const uint4 t = ld_global_v4(p.rope + (size_t)m * p.head_dim + (nr % p.head_dim));
                        const uint32_t* tw = &t.x;
                        uint32_t* ow = &o.x;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float cs, sn;
                            unpack_bf16x2(tw[k], cs, sn);
                            ow[k] = pack_bf16x2(__fmaf_rn(v[2 * k], cs, -__fmul_rn(v[2 * k + 1], sn)),
                                                __fmaf_rn(v[2 * k + 1], cs, __fmul_rn(v[2 * k], sn)));
                        }
                    } else {
                        o.x = pack_bf16x2(v[0], v[1]);
                        o.y = pack_bf16x2(v[2], v[3]);
                        o.z = pack_bf16x2(v[4], v[5]);
                        o.w = pack_bf16x2(v[6], v[7]);
                    }
                    __nv_bfloat16* dst = is_q ? p.outQ + (size_t)m * p.q_dim + nr
                                              : (is_k ? p.outK + (size_t)(pos + m) * p.k_dim + nr
                                                      : p.outV + (size_t)(pos + m) * p.v_dim + nr);
                    st_global_v4(dst, o);
                } else {
                    // GeGLU: a = gate partial sums (lanes g*8..), b = up partial sums (lanes 64 + g*8..)
                    const int h = lane0 + g * 8;
                    if (h >= p.half) continue;
                    float q[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float gt = __bfloat162float(__float2bfloat16_rn(a[j] * alpha));
                        const float up = __bfloat162float(__float2bfloat16_rn(b[j] * alpha));
                        q[j] = clamp448(__fmul_rn(__fmul_rn(det_gelu_tanh(gt), up), inv_os));
                    }
                    uint2 o8;
                    o8.x = f32x4_to_e4m3x4(q[0], q[1], q[2], q[3]);
                    o8.y = f32x4_to_e4m3x4(q[4], q[5], q[6], q[7]);
                    st_global_v2(p.out8 + (size_t)m * p.half + h, o8);
                }
            }
        } else if (!*abort_flag) {
            // large-M kernel with split-K: lanes = rows m, columns = n (scalar, rarely used)
            const uint32_t red_addr = tc::smem_u32(red);
            uint32_t rank_base[16];
#pragma unroll
            for (int r = 0; r < 16; ++r) rank_base[r] = tc::dsmem_map(red_addr, (uint32_t)r < S ? r : 0);
            const int cols_per = (BN + (int)S - 1) / (int)S;
            const int cbeg = (int)rank * cols_per;
            const int cend = cbeg + cols_per < BN ? cbeg + cols_per : BN;
            const int tl = warp * 32 + lane;
            for (int c = cbeg; c < cend; ++c) {
                const int gcol = col0 + c;
                if (gcol >= p.N) break;
                const float acc = reduce_ranks<16>(rank_base, S, (uint32_t)(c * 128 + tl) * 4u);
                if (lrow < p.M) {
                    const float f = scale_bias(acc, alpha, p.bias ? __bfloat162float(p.bias[gcol]) : 0.0f, p.bias != nullptr);
                    p.out[(size_t)lrow * p.N + gcol] = __float2bfloat16_rn(f);
                }
            }
        }
        if (S > 1 || EPI == EPI_GATE_RES_NORM_FP8) tc::cluster_sync_all();
    }

    // ---------------- teardown
    tc::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // give copies that were issued but never consumed a bounded chance to land
        for (int i = *consumed; i < *issued; ++i) {
            const int s = i % STAGES;
            for (int it = 0; it < 4096; ++it) {
                if (tc::mbar_try_wait(&full[s], (i / STAGES) & 1)) break;
                __nanosleep(256);
            }
        }
    }
    __syncthreads();
    if (warp == 2) tc::tmem_dealloc(tmem_d, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------ host launch
struct TmapKey {
    const void* base; uint64_t rows, row_bytes, pitch; uint32_t box_rows;
    bool operator==(const TmapKey& o) const {
        return base == o.base && rows == o.rows && row_bytes == o.row_bytes && pitch == o.pitch && box_rows == o.box_rows;
    }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey& k) const {
        size_t h = std::hash<const void*>()(k.base);
        h ^= k.rows * 0x9e3779b97f4a7c15ull + (h << 6);
        h ^= k.row_bytes * 0xc2b2ae3d27d4eb4full + (h >> 3);
        h ^= (k.pitch << 8) ^ k.box_rows;
        return h;
    }
};
static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmaps;

int get_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t pitch,
                   uint32_t box_rows) {
    TmapKey k{base, rows, row_bytes, pitch, box_rows};
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_tmaps.find(k);
        if (it != g_tmaps.end()) { *out = it->second; return FRT_OK; }
    }
    int rc = make_tmap_2d_u8(out, base, rows, row_bytes, pitch, box_rows);
    if (rc) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_tmaps.size() > 65536) g_tmaps.clear();
    g_tmaps[k] = *out;
    return FRT_OK;
}

// K counts elements; a row holds K bytes (FP8) or K / 2 bytes (packed NVFP4)
template <int BN, bool SWAP, int EPI, bool FP4 = false>
static int launch_gemm(const void* A, const void* W, GemmParams p, int K, int splits, bool pdl, cudaStream_t stream) {
    using Cfg = GemmCfg<BN, FP4>;
    static PerDeviceOnce attr_once;
    int attr_dev = 0;
    if (attr_once.need(attr_dev)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel<BN, SWAP, EPI, FP4>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        e = cudaFuncSetAttribute(gemm_fp8_kernel<BN, SWAP, EPI, FP4>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        attr_once.set(attr_dev);
    }
    const void* lane_ptr = SWAP ? W : A;
    const void* col_ptr = SWAP ? A : W;
    p.lane_rows = SWAP ? p.N : p.M;
    p.col_rows = SWAP ? p.M : p.N;
    p.w_is_lane = SWAP ? 1 : 0;
    if (FP4) {
        if (SWAP) { const uint8_t* t = p.sf_lane; p.sf_lane = p.sf_col; p.sf_col = t; }   // callers pass (A, W) order
        p.sf_katoms = K / 64;
        p.sf_col_rblocks = (p.col_rows + 127) / 128;
    }
    const uint64_t row_bytes = FP4 ? (uint64_t)K / 2 : (uint64_t)K;
    CUtensorMap tmL, tmC;
    int rc = get_tmap_2d_u8(&tmL, lane_ptr, (uint64_t)p.lane_rows, row_bytes, row_bytes,
                            EPI == EPI_GEGLU_FP8 ? 64 : 128);
    if (rc) return rc;
    rc = get_tmap_2d_u8(&tmC, col_ptr, (uint64_t)p.col_rows, row_bytes, row_bytes, BN);
    if (rc) return rc;

    const int lane_tiles = EPI == EPI_GEGLU_FP8 ? (p.half + 63) / 64 : (p.lane_rows + 127) / 128;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(lane_tiles, (p.col_rows + BN - 1) / BN, splits);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = splits;
    ++na;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_fp8_kernel<BN, SWAP, EPI, FP4>, tmL, tmC, p);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}

// Split-K factor.  Measured on B200 at M = 50 (graph of back-to-back launches): the cluster exchange costs about
// as much as streaming 64 KB per CTA, so splitting pays only while it at least halves the bytes per CTA and the
// grid still fits well inside one wave; clusters larger than 4 were never faster.
static int pick_splits(int tiles, int kb_total, int requested) {
    if (requested > 0) {
        int s = requested > 16 ? 16 : requested;
        return s > kb_total ? kb_total : s;
    }
    int s = 1;
    while (s < 4 && tiles * s * 2 <= 120 && s * 2 <= kb_total) s *= 2;
    return s;
}

// fused projection + gated residual + adaRMS + FP8: one cluster of (N / 128 tiles) x S CTAs
static int launch_gemm_gate_res_norm(const void* A, const void* W, GemmParams p, int K, int splits, bool pdl,
                                     cudaStream_t stream) {
    constexpr int BN = 64;
    using Cfg = GemmCfg<BN>;
    auto kern = gemm_fp8_kernel<BN, true, EPI_GATE_RES_NORM_FP8>;
    static PerDeviceOnce attr_once;
    int attr_dev = 0;
    if (attr_once.need(attr_dev)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        attr_once.set(attr_dev);
    }
    p.lane_rows = p.N;
    p.col_rows = p.M;
    p.w_is_lane = 1;
    CUtensorMap tmL, tmC;
    int rc = get_tmap_2d_u8(&tmL, W, (uint64_t)p.N, (uint64_t)K, (uint64_t)K, 128);
    if (rc) return rc;
    rc = get_tmap_2d_u8(&tmC, A, (uint64_t)p.M, (uint64_t)K, (uint64_t)K, BN);
    if (rc) return rc;
    const int tiles = p.N / 128;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, 1, splits);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = tiles;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = splits;
    ++na;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmL, tmC, p);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}

template <int EPI>
static int dispatch_small_m(const void* A, const void* W, GemmParams p, int K, int M, int tiles, int splits,
                            bool pdl, cudaStream_t s) {
    int sp = pick_splits(tiles, p.kb_total, splits);
    if (M <= 16) return launch_gemm<16, true, EPI>(A, W, p, K, sp, pdl, s);
    if (M <= 32) return launch_gemm<32, true, EPI>(A, W, p, K, sp, pdl, s);
    if (M <= 64) return launch_gemm<64, true, EPI>(A, W, p, K, sp, pdl, s);
    if (M <= 128) return launch_gemm<128, true, EPI>(A, W, p, K, sp, pdl, s);
    return launch_gemm<256, true, EPI>(A, W, p, K, sp, pdl, s);
}

#include "gemm_persistent.cuh"
#include "gemm_pair.cuh"
#include "gemm_tok.cuh"

template <int EPI>
static int dispatch_small_m_nvfp4(const void* A, const void* W, GemmParams p, int K, int M, int tiles, int splits,
                                  bool pdl, cudaStream_t s) {
    int sp = pick_splits(tiles, p.kb_total, splits);
    if (M <= 32) return launch_gemm<32, true, EPI, true>(A, W, p, K, sp, pdl, s);
    if (M <= 64) return launch_gemm<64, true, EPI, true>(A, W, p, K, sp, pdl, s);
    if (M <= 128) return launch_gemm<128, true, EPI, true>(A, W, p, K, sp, pdl, s);
    return launch_gemm<256, true, EPI, true>(A, W, p, K, sp, pdl, s);
}

}  // namespace frt

using namespace frt;

// flags bits 8-9: tile-width hint of the token-major small-M kernel (1 = 64, 2 = 128, 3 = 256 weight rows)
static inline int tok_bn_hint(int flags) {
    const int h = (flags >> 8) & 3;
    return h == 1 ? 64 : h == 2 ? 128 : h == 3 ? 256 : 0;
}
static inline int tok_split_hint(int splits) {
    return (splits == 1 || splits == 2 || splits == 4 || splits == 8) ? splits : 0;
}
// the token-major kernel serves up to 128 rows (one accumulator tile: the weights stream once), K in whole 128-byte
// k-blocks, 16-byte output rows; flags bit 4 keeps the swapped (weights-on-lanes) kernel.  With a pinned tile width or
// split it also takes 129..256 rows (two row tiles; measured slower than the swapped kernel there).
static inline bool tok_eligible(int M, int N, int K, int flags, int splits = 0) {
    const bool pinned = ((flags >> 8) & 3) != 0 || splits == 1 || splits == 2 || splits == 4 || splits == 8;
    return (M <= 128 || (M <= 256 && pinned)) && (K % 128) == 0 && (N % 8) == 0 && !(flags & 16);
}

extern "C" {

// D(M,N) bf16 = alpha_host * (*d_scale_a) * (*d_scale_b) * A(M,K) . W(N,K)^T + bias
// A, W: FP8 E4M3 row-major, K contiguous.  K % 16 == 0; A, W 16-byte aligned.
// splits: 0 = choose, otherwise the split-K factor (clamped to [1, 8]).
// flags: bit0 = programmatic dependent launch; bit1 = one-tile-per-CTA kernel for M > 256; bit3 = force the CTA-pair
// kernel (256 x 256 tiles, M > 256, N >= 256, no split-K; chosen by itself for long tile lists), bit5 = never use it.
int frt_b200_gemm_fp8_nt(const void* A, const void* W, void* D, int M, int N, int K, const float* d_scale_a,
                         const float* d_scale_b, float alpha_host, const void* bias, int splits, int flags,
                         void* stream) {
    if (!A || !W || !D || M < 0 || N <= 0 || K <= 0) return FRT_ERR_INVALID;
    if (K % 16) return FRT_ERR_UNSUPPORTED;
    if (M == 0) return FRT_OK;
    GemmParams p = {};
    p.out = (__nv_bfloat16*)D;
    p.sa = d_scale_a;
    p.sb = d_scale_b;
    p.alpha_host = alpha_host;
    p.bias = (const __nv_bfloat16*)bias;
    p.M = M;
    p.N = N;
    p.kb_total = (K + 127) / 128;
    cudaStream_t s = (cudaStream_t)stream;
    bool pdl = flags & 1;
    if (tok_eligible(M, N, K, flags, splits)) {
        TokParams t = {};
        t.M = M; t.N = N; t.sa = d_scale_a; t.sb = d_scale_b; t.alpha_host = alpha_host;
        t.out = (__nv_bfloat16*)D; t.bias = (const __nv_bfloat16*)bias;
        int rc = dispatch_gemm_tok<TOK_PRO_TMA, TOK_EPI_BF16>(A, W, t, K, tok_bn_hint(flags), tok_split_hint(splits), pdl, s);
        if (rc != FRT_ERR_UNSUPPORTED) return rc;
    }
    if (M <= 256) return dispatch_small_m<EPI_BF16>(A, W, p, K, M, (N + 127) / 128, splits, pdl, s);
    int sp = splits > 0 ? pick_splits(1, p.kb_total, splits > 8 ? 8 : splits) : 1;
    // One 256 x 256 tile per CTA pair (cta_group::2): measured 3-10 % faster than the one-CTA persistent kernel once
    // the tile list fills at least two waves of pairs and K >= 2048 (e.g. 20480 x 14336 x 3072: 698 vs 744 us), a few
    // percent slower on short lists and at K = 1024.  flags bit 3 forces it, flags bit 5 keeps the one-CTA kernel.
    const long long tiles256 = (long long)((M + 255) / 256) * ((N + 255) / 256);
    const bool pair_pays = tiles256 >= 148 && K >= 2048 && !(flags & 32) && !(flags & 2);
    if (sp == 1 && ((flags & 8) || pair_pays) && N >= 256) return launch_gemm_pair(A, W, p, K, pdl, s);
    if (sp == 1 && !(flags & 2)) {      // flags bit1 keeps the one-tile-per-CTA kernel (for comparison runs)
        // 128-column tiles only where the 256-column tile list leaves more than half of the SMs idle (2048 x 1024: 64
        // wide tiles for 148 SMs: 9.6 -> 8.6 us); from one wave on the wide tile wins (2048 x 3072 x 3072: 24.9 us wide,
        // 32.4 us narrow)
        const long long wide_tiles = (long long)((M + 127) / 128) * ((N + 255) / 256);
        const bool narrow = N > 64 && wide_tiles * 2 <= device_sm_count();
        if (N >= 256 && !narrow) return launch_gemm_persistent<256, EPI_P_BF16>(A, W, p, K, pdl, s);
        if (N > 64) return launch_gemm_persistent<128, EPI_P_BF16>(A, W, p, K, pdl, s);
    }
    if (N >= 256) return launch_gemm<256, false, EPI_BF16>(A, W, p, K, sp, pdl, s);
    if (N > 64) return launch_gemm<128, false, EPI_BF16>(A, W, p, K, sp, pdl, s);
    return launch_gemm<64, false, EPI_BF16>(A, W, p, K, sp, pdl, s);
}

// The same product with the weights stored (K, N) row-major -- GemmRunner::fp8_nn_dev, the reference's default
// ("kn") layout (csrc/bindings.cpp:706-716, flash_rt/models/pi05/pipeline_rtx.py:550-562):
//   D(M,N) bf16 = alpha_host * (*d_scale_a) * (*d_scale_b) * A(M,K) . B(K,N) + bias.
// The weight tiles arrive as boxes of 128 K-rows x 128 N-bytes and feed the MMA as an MN-major operand; accumulation
// order and result are those of frt_b200_gemm_fp8_nt on the transposed weights (bit for bit).  K % 128 == 0,
// N % 16 == 0; M <= 256 runs the token-major kernel, larger M the persistent kernel (N >= 128).
int frt_b200_gemm_fp8_nn(const void* A, const void* B, void* D, int M, int N, int K, const float* d_scale_a,
                         const float* d_scale_b, float alpha_host, const void* bias, int splits, int flags,
                         void* stream) {
    if (!A || !B || !D || M < 0 || N <= 0 || K <= 0) return FRT_ERR_INVALID;
    if ((K % 128) || (N % 16) || N < 128) return FRT_ERR_UNSUPPORTED;
    if (M == 0) return FRT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool pdl = flags & 1;
    if (M <= 256) {
        TokParams t = {};
        t.M = M; t.N = N; t.sa = d_scale_a; t.sb = d_scale_b; t.alpha_host = alpha_host;
        t.out = (__nv_bfloat16*)D; t.bias = (const __nv_bfloat16*)bias; t.w_kn = 1;
        return dispatch_gemm_tok<TOK_PRO_TMA, TOK_EPI_BF16>(A, B, t, K, tok_bn_hint(flags), tok_split_hint(splits), pdl, s);
    }
    GemmParams p = {};
    p.out = (__nv_bfloat16*)D;
    p.sa = d_scale_a;
    p.sb = d_scale_b;
    p.alpha_host = alpha_host;
    p.bias = (const __nv_bfloat16*)bias;
    p.M = M;
    p.N = N;
    p.kb_total = K / 128;
    p.w_kn = 1;
    if (N >= 256) return launch_gemm_persistent<256, EPI_P_BF16>(A, B, p, K, pdl, s);
    return launch_gemm_persistent<128, EPI_P_BF16>(A, B, p, K, pdl, s);
}

// QKV projection with the RoPE + split + KV-append epilogue fused (M <= 256):
//   row = alpha * A(M,K) . W(N,K)^T rounded to bf16, N = q_dim + k_dim + v_dim; q and k parts rotated pairwise
//   with rope (M, head_dim) = [cos0, sin0, ...]; Q -> (M, q_dim); K, V rows -> row (*devpos + m) (devpos NULL: m).
// Byte-identical to frt_b200_gemm_fp8_nt followed by frt_b200_qkv_split_rope.
int frt_b200_gemm_fp8_nt_rope_split(const void* A, const void* W, int M, int K, const float* d_scale_a,
                                    const float* d_scale_b, const void* rope, void* Q, void* Kout, void* Vout,
                                    const int* devpos, int q_dim, int k_dim, int v_dim, int head_dim, int splits,
                                    int flags, void* stream) {
    if (!A || !W || !rope || !Q || !Kout || !Vout || M < 0 || K <= 0) return FRT_ERR_INVALID;
    if (q_dim <= 0 || k_dim <= 0 || v_dim <= 0 || head_dim <= 0) return FRT_ERR_INVALID;
    if ((K % 16) || M > 256 || (head_dim & 1) || (q_dim % head_dim) || (k_dim % head_dim) || (q_dim & 1) ||
        (k_dim & 1))
        return FRT_ERR_UNSUPPORTED;
    if (M == 0) return FRT_OK;
    GemmParams p = {};
    p.sa = d_scale_a;
    p.sb = d_scale_b;
    p.alpha_host = 1.0f;
    p.M = M;
    p.N = q_dim + k_dim + v_dim;
    p.kb_total = (K + 127) / 128;
    p.rope = (const __nv_bfloat16*)rope;
    p.outQ = (__nv_bfloat16*)Q;
    p.outK = (__nv_bfloat16*)Kout;
    p.outV = (__nv_bfloat16*)Vout;
    p.devpos = devpos;
    p.q_dim = q_dim;
    p.k_dim = k_dim;
    p.v_dim = v_dim;
    p.head_dim = head_dim;
    if (tok_eligible(M, p.N, K, flags) && M <= 128 && (head_dim % 8) == 0) {
        TokParams t = {};
        t.M = M; t.N = p.N; t.sa = d_scale_a; t.sb = d_scale_b; t.alpha_host = 1.0f;
        t.rope = p.rope; t.outQ = p.outQ; t.outK = p.outK; t.outV = p.outV; t.devpos = devpos;
        t.q_dim = q_dim; t.k_dim = k_dim; t.v_dim = v_dim; t.head_dim = head_dim;
        int rc = dispatch_gemm_tok<TOK_PRO_TMA, TOK_EPI_ROPE>(A, W, t, K, tok_bn_hint(flags), tok_split_hint(splits),
                                                             flags & 1, (cudaStream_t)stream);
        if (rc != FRT_ERR_UNSUPPORTED) return rc;
    }
    return dispatch_small_m<EPI_ROPE_SPLIT>(A, W, p, K, M, (p.N + 127) / 128, splits, flags & 1, (cudaStream_t)stream);
}

// gate|up projection with the GeGLU -> FP8 epilogue fused (M <= 256):
//   W (2*half, K): rows [0, half) = gate, [half, 2*half) = up.  out8 (M, half) =
//   e4m3(clamp(gelu_tanh(bf16(gate)) * bf16(up) * (1 / *d_out_scale), +-448)).  half % 64 == 0.
// Byte-identical to frt_b200_gemm_fp8_nt followed by frt_b200_geglu_fp8.  flags bit 6: SiLU gate instead of GELU
// (SwiGLU; M <= 128, K % 128 == 0: the token-major kernel), byte-identical to frt_b200_geglu_fp8 with its bit 1.
int frt_b200_gemm_fp8_nt_geglu_fp8(const void* A, const void* W, void* out8, int M, int half, int K,
                                   const float* d_scale_a, const float* d_scale_b, const float* d_out_scale,
                                   int splits, int flags, void* stream) {
    if (!A || !W || !out8 || !d_out_scale || M < 0 || half <= 0 || K <= 0) return FRT_ERR_INVALID;
    if ((K % 16) || M > 256 || (half % 64)) return FRT_ERR_UNSUPPORTED;
    if (M == 0) return FRT_OK;
    GemmParams p = {};
    p.sa = d_scale_a;
    p.sb = d_scale_b;
    p.alpha_host = 1.0f;
    p.M = M;
    p.N = 2 * half;
    p.kb_total = (K + 127) / 128;
    p.out8 = (uint8_t*)out8;
    p.out_scale = d_out_scale;
    p.half = half;
    // SiLU gate (bit 6) and the hardware-tanh GELU (bit 7): built in the token-major kernel only
    const bool silu = (flags & 64) != 0, fast = (flags & 128) != 0;
    if (silu && fast) return FRT_ERR_INVALID;
    if ((silu || fast) && !(tok_eligible(M, p.N, K, flags) && M <= 128)) return FRT_ERR_UNSUPPORTED;
    if (tok_eligible(M, p.N, K, flags) && M <= 128 && (half % 64) == 0) {
        TokParams t = {};
        t.M = M; t.N = p.N; t.sa = d_scale_a; t.sb = d_scale_b; t.alpha_host = 1.0f;
        t.out8 = (uint8_t*)out8; t.out_scale = d_out_scale; t.half = half; t.gate_act = silu ? 1 : fast ? 2 : 0;
        int rc = dispatch_gemm_tok<TOK_PRO_TMA, TOK_EPI_GEGLU>(A, W, t, K, tok_bn_hint(flags), tok_split_hint(splits),
                                                              flags & 1, (cudaStream_t)stream);
        if (rc != FRT_ERR_UNSUPPORTED || silu || fast) return rc;
    }
    return dispatch_small_m<EPI_GEGLU_FP8>(A, W, p, K, M, half / 64, splits, flags & 1, (cudaStream_t)stream);
}

// NVFP4 block-scaled GEMM: D(M,N) bf16 = alpha * (*d_alpha) * (A . SFA)(M,K) . (W . SFW)(N,K)^T + bias.
// A, W: packed e2m1, two per byte, K contiguous (row = K / 2 bytes); SFA, SFW: unsigned-E4M3 scales per 16
// elements in 512-byte atoms of 128 rows x 4 blocks (frt_b200_nvfp4_sf_bytes; padding zero-filled).
// K % 256 == 0.  d_alpha: optional device float (e.g. the product of two FP32 global scales).
int frt_b200_gemm_nvfp4_nt(const void* A, const void* SFA, const void* W, const void* SFW, void* D, int M, int N,
                           int K, float alpha, const float* d_alpha, const void* bias, int splits, int flags,
                           void* stream) {
    if (!A || !SFA || !W || !SFW || !D || M < 0 || N <= 0 || K <= 0) return FRT_ERR_INVALID;
    if (K % 256) return FRT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(SFA) & 15) || (reinterpret_cast<uintptr_t>(SFW) & 15)) return FRT_ERR_INVALID;
    if (M == 0) return FRT_OK;
    GemmParams p = {};
    p.out = (__nv_bfloat16*)D;
    p.sa = d_alpha;
    p.alpha_host = alpha;
    p.bias = (const __nv_bfloat16*)bias;
    p.M = M;
    p.N = N;
    p.kb_total = K / 256;
    p.sf_lane = (const uint8_t*)SFA;
    p.sf_col = (const uint8_t*)SFW;
    cudaStream_t s = (cudaStream_t)stream;
    bool pdl = flags & 1;
    if (M <= 256) return dispatch_small_m_nvfp4<EPI_BF16>(A, W, p, K, M, (N + 127) / 128, splits, pdl, s);
    int sp = splits > 0 ? pick_splits(1, p.kb_total, splits > 8 ? 8 : splits) : 1;
    // Persistent kernel with two 128-column accumulators: measured faster than the 128 x 256 one-tile kernel while
    // the per-tile prologue / epilogue dominates (K < 3072); at larger K the wider tile's lower operand traffic wins.
    if (sp == 1 && N > 64 && !(flags & 2) && (K < 3072 || N < 256 || (flags & 4)))
        return launch_gemm_persistent<128, EPI_P_BF16, true>(A, W, p, K, pdl, s);
    if (N >= 256) return launch_gemm<256, false, EPI_BF16, true>(A, W, p, K, sp, pdl, s);
    if (N > 64) return launch_gemm<128, false, EPI_BF16, true>(A, W, p, K, sp, pdl, s);
    return launch_gemm<64, false, EPI_BF16, true>(A, W, p, K, sp, pdl, s);
}

// NVFP4 QKV projection with the RoPE + split + KV-append epilogue (M <= 256); arguments as
// frt_b200_gemm_fp8_nt_rope_split with the operand scales replaced by the block-scale buffers.
int frt_b200_gemm_nvfp4_nt_rope_split(const void* A, const void* SFA, const void* W, const void* SFW, int M, int K,
                                      float alpha, const void* rope, void* Q, void* Kout, void* Vout,
                                      const int* devpos, int q_dim, int k_dim, int v_dim, int head_dim, int splits,
                                      int flags, void* stream) {
    if (!A || !SFA || !W || !SFW || !rope || !Q || !Kout || !Vout || M < 0 || K <= 0) return FRT_ERR_INVALID;
    if (q_dim <= 0 || k_dim <= 0 || v_dim <= 0 || head_dim <= 0) return FRT_ERR_INVALID;
    if ((K % 256) || M > 256 || (head_dim & 1) || (q_dim % head_dim) || (k_dim % head_dim) || (q_dim & 1) ||
        (k_dim & 1))
        return FRT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(SFA) & 15) || (reinterpret_cast<uintptr_t>(SFW) & 15)) return FRT_ERR_INVALID;
    if (M == 0) return FRT_OK;
    GemmParams p = {};
    p.alpha_host = alpha;
    p.M = M;
    p.N = q_dim + k_dim + v_dim;
    p.kb_total = K / 256;
    p.sf_lane = (const uint8_t*)SFA;
    p.sf_col = (const uint8_t*)SFW;
    p.rope = (const __nv_bfloat16*)rope;
    p.outQ = (__nv_bfloat16*)Q;
    p.outK = (__nv_bfloat16*)Kout;
    p.outV = (__nv_bfloat16*)Vout;
    p.devpos = devpos;
    p.q_dim = q_dim;
    p.k_dim = k_dim;
    p.v_dim = v_dim;
    p.head_dim = head_dim;
    return dispatch_small_m_nvfp4<EPI_ROPE_SPLIT>(A, W, p, K, M, (p.N + 127) / 128, splits, flags & 1,
                                                  (cudaStream_t)stream);
}

// Row-parallel projection of the action expert with the following norm kernel fused (M <= 64, N = 128 .. 1024):
//   o = bf16(sa * sb * A . W^T); residual <- bf16(residual + o * gate); rms over the N features of each row;
//   out8 = e4m3(clamp(((residual * rms) * (1 + scale) + shift) * (1 / *d_out_scale), +-448)),
//   gate (N,) and style = [scale (N) | shift (N)] shared by all rows.  Stands for frt_b200_gemm_fp8_nt followed by
//   frt_b200_norm_fp8 (gate_residual_ada_norm_fp8) with unit norm weight: same rounding points; the row sum of
//   squares is accumulated in a different (fixed) order, so FP8 codes may differ in the last place on rare rows.
// splits: 1 or 2 (0 = 2 when K >= 2048).
int frt_b200_gemm_fp8_nt_gate_res_norm_fp8(const void* A, const void* W, int M, int N, int K, const float* d_scale_a,
                                           const float* d_scale_b, void* residual, const void* gate, const void* style,
                                           void* out8, const float* d_out_scale, float eps, int splits, int flags,
                                           void* stream) {
    if (!A || !W || !residual || !gate || !style || !out8 || !d_out_scale || M < 0 || N <= 0 || K <= 0)
        return FRT_ERR_INVALID;
    if ((K % 16) || M > 64 || (N % 128) || N > 1024) return FRT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(residual) & 15) || (reinterpret_cast<uintptr_t>(gate) & 15) ||
        (reinterpret_cast<uintptr_t>(style) & 15) || (reinterpret_cast<uintptr_t>(out8) & 7))
        return FRT_ERR_INVALID;
    if (M == 0) return FRT_OK;
    GemmParams p = {};
    p.sa = d_scale_a;
    p.sb = d_scale_b;
    p.alpha_host = 1.0f;
    p.M = M;
    p.N = N;
    p.kb_total = (K + 127) / 128;
    p.resid = (__nv_bfloat16*)residual;
    p.gate = (const __nv_bfloat16*)gate;
    p.style = (const __nv_bfloat16*)style;
    p.out8 = (uint8_t*)out8;
    p.out_scale = d_out_scale;
    p.eps = eps;
    int sp = splits > 0 ? (splits > 2 ? 2 : splits) : (K >= 2048 ? 2 : 1);
    if (sp > p.kb_total) sp = p.kb_total;
    return launch_gemm_gate_res_norm(A, W, p, K, sp, flags & 1, (cudaStream_t)stream);
}

// FFN-up projection with bias + GELU(tanh) + FP8 quantise in the epilogue (M > 256):
//   out8 (M, N) e4m3 = clamp(gelu_tanh(bf16(alpha * A . W^T) + bias) * (1 / *d_out_scale), +-448)
// Byte-identical to frt_b200_gemm_fp8_nt followed by frt_b200_bias_gelu_quantize_fp8.  N % 8 == 0.
int frt_b200_gemm_fp8_nt_bias_gelu_fp8(const void* A, const void* W, void* out8, int M, int N, int K,
                                       const float* d_scale_a, const float* d_scale_b, const void* bias,
                                       const float* d_out_scale, int flags, void* stream) {
    if (!A || !W || !out8 || !d_out_scale || M < 0 || N <= 0 || K <= 0) return FRT_ERR_INVALID;
    if ((K % 16) || (N % 8) || M <= 256 || N < 128) return FRT_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(out8) & 7) return FRT_ERR_INVALID;
    GemmParams p = {};
    p.sa = d_scale_a;
    p.sb = d_scale_b;
    p.alpha_host = 1.0f;
    p.bias = (const __nv_bfloat16*)bias;
    p.M = M;
    p.N = N;
    p.kb_total = (K + 127) / 128;
    p.out8 = (uint8_t*)out8;
    p.out_scale = d_out_scale;
    p.fast_act = (flags & 128) ? 1 : 0;
    if (p.fast_act) {
        if (N >= 256)
            return launch_gemm_persistent<256, EPI_P_BIAS_GELU_FAST_FP8>(A, W, p, K, flags & 1, (cudaStream_t)stream);
        return launch_gemm_persistent<128, EPI_P_BIAS_GELU_FAST_FP8>(A, W, p, K, flags & 1, (cudaStream_t)stream);
    }
    if (N >= 256) return launch_gemm_persistent<256, EPI_P_BIAS_GELU_FP8>(A, W, p, K, flags & 1, (cudaStream_t)stream);
    return launch_gemm_persistent<128, EPI_P_BIAS_GELU_FP8>(A, W, p, K, flags & 1, (cudaStream_t)stream);
}

// Row-parallel projection with the gated residual update fused (M <= 128, N % 64 == 0, K % 128 == 0):
//   o = bf16(sa * sb * A . W^T);  residual(M, N) <- bf16(residual + o * gate),  gate (N,) shared by all rows;
//   stats_out[tile][m] (row pitch 128 floats, N / tile_width rows; may be NULL) = sum over the tile's features of the
//   squares of the UNROUNDED updated residual -- the first pass of gate_residual_ada_norm_fp8
//   (csrc/kernels/fusion.cu:41-47); frt_b200_norm_gemm_fp8_nt_* finishes the norm inside the next projection.
// *stat_tiles (host int, may be NULL) receives the number of statistics rows written.
// The same launch, which also leaves the next projection's FP8 operand WITHOUT the 1 / rms factor of the norm between
// them (q8_out may be NULL: then exactly the entry point above):
//   q8_out[m][n] = e4m3(clamp(bf16(residual[m][n]) * (1 + next_scale[n]) / *d_q8_scale, +-448)),
// next_scale = the scale third of the NEXT adaRMS style row (N bf16).  A row's 1 / rms commutes with the projection
//   W . (rms * x * (1 + scale) + shift) = rms * (W . (x * (1 + scale))) + W . shift,
// so frt_b200_gemm_fp8_nt_*_rowscale applies it, and the precomputed W . shift, in its finish: no CTA of the next
// projection waits for the row statistics before its MMAs.  Stands for gate_residual_ada_norm_fp8
// (csrc/kernels/fusion.cu:15-81) with the quantisation point moved in front of the row scale; E4M3 is a floating-point
// format, so the relative rounding error of an element is the same on either side of the scale.
int frt_b200_gemm_fp8_nt_gate_residual_q8(const void* A, const void* W, int M, int N, int K, const float* d_scale_a,
                                          const float* d_scale_b, void* residual, const void* gate, float* stats_out,
                                          int* stat_tiles, const void* next_scale, void* q8_out,
                                          const float* d_q8_scale, int splits, int flags, void* stream) {
    if (!A || !W || !residual || !gate || M < 0 || N <= 0 || K <= 0) return FRT_ERR_INVALID;
    if (q8_out && (!next_scale || !d_q8_scale)) return FRT_ERR_INVALID;
    if ((K % 128) || M > 128 || (N % 64)) return FRT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(residual) & 15) || (reinterpret_cast<uintptr_t>(gate) & 15)) return FRT_ERR_INVALID;
    if (q8_out && ((reinterpret_cast<uintptr_t>(q8_out) & 7) || (reinterpret_cast<uintptr_t>(next_scale) & 15)))
        return FRT_ERR_INVALID;
    TokParams t = {};
    t.M = M; t.N = N; t.sa = d_scale_a; t.sb = d_scale_b; t.alpha_host = 1.0f;
    t.resid = (__nv_bfloat16*)residual; t.gate = (const __nv_bfloat16*)gate; t.stats_out = stats_out;
    t.q8_out = (uint8_t*)q8_out; t.q8_mod = (const __nv_bfloat16*)next_scale; t.q8_scale = d_q8_scale;
    TokPlan pl;
    int bn = tok_bn_hint(flags);
    if (bn == 0 && (N % 128)) bn = 64;
    if (!tok_plan(N, K, 1, M < 128 ? (M > 0 ? M : 1) : 128, TOK_EPI_RESID, TOK_PRO_TMA, tok_sm_count(), bn,
                  tok_split_hint(splits), &pl))
        return FRT_ERR_UNSUPPORTED;
    if (stat_tiles) *stat_tiles = N / pl.BN;
    if (M == 0) return FRT_OK;
    if (pl.BN == 128)
        return launch_gemm_tok<128, TOK_PRO_TMA, TOK_EPI_RESID>(A, W, t, K, pl, flags & 1, (cudaStream_t)stream);
    return launch_gemm_tok<64, TOK_PRO_TMA, TOK_EPI_RESID>(A, W, t, K, pl, flags & 1, (cudaStream_t)stream);
}

// Without the extra operand.
int frt_b200_gemm_fp8_nt_gate_residual(const void* A, const void* W, int M, int N, int K, const float* d_scale_a,
                                       const float* d_scale_b, void* residual, const void* gate, float* stats_out,
                                       int* stat_tiles, int splits, int flags, void* stream) {
    return frt_b200_gemm_fp8_nt_gate_residual_q8(A, W, M, N, K, d_scale_a, d_scale_b, residual, gate, stats_out,
                                                 stat_tiles, nullptr, nullptr, nullptr, splits, flags, stream);
}

// QKV projection of an operand written by frt_b200_gemm_fp8_nt_gate_residual_q8 (M <= 128, K % 128 == 0):
//   row[m][n] = bf16(sa * sb * (A . W^T)[m][n] * rms[m] + col_term[n]),
//   rms[m] = 1 / sqrt(sum_t stats_in[t][m] / K + eps)   (stats_in: n_stat rows of 128 floats, summed in order),
//   col_term (N fp32) = W . shift of the norm's style row, computed once per (step, layer) by the caller;
// then the RoPE + split + KV-append epilogue of frt_b200_gemm_fp8_nt_rope_split.
int frt_b200_gemm_fp8_nt_rope_split_rowscale(const void* A, const void* W, int M, int K, const float* d_scale_a,
                                             const float* d_scale_b, const float* stats_in, int n_stat, float eps,
                                             const float* col_term, const void* rope, void* Q, void* Kout, void* Vout,
                                             const int* devpos, int q_dim, int k_dim, int v_dim, int head_dim,
                                             int splits, int flags, void* stream) {
    if (!A || !W || !stats_in || !col_term || !rope || !Q || !Kout || !Vout || M < 0 || K <= 0 || n_stat <= 0)
        return FRT_ERR_INVALID;
    if (q_dim <= 0 || k_dim <= 0 || v_dim <= 0 || head_dim <= 0) return FRT_ERR_INVALID;
    if ((K % 128) || M > 128 || (head_dim % 8) || (q_dim % head_dim) || (k_dim % head_dim) || (v_dim % 8))
        return FRT_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(col_term) & 15) return FRT_ERR_INVALID;
    if (M == 0) return FRT_OK;
    TokParams t = {};
    t.M = M; t.N = q_dim + k_dim + v_dim; t.sa = d_scale_a; t.sb = d_scale_b; t.alpha_host = 1.0f;
    t.rope = (const __nv_bfloat16*)rope; t.outQ = (__nv_bfloat16*)Q; t.outK = (__nv_bfloat16*)Kout;
    t.outV = (__nv_bfloat16*)Vout; t.devpos = devpos;
    t.q_dim = q_dim; t.k_dim = k_dim; t.v_dim = v_dim; t.head_dim = head_dim;
    t.stats_in = stats_in; t.n_stat = n_stat; t.eps = eps; t.col_term = col_term;
    return dispatch_gemm_tok<TOK_PRO_TMA, TOK_EPI_ROPE>(A, W, t, K, tok_bn_hint(flags), tok_split_hint(splits),
                                                       flags & 1, (cudaStream_t)stream);
}

// gate|up projection of such an operand: gate / up values = bf16(sa * sb * acc * rms[m] + col_term[n]) (col_term has
// 2 * half entries, gate rows first), then the GeGLU -> FP8 epilogue of frt_b200_gemm_fp8_nt_geglu_fp8
// (M <= 128, half % 64 == 0, K % 128 == 0).
int frt_b200_gemm_fp8_nt_geglu_fp8_rowscale(const void* A, const void* W, void* out8, int M, int half, int K,
                                            const float* d_scale_a, const float* d_scale_b, const float* stats_in,
                                            int n_stat, float eps, const float* col_term, const float* d_out_scale,
                                            int splits, int flags, void* stream) {
    if (!A || !W || !out8 || !stats_in || !col_term || !d_out_scale || M < 0 || half <= 0 || K <= 0 || n_stat <= 0)
        return FRT_ERR_INVALID;
    if ((K % 128) || M > 128 || (half % 64)) return FRT_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(col_term) & 15) return FRT_ERR_INVALID;
    if (M == 0) return FRT_OK;
    TokParams t = {};
    t.M = M; t.N = 2 * half; t.sa = d_scale_a; t.sb = d_scale_b; t.alpha_host = 1.0f;
    t.out8 = (uint8_t*)out8; t.out_scale = d_out_scale; t.half = half; t.gate_act = (flags & 128) ? 2 : 0;
    t.stats_in = stats_in; t.n_stat = n_stat; t.eps = eps; t.col_term = col_term;
    return dispatch_gemm_tok<TOK_PRO_TMA, TOK_EPI_GEGLU>(A, W, t, K, tok_bn_hint(flags), tok_split_hint(splits),
                                                        flags & 1, (cudaStream_t)stream);
}

// QKV projection whose FP8 input is produced inside the kernel from the residual stream (M <= 128, K = 128, 256, 512
// per split): a = e4m3(clamp(((x * rms) * (1 + scale) + shift) / *d_scale_a, +-448)) with
//   rms[m] = 1 / sqrt(sum_t stats_in[t][m] / K + eps)  (stats_in: n_stat rows of 128 floats, summed in order),
//   style = [scale (K) | shift (K)] one bf16 row shared by all tokens (unit norm weight),
// followed by the projection and the RoPE + split + KV-append epilogue of frt_b200_gemm_fp8_nt_rope_split.
// Stands for gate_residual_ada_norm_fp8 (second pass, csrc/kernels/fusion.cu:48-81) + fp8_nn_dev + qkv_split_rope.
int frt_b200_norm_gemm_fp8_nt_rope_split(const void* x, const float* stats_in, int n_stat, const void* style, float eps,
                                         const void* W, int M, int K, const float* d_scale_a, const float* d_scale_b,
                                         const void* rope, void* Q, void* Kout, void* Vout, const int* devpos,
                                         int q_dim, int k_dim, int v_dim, int head_dim, int splits, int flags,
                                         void* stream) {
    if (!x || !stats_in || !style || !W || !rope || !Q || !Kout || !Vout || !d_scale_a || M < 0 || K <= 0 || n_stat <= 0)
        return FRT_ERR_INVALID;
    if (q_dim <= 0 || k_dim <= 0 || v_dim <= 0 || head_dim <= 0) return FRT_ERR_INVALID;
    if ((K % 128) || M > 128 || (head_dim % 8) || (q_dim % head_dim) || (k_dim % head_dim) || (v_dim % 8))
        return FRT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(style) & 15)) return FRT_ERR_INVALID;
    if (M == 0) return FRT_OK;
    TokParams t = {};
    t.M = M; t.N = q_dim + k_dim + v_dim; t.sa = d_scale_a; t.sb = d_scale_b; t.alpha_host = 1.0f;
    t.rope = (const __nv_bfloat16*)rope; t.outQ = (__nv_bfloat16*)Q; t.outK = (__nv_bfloat16*)Kout;
    t.outV = (__nv_bfloat16*)Vout; t.devpos = devpos;
    t.q_dim = q_dim; t.k_dim = k_dim; t.v_dim = v_dim; t.head_dim = head_dim;
    t.x = (const __nv_bfloat16*)x; t.stats_in = stats_in; t.n_stat = n_stat; t.style = (const __nv_bfloat16*)style;
    t.eps = eps;
    return dispatch_gemm_tok<TOK_PRO_NORM, TOK_EPI_ROPE>(nullptr, W, t, K, tok_bn_hint(flags), tok_split_hint(splits),
                                                        flags & 1, (cudaStream_t)stream);
}

// gate|up projection with the same in-kernel adaRMS -> FP8 producer in front and the GeGLU -> FP8 epilogue of
// frt_b200_gemm_fp8_nt_geglu_fp8 behind (M <= 128, half % 128 == 0).
int frt_b200_norm_gemm_fp8_nt_geglu_fp8(const void* x, const float* stats_in, int n_stat, const void* style, float eps,
                                        const void* W, void* out8, int M, int half, int K, const float* d_scale_a,
                                        const float* d_scale_b, const float* d_out_scale, int splits, int flags,
                                        void* stream) {
    if (!x || !stats_in || !style || !W || !out8 || !d_scale_a || !d_out_scale || M < 0 || half <= 0 || K <= 0 ||
        n_stat <= 0)
        return FRT_ERR_INVALID;
    if ((K % 128) || M > 128 || (half % 64)) return FRT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(style) & 15)) return FRT_ERR_INVALID;
    if (M == 0) return FRT_OK;
    TokParams t = {};
    t.M = M; t.N = 2 * half; t.sa = d_scale_a; t.sb = d_scale_b; t.alpha_host = 1.0f;
    t.out8 = (uint8_t*)out8; t.out_scale = d_out_scale; t.half = half; t.gate_act = (flags & 128) ? 2 : 0;
    t.x = (const __nv_bfloat16*)x; t.stats_in = stats_in; t.n_stat = n_stat; t.style = (const __nv_bfloat16*)style;
    t.eps = eps;
    return dispatch_gemm_tok<TOK_PRO_NORM, TOK_EPI_GEGLU>(nullptr, W, t, K, tok_bn_hint(flags), tok_split_hint(splits),
                                                         flags & 1, (cudaStream_t)stream);
}

}  // extern "C"
namespace frt {
int* gemm_status_device_ptr() {
    void* p = nullptr;
    return cudaGetSymbolAddress(&p, g_gemm_status) == cudaSuccess ? static_cast<int*>(p) : nullptr;
}
}  // namespace frt
extern "C" {

// returns and clears the device-side status word of the GEMM kernels (0 = no bounded wait ever gave up)
int frt_b200_gemm_status(int reset) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int));
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    if (reset && v) {
        int z = 0;
        cudaMemcpyToSymbol(g_gemm_status, &z, sizeof(int));
    }
    return v;
}


}  // extern "C"

#ifdef FRT_PHASE_STAMPS
// not part of the ABI: the GEMM half of frt_b200_phase_stamps_read (attention.cu)
extern "C" __attribute__((visibility("hidden"))) int frt_b200_gemm_phase_stamps(unsigned long long* host, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(host, g_tok_trace, sizeof(unsigned long long) * 8 * 160 * 16);
    if (reset) {
        g_tok_trace_slot = 0;
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_tok_trace) == cudaSuccess && ptr)
            cudaMemset(ptr, 0, sizeof(unsigned long long) * 8 * 160 * 16);
    }
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}
#endif
