// Flash attention forward for sm_100a: bf16 Q/K/V, tcgen05 MMAs with S and O
// accumulators in TMEM, TMA-fed operands, non-causal, MHA / GQA / MQA.
//
// Replaces, for sm_100a, the reference attention entry points
//   fa2.fwd_bf16 / fwd_bf16_seqused[_splitkv]   csrc/fa2_bindings.cpp:142-183 -> csrc/attention/fa2_wrapper.cu
//   (call site RtxFlashAttnBackend.decoder_attn, flash_rt/hardware/rtx/attn_backend.py:633-660)
// and covers the two shapes of the denoise path:
//   * MQA cross-attention of the action expert: 50 x 8 query rows of width 256
//     against one KV head of 768 prefix + 50 fresh keys;
//   * long bidirectional self-attention of a video DiT (head_dim 128).
//
// Work split.  The G = Hq / Hkv query heads that share a KV head are packed into
// the MMA M-dimension (row = token * G + head-in-group), so one 128-row tile holds
// 128 / G tokens and K/V are read once for all of them.  grid = (row tiles,
// Hkv * batch, kv splits).  The kv splits of one tile form a thread-block cluster
// (1 x 1 x C, C <= 8): each CTA runs an online-softmax pass over its slice of the
// keys, then the partial (max, sum, O) triples are combined through distributed
// shared memory, each CTA finishing 1/C of the head dimension.  No global scratch.
//
// Per CTA and per chunk of BKV keys:  S = Q K^T (UMMA 128 x BKV x 16, both operands
// K-major) -> TMEM;  four softmax warps (one thread per row) read S with tcgen05.ld,
// keep the running max / sum, write P as bf16 into shared memory in the 128-byte
// swizzled K-major layout;  O += P V (UMMA 128 x D x 16, V is the MN-major B
// operand straight from its (key, d) layout).
//
// Floating point: cosine >= 0.999 and max-abs <= 2e-2 x RMS against the fp32
// reference is the acceptance bar; exp2 uses the hardware approximation.
#include "common.cuh"
#include "tc05.cuh"

#include <mutex>
#include <type_traits>

namespace frt {

__device__ int g_attn_status = 0;   // 0 ok; otherwise first failure code | (blockIdx.x << 8)

// ------------------------------------------------------------------ tensor maps (bf16, up to 5-D)
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static PFN_encodeTiled g_encode_attn = nullptr;
static std::mutex g_attn_mu;

static int ensure_encode_attn() {
    std::lock_guard<std::mutex> lk(g_attn_mu);
    if (g_encode_attn) return FRT_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) return FRT_ERR_UNSUPPORTED;
    g_encode_attn = (PFN_encodeTiled)fn;
    return FRT_OK;
}

// dims[0] is the contiguous one (elements); strides_bytes[i] is the pitch of dims[i+1]
static int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box) {
    int rc = ensure_encode_attn();
    if (rc) return rc;
    if (reinterpret_cast<uintptr_t>(base) & 15) return FRT_ERR_INVALID;
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; e[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) {
        if (strides_bytes[i] & 15) return FRT_ERR_INVALID;
        s[i] = strides_bytes[i];
    }
    CUresult r = g_encode_attn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), d, s, b, e,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? FRT_OK : FRT_ERR_INVALID;
}

namespace tc {
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
        "[%2];" ::"r"(smem_u32(smem_dst)),
        "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, "
        "%7}], [%2];" ::"r"(smem_u32(smem_dst)),
        "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
}  // namespace tc

// ------------------------------------------------------------------ kernel
struct AttnParams {
    __nv_bfloat16* O;            // (B, Sq, Hq, D) with the strides below (elements)
    uint8_t* O_fp8;              // optional second result: e4m3(clamp(O / *out_scale)), same indexing, or null
    const float* out_scale;      // device scalar for O_fp8
    float* lse;                  // optional (B, Hq, Sq) fp32 natural-log-sum-exp, or null
    const int* seqused_k;        // optional device int: number of valid keys (<= Skv), or null
    long long o_bs, o_rs, o_hs;
    int B, Sq, Skv, Hq, Hkv, G;
    int chunks_total;            // ceil(Skv / BKV)
    int kv_static_rows;          // leading K/V rows that the previous kernel in the stream does not write
    // split-KV through global scratch (same buffers and layouts as the reference's FA2 split-kv path):
    float* o_accum;              // (splits, B, Hq, Sq, D) fp32, each split's O already divided by its row sum
    float* lse_accum;            // (splits, B, Hq, Sq) fp32, log2-domain log-sum-exp of the split (-inf if empty)
    unsigned* counters;          // 2 words per (row tile, kv head, batch): arrivals (monotonic), spare; zero before first use
    float scale_log2;            // softmax_scale * log2(e)
    int flags;                   // the entry point's flags (head_dim-256 kernel: bit 2 keeps one CTA per (tile, split), bit 3 the global-scratch combine)
#ifdef FRT_PHASE_STAMPS
    int trace_slot;
#endif
};

template <int D, int BKV>
struct AttnCfg {
    static constexpr int DB = D / 64;                      // 64-element (128-byte) blocks along the head dim
    static constexpr int Q_BYTES = 128 * D * 2;
    static constexpr int KV_BYTES = BKV * D * 2;           // one of K or V
    static constexpr int PB = (BKV + 63) / 64;             // 64-key blocks of P
    static constexpr int P_BYTES = PB * 128 * 128;
    static constexpr int OFF_K = Q_BYTES;
    static constexpr int OFF_V = OFF_K + KV_BYTES;
    static constexpr int OFF_P = OFF_V + KV_BYTES;
    static constexpr int DATA_BYTES = OFF_P + P_BYTES;
    static constexpr int RED_BYTES = D * 128 * 4;          // partial O staged as [d][row] fp32
    static constexpr int ML_BYTES = 2 * 128 * 4;
    static constexpr int BODY = (DATA_BYTES > RED_BYTES ? DATA_BYTES : RED_BYTES);
    static constexpr int SMEM_BYTES = BODY + ML_BYTES + 256 + 1024;
    static constexpr int S_COL = 0;
    static constexpr int O_COL = 256;
    static constexpr int TMEM_COLS = 512;
    static_assert(BKV % 16 == 0 && BKV <= 256, "key chunk must be a multiple of 16, at most 256");
    static_assert(D % 64 == 0 && D <= 256, "head dim must be a multiple of 64, at most 256");
    static_assert(KV_BYTES % 1024 == 0 && Q_BYTES % 1024 == 0, "tiles must keep 1024-byte alignment");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

enum { AERR_PRODUCER = 0x11, AERR_MMA = 0x12, AERR_SOFTMAX = 0x13 };

#define ATTN_WAIT(bar, parity, code)                                                     \
    do {                                                                                 \
        if (!tc::mbar_wait_until((bar), (parity), deadline, abort_flag)) {               \
            if (!*abort_flag) atomicCAS(&g_attn_status, 0, (code) | (blockIdx.x << 8));  \
            *abort_flag = 1;                                                             \
        }                                                                                \
    } while (0)

template <int D, int BKV>
__global__ void __launch_bounds__(192, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, AttnParams p) {
    using Cfg = AttnCfg<D, BKV>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = smem + Cfg::OFF_K;
    uint8_t* sV = smem + Cfg::OFF_V;
    uint8_t* sP = smem + Cfg::OFF_P;
    float* red = reinterpret_cast<float*>(smem);                       // aliases the operand tiles after the last MMA
    float* s_m = reinterpret_cast<float*>(smem + Cfg::BODY);           // per-row running max (log2 domain)
    float* s_l = s_m + 128;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::BODY + Cfg::ML_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;
    uint64_t* v_full = bars + 2;
    uint64_t* kv_empty = bars + 3;    // K and V tiles may be overwritten (PV of the chunk has completed)
    uint64_t* s_full = bars + 4;      // S = Q K^T is in TMEM
    uint64_t* p_ready = bars + 5;     // P is in shared memory, O has been rescaled (128 arrivals)
    uint64_t* o_full = bars + 6;      // O += P V has completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint64_t deadline = tc::global_timer_ns() + FRT_KERNEL_DEADLINE_NS;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // kv splits are either the CTAs of a cluster (combined through DSMEM) or, when scratch buffers are given,
    // independent CTAs along grid z (combined through global memory)
    const bool via_scratch = p.o_accum != nullptr;
    const uint32_t C = via_scratch ? gridDim.z : tc::cluster_nctarank();
    const uint32_t rank = via_scratch ? blockIdx.z : tc::cluster_ctarank();
    unsigned cnt_base = 0;       // thread 0, scratch path: the tile's arrival count when this launch started
    const int tile = blockIdx.x;
    const int hk = blockIdx.y % p.Hkv;
    const int b = blockIdx.y / p.Hkv;
    const int tok0 = tile * (128 / p.G);                                // first token of this row tile
    const int c_begin = (int)((long long)p.chunks_total * rank / C);
    const int c_end = (int)((long long)p.chunks_total * (rank + 1) / C);
    const int nchunks = c_end - c_begin;
    const int dper = D / (int)C;                      // head-dim columns finished by each rank (C is a power of two)
    const int swz = (dper >> 2) - 1 < 7 ? (dper >> 2) - 1 : 7;

    if (threadIdx.x == 0) {
        tc::mbar_init(q_full, 1);
        tc::mbar_init(k_full, 1);
        tc::mbar_init(v_full, 1);
        tc::mbar_init(kv_empty, 1);
        tc::mbar_init(s_full, 1);
        tc::mbar_init(p_ready, 128);
        tc::mbar_init(o_full, 1);
        *abort_flag = 0;
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&tmQ);
        tc::tma_prefetch_desc(&tmK);
        tc::tma_prefetch_desc(&tmV);
    }
    if (warp == 5) {
        tc::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_S = tmem + Cfg::S_COL;
    const uint32_t tmem_O = tmem + Cfg::O_COL;

    pdl_launch_dependents();

    if (warp == 4 && lane == 0) {
        // ---------------- TMA producer
        auto load_kv = [&](int chunk) {
            const int key0 = chunk * BKV;
            tc::mbar_arrive_expect_tx(k_full, Cfg::KV_BYTES);
            for (int db = 0; db < Cfg::DB; ++db)
                tc::tma_load_4d(sK + db * (BKV * 128), &tmK, k_full, db * 64, hk, key0, b);
            tc::mbar_arrive_expect_tx(v_full, Cfg::KV_BYTES);
            for (int db = 0; db < Cfg::DB; ++db)
                tc::tma_load_4d(sV + db * (BKV * 128), &tmV, v_full, db * 64, hk, key0, b);
        };
        // keys that the previous kernel does not write (the prefix) can be fetched while it still runs
        const bool early = nchunks > 0 && (c_begin + 1) * BKV <= p.kv_static_rows;
        if (early) load_kv(c_begin);
        pdl_wait();                   // Q and the freshly appended K/V rows come from the previous kernel
        tc::mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
        for (int db = 0; db < Cfg::DB; ++db)
            tc::tma_load_5d(sQ + db * (128 * 128), &tmQ, q_full, db * 64, 0, hk, tok0, b);
        for (int i = early ? 1 : 0; i < nchunks && !*abort_flag; ++i) {
            if (i > 0) ATTN_WAIT(kv_empty, (uint32_t)((i - 1) & 1), AERR_PRODUCER);
            if (*abort_flag) break;
            load_kv(c_begin + i);
        }
    } else if (warp == 5 && lane == 0) {
        pdl_wait();
        // ---------------- MMA issuer
        constexpr uint32_t idesc_s = tc::make_idesc(1, 1, 0, 0, 128, BKV);   // bf16 x bf16, both K-major
        constexpr uint32_t idesc_o = tc::make_idesc(1, 1, 0, 1, 128, D);     // B (= V) is MN-major
        // descriptors differ only in their start-address field (units of 16 bytes): build the bases once
        const uint64_t dq_base = tc::make_desc_kmajor_sw128(tc::smem_u32(sQ));
        const uint64_t dk_base = tc::make_desc_kmajor_sw128(tc::smem_u32(sK));
        const uint64_t dp_base = tc::make_desc_kmajor_sw128(tc::smem_u32(sP));
        const uint64_t dv_base = tc::make_desc_mnmajor_sw128(tc::smem_u32(sV), BKV * 128);
        ATTN_WAIT(q_full, 0u, AERR_MMA);
        for (int i = 0; i < nchunks && !*abort_flag; ++i) {
            const uint32_t ph = (uint32_t)(i & 1);
            ATTN_WAIT(k_full, ph, AERR_MMA);
            if (*abort_flag) break;
            tc::tc_fence_after_sync();
            // S = Q K^T : D / 16 steps of K = 16; a step advances 32 bytes inside a 128-byte block
#pragma unroll
            for (int k = 0; k < D / 16; ++k)
                tc::mma_f16(tmem_S, dq_base + (uint64_t)((k / 4) * ((128 * 128) >> 4) + 2 * (k % 4)),
                            dk_base + (uint64_t)((k / 4) * ((BKV * 128) >> 4) + 2 * (k % 4)), idesc_s, k > 0 ? 1u : 0u);
            tc::mma_commit(s_full);
            ATTN_WAIT(p_ready, ph, AERR_MMA);
            ATTN_WAIT(v_full, ph, AERR_MMA);
            if (*abort_flag) break;
            tc::tc_fence_after_sync();
            // O += P V : BKV / 16 steps over the keys
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k)
                tc::mma_f16(tmem_O, dp_base + (uint64_t)((k / 4) * ((128 * 128) >> 4) + 2 * (k % 4)),
                            dv_base + (uint64_t)(k * ((16 * 128) >> 4)), idesc_o, (i > 0 || k > 0) ? 1u : 0u);
            tc::mma_commit(kv_empty);
            tc::mma_commit(o_full);
        }
    } else if (warp < 4) {
        // ---------------- softmax: thread = row (TMEM lane 32*warp + lane)
        pdl_wait();
        if (via_scratch && threadIdx.x == 0) {
            // The tile's arrival counter only ever grows, by 256 per launch (each of its C CTAs adds 256 / C, whatever
            // C is, so launches of different shapes may share a counter); every earlier launch has completed here and
            // this CTA has not arrived yet, so rounding down to a multiple of 256 gives the count this launch started from.
            const unsigned tid = (unsigned)((b * p.Hkv + hk) * gridDim.x + tile);
            unsigned seen;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.counters + 2 * tid) : "memory");
            cnt_base = seen & ~255u;
        }
        int kv_len = p.Skv;
        if (p.seqused_k) { int u = *p.seqused_k; kv_len = u < kv_len ? u : kv_len; }
        const int row = warp * 32 + lane;
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        float m_run = -INFINITY, l_run = 0.0f;
        for (int i = 0; i < nchunks; ++i) {
            const uint32_t ph = (uint32_t)(i & 1);
            ATTN_WAIT(s_full, ph, AERR_SOFTMAX);
            __syncwarp();
            if (__any_sync(0xffffffffu, *abort_flag != 0)) break;      // leave the loop as a whole warp
            tc::tc_fence_after_sync();
            const int key0 = (c_begin + i) * BKV;
            float s[BKV];
#pragma unroll
            for (int c = 0; c < BKV; c += 16) {
                uint32_t v[16];
                tc::tmem_ld16(tmem_S + lane_off + c, v);
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    s[c + j] = (key0 + c + j < kv_len) ? __uint_as_float(v[j]) * p.scale_log2 : -INFINITY;
            }
            float mx = m_run;
#pragma unroll
            for (int j = 0; j < BKV; ++j) mx = fmaxf(mx, s[j]);
            const float m_use = (mx == -INFINITY) ? 0.0f : mx;
            const float alpha = tc::ex2_approx(m_run - m_use);       // m_run = -inf -> 0
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < BKV; ++j) {
                s[j] = tc::ex2_approx(s[j] - m_use);
                sum += s[j];
            }
            l_run = l_run * alpha + sum;
            m_run = mx;
            // P -> shared memory, K-major rows of 128 bytes, 16-byte chunk index xor (row & 7)
#pragma unroll
            for (int c8 = 0; c8 < BKV / 8; ++c8) {
                uint4 w;
                w.x = pack_bf16x2(s[c8 * 8 + 0], s[c8 * 8 + 1]);
                w.y = pack_bf16x2(s[c8 * 8 + 2], s[c8 * 8 + 3]);
                w.z = pack_bf16x2(s[c8 * 8 + 4], s[c8 * 8 + 5]);
                w.w = pack_bf16x2(s[c8 * 8 + 6], s[c8 * 8 + 7]);
                const int blk = c8 / 8, ch = c8 % 8;
                *reinterpret_cast<uint4*>(sP + blk * (128 * 128) + row * 128 + ((ch ^ (row & 7)) << 4)) = w;
            }
            // rescale the running O (the previous P V has completed: o_full phase i-1)
            if (i > 0) {
                ATTN_WAIT(o_full, (uint32_t)((i - 1) & 1), AERR_SOFTMAX);
                __syncwarp();
                tc::tc_fence_after_sync();
                // tcgen05.ld / st are warp-collective: the decision to rescale must be uniform across the warp
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        uint32_t v[32];
                        tc::tmem_ld32(tmem_O + lane_off + c, v);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
                        tc::tmem_st32(tmem_O + lane_off + c, v);
                    }
                    tc::tmem_st_wait();
                }
            }
            tc::fence_proxy_async_smem();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(p_ready);
        }
        // ---------------- stage the partial result for the cluster combine
        if (nchunks > 0) {
            ATTN_WAIT(o_full, (uint32_t)((nchunks - 1) & 1), AERR_SOFTMAX);
            tc::tc_fence_after_sync();
        }
        __syncwarp();
        s_m[row] = m_run;
        s_l[row] = l_run;
        if (via_scratch) {
            // partial of this row (O / l, log2-domain lse) -> shared memory, row-major with xor-swizzled 16-byte
            // chunks; the whole CTA then copies full rows to the global scratch with coalesced stores
            const bool aborted = __any_sync(0xffffffffu, *abort_flag != 0);
            if (!aborted) {
                const float invl = l_run > 0.0f ? 1.0f / l_run : 0.0f;
                s_m[row] = l_run > 0.0f ? m_run + log2f(l_run) : -INFINITY;
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    uint32_t v[32];
                    if (nchunks > 0) {                   // warp-uniform: tcgen05.ld is warp-collective
                        tc::tmem_ld32(tmem_O + lane_off + c, v);
                        tc::tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = 0u;
                    }
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        const int ch = (c >> 2) + j4;
                        *reinterpret_cast<float4*>(&red[(size_t)row * D + ((ch ^ (row & 7)) << 2)]) =
                            make_float4(__uint_as_float(v[j4 * 4]) * invl, __uint_as_float(v[j4 * 4 + 1]) * invl,
                                        __uint_as_float(v[j4 * 4 + 2]) * invl, __uint_as_float(v[j4 * 4 + 3]) * invl);
                    }
                }
            }
        } else if (!__any_sync(0xffffffffu, *abort_flag != 0)) {
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                uint32_t v[32];
                if (nchunks > 0) {
                    tc::tmem_ld32(tmem_O + lane_off + c, v);
                    tc::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                }
                // staged as [slice of dper columns][row][dper] with the 16-byte chunks of a row xor-swizzled by
                // (row & mask): conflict-free 16-byte writes here and 16-byte remote reads in the combine
#pragma unroll
                for (int j4 = 0; j4 < 8; ++j4) {
                    const int d = c + j4 * 4;
                    const int slice = d / dper, ch = (d % dper) >> 2;
                    float4 w4 = make_float4(__uint_as_float(v[j4 * 4]), __uint_as_float(v[j4 * 4 + 1]),
                                            __uint_as_float(v[j4 * 4 + 2]), __uint_as_float(v[j4 * 4 + 3]));
                    *reinterpret_cast<float4*>(&red[((size_t)(slice * 128 + row)) * dper + ((ch ^ (row & swz)) << 2)]) = w4;
                }
            }
        }
    }
    __syncwarp();
    if (via_scratch) {
        // ---------------- combine through global scratch.  All CTAs of the grid are co-resident (the host keeps
        // the grid within one wave), each publishes its partial, waits (bounded) for the C partials of its tile and
        // finishes D / C columns of every row.  Every global access below is coalesced: consecutive lanes touch
        // consecutive 16-byte chunks of one row.
        const unsigned tile_id = (unsigned)((b * p.Hkv + hk) * gridDim.x + tile);
        unsigned* cnt = p.counters + 2 * tile_id;
        const size_t split_stride = (size_t)p.B * p.Hq * p.Sq;
        __syncthreads();
        // G divides 128, so it is a power of two: row -> (token, head) by shift / mask
        const int gshift = 31 - __clz(p.G);
        int rows_valid = (p.Sq - tok0) << gshift;
        rows_valid = rows_valid > 128 ? 128 : rows_valid;
        if (!*abort_flag) {
#pragma unroll 4
            for (int r = warp; r < rows_valid; r += 6) {
                const int t = tok0 + (r >> gshift);
                const int hq = hk * p.G + (r & (p.G - 1));
                const size_t ridx = rank * split_stride + ((size_t)b * p.Hq + hq) * p.Sq + t;
                float4* dst = reinterpret_cast<float4*>(p.o_accum + ridx * D);
#pragma unroll
                for (int ch = lane; ch < D / 4; ch += 32)
                    __stcg(dst + ch, *reinterpret_cast<const float4*>(&red[(size_t)r * D + ((ch ^ (r & 7)) << 2)]));
                if (lane == 0) __stcg(p.lse_accum + ridx, s_m[r]);
            }
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(cnt), "r"(256u / C) : "memory");
            bool ok = false;
            for (uint32_t it = 0;; ++it) {
                unsigned seen;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(cnt) : "memory");
                if (seen - cnt_base >= 256u) { ok = true; break; }
                if (*abort_flag) break;
                if ((it & 15) == 15 && tc::global_timer_ns() > deadline) break;
                __nanosleep(20);
            }
            if (!ok) {
                if (!*abort_flag) atomicCAS(&g_attn_status, 0, AERR_SOFTMAX | (blockIdx.x << 8));
                *abort_flag = 1;
            }
        }
        __syncthreads();
        if (!*abort_flag) {
            const int cpr = dper >> 2;                            // 16-byte chunks of this rank's slice per row
            const int d0 = (int)rank * dper;
            const float inv_os = p.O_fp8 ? __fdiv_rn(1.0f, *p.out_scale) : 0.0f;
            const int cshift = 31 - __clz(cpr);                   // cpr is a power of two
#pragma unroll 2
            for (int idx = threadIdx.x; idx < rows_valid * cpr; idx += 192) {
                const int r = idx >> cshift, ch = idx & (cpr - 1);
                const int t = tok0 + (r >> gshift);
                const int hq = hk * p.G + (r & (p.G - 1));
                const size_t r0 = ((size_t)b * p.Hq + hq) * p.Sq + t;
                float w[8];
                float4 x[8];
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx) {
                    if ((uint32_t)sidx < C) {
                        w[sidx] = __ldcg(p.lse_accum + sidx * split_stride + r0);
                        x[sidx] = __ldcg(reinterpret_cast<const float4*>(p.o_accum + (sidx * split_stride + r0) * D + d0) + ch);
                    } else {
                        w[sidx] = -INFINITY;
                        x[sidx] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                float M = -INFINITY;
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx) M = fmaxf(M, w[sidx]);
                float Lw = 0.0f;
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx) {
                    w[sidx] = (w[sidx] == -INFINITY) ? 0.0f : tc::ex2_approx(w[sidx] - M);
                    Lw += w[sidx];
                }
                const float invL = Lw > 0.0f ? 1.0f / Lw : 0.0f;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx) {
                    const float ws = w[sidx] * invL;
                    a0 += ws * x[sidx].x; a1 += ws * x[sidx].y; a2 += ws * x[sidx].z; a3 += ws * x[sidx].w;
                }
                const size_t o = (size_t)b * p.o_bs + (size_t)t * p.o_rs + (size_t)hq * p.o_hs + d0 + ch * 4;
                uint2 ob;
                ob.x = pack_bf16x2(a0, a1);
                ob.y = pack_bf16x2(a2, a3);
                st_global_v2(p.O + o, ob);
                if (p.O_fp8) {
                    float q0, q1, q2, q3;                         // quantise the bf16-rounded value
                    unpack_bf16x2(ob.x, q0, q1);
                    unpack_bf16x2(ob.y, q2, q3);
                    *reinterpret_cast<uint32_t*>(p.O_fp8 + o) =
                        f32x4_to_e4m3x4(clamp448(__fmul_rn(q0, inv_os)), clamp448(__fmul_rn(q1, inv_os)),
                                        clamp448(__fmul_rn(q2, inv_os)), clamp448(__fmul_rn(q3, inv_os)));
                }
                if (p.lse && rank == 0 && ch == 0)
                    p.lse[r0] = (Lw > 0.0f) ? (M + log2f(Lw)) * 0.6931471805599453f : -INFINITY;
            }
        }
        tc::tc_fence_before_sync();
        __syncthreads();
        if (warp == 5) tc::tmem_dealloc(tmem, Cfg::TMEM_COLS);
        return;
    }
    tc::cluster_sync_all();

    // ---------------- combine across the kv splits (cluster path): this CTA finishes D / C columns
    if (warp < 4 && !*abort_flag) {
        const int row = warp * 32 + lane;
        const int d0 = (int)rank * dper;
        const int t = tok0 + row / p.G;
        const int hq = hk * p.G + row % p.G;
        if (t < p.Sq) {
            float w[8];
            float M = -INFINITY;
            const uint32_t a_m = tc::smem_u32(&s_m[row]);
            const uint32_t a_l = tc::smem_u32(&s_l[row]);
            for (uint32_t s = 0; s < C; ++s) {
                w[s] = tc::dsmem_ld_f32(tc::dsmem_map(a_m, s));
                M = fmaxf(M, w[s]);
            }
            float L = 0.0f;
            for (uint32_t s = 0; s < C; ++s) {
                w[s] = (w[s] == -INFINITY) ? 0.0f : tc::ex2_approx(w[s] - M);
                L += w[s] * tc::dsmem_ld_f32(tc::dsmem_map(a_l, s));
            }
            const float invL = L > 0.0f ? 1.0f / L : 0.0f;
            for (uint32_t s = 0; s < C; ++s) w[s] *= invL;
            const size_t obase = (size_t)b * p.o_bs + (size_t)t * p.o_rs + (size_t)hq * p.o_hs;
            const float inv_os = p.O_fp8 ? __fdiv_rn(1.0f, *p.out_scale) : 0.0f;
            const uint32_t my_row = tc::smem_u32(&red[((size_t)((int)rank * 128 + row)) * dper]);
            uint32_t rbase[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) rbase[s] = tc::dsmem_map(my_row, (uint32_t)s < C ? s : 0);
            for (int d = 0; d < dper; d += 8) {
                float acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
                const uint32_t off0 = (uint32_t)((((d >> 2)) ^ (row & swz)) << 4);
                const uint32_t off1 = (uint32_t)((((d >> 2) + 1) ^ (row & swz)) << 4);
#pragma unroll
                for (int g = 0; g < 8; g += 2) {
                    if ((uint32_t)g >= C) break;
                    // four 16-byte remote loads in flight per block: ranks g, g+1 x two chunks
                    float4 x0, x1, y0, y1;
                    asm volatile(
                        "ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%16];\n\t"
                        "ld.shared::cluster.v4.f32 {%4,%5,%6,%7}, [%17];\n\t"
                        "ld.shared::cluster.v4.f32 {%8,%9,%10,%11}, [%18];\n\t"
                        "ld.shared::cluster.v4.f32 {%12,%13,%14,%15}, [%19];"
                        : "=f"(x0.x), "=f"(x0.y), "=f"(x0.z), "=f"(x0.w), "=f"(x1.x), "=f"(x1.y), "=f"(x1.z), "=f"(x1.w),
                          "=f"(y0.x), "=f"(y0.y), "=f"(y0.z), "=f"(y0.w), "=f"(y1.x), "=f"(y1.y), "=f"(y1.z), "=f"(y1.w)
                        : "r"(rbase[g] + off0), "r"(rbase[g] + off1),
                          "r"(rbase[(uint32_t)(g + 1) < C ? g + 1 : g] + off0),
                          "r"(rbase[(uint32_t)(g + 1) < C ? g + 1 : g] + off1)
                        : "memory");
                    const float w0 = w[g], w1 = (uint32_t)(g + 1) < C ? w[g + 1] : 0.0f;
                    acc[0] += w0 * x0.x; acc[1] += w0 * x0.y; acc[2] += w0 * x0.z; acc[3] += w0 * x0.w;
                    acc[4] += w0 * x1.x; acc[5] += w0 * x1.y; acc[6] += w0 * x1.z; acc[7] += w0 * x1.w;
                    acc[0] += w1 * y0.x; acc[1] += w1 * y0.y; acc[2] += w1 * y0.z; acc[3] += w1 * y0.w;
                    acc[4] += w1 * y1.x; acc[5] += w1 * y1.y; acc[6] += w1 * y1.z; acc[7] += w1 * y1.w;
                }
                uint4 o;
                o.x = pack_bf16x2(acc[0], acc[1]);
                o.y = pack_bf16x2(acc[2], acc[3]);
                o.z = pack_bf16x2(acc[4], acc[5]);
                o.w = pack_bf16x2(acc[6], acc[7]);
                st_global_v4(p.O + obase + d0 + d, o);
                if (p.O_fp8) {
                    // quantise the bf16-rounded value, as a separate quantise kernel reading O would
                    float q[8];
                    unpack_bf16x2(o.x, q[0], q[1]);
                    unpack_bf16x2(o.y, q[2], q[3]);
                    unpack_bf16x2(o.z, q[4], q[5]);
                    unpack_bf16x2(o.w, q[6], q[7]);
                    uint2 o8;
                    o8.x = f32x4_to_e4m3x4(clamp448(__fmul_rn(q[0], inv_os)), clamp448(__fmul_rn(q[1], inv_os)),
                                           clamp448(__fmul_rn(q[2], inv_os)), clamp448(__fmul_rn(q[3], inv_os)));
                    o8.y = f32x4_to_e4m3x4(clamp448(__fmul_rn(q[4], inv_os)), clamp448(__fmul_rn(q[5], inv_os)),
                                           clamp448(__fmul_rn(q[6], inv_os)), clamp448(__fmul_rn(q[7], inv_os)));
                    st_global_v2(p.O_fp8 + obase + d0 + d, o8);
                }
            }
            if (p.lse && rank == 0)
                p.lse[((size_t)b * p.Hq + hq) * p.Sq + t] = (L > 0.0f) ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
        }
    }
    tc::cluster_sync_all();

    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) tc::tmem_dealloc(tmem, Cfg::TMEM_COLS);
}

#include "attention_pair.cuh"
#include "attention_d256.cuh"

template <int D, int BKV>
static int launch_attn(const void* Q, const void* K, const void* V, AttnParams p, const long long* qs,
                       const long long* ks, const long long* vs, int splits, bool pdl, cudaStream_t stream) {
    using Cfg = AttnCfg<D, BKV>;
    static PerDeviceOnce attr_once;
    int attr_dev = 0;
    if (attr_once.need(attr_dev)) {
        cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<D, BKV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        attr_once.set(attr_dev);
    }
    // Q as {d, head-in-group, kv head, token, batch}; strides in elements: qs = {batch, row, head}
    CUtensorMap tmQ, tmK, tmV;
    {
        uint64_t dims[5] = {(uint64_t)D, (uint64_t)p.G, (uint64_t)p.Hkv, (uint64_t)p.Sq, (uint64_t)p.B};
        uint64_t str[4] = {(uint64_t)qs[2] * 2, (uint64_t)qs[2] * 2 * p.G, (uint64_t)qs[1] * 2, (uint64_t)qs[0] * 2};
        uint32_t box[5] = {64, (uint32_t)p.G, 1, (uint32_t)(128 / p.G), 1};
        int rc = make_tmap_bf16(&tmQ, Q, 5, dims, str, box);
        if (rc) return rc;
    }
    {
        uint64_t dims[4] = {(uint64_t)D, (uint64_t)p.Hkv, (uint64_t)p.Skv, (uint64_t)p.B};
        uint64_t strk[3] = {(uint64_t)ks[2] * 2, (uint64_t)ks[1] * 2, (uint64_t)ks[0] * 2};
        uint64_t strv[3] = {(uint64_t)vs[2] * 2, (uint64_t)vs[1] * 2, (uint64_t)vs[0] * 2};
        uint32_t box[4] = {64, 1, (uint32_t)BKV, 1};
        int rc = make_tmap_bf16(&tmK, K, 4, dims, strk, box);
        if (rc) return rc;
        rc = make_tmap_bf16(&tmV, V, 4, dims, strv, box);
        if (rc) return rc;
    }
    p.chunks_total = (p.Skv + BKV - 1) / BKV;
    if (splits > p.chunks_total) splits = p.chunks_total;
    if (splits < 1) splits = 1;
    while (splits & (splits - 1)) --splits;            // power of two: each rank finishes D / splits columns
    const int tiles = (p.Sq * p.G + 127) / 128;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, p.Hkv * p.B, splits);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = p.o_accum ? 1 : splits;
    ++na;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (p.o_accum && splits > 1) {
        // the CTAs of a tile wait for one another: the whole grid has to be resident at once
        int sms = 0, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if ((long long)tiles * p.Hkv * p.B * splits > sms) return FRT_ERR_UNSUPPORTED;
    }
    if (splits == 1) p.o_accum = nullptr;              // nothing to combine: plain path
    cudaError_t e = cudaLaunchKernelEx(&cfg, attn_fwd_kernel<D, BKV>, tmQ, tmK, tmV, p);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}

}  // namespace frt

using namespace frt;

extern "C" {

// Non-causal attention forward, bf16.  Layouts (strides in elements, innermost head_dim contiguous):
//   Q, O: (batch, seqlen_q, num_heads_q, head_dim)   q_strides / o_strides = {batch, row, head}
//   K, V: (batch, seqlen_k, num_heads_kv, head_dim)  k_strides / v_strides = {batch, row, head}
// O_fp8 / out_scale: optional fused e4m3 copy of O (null to skip).  lse: optional (batch, heads_q, seqlen_q).
// seqused_k: optional device int limiting the valid keys.  kv_splits: 0 = choose, else 1..8 (rounded down to a
// power of two).  kv_static_rows: number of leading K/V rows NOT written by the previous kernel in the stream
// (they may be fetched before that kernel finishes when flags bit0 is set); 0 if unsure.
// o_accum / lse_accum / counters: optional split-KV scratch, all three or none.  o_accum (splits, batch, heads_q,
// seqlen_q, head_dim) fp32, lse_accum (splits, batch, heads_q, seqlen_q) fp32 (the reference's FA2 split-kv
// buffers), counters: 2 unsigned per (128-row tile, kv head, batch), zeroed once by the caller (a tile's count only
// grows, by 256 per launch; a launch reads where it starts).  With scratch the kv splits are ordinary CTAs that combine through global memory (faster than the
// cluster exchange at the action-expert shape); the grid must fit the device in one wave (else -2).
int frt_b200_attention_fwd_bf16(const void* Q, const void* K, const void* V, void* O, void* O_fp8,
                                const float* out_scale, float* lse, const int* seqused_k, int batch, int seqlen_q,
                                int seqlen_k, int num_heads_q, int num_heads_kv, int head_dim,
                                const long long* q_strides, const long long* k_strides, const long long* v_strides,
                                const long long* o_strides, float softmax_scale, int kv_splits, int kv_static_rows,
                                float* o_accum, float* lse_accum, void* counters, int flags, void* stream) {
    if (!Q || !K || !V || !O || !q_strides || !k_strides || !v_strides || !o_strides) return FRT_ERR_INVALID;
    if (batch <= 0 || seqlen_q < 0 || seqlen_k <= 0 || num_heads_q <= 0 || num_heads_kv <= 0) return FRT_ERR_INVALID;
    if (O_fp8 && !out_scale) return FRT_ERR_INVALID;
    if (num_heads_q % num_heads_kv) return FRT_ERR_INVALID;
    const int G = num_heads_q / num_heads_kv;
    if (G > 128 || (128 % G)) return FRT_ERR_UNSUPPORTED;
    if (head_dim != 128 && head_dim != 256) return FRT_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(O) & 15) || (o_strides[1] & 7) || (o_strides[2] & 7) || (o_strides[0] & 7))
        return FRT_ERR_INVALID;
    if (seqlen_q == 0) return FRT_OK;
    AttnParams p = {};
    p.O = (__nv_bfloat16*)O;
    p.O_fp8 = (uint8_t*)O_fp8;
    p.out_scale = out_scale;
    p.lse = lse;
    p.seqused_k = seqused_k;
    p.o_bs = o_strides[0];
    p.o_rs = o_strides[1];
    p.o_hs = o_strides[2];
    p.B = batch;
    p.Sq = seqlen_q;
    p.Skv = seqlen_k;
    p.Hq = num_heads_q;
    p.Hkv = num_heads_kv;
    p.G = G;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.kv_static_rows = kv_static_rows;
    p.flags = flags;
    if (o_accum && lse_accum && counters) {
        p.o_accum = o_accum;
        p.lse_accum = lse_accum;
        p.counters = (unsigned*)counters;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const bool pdl = flags & 1;
    const int tiles = ((seqlen_q * G + 127) / 128) * num_heads_kv * batch;
    if (head_dim == 256) {
        // pipelined kernel (64-key chunks, double-buffered K/V and S, P in tensor memory): whenever the splits combine
        // through the caller's scratch, or there is nothing to combine; flags bit 1 keeps the single-tile kernel
        if (!(flags & 2)) {
            const int chunks64 = (seqlen_k + 63) / 64;
            int sp64 = kv_splits > 0 ? kv_splits : (tiles >= 74 ? 1 : (chunks64 < 8 ? chunks64 : 8));
            if (sp64 > 8) sp64 = 8;
            if (p.o_accum || sp64 == 1)
                return launch_attn_d256(Q, K, V, p, q_strides, k_strides, v_strides, p.o_accum ? sp64 : 1, pdl, s);
        }
        constexpr int BKV = 112;
        int chunks = (seqlen_k + BKV - 1) / BKV;
        int sp = kv_splits > 0 ? kv_splits : (tiles >= 74 ? 1 : (chunks < 8 ? chunks : 8));
        if (sp > 8) sp = 8;
        return launch_attn<256, BKV>(Q, K, V, p, q_strides, k_strides, v_strides, sp, pdl, s);
    }
    constexpr int BKV = 128;
    int chunks = (seqlen_k + BKV - 1) / BKV;
    int sp = kv_splits > 0 ? kv_splits : (tiles >= 74 ? 1 : (chunks < 8 ? chunks : 8));
    if (sp > 8) sp = 8;
    // one split and at least two row tiles: the two-tile ping-pong kernel (softmax overlapped with the MMAs)
    if (sp == 1 && (seqlen_q * G + 127) / 128 >= 2)
        return launch_attn_pair(Q, K, V, p, q_strides, k_strides, v_strides, pdl, s);
    return launch_attn<128, BKV>(Q, K, V, p, q_strides, k_strides, v_strides, sp, pdl, s);
}

// ------------------------------------------------------------------ variant with built-in scratch
// Some hosts of this library may not allocate device memory at the point where they need attention with split KV:
// a real-time control loop that has frozen its memory map, a plugin running inside another runtime's captured or
// pooled-memory region, an embedding that only hands out fixed buffers.  For them the split-KV scratch lives in
// this module: a fixed array in device global memory that every GPU loading the library carries until the
// process exits.
#define FRT_STATIC_ATTN_MAX_SPLITS 8
#define FRT_STATIC_ATTN_MAX_ROWS 512          /* batch * heads_q * seqlen_q */
#define FRT_STATIC_ATTN_MAX_HEAD_DIM 256
#define FRT_STATIC_ATTN_MAX_TILES 64          /* 128-row tiles x kv heads x batch */
#define FRT_STATIC_O_BYTES ((size_t)FRT_STATIC_ATTN_MAX_SPLITS * FRT_STATIC_ATTN_MAX_ROWS * FRT_STATIC_ATTN_MAX_HEAD_DIM * 4)
#define FRT_STATIC_LSE_BYTES ((size_t)FRT_STATIC_ATTN_MAX_SPLITS * FRT_STATIC_ATTN_MAX_ROWS * 4)
#define FRT_STATIC_CNT_BYTES ((size_t)FRT_STATIC_ATTN_MAX_TILES * 2 * 4)
static __device__ __align__(256) unsigned char g_attn_static_scratch[FRT_STATIC_O_BYTES + FRT_STATIC_LSE_BYTES +
                                                                     FRT_STATIC_CNT_BYTES];
// In host code the array's name is only a handle; the device address is asked for once per device (under g_attn_mu).
static void* g_attn_static_ptr[64] = {nullptr};

// Same operation and arguments as frt_b200_attention_fwd_bf16 without the three scratch pointers: the split-KV
// partials go to the module's own fixed device array (about 4.2 MB per GPU).  Limits: kv_splits <= 8,
// batch * num_heads_q * seqlen_q <= 512, head_dim <= 256, at most 64 (row tile, kv head, batch) triples; anything
// larger returns -4.  Nothing is allocated or freed by this call.  The first call on each device looks up the
// array's device address (cudaGetSymbolAddress) and clears the arrival counters with a memset enqueued on the
// caller's stream in front of the kernel: make that first call before any stream capture (inside a capture it is
// refused with -1).  Every call uses the same array, which keeps whatever the previous call left in it (the kernel
// overwrites the partials it reads and its arrival counters only ever grow), so two calls whose kernels can overlap on the
// GPU -- different streams, or graph branches -- would corrupt each other.  After a call whose bounded wait gave up
// (frt_b200_attention_status != 0) the counters are stale: frt_b200_attention_status(1) clears them as well.
int frt_b200_attention_fwd_bf16_static_scratch(const void* Q, const void* K, const void* V, void* O, void* O_fp8,
                                               const float* out_scale, float* lse, const int* seqused_k, int batch,
                                               int seqlen_q, int seqlen_k, int num_heads_q, int num_heads_kv,
                                               int head_dim, const long long* q_strides, const long long* k_strides,
                                               const long long* v_strides, const long long* o_strides,
                                               float softmax_scale, int kv_splits, int kv_static_rows, int flags,
                                               void* stream) {
    if (!Q || !K || !V || !O || !q_strides || !k_strides || !v_strides || !o_strides) return FRT_ERR_INVALID;
    if (batch <= 0 || seqlen_q < 0 || seqlen_k <= 0 || num_heads_q <= 0 || num_heads_kv <= 0 ||
        (num_heads_q % num_heads_kv))
        return FRT_ERR_INVALID;
    if (O_fp8 && !out_scale) return FRT_ERR_INVALID;
    const long long rows = (long long)batch * num_heads_q * seqlen_q;
    const int G = num_heads_q / num_heads_kv;
    const long long tiles = (((long long)seqlen_q * G + 127) / 128) * num_heads_kv * batch;
    if (kv_splits > FRT_STATIC_ATTN_MAX_SPLITS || rows > FRT_STATIC_ATTN_MAX_ROWS ||
        head_dim > FRT_STATIC_ATTN_MAX_HEAD_DIM || tiles > FRT_STATIC_ATTN_MAX_TILES)
        return -4;   // larger than the built-in scratch
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    if (dev < 0 || dev >= 64) return FRT_ERR_UNSUPPORTED;
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_attn_mu);
        if (!g_attn_static_ptr[dev]) {
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            e = cudaStreamIsCapturing((cudaStream_t)stream, &cap);
            if (e != cudaSuccess) return FRT_CUDA_ERR(e);
            if (cap != cudaStreamCaptureStatusNone) return FRT_ERR_INVALID;   // set-up call must precede any capture
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_attn_static_scratch);
            if (e != cudaSuccess || !ptr) return e != cudaSuccess ? FRT_CUDA_ERR(e) : FRT_ERR_INVALID;
            e = cudaMemsetAsync(static_cast<unsigned char*>(ptr) + FRT_STATIC_O_BYTES + FRT_STATIC_LSE_BYTES, 0,
                                FRT_STATIC_CNT_BYTES, (cudaStream_t)stream);
            if (e != cudaSuccess) return FRT_CUDA_ERR(e);
            g_attn_static_ptr[dev] = ptr;
        }
        base = static_cast<unsigned char*>(g_attn_static_ptr[dev]);
    }
    return frt_b200_attention_fwd_bf16(Q, K, V, O, O_fp8, out_scale, lse, seqused_k, batch, seqlen_q, seqlen_k,
                                       num_heads_q, num_heads_kv, head_dim, q_strides, k_strides, v_strides, o_strides,
                                       softmax_scale, kv_splits, kv_static_rows, reinterpret_cast<float*>(base),
                                       reinterpret_cast<float*>(base + FRT_STATIC_O_BYTES),
                                       base + FRT_STATIC_O_BYTES + FRT_STATIC_LSE_BYTES, flags, stream);
}

}  // extern "C"
namespace frt {
int* attention_status_device_ptr() {
    void* p = nullptr;
    return cudaGetSymbolAddress(&p, g_attn_status) == cudaSuccess ? static_cast<int*>(p) : nullptr;
}
}  // namespace frt
extern "C" {

// returns (and optionally clears) the attention kernels' device status word; 0 = no bounded wait gave up.
// code 0x11 = TMA producer, 0x12 = MMA issuer, 0x13 = softmax warps.  Synchronises the device.  Clearing a
// non-zero status also clears the arrival counters of the built-in scratch on the current device (a kernel that
// gave up leaves them mid-count, and the static-scratch caller has no buffer of its own to re-zero).
int frt_b200_attention_status(int reset) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int));
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    if (reset && v) {
        int z = 0;
        cudaMemcpyToSymbol(g_attn_status, &z, sizeof(int));
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
            std::lock_guard<std::mutex> lk(g_attn_mu);
            if (g_attn_static_ptr[dev]) {
                cudaMemset(static_cast<unsigned char*>(g_attn_static_ptr[dev]) + FRT_STATIC_O_BYTES +
                               FRT_STATIC_LSE_BYTES, 0, FRT_STATIC_CNT_BYTES);
                cudaDeviceSynchronize();
            }
        }
    }
    return v;
}

// Diagnostics (no counterpart in the reference): device-timer phase stamps of the last 8 launches of the token-major
// GEMM (gemm_host: 8 x 160 CTAs x 16 stamps) and of the head_dim-256 attention kernel (attn_host: 8 x 128 x 16), in
// nanoseconds of %globaltimer.  Only a library built with -DFRT_PHASE_STAMPS records them; otherwise -2.
// reset != 0 restarts the launch slots at 0 and clears the stamps (after copying them out).  Synchronises the device.
#ifdef FRT_PHASE_STAMPS
extern "C" int frt_b200_gemm_phase_stamps(unsigned long long* host, int reset);
#endif
int frt_b200_phase_stamps_read(unsigned long long* gemm_host, unsigned long long* attn_host, int reset) {
#ifdef FRT_PHASE_STAMPS
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    if (gemm_host) {
        int rc = frt_b200_gemm_phase_stamps(gemm_host, reset);
        if (rc) return rc;
    }
    if (attn_host) {
        e = cudaMemcpyFromSymbol(attn_host, g_attn_trace, sizeof(unsigned long long) * 8 * 128 * 16);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    }
    if (reset) {
        g_attn_trace_slot = 0;
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_attn_trace) == cudaSuccess && ptr)
            cudaMemset(ptr, 0, sizeof(unsigned long long) * 8 * 128 * 16);
    }
    return FRT_OK;
#else
    (void)gemm_host; (void)attn_host; (void)reset;
    return FRT_ERR_UNSUPPORTED;
#endif
}

}  // extern "C"
