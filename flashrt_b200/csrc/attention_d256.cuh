// Pipelined flash attention for head_dim 256 (the action expert's MQA cross-attention), sm_100a.
//
// Included by attention.cu inside namespace frt (AttnParams, tensor-map helpers, ATTN_WAIT).
//
// The single-tile kernel keeps one K and one V chunk of 112 keys in shared memory (Q + K + V + P fill it), so every
// chunk pays a full TMA round trip before its MMAs: measured 4.5 us per additional chunk.  Here
//   * chunks are 64 keys, K/V are double-buffered (Q 64 KB + 2 x (32 + 32) KB), the producer runs two chunks ahead;
//   * S is double-buffered in TMEM (2 x 64 columns) so QK(j+1) is issued before the softmax of chunk j has finished;
//   * P (bf16) overlays its S buffer and feeds the PV MMA as the A operand from TMEM -- no shared-memory round trip;
//   * the row of S lives in registers (one tcgen05.wait per chunk); O is rescaled only when a row maximum grows by
//     more than 2^8.
// KV splits: none (gridDim.z = 1, result written directly) or through the caller's scratch.  The scratch path is
// built around bulk copies: a split's normalised O leaves as bf16 in column slices [slice][row][D / C] -- one
// contiguous block per (row tile, split), written by ONE cp.async.bulk from shared memory -- then the arrival
// counter, and every split fetches its own column slice of all C partials with C bulk loads and combines them out
// of shared memory.  (Measured at the action-expert shape with per-thread fp32 stores and loads instead: 2.4 us to
// publish, 4.9 us to combine -- five dependent L2 round trips per thread -- out of 14.5 us per launch.)
// Warps: 0-3 softmax (thread = row), 4 TMA, 5 MMA.
#pragma once

#ifdef FRT_PHASE_STAMPS
__device__ unsigned long long g_attn_trace[8][128][16];
static int g_attn_trace_slot = 0;
#define ATT_STAMP(i) do { if (threadIdx.x == 0) g_attn_trace[p.trace_slot][(blockIdx.z * gridDim.x + blockIdx.x) % 128][i] = tc::global_timer_ns(); } while (0)
#define ATT_STAMP_ANY(i) do { g_attn_trace[p.trace_slot][(blockIdx.z * gridDim.x + blockIdx.x) % 128][i] = tc::global_timer_ns(); } while (0)
#else
#define ATT_STAMP(i)
#define ATT_STAMP_ANY(i)
#endif

struct D256Cfg {
    static constexpr int D = 256, BKV = 64;
    static constexpr int Q_BYTES = 128 * D * 2;            // 64 KB
    static constexpr int KV_BYTES = BKV * D * 2;           // 32 KB, one of K or V, one stage
    static constexpr int OFF_K = Q_BYTES;
    static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
    // operand tiles of a CTA that owns D / dq columns of V: Q, two stages of K, two stages of its part of V (192 KB for
    // dq = 1, 144 KB for dq = 4; the combine re-uses the first 74 KB after the last MMA)
    static constexpr int data_bytes(int dq) { return OFF_V + 2 * (KV_BYTES / dq); }
    static constexpr int ML_BYTES = 128 * 4;
    // cluster exchange (XC): one receive slot per kv split, [128 rows][64 / C columns] bf16 + 128 log-sum-exps
    static constexpr int recv_bytes(int dq) { return 128 * (D / dq) * 2 + 8 * 512; }
    static constexpr int OFF_RECV(int dq) { return data_bytes(dq) + ML_BYTES + 256; }
    static constexpr int smem_bytes(int dq, bool xc = false) { return OFF_RECV(dq) + (xc ? recv_bytes(dq) : 0) + 1024; }
    // ragged launch: full tiles in four parts, a last tile of at most RAGGED_ROWS rows in two (slots of
    // rows x (128 / C columns bf16 + one float) from each of C splits: at most 8 x 32 x 36 bytes)
    static constexpr int RAGGED_ROWS = 32;
    static constexpr int ragged_smem_bytes() {
        const int tail = OFF_RECV(2) + 8 * RAGGED_ROWS * 36 + 1024;
        return tail > smem_bytes(4, true) ? tail : smem_bytes(4, true);
    }
    static constexpr int S_COL = 0;                        // two S buffers of 64 columns
    static constexpr int O_COL = 128;
    static constexpr int TMEM_COLS = 512;
    static constexpr float RESCALE_THRESHOLD = 8.0f;
};

// DQ: the head dim of V / O is cut into DQ parts, one CTA each (scratch path only).  Every part repeats Q.K^T and the
// softmax of its (row tile, kv split) and computes P.V for D / DQ columns, so that the accumulator a CTA has to move
// out of tensor memory -- the longest single step of the scratch path: 3 us for 128 x 256 fp32 -- shrinks by DQ and
// the grid covers 4 x more SMs.
//
// XC (with DQ = 4): the C kv splits of a (row tile, head-dim part) are the CTAs of one thread-block cluster (1 x 1 x C)
// and exchange their partials through distributed shared memory instead of the global scratch: the thread of a row
// pushes, straight from registers with st.async, the 64 / C columns that split s finishes (normalised, bf16) and the
// row's log-sum-exp into split s's receive slot, the bytes counted on s's mbarrier; it then waits for its own slot to
// fill and combines and stores its row.  No fence, no CTA barrier, no counter and no L2 round trip between the last
// MMA and the result (measured per launch at the action-expert shape: publish 0.5 us + fence and barrier 0.7 + arrival
// 1.9 + combine 1.4 through the scratch).  Nothing of a CTA is read by a peer and a CTA leaves only after every peer's
// push has landed, so there is no cluster barrier at the end; the one that orders the peers' mbarrier initialisation
// before the first push is split: arrive after the set-up, wait just before pushing.
// DQT = 0 (cluster exchange only): the number of parts is a run-time argument, so that the CTAs of a ragged launch --
// full tiles in four parts, the last tile in two -- run the same instructions: with one body per part count the 16 CTAs
// of the last tile found their variant cold in the instruction cache of whatever SM they landed on (every phase of them
// ran 0.3-0.5 us behind the same phase of the other 96 CTAs on its first pass and at their speed on its second).
template <int DQT, bool XC>
__device__ __forceinline__ void attn_d256_body(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                                               const AttnParams& p, const int tile, const int dq, const int ntiles,
                                               const int parts) {
    using Cfg = D256Cfg;
    static_assert(DQT != 0 || XC, "run-time part count: cluster exchange only");
    constexpr int D = Cfg::D, BKV = Cfg::BKV;
    constexpr int DVC = DQT ? D / DQT : 64;                // compile-time columns of V / O of this CTA (DQT != 0)
    const int DQ = DQT ? DQT : parts;
    const int DV = D / DQ;                                 // columns of V / O of this CTA
    const int V_BYTES = BKV * DV * 2;                      // one V stage
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = smem + Cfg::OFF_K;
    uint8_t* sV = smem + Cfg::OFF_V;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::data_bytes(DQ) + Cfg::ML_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;      // [2]
    uint64_t* v_full = bars + 3;      // [2]
    uint64_t* kv_empty = bars + 5;    // [2]
    uint64_t* s_full = bars + 7;      // [2] one per S buffer
    uint64_t* p_ready = bars + 9;     // [2] 128 arrivals per chunk, one barrier per S / P buffer
    uint64_t* o_full = bars + 11;     // PV of a chunk has completed (read only where the count is known to within one)
    uint64_t* o_done = bars + 12;     // every PV of this CTA has completed
    uint64_t* c_full = bars + 13;     // the C column slices of the combine have landed
    uint64_t* q_part = bars + 14;     // [3] the second .. fourth 64-column block of Q (q_full covers the first)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint64_t deadline = tc::global_timer_ns() + FRT_KERNEL_DEADLINE_NS;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    ATT_STAMP(0);
    const bool via_scratch = p.o_accum != nullptr;
    const uint32_t C = gridDim.z;
    const uint32_t rank = blockIdx.z;
    const int hk = blockIdx.y % p.Hkv;
    const int b = blockIdx.y / p.Hkv;
    const int tok0 = tile * (128 / p.G);
    const int gshift = 31 - __clz(p.G);
    int rows_valid = (p.Sq - tok0) << gshift;                       // query rows (token x head-in-group) of this tile
    rows_valid = rows_valid > 128 ? 128 : rows_valid;
    uint8_t* cbuf = smem;                                           // the C column slices of the combine, up to 64 KB
    const int c_begin = (int)((long long)p.chunks_total * rank / C);
    const int c_end = (int)((long long)p.chunks_total * (rank + 1) / C);
    const int nchunks = c_end - c_begin;
    unsigned cnt_base = 0;                                          // thread 0, scratch path

    if (threadIdx.x == 0) {
        tc::mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(&k_full[i], 1);
            tc::mbar_init(&v_full[i], 1);
            tc::mbar_init(&kv_empty[i], 1);
            tc::mbar_init(&s_full[i], 1);
        }
        tc::mbar_init(&p_ready[0], 128);
        tc::mbar_init(&p_ready[1], 128);
        tc::mbar_init(o_full, 1);
        tc::mbar_init(o_done, 1);
        tc::mbar_init(c_full, 1);
        for (int i = 0; i < 3; ++i) tc::mbar_init(&q_part[i], 1);
        *abort_flag = 0;
        tc::mbar_fence_init();
        if constexpr (XC)       // every peer pushes rows_valid x (64 / C columns bf16 + one float) into this CTA
            tc::mbar_arrive_expect_tx(c_full, (C - 1) * (uint32_t)rows_valid * ((uint32_t)(DV / C) * 2u + 4u));
        tc::tma_prefetch_desc(&tmQ);
        tc::tma_prefetch_desc(&tmK);
        tc::tma_prefetch_desc(&tmV);
    }
    if (warp == 5) {
        tc::tmem_alloc(tmem_slot, (DQ == 1 ? 512 : 256));
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    // every peer's c_full must be initialised before anyone pushes into it: all threads arrive here, the softmax warps
    // wait just before their first push (by then the barrier has long completed: nothing of it is on the way to the
    // first MMA)
    if constexpr (XC) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

    pdl_launch_dependents();

    if (warp == 4 && lane == 0) {
        // ---------------- TMA producer
        auto load_kv = [&](int j) {
            const int st = j & 1;
            const int key0 = (c_begin + j) * BKV;
            tc::mbar_arrive_expect_tx(&k_full[st], Cfg::KV_BYTES);
            for (int db = 0; db < 4; ++db)
                tc::tma_load_4d(sK + st * Cfg::KV_BYTES + db * (BKV * 128), &tmK, &k_full[st], db * 64, hk, key0, b);
            tc::mbar_arrive_expect_tx(&v_full[st], V_BYTES);
            for (int db = 0; db < DV / 64; ++db)
                tc::tma_load_4d(sV + st * V_BYTES + db * (BKV * 128), &tmV, &v_full[st], dq * DV + db * 64, hk, key0, b);
        };
        // chunks that lie inside the rows the previous kernel does not write may be fetched while it still runs
        int early = 0;
        while (early < 2 && early < nchunks && (c_begin + early + 1) * BKV <= p.kv_static_rows) {
            load_kv(early);
            ++early;
        }
        pdl_wait();
        ATT_STAMP_ANY(1);
        // Q arrives as four 64-column blocks, each on its own barrier: the first chunk's Q.K^T starts on the first block
        // while the others are still in flight
        for (int db = 0; db < 4; ++db) {
            uint64_t* qb = db == 0 ? q_full : &q_part[db - 1];
            tc::mbar_arrive_expect_tx(qb, Cfg::Q_BYTES / 4);
            tc::tma_load_5d(sQ + db * (128 * 128), &tmQ, qb, db * 64, 0, hk, tok0, b);
        }
        for (int j = early; j < nchunks && !*abort_flag; ++j) {
            if (j >= 2) ATTN_WAIT(&kv_empty[j & 1], (uint32_t)(((j >> 1) - 1) & 1), AERR_PRODUCER);
            if (*abort_flag) break;
            load_kv(j);
        }
    } else if (warp == 5 && lane == 0) {
        // ---------------- MMA issuer
        constexpr uint32_t idesc_s = tc::make_idesc(1, 1, 0, 0, 128, BKV);
        const uint32_t idesc_o = tc::make_idesc(1, 1, 0, 1, 128, (uint32_t)DV);    // A = P from TMEM, B = V MN-major
        const uint64_t dq_base = tc::make_desc_kmajor_sw128(tc::smem_u32(sQ));
        const uint64_t dk_base = tc::make_desc_kmajor_sw128(tc::smem_u32(sK));
        const uint64_t dv_base = tc::make_desc_mnmajor_sw128(tc::smem_u32(sV), BKV * 128);
        auto qk = [&](int j) {
            const uint64_t dk = dk_base + (uint64_t)((j & 1) * (Cfg::KV_BYTES >> 4));
            const uint32_t d_tm = tmem + Cfg::S_COL + (j & 1) * 64;
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
                if (j == 0 && k > 0 && (k % 4) == 0) {          // next 64-column block of Q (first chunk only)
                    ATTN_WAIT(&q_part[k / 4 - 1], 0u, AERR_MMA);
                    if (*abort_flag) return;
                    tc::tc_fence_after_sync();
                }
                tc::mma_f16(d_tm, dq_base + (uint64_t)((k / 4) * ((128 * 128) >> 4) + 2 * (k % 4)),
                            dk + (uint64_t)((k / 4) * ((BKV * 128) >> 4) + 2 * (k % 4)), idesc_s, k > 0 ? 1u : 0u);
            }
            tc::mma_commit(&s_full[j & 1]);
        };
        ATTN_WAIT(q_full, 0u, AERR_MMA);
        ATT_STAMP_ANY(2);
        if (nchunks > 0 && !*abort_flag) {
            ATTN_WAIT(&k_full[0], 0u, AERR_MMA);
            if (!*abort_flag) {
                tc::tc_fence_after_sync();
                qk(0);
            }
        }
        for (int j = 0; j < nchunks && !*abort_flag; ++j) {
            if (j + 1 < nchunks) {      // S of the next chunk goes to the other buffer while the softmax works on this one
                ATTN_WAIT(&k_full[(j + 1) & 1], (uint32_t)(((j + 1) >> 1) & 1), AERR_MMA);
                if (*abort_flag) break;
                tc::tc_fence_after_sync();
                qk(j + 1);
            }
            ATTN_WAIT(&p_ready[j & 1], (uint32_t)((j >> 1) & 1), AERR_MMA);
            ATTN_WAIT(&v_full[j & 1], (uint32_t)((j >> 1) & 1), AERR_MMA);
            if (*abort_flag) break;
            tc::tc_fence_after_sync();
            const uint64_t dv = dv_base + (uint64_t)((j & 1) * (V_BYTES >> 4));
            const uint32_t a_tm = tmem + Cfg::S_COL + (j & 1) * 64;
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k)
                tc::mma_f16_ts(tmem + Cfg::O_COL, a_tm + 8 * k, dv + (uint64_t)(k * ((16 * 128) >> 4)), idesc_o,
                               (j > 0 || k > 0) ? 1u : 0u);
            tc::mma_commit(&kv_empty[j & 1]);
            tc::mma_commit(o_full);
        }
        if (!*abort_flag) tc::mma_commit(o_done);
        ATT_STAMP_ANY(3);
    } else if (warp < 4) {
        // ---------------- softmax: thread = row
        pdl_wait();
        if (!XC && via_scratch && threadIdx.x == 0) {
            // Arrival counter of this tile: it only ever grows, by 256 per launch (each of the C * DQ CTAs adds
            // 256 / (C * DQ)).  Every earlier launch has completed here and this CTA has not arrived yet, so rounding
            // down to a multiple of 256 gives the count this launch started from.
            const unsigned tid = (unsigned)((b * p.Hkv + hk) * ntiles + tile);
            unsigned seen;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.counters + 2 * tid) : "memory");
            cnt_base = seen & ~255u;
        }
        int kv_len = p.Skv;
        if (p.seqused_k) { int u = *p.seqused_k; kv_len = u < kv_len ? u : kv_len; }
        // read here, not where it is used: the load is an L2 round trip (0.6-1.2 us, by the distance of the SM from the
        // line's L2 slice) that would otherwise sit between the last partial's arrival and the result
        const float inv_os_early = (XC && p.O_fp8) ? __fdiv_rn(1.0f, *p.out_scale) : 0.0f;
        const int row = warp * 32 + lane;
        const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
        const uint32_t tmem_O = tmem + Cfg::O_COL + lane_off;
        float m_run = -INFINITY, l_run = 0.0f;
        bool alive = true;
        for (int j = 0; j < nchunks; ++j) {
            ATTN_WAIT(&s_full[j & 1], (uint32_t)((j >> 1) & 1), AERR_SOFTMAX);
            __syncwarp();
            if (__any_sync(0xffffffffu, *abort_flag != 0)) { alive = false; break; }
            tc::tc_fence_after_sync();
            if (j == 0) ATT_STAMP(4);
            const uint32_t tmem_S = tmem + Cfg::S_COL + (j & 1) * 64 + lane_off;
            const int valid = kv_len - (c_begin + j) * BKV;
            uint32_t sv[BKV];
            tc::tmem_ld32(tmem_S + 0, sv + 0);
            tc::tmem_ld32(tmem_S + 32, sv + 32);
            tc::tmem_ld_wait();
            if (valid < BKV) {
#pragma unroll
                for (int i = 0; i < BKV; ++i)
                    if (i >= valid) sv[i] = 0xff800000u;        // -inf
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < BKV; i += 4) {
#pragma unroll
                for (int q = 0; q < 4; ++q) mx4[q] = fmaxf(mx4[q], __uint_as_float(sv[i + q]));
            }
            const float mx_s = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            const bool grow = mx_s > m_run + Cfg::RESCALE_THRESHOLD || (m_run == -INFINITY && mx_s > -INFINITY);
            const float m_new = grow ? mx_s : m_run;
            if (__any_sync(0xffffffffu, grow && j > 0)) {
                // O holds the chunks up to j - 1: their PV must have completed before it is rescaled.  s_full(j) was
                // committed after PV(j - 2), so o_full has completed j - 1 or j times here: the parity wait is exact
                ATTN_WAIT(o_full, (uint32_t)((j - 1) & 1), AERR_SOFTMAX);
                __syncwarp();
                tc::tc_fence_after_sync();
                const float alpha = grow ? tc::ex2_approx(m_run - m_new) : 1.0f;
                l_run *= alpha;
#pragma unroll 1
                for (int c = 0; c < DV; c += 32) {
                    uint32_t v[32];
                    tc::tmem_ld32(tmem_O + c, v);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                    tc::tmem_st32(tmem_O + c, v);
                }
                tc::tmem_st_wait();
            }
            m_run = m_new;
            const float m_use = (m_run == -INFINITY) ? 0.0f : m_run;
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < BKV; c += 32) {
                uint32_t u[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float a = tc::ex2_approx(__fmaf_rn(__uint_as_float(sv[c + 2 * i]), p.scale_log2, -m_use));
                    const float bb = tc::ex2_approx(__fmaf_rn(__uint_as_float(sv[c + 2 * i + 1]), p.scale_log2, -m_use));
                    sum4[i & 3] += a + bb;
                    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(u[i]) : "f"(bb), "f"(a));   // low half = first key
                }
                tc::tmem_st16(tmem_S + (c >> 1), u);
            }
            tc::tmem_st_wait();
            l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&p_ready[j & 1]);
            if (j == 0) ATT_STAMP(5);
        }
        ATT_STAMP(6);
        // ---------------- the accumulated O of this split (o_full may be two completions behind here: use o_done)
        if (alive) {
            if (nchunks > 0) ATTN_WAIT(o_done, 0u, AERR_SOFTMAX);
            __syncwarp();
            alive = !__any_sync(0xffffffffu, *abort_flag != 0);
        }
        ATT_STAMP(7);
        if (alive) {
            tc::tc_fence_after_sync();
            const float invl = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            if constexpr (XC) {
                // ---------------- cluster exchange: slice s of this partial (columns [s dper, (s + 1) dper) of the part)
                // goes to split s's receive slot of this split; 64 columns at a time (one or more whole slices, or half a
                // slice of 128 / 2 columns)
                const float lse2 = l_run > 0.0f ? m_run + log2f(l_run) : -INFINITY;
                uint8_t* recv = smem + Cfg::OFF_RECV(DQ);
                const uint32_t recv_u32 = tc::smem_u32(recv);
                const uint32_t bar_u32 = tc::smem_u32(c_full);
                const int dper = DV / (int)C;                   // 8 .. 64 columns per slice
                // slot of a source split: [rows_valid][dper] bf16, then rows_valid log-sum-exps
                const uint32_t slot = ((uint32_t)rows_valid * ((uint32_t)dper * 2u + 4u) + 15u) & ~15u;
                const uint32_t my_data = rank * slot + (uint32_t)row * (uint32_t)dper * 2u;
                const uint32_t my_lse = rank * slot + (uint32_t)rows_valid * (uint32_t)dper * 2u + (uint32_t)row * 4u;
                asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
                if (row < rows_valid) {                         // the log-sum-exp of the row: once to every split
#pragma unroll
                    for (uint32_t s = 0; s < 8; ++s) {
                        if (s >= C) break;
                        if (s == rank) *reinterpret_cast<float*>(recv + my_lse) = lse2;
                        else tc::st_async_b32(tc::dsmem_map(recv_u32 + my_lse, s), tc::dsmem_map(bar_u32, s),
                                              __float_as_uint(lse2));
                    }
                }
#pragma unroll 1
                for (int c = 0; c < DV; c += 64) {
                    uint32_t va[64];
                    if (nchunks > 0) {                          // warp-uniform: the loads are warp-collective
                        tc::tmem_ld32(tmem_O + c, va);
                        tc::tmem_ld32(tmem_O + c + 32, va + 32);
                        tc::tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int i = 0; i < 64; ++i) va[i] = 0u;
                    }
                    uint32_t pk[32];                            // 64 columns of the row, normalised, as bf16 pairs
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        pk[i] = pack_bf16x2(__uint_as_float(va[2 * i]) * invl, __uint_as_float(va[2 * i + 1]) * invl);
                    if (c == 0) ATT_STAMP(13);
                    auto push = [&](auto dper_c) {
                        constexpr int DPER = decltype(dper_c)::value;        // columns of a slice inside this block
                        constexpr int NS = 64 / DPER;                          // slices (or 1: half a 128-column slice)
#pragma unroll
                        for (int i = 0; i < NS; ++i) {
                            const uint32_t s = (uint32_t)((c + i * DPER) >> (31 - __clz(dper)));
                            const uint32_t off = my_data + (uint32_t)(((c + i * DPER) & (dper - 1)) * 2);
                            const uint32_t* w = pk + i * (DPER / 2);
                            if (row >= rows_valid) {
                            } else if (s == rank) {             // the own slice: plain stores into the own slot
#pragma unroll
                                for (int q = 0; q < DPER / 8; ++q)
                                    *reinterpret_cast<uint4*>(recv + off + 16 * q) =
                                        make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                            } else {
                                const uint32_t peer_bar = tc::dsmem_map(bar_u32, s);
                                const uint32_t peer_data = tc::dsmem_map(recv_u32 + off, s);
#pragma unroll
                                for (int q = 0; q < DPER / 8; ++q)
                                    tc::st_async_v4(peer_data + 16 * q, peer_bar, w[4 * q], w[4 * q + 1], w[4 * q + 2],
                                                    w[4 * q + 3]);
                            }
                        }
                    };
                    if (dper == 8) push(std::integral_constant<int, 8>{});
                    else if (dper == 16) push(std::integral_constant<int, 16>{});
                    else if (dper == 32) push(std::integral_constant<int, 32>{});
                    else push(std::integral_constant<int, 64>{});
                }
                ATT_STAMP(14);
                ATT_STAMP(8);
            } else if (via_scratch) {
                constexpr int DV = DVC;                         // compile-time here (never the run-time-parts variant)
                // O / l as bf16 straight from registers to the scratch in column slices [slice][row][D / C]: the 64
                // bytes a thread writes per 32 columns are adjacent to its neighbours' (the rows of a slice are
                // contiguous), so a warp's store covers 2 KB without gaps.  Log2-domain lse alongside.
                const int dper = DV / (int)C;                  // columns per slice: a multiple of 8
                const size_t split_stride = (size_t)p.B * p.Hq * p.Sq;
                const size_t row0 = ((size_t)(b * p.Hkv + hk) * p.Sq << gshift) + (size_t)tile * 128;
                // block of (tile, split): rows_valid x D bf16; inside it the part of this dq: rows_valid x DV
                uint8_t* blk = reinterpret_cast<uint8_t*>(p.o_accum) + (rank * split_stride + row0) * (size_t)(D * 2) +
                               (size_t)dq * rows_valid * (DV * 2);
                if (row < rows_valid && dq == 0)
                    __stcg(p.lse_accum + rank * split_stride + row0 + row,
                           l_run > 0.0f ? m_run + log2f(l_run) : -INFINITY);
                // 64 columns per step, the next step's tensor-memory load in flight while this one is converted
                // dper is a power of two (>= 8): slice = column >> dsh.  These threads run one warp per scheduler, so every
                // instruction of the address arithmetic is exposed latency: shifts and 32-bit offsets, no divisions
                const int dsh = 31 - __clz(dper);
                const uint32_t slice_stride = (uint32_t)rows_valid * (uint32_t)dper * 2u;
                uint8_t* rowp = blk + (uint32_t)row * (uint32_t)dper * 2u;
                auto emit = [&](const uint32_t* v, int c) {
                    if (row < rows_valid) {
#pragma unroll
                        for (int j8 = 0; j8 < 8; ++j8) {                // 8 columns = 16 bytes at a time
                            const int cc = c + 8 * j8;
                            uint4* dst = reinterpret_cast<uint4*>(rowp + (uint32_t)(cc >> dsh) * slice_stride +
                                                                  (uint32_t)(cc & (dper - 1)) * 2u);
                            const uint32_t* w = v + 8 * j8;
                            uint4 o;
                            o.x = pack_bf16x2(__uint_as_float(w[0]) * invl, __uint_as_float(w[1]) * invl);
                            o.y = pack_bf16x2(__uint_as_float(w[2]) * invl, __uint_as_float(w[3]) * invl);
                            o.z = pack_bf16x2(__uint_as_float(w[4]) * invl, __uint_as_float(w[5]) * invl);
                            o.w = pack_bf16x2(__uint_as_float(w[6]) * invl, __uint_as_float(w[7]) * invl);
                            __stcg(dst, o);
                        }
                    }
                };
                uint32_t va[64], vb[64];
                if (nchunks > 0) {                              // warp-uniform: the loads are warp-collective
                    tc::tmem_ld32(tmem_O + 0, va);
                    tc::tmem_ld32(tmem_O + 32, va + 32);
                    if constexpr (DV >= 128) {
#pragma unroll
                        for (int c = 0; c < DV; c += 128) {
                            tc::tmem_ld_wait();
                            tc::tmem_ld32(tmem_O + c + 64, vb);
                            tc::tmem_ld32(tmem_O + c + 96, vb + 32);
                            emit(va, c);
                            tc::tmem_ld_wait();
                            if (c + 128 < DV) {
                                tc::tmem_ld32(tmem_O + c + 128, va);
                                tc::tmem_ld32(tmem_O + c + 160, va + 32);
                            }
                            emit(vb, c + 64);
                        }
                    } else {
                        tc::tmem_ld_wait();
                        ATT_STAMP(13);
                        emit(va, 0);
                        ATT_STAMP(14);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i) va[i] = 0u;
#pragma unroll 1
                    for (int c = 0; c < DV; c += 64) emit(va, c);
                }
            } else {
                // single split: the result leaves directly, one row per thread
                const int tok = tok0 + row / p.G;
                const int hq = hk * p.G + row % p.G;
                const bool store = tok < p.Sq;
                const float inv_os = p.O_fp8 ? __fdiv_rn(1.0f, *p.out_scale) : 0.0f;
                const size_t obase = (size_t)b * p.o_bs + (size_t)(store ? tok : 0) * p.o_rs + (size_t)hq * p.o_hs;
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    uint32_t v[32];
                    if (nchunks > 0) {
                        tc::tmem_ld32(tmem_O + c, v);
                        tc::tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0u;
                    }
                    if (store) {
#pragma unroll
                        for (int i8 = 0; i8 < 4; ++i8) {
                            uint4 o;
                            uint32_t* ow = &o.x;
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                ow[i] = pack_bf16x2(__uint_as_float(v[i8 * 8 + 2 * i]) * invl,
                                                    __uint_as_float(v[i8 * 8 + 2 * i + 1]) * invl);
                            st_global_v4(p.O + obase + c + i8 * 8, o);
                            if (p.O_fp8) {
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
                                st_global_v2(p.O_fp8 + obase + c + i8 * 8, o8);
                            }
                        }
                    }
                }
                if (store && p.lse)
                    p.lse[((size_t)b * p.Hq + hq) * p.Sq + tok] =
                        (l_run > 0.0f) ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
            }
        }
        if constexpr (XC) {
            // ---------------- every peer's slice of this split's columns has landed: combine and store.  One item =
            // (row, 8 columns), spread over the four softmax warps whatever their rows (a short last tile has its rows in
            // one warp), so a thread reads slots that other threads filled: a named barrier, reached by the four warps
            // on every path, orders the plain stores of the own slice
            if (!*abort_flag) ATTN_WAIT(c_full, 0u, AERR_SOFTMAX);
            ATT_STAMP(10);
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!*abort_flag) {
                const uint8_t* recv = smem + Cfg::OFF_RECV(DQ);
                const int dper = DV / (int)C;
                const uint32_t slot = ((uint32_t)rows_valid * ((uint32_t)dper * 2u + 4u) + 15u) & ~15u;
                const uint32_t lse_off = (uint32_t)rows_valid * (uint32_t)dper * 2u;
                const int cshift = 31 - __clz(dper >> 3);        // 16-byte chunks per slice row: a power of two
                const float inv_os = inv_os_early;
                for (int it = threadIdx.x; it < (rows_valid << cshift); it += 128) {
                    const int r = it >> cshift, ch = it & ((1 << cshift) - 1);
                    const int t = tok0 + (r >> gshift);
                    const int hq = hk * p.G + (r & (p.G - 1));
                    float w[8];
#pragma unroll
                    for (int sidx = 0; sidx < 8; ++sidx)
                        w[sidx] = (uint32_t)sidx < C
                                      ? *reinterpret_cast<const float*>(recv + sidx * slot + lse_off + (uint32_t)r * 4u)
                                      : -INFINITY;
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
#pragma unroll
                    for (int sidx = 0; sidx < 8; ++sidx) w[sidx] *= invL;
                    float a[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) a[i] = 0.0f;
#pragma unroll
                    for (uint32_t sidx = 0; sidx < 8; ++sidx) {
                        if (sidx >= C) break;
                        const uint4 x = *reinterpret_cast<const uint4*>(recv + sidx * slot +
                                                                        (uint32_t)r * (uint32_t)dper * 2u + ch * 16);
                        const float ws = w[sidx];
                        float f0, f1;
                        unpack_bf16x2(x.x, f0, f1); a[0] += ws * f0; a[1] += ws * f1;
                        unpack_bf16x2(x.y, f0, f1); a[2] += ws * f0; a[3] += ws * f1;
                        unpack_bf16x2(x.z, f0, f1); a[4] += ws * f0; a[5] += ws * f1;
                        unpack_bf16x2(x.w, f0, f1); a[6] += ws * f0; a[7] += ws * f1;
                    }
                    const size_t o = (size_t)b * p.o_bs + (size_t)t * p.o_rs + (size_t)hq * p.o_hs + dq * DV +
                                     (int)rank * dper + ch * 8;
                    uint4 ob;
                    ob.x = pack_bf16x2(a[0], a[1]);
                    ob.y = pack_bf16x2(a[2], a[3]);
                    ob.z = pack_bf16x2(a[4], a[5]);
                    ob.w = pack_bf16x2(a[6], a[7]);
                    st_global_v4(p.O + o, ob);
                    if (p.O_fp8) {
                        float q[8];
                        unpack_bf16x2(ob.x, q[0], q[1]);
                        unpack_bf16x2(ob.y, q[2], q[3]);
                        unpack_bf16x2(ob.z, q[4], q[5]);
                        unpack_bf16x2(ob.w, q[6], q[7]);
                        uint2 o8;
                        o8.x = f32x4_to_e4m3x4(clamp448(__fmul_rn(q[0], inv_os)), clamp448(__fmul_rn(q[1], inv_os)),
                                               clamp448(__fmul_rn(q[2], inv_os)), clamp448(__fmul_rn(q[3], inv_os)));
                        o8.y = f32x4_to_e4m3x4(clamp448(__fmul_rn(q[4], inv_os)), clamp448(__fmul_rn(q[5], inv_os)),
                                               clamp448(__fmul_rn(q[6], inv_os)), clamp448(__fmul_rn(q[7], inv_os)));
                        st_global_v2(p.O_fp8 + o, o8);
                    }
                    if (p.lse && rank == 0 && dq == 0 && ch == 0)
                        p.lse[((size_t)b * p.Hq + hq) * p.Sq + t] =
                            (Lw > 0.0f) ? (M + log2f(Lw)) * 0.6931471805599453f : -INFINITY;
                }
            }
            ATT_STAMP(11);
        }
    }
    __syncwarp();
    if (!XC && via_scratch) {
        // ---------------- combine through global scratch.  Block of (batch, kv head, tile, split) in o_accum, as bf16:
        // rows_valid x D, stored [slice][row][D / C]; the rows of all tiles of one (split, batch, kv head) are packed
        // back to back, so the caller's (splits, batch, heads, seqlen_q, D) fp32 buffer is always large enough.
        const unsigned tile_id = (unsigned)((b * p.Hkv + hk) * ntiles + tile);
        const unsigned arrivals = C * DQ;        // one counter per tile: all kv splits of all DQ parts
        unsigned* cnt = p.counters + 2 * tile_id;
        const size_t split_stride = (size_t)p.B * p.Hq * p.Sq;            // rows per split in the scratch
        const size_t row0 = ((size_t)(b * p.Hkv + hk) * p.Sq << gshift) + (size_t)tile * 128;
        const int dper = DV / (int)C;
        const uint32_t slice_bytes = (uint32_t)rows_valid * dper * 2;
        const size_t part_off = (size_t)dq * rows_valid * (DV * 2);
        uint8_t* gbase = reinterpret_cast<uint8_t*>(p.o_accum);
        float* s_w = reinterpret_cast<float*>(smem + 65536);        // [row][8] combine weights
        float* s_l = s_w + 128 * 8;                                  // [split][row] log-sum-exps of the partials
        // the log-sum-exps of a tile are rows_valid consecutive floats per split: fetched with the slices when aligned
        const bool lse_bulk = ((split_stride | row0 | (size_t)rows_valid) & 3) == 0 &&
                              (reinterpret_cast<uintptr_t>(p.lse_accum) & 15) == 0;
        ATT_STAMP(8);
        __threadfence();
        __syncthreads();
        ATT_STAMP(9);
        if (threadIdx.x == 0) {
            // arrive without waiting for the old value (every thread fenced its part of the partial before the barrier
            // above, so a relaxed add publishes it), then poll
            asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(cnt), "r"(256u / arrivals) : "memory");
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
            } else {
                // this split's column slice of all C partials: C bulk loads of rows_valid x dper bf16
                asm volatile("fence.proxy.async;" ::: "memory");
                tc::mbar_arrive_expect_tx(c_full, C * slice_bytes + (lse_bulk ? C * (uint32_t)rows_valid * 4u : 0u));
                for (uint32_t sidx = 0; sidx < C; ++sidx) {
                    tc::bulk_load(cbuf + sidx * slice_bytes,
                                  gbase + (sidx * split_stride + row0) * (size_t)(D * 2) + part_off +
                                      (size_t)rank * slice_bytes,
                                  slice_bytes, c_full);
                    if (lse_bulk)
                        tc::bulk_load(s_l + sidx * 128, p.lse_accum + sidx * split_stride + row0,
                                      (uint32_t)rows_valid * 4u, c_full);
                }
            }
        }
        __syncthreads();
        ATT_STAMP(10);
        if (!*abort_flag) {
            // weights of the C partials of a row from their log-sum-exps
            if (lse_bulk) ATTN_WAIT(c_full, 0u, AERR_SOFTMAX);
            if ((int)threadIdx.x < rows_valid && !*abort_flag) {
                const int r = threadIdx.x;
                const int t = tok0 + (r >> gshift);
                const int hq = hk * p.G + (r & (p.G - 1));
                const size_t r0 = ((size_t)b * p.Hq + hq) * p.Sq + t;
                float w[8];
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx)
                    w[sidx] = (uint32_t)sidx < C
                                  ? (lse_bulk ? s_l[sidx * 128 + r] : __ldcg(p.lse_accum + sidx * split_stride + row0 + r))
                                  : -INFINITY;
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
#pragma unroll
                for (int sidx = 0; sidx < 8; ++sidx) s_w[r * 8 + sidx] = w[sidx] * invL;
                if (p.lse && rank == 0 && dq == 0) p.lse[r0] = (Lw > 0.0f) ? (M + log2f(Lw)) * 0.6931471805599453f : -INFINITY;
            }
            if (!lse_bulk) ATTN_WAIT(c_full, 0u, AERR_SOFTMAX);
        }
        __syncthreads();
        if (!*abort_flag) {
            const int cpr = dper >> 3;                       // 16-byte chunks (8 columns) per slice row
            const int d0 = dq * DV + (int)rank * dper;
            const float inv_os = p.O_fp8 ? __fdiv_rn(1.0f, *p.out_scale) : 0.0f;
            const int cshift = 31 - __clz(cpr);
            for (int idx = threadIdx.x; idx < rows_valid * cpr; idx += 192) {
                const int r = idx >> cshift, ch = idx & (cpr - 1);
                const int t = tok0 + (r >> gshift);
                const int hq = hk * p.G + (r & (p.G - 1));
                float a[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) a[i] = 0.0f;
#pragma unroll
                for (uint32_t sidx = 0; sidx < 8; ++sidx) {             // all loads of the row in flight at once
                    if (sidx >= C) break;
                    const uint4 x = *reinterpret_cast<const uint4*>(cbuf + sidx * slice_bytes + ((uint32_t)r * cpr + ch) * 16u);
                    const float ws = s_w[r * 8 + sidx];
                    float f0, f1;
                    unpack_bf16x2(x.x, f0, f1); a[0] += ws * f0; a[1] += ws * f1;
                    unpack_bf16x2(x.y, f0, f1); a[2] += ws * f0; a[3] += ws * f1;
                    unpack_bf16x2(x.z, f0, f1); a[4] += ws * f0; a[5] += ws * f1;
                    unpack_bf16x2(x.w, f0, f1); a[6] += ws * f0; a[7] += ws * f1;
                }
                const size_t o = (size_t)b * p.o_bs + (size_t)t * p.o_rs + (size_t)hq * p.o_hs + d0 + ch * 8;
                uint4 ob;
                ob.x = pack_bf16x2(a[0], a[1]);
                ob.y = pack_bf16x2(a[2], a[3]);
                ob.z = pack_bf16x2(a[4], a[5]);
                ob.w = pack_bf16x2(a[6], a[7]);
                st_global_v4(p.O + o, ob);
                if (p.O_fp8) {
                    float q[8];
                    unpack_bf16x2(ob.x, q[0], q[1]);
                    unpack_bf16x2(ob.y, q[2], q[3]);
                    unpack_bf16x2(ob.z, q[4], q[5]);
                    unpack_bf16x2(ob.w, q[6], q[7]);
                    uint2 o8;
                    o8.x = f32x4_to_e4m3x4(clamp448(__fmul_rn(q[0], inv_os)), clamp448(__fmul_rn(q[1], inv_os)),
                                           clamp448(__fmul_rn(q[2], inv_os)), clamp448(__fmul_rn(q[3], inv_os)));
                    o8.y = f32x4_to_e4m3x4(clamp448(__fmul_rn(q[4], inv_os)), clamp448(__fmul_rn(q[5], inv_os)),
                                           clamp448(__fmul_rn(q[6], inv_os)), clamp448(__fmul_rn(q[7], inv_os)));
                    st_global_v2(p.O_fp8 + o, o8);
                }
            }
        }
        __syncthreads();
        ATT_STAMP(11);
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) tc::tmem_dealloc(tmem, (DQ == 1 ? 512 : 256));
    ATT_STAMP(12);
}

template <int DQ, bool XC>
__global__ void __launch_bounds__(192, 1)
attn_d256_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    attn_d256_body<XC ? 0 : DQ, XC>(tmQ, tmK, tmV, p, (int)blockIdx.x / DQ, (int)blockIdx.x % DQ, (int)gridDim.x / DQ,
                                    DQ);
}

// Cluster exchange with a ragged last row tile: the full tiles in four head-dim parts, the last one in two.  A CTA of
// this size runs alone on its SM, and the B200s measured hold 15 clusters of eight such CTAs (the number depends on which
// SMs of a part are enabled; the host asks the occupancy API): at the action-expert shape -- 400 query rows, 3 full tiles and
// one of 16 rows -- 16 clusters do not fit but 3 x 4 + 2 do.  blockIdx.x 0 and 1: the halves of the last tile (they
// have the longer way to go and start first); above: part (x - 2) % 4 of tile (x - 2) / 4.  The last tile has at most
// RAGGED_ROWS rows, which keeps its receive slots, and with them the shared memory of the launch, small enough for a
// CTA of the previous kernel to stay resident beside it (the early start under programmatic dependent launch).
__global__ void __launch_bounds__(192, 1)
attn_d256_ragged_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    const int ntiles = ((int)gridDim.x - 2) / 4 + 1;
    const int x = (int)blockIdx.x - 2;
    const bool last = x < 0;
    attn_d256_body<0, true>(tmQ, tmK, tmV, p, last ? ntiles - 1 : x / 4, last ? (int)blockIdx.x : x % 4, ntiles,
                            last ? 2 : 4);
}

static int launch_attn_d256(const void* Q, const void* K, const void* V, AttnParams p, const long long* qs,
                            const long long* ks, const long long* vs, int splits, bool pdl, cudaStream_t stream) {
    using Cfg = D256Cfg;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return FRT_ERR_UNSUPPORTED;
    static bool attr_done[64] = {false};                 // the attribute is per device
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_d256_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Cfg::smem_bytes(1));
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        e = cudaFuncSetAttribute(attn_d256_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::smem_bytes(4));
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        e = cudaFuncSetAttribute(attn_d256_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::smem_bytes(4, true));
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        e = cudaFuncSetAttribute(attn_d256_ragged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::ragged_smem_bytes());
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        attr_done[dev] = true;
    }
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    CUtensorMap tmQ, tmK, tmV;
    {
        uint64_t dims[5] = {(uint64_t)Cfg::D, (uint64_t)p.G, (uint64_t)p.Hkv, (uint64_t)p.Sq, (uint64_t)p.B};
        uint64_t str[4] = {(uint64_t)qs[2] * 2, (uint64_t)qs[2] * 2 * p.G, (uint64_t)qs[1] * 2, (uint64_t)qs[0] * 2};
        uint32_t box[5] = {64, (uint32_t)p.G, 1, (uint32_t)(128 / p.G), 1};
        int rc = make_tmap_bf16(&tmQ, Q, 5, dims, str, box);
        if (rc) return rc;
    }
    {
        uint64_t dims[4] = {(uint64_t)Cfg::D, (uint64_t)p.Hkv, (uint64_t)p.Skv, (uint64_t)p.B};
        uint64_t strk[3] = {(uint64_t)ks[2] * 2, (uint64_t)ks[1] * 2, (uint64_t)ks[0] * 2};
        uint64_t strv[3] = {(uint64_t)vs[2] * 2, (uint64_t)vs[1] * 2, (uint64_t)vs[0] * 2};
        uint32_t box[4] = {64, 1, (uint32_t)Cfg::BKV, 1};
        int rc = make_tmap_bf16(&tmK, K, 4, dims, strk, box);
        if (rc) return rc;
        rc = make_tmap_bf16(&tmV, V, 4, dims, strv, box);
        if (rc) return rc;
    }
#ifdef FRT_PHASE_STAMPS
    p.trace_slot = g_attn_trace_slot;
    g_attn_trace_slot = (g_attn_trace_slot + 1) % 8;
#endif
    p.chunks_total = (p.Skv + Cfg::BKV - 1) / Cfg::BKV;
    if (splits > p.chunks_total) splits = p.chunks_total;
    if (splits < 1) splits = 1;
    while (splits & (splits - 1)) --splits;            // power of two: each split finishes D / splits columns
    if (splits == 1) p.o_accum = nullptr;
    const int tiles = (p.Sq * p.G + 127) / 128;
    int dq = 1;
    if (p.o_accum) {
        const long long ctas = (long long)tiles * p.Hkv * p.B * splits;
        if (ctas > sms) return FRT_ERR_UNSUPPORTED;    // the CTAs of a tile wait for one another
        // four head-dim parts per (tile, split) while the whole grid still fits one wave and a slice keeps 8 columns
        if (ctas * 4 <= sms && 64 / splits >= 8 && !(p.flags & 4)) dq = 4;
    }
    // with four head-dim parts the kv splits of a (tile, part) exchange their partials as one cluster (flags bit 3
    // keeps the global scratch) -- when the device can hold all those clusters at once: CTAs of this size run one per
    // SM and how many clusters of them fit depends on the part's enabled SMs.  Otherwise the last tile in two parts, if
    // that fits; otherwise the scratch.
    bool xc = dq == 4 && !(p.flags & 8);
    bool ragged = false;
    if (xc) {
        int lg = 0;
        while ((1 << lg) < splits) ++lg;                     // splits is 2, 4 or 8 here
        static int max_clusters[64][4][2];                   // [device][log2 splits][ragged], 0 = not asked yet
        auto fits = [&](bool rg, int need) {
            int& m = max_clusters[dev][lg][rg ? 1 : 0];
            if (m == 0) {
                cudaLaunchConfig_t q = {};
                q.gridDim = dim3(rg ? 4 * (tiles - 1) + 2 : tiles * 4, p.Hkv * p.B, splits);
                q.blockDim = dim3(192);
                q.dynamicSmemBytes = rg ? Cfg::ragged_smem_bytes() : Cfg::smem_bytes(4, true);
                cudaLaunchAttribute qa[1];
                qa[0].id = cudaLaunchAttributeClusterDimension;
                qa[0].val.clusterDim.x = 1;
                qa[0].val.clusterDim.y = 1;
                qa[0].val.clusterDim.z = (unsigned)splits;
                q.attrs = qa;
                q.numAttrs = 1;
                int n = 0;
                cudaError_t qe = rg ? cudaOccupancyMaxActiveClusters(&n, attn_d256_ragged_kernel, &q)
                                    : cudaOccupancyMaxActiveClusters(&n, attn_d256_kernel<4, true>, &q);
                m = (qe == cudaSuccess && n > 0) ? n : -1;
                if (qe != cudaSuccess) cudaGetLastError();
            }
            return need <= m;
        };
        if (!fits(false, tiles * 4 * p.Hkv * p.B)) {
            const int tail_rows = p.Sq * p.G - 128 * (tiles - 1);
            if (tail_rows <= Cfg::RAGGED_ROWS && fits(true, (4 * (tiles - 1) + 2) * p.Hkv * p.B)) ragged = true;
            else xc = false;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ragged ? 4 * (tiles - 1) + 2 : tiles * dq, p.Hkv * p.B, splits);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = ragged ? Cfg::ragged_smem_bytes() : Cfg::smem_bytes(dq, xc);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (xc) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = (unsigned)splits;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = ragged    ? cudaLaunchKernelEx(&cfg, attn_d256_ragged_kernel, tmQ, tmK, tmV, p)
                    : xc      ? cudaLaunchKernelEx(&cfg, attn_d256_kernel<4, true>, tmQ, tmK, tmV, p)
                    : dq == 4 ? cudaLaunchKernelEx(&cfg, attn_d256_kernel<4, false>, tmQ, tmK, tmV, p)
                              : cudaLaunchKernelEx(&cfg, attn_d256_kernel<1, false>, tmQ, tmK, tmV, p);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}
