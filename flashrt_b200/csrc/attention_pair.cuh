// Long-sequence flash attention (head_dim 128) for sm_100a: two 128-row query tiles per CTA in ping-pong.
//
// Included by attention.cu inside namespace frt (it uses AttnParams, the tensor-map helpers and ATTN_WAIT).
//
// Why a second kernel: with one query tile per CTA the tensor core idles while the softmax warps work on S and
// the softmax warps idle during the MMAs.  Here a CTA owns two query tiles A and B that share every K/V chunk:
//   tensor core : QK(A,j+1) and PV(B,j) run while the softmax warps of A work on S_A(j+1), and vice versa;
//   shared mem  : K/V chunks are double-buffered and fetched once for 256 query rows;
//   TMEM        : S_A, S_B (128 fp32 columns each) and O_A, O_B (128 each) fill the 512 columns; P (bf16) is
//                 written over the first 64 columns of its S and feeds the PV MMA as the A operand from TMEM,
//                 so P never goes through shared memory;
//   rescale     : O is rescaled only when a row maximum grows by more than 2^8 (the stale maximum keeps P <= 256
//                 and the final normalisation by the row sum makes the result independent of it).
// Warps: 0-3 softmax of tile A (thread = row), 4-7 softmax of tile B, 8 TMA producer, 9 MMA issuer + TMEM owner.
// Ordering: all tcgen05 operations are issued by one thread and execute in issue order; s_full(t, j) is committed
// after QK(t, j), which was issued after PV(t, j-1), so a softmax warp that sees s_full(t, j) may overwrite
// P(t, j-1) and rescale O_t; PV(t, j) is issued only after p_ready(t, j).
#pragma once

struct PairCfg {
    static constexpr int D = 128, BKV = 128;
    static constexpr int Q_BYTES = 128 * D * 2;          // one query tile
    static constexpr int KV_BYTES = BKV * D * 2;         // one of K or V, one stage
    static constexpr int OFF_K = 2 * Q_BYTES;
    static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
    static constexpr int DATA_BYTES = OFF_V + 2 * KV_BYTES;
    static constexpr int SMEM_BYTES = DATA_BYTES + 256 + 1024;
    static constexpr int TMEM_COLS = 512;
    static constexpr float RESCALE_THRESHOLD = 8.0f;     // log2 domain
};

__global__ void __launch_bounds__(320, 1)
attn_pair_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, AttnParams p) {
    using Cfg = PairCfg;
    constexpr int D = Cfg::D, BKV = Cfg::BKV;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sQ = smem;
    uint8_t* sK = smem + Cfg::OFF_K;
    uint8_t* sV = smem + Cfg::OFF_V;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::DATA_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;      // [2]
    uint64_t* v_full = bars + 3;      // [2]
    uint64_t* kv_empty = bars + 5;    // [2]
    uint64_t* s_full = bars + 7;      // [2] per tile
    uint64_t* p_ready = bars + 9;     // [2] per tile, 128 arrivals
    uint64_t* o_done = bars + 11;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint64_t deadline = tc::global_timer_ns() + FRT_KERNEL_DEADLINE_NS;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int hk = blockIdx.y % p.Hkv;
    const int b = blockIdx.y / p.Hkv;
    const int tok_per_tile = 128 / p.G;
    const int tok0 = blockIdx.x * 2 * tok_per_tile;
    const int nchunks = p.chunks_total;

    if (threadIdx.x == 0) {
        tc::mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            tc::mbar_init(&k_full[i], 1);
            tc::mbar_init(&v_full[i], 1);
            tc::mbar_init(&kv_empty[i], 1);
            tc::mbar_init(&s_full[i], 1);
            tc::mbar_init(&p_ready[i], 128);
        }
        tc::mbar_init(o_done, 1);
        *abort_flag = 0;
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&tmQ);
        tc::tma_prefetch_desc(&tmK);
        tc::tma_prefetch_desc(&tmV);
    }
    if (warp == 9) {
        tc::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    pdl_launch_dependents();

    if (warp == 8 && lane == 0) {
        // ---------------- TMA producer
        pdl_wait();
        tc::mbar_arrive_expect_tx(q_full, 2 * Cfg::Q_BYTES);
        for (int t = 0; t < 2; ++t)
            for (int db = 0; db < 2; ++db)
                tc::tma_load_5d(sQ + t * Cfg::Q_BYTES + db * (128 * 128), &tmQ, q_full, db * 64, 0, hk,
                                tok0 + t * tok_per_tile, b);
        for (int j = 0; j < nchunks && !*abort_flag; ++j) {
            const int st = j & 1;
            if (j >= 2) ATTN_WAIT(&kv_empty[st], (uint32_t)(((j >> 1) - 1) & 1), AERR_PRODUCER);
            if (*abort_flag) break;
            const int key0 = j * BKV;
            tc::mbar_arrive_expect_tx(&k_full[st], Cfg::KV_BYTES);
            for (int db = 0; db < 2; ++db)
                tc::tma_load_4d(sK + st * Cfg::KV_BYTES + db * (BKV * 128), &tmK, &k_full[st], db * 64, hk, key0, b);
            tc::mbar_arrive_expect_tx(&v_full[st], Cfg::KV_BYTES);
            for (int db = 0; db < 2; ++db)
                tc::tma_load_4d(sV + st * Cfg::KV_BYTES + db * (BKV * 128), &tmV, &v_full[st], db * 64, hk, key0, b);
        }
    } else if (warp == 9 && lane == 0) {
        // ---------------- MMA issuer
        constexpr uint32_t idesc_s = tc::make_idesc(1, 1, 0, 0, 128, BKV);   // bf16 x bf16, both K-major
        constexpr uint32_t idesc_o = tc::make_idesc(1, 1, 0, 1, 128, D);     // A = P from TMEM, B = V MN-major
        // descriptors differ only in their start-address field (units of 16 bytes): build the bases once
        const uint64_t dq_base = tc::make_desc_kmajor_sw128(tc::smem_u32(sQ));
        const uint64_t dk_base = tc::make_desc_kmajor_sw128(tc::smem_u32(sK));
        const uint64_t dv_base = tc::make_desc_mnmajor_sw128(tc::smem_u32(sV), BKV * 128);
        auto qk = [&](int t, int j) {
            const uint64_t dq = dq_base + (uint64_t)(t * (Cfg::Q_BYTES >> 4));
            const uint64_t dk = dk_base + (uint64_t)((j & 1) * (Cfg::KV_BYTES >> 4));
            const uint32_t d_tm = tmem + t * 128;
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
                // 64-element block k / 4 (16 KB apart), 32 bytes per K = 16 step inside the 128-byte row
                const uint64_t off = (uint64_t)((k / 4) * ((128 * 128) >> 4) + 2 * (k % 4));
                tc::mma_f16(d_tm, dq + off, dk + off, idesc_s, k > 0 ? 1u : 0u);
            }
            tc::mma_commit(&s_full[t]);
        };
        auto pv = [&](int t, int j) {
            const uint64_t dv = dv_base + (uint64_t)((j & 1) * (Cfg::KV_BYTES >> 4));
            const uint32_t d_tm = tmem + 256 + t * 128, a_tm = tmem + t * 128;
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k)       // 16 keys = 16 rows of 128 bytes further on
                tc::mma_f16_ts(d_tm, a_tm + 8 * k, dv + (uint64_t)(k * ((16 * 128) >> 4)), idesc_o,
                               (j > 0 || k > 0) ? 1u : 0u);
        };
        ATTN_WAIT(q_full, 0u, AERR_MMA);
        if (nchunks > 0 && !*abort_flag) {
            ATTN_WAIT(&k_full[0], 0u, AERR_MMA);
            if (!*abort_flag) {
                tc::tc_fence_after_sync();
                qk(0, 0);
                qk(1, 0);
            }
        }
        for (int j = 0; j < nchunks && !*abort_flag; ++j) {
            const int st = j & 1;
            const uint32_t ph = (uint32_t)(j & 1);
            ATTN_WAIT(&p_ready[0], ph, AERR_MMA);
            ATTN_WAIT(&v_full[st], (uint32_t)((j >> 1) & 1), AERR_MMA);
            if (*abort_flag) break;
            tc::tc_fence_after_sync();
            pv(0, j);
            if (j + 1 < nchunks) {
                ATTN_WAIT(&k_full[(j + 1) & 1], (uint32_t)(((j + 1) >> 1) & 1), AERR_MMA);
                if (*abort_flag) break;
                tc::tc_fence_after_sync();
                qk(0, j + 1);
            }
            ATTN_WAIT(&p_ready[1], ph, AERR_MMA);
            if (*abort_flag) break;
            tc::tc_fence_after_sync();
            pv(1, j);
            tc::mma_commit(&kv_empty[st]);
            if (j + 1 < nchunks) qk(1, j + 1);
        }
        if (!*abort_flag) tc::mma_commit(o_done);
    } else if (warp < 8) {
        // ---------------- softmax: tile t, thread = row
        pdl_wait();
        const int t = warp >> 2;
        const int w4 = warp & 3;
        const int row = w4 * 32 + lane;
        const uint32_t lane_off = (uint32_t)(w4 * 32) << 16;
        const uint32_t tmem_S = tmem + t * 128 + lane_off;      // P (bf16) overlays its first 64 columns
        const uint32_t tmem_O = tmem + 256 + t * 128 + lane_off;
        int kv_len = p.Skv;
        if (p.seqused_k) { int u = *p.seqused_k; kv_len = u < kv_len ? u : kv_len; }
        float m_run = -INFINITY, l_run = 0.0f;
        bool alive = true;
        for (int j = 0; j < nchunks; ++j) {
            ATTN_WAIT(&s_full[t], (uint32_t)(j & 1), AERR_SOFTMAX);
            __syncwarp();
            if (__any_sync(0xffffffffu, *abort_flag != 0)) { alive = false; break; }
            tc::tc_fence_after_sync();
            const int valid = kv_len - j * BKV;                 // keys of this chunk that count (warp-uniform)
            // the whole row of S (128 fp32) comes into registers with one wait
            uint32_t sv[BKV];
            tc::tmem_ld32(tmem_S + 0, sv + 0);
            tc::tmem_ld32(tmem_S + 32, sv + 32);
            tc::tmem_ld32(tmem_S + 64, sv + 64);
            tc::tmem_ld32(tmem_S + 96, sv + 96);
            tc::tmem_ld_wait();
            if (valid < BKV) {                                  // last, partial chunk (warp-uniform branch)
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
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float mx_s = mx * p.scale_log2;               // scale_log2 > 0
            // keep the stale maximum unless it is exceeded by more than the threshold
            const bool grow = mx_s > m_run + Cfg::RESCALE_THRESHOLD || (m_run == -INFINITY && mx_s > -INFINITY);
            const float m_new = grow ? mx_s : m_run;
            if (__any_sync(0xffffffffu, grow && j > 0)) {       // warp-uniform: tcgen05.ld / st are collective
                const float alpha = grow ? tc::ex2_approx(m_run - m_new) : 1.0f;   // m_run = -inf -> 0
                l_run *= alpha;
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
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
            // P = 2^(s * scale - m) (2^-inf = 0 for masked keys), row sum, bf16 pairs into TMEM over S
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
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            tc::tmem_st_wait();
            l_run += sum;
            tc::tc_fence_before_sync();
            tc::mbar_arrive(&p_ready[t]);
        }
        // ---------------- result: O / l -> bf16 (and optional e4m3 copy), one row per thread
        if (alive) {
            if (nchunks > 0) ATTN_WAIT(o_done, 0u, AERR_SOFTMAX);
            __syncwarp();
            if (!__any_sync(0xffffffffu, *abort_flag != 0)) {
                tc::tc_fence_after_sync();
                const int tok = tok0 + t * tok_per_tile + row / p.G;
                const int hq = hk * p.G + row % p.G;
                const bool store = tok < p.Sq;
                const float invl = l_run > 0.0f ? 1.0f / l_run : 0.0f;
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
    }
    __syncwarp();
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 9) tc::tmem_dealloc(tmem, Cfg::TMEM_COLS);
}

static int launch_attn_pair(const void* Q, const void* K, const void* V, AttnParams p, const long long* qs,
                            const long long* ks, const long long* vs, bool pdl, cudaStream_t stream) {
    using Cfg = PairCfg;
    static PerDeviceOnce attr_once;
    int attr_dev = 0;
    if (attr_once.need(attr_dev)) {
        cudaError_t e = cudaFuncSetAttribute(attn_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Cfg::SMEM_BYTES);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        attr_once.set(attr_dev);
    }
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
    p.chunks_total = (p.Skv + Cfg::BKV - 1) / Cfg::BKV;
    p.o_accum = nullptr;
    const int tiles = (p.Sq * p.G + 127) / 128;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((tiles + 1) / 2, p.Hkv * p.B, 1);
    cfg.blockDim = dim3(320);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, attn_pair_kernel, tmQ, tmK, tmV, p);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}
