// Small-M FP8 GEMM with the TOKENS on the 128 TMEM lanes and the WEIGHTS on the accumulator columns, sm_100a.
//
// Included by gemm_fp8.cu inside namespace frt (tensor-map cache, status word, arithmetic helpers).
//
// Why this orientation for M <= 128 activation rows: a tcgen05.mma (kind::f8f6f4, K = 32) costs the issuing
// thread about 160 cycles whatever its shape (measured: 128 x 256, 128 x 64 and 64 x 8 all take the same time), so
// the launch-latency-bound GEMMs of the denoise loop want as many weight bytes per instruction as possible and as
// few instructions per CTA as possible:
//   * weights on N: up to 256 weight rows x 32 K-bytes = 8 KB per instruction (the swapped kernel moves 4 KB);
//   * split-K over a thread-block cluster (1 x 1 x S, S <= 8): a CTA owns BN weight rows x K / S, i.e. 2-4 k-blocks
//     of 128 bytes = 8-16 instructions, and a launch spreads over 80-128 SMs instead of 32-64;
//   * an accumulator row is one token: a thread that finishes (token, 8 features) holds 8 CONSECUTIVE output
//     features, so RoPE pairs, GeGLU (gate column j and up column 128 + j of the same tile), the gated residual
//     update and the row sum of squares all stay inside a thread or a group of 8-16 neighbouring lanes.
// Split-K partials are staged in shared memory as rows of fp32 (16-byte chunks xor-swizzled by the row) and summed
// in fixed order 0, 1, ... through distributed shared memory; rank r of the cluster finishes a contiguous range of
// tokens.  No global workspace; results are deterministic.
//
// A operand: FP8 activations by TMA (PRO_TMA), or produced inside the kernel (PRO_NORM): every CTA reads the bf16
// residual rows of its K-slice, the per-tile partial sums of squares left by the previous projection's epilogue
// (EPI_RESID below) and the adaRMS style row, and writes the modulated FP8 operand straight into the swizzled
// shared-memory tile -- the norm kernel between two projections disappears.  Stands for
// gate_residual_ada_norm_fp8 (csrc/kernels/fusion.cu:15-81) + GemmRunner::fp8_nn_dev of the reference.
//
// Epilogues: bf16 (+bias); RoPE + q/k/v split + KV append (csrc/kernels/rope.cu:135-277); GeGLU -> FP8
// (csrc/kernels/activation.cu:249-279); gated residual update + per-tile row sums of squares
// (csrc/kernels/fusion.cu:41-64, first pass).
//
// Warps: 0 (lane 0) TMA producer, 1 (lane 0) MMA issuer, 2 TMEM owner; all 8 warps stage and finish the tile.
// Every wait is bounded by the kernel deadline; on expiry the status word is set, the work is skipped and every
// thread still reaches the cluster barriers and the TMEM release.
#pragma once

enum { TOK_EPI_BF16 = 0, TOK_EPI_ROPE = 1, TOK_EPI_GEGLU = 2, TOK_EPI_RESID = 3 };
enum { TOK_PRO_TMA = 0, TOK_PRO_NORM = 1 };
enum { TOK_STAT_STRIDE = 128 };          // floats between the per-tile rows of a statistics buffer

struct TokParams {
    int M, N;                  // activation rows (all m-tiles), output features
    int nkb;                   // 128-byte k-blocks per split
    int stages;                // shared-memory ring depth (>= nkb when the A operand is produced in the kernel)
    int stage_rows;            // rows of the fp32 staging area = tokens of an m-tile rounded up to 32
    const float* sa;           // device scalars (may be null = 1): activation / weight scale
    const float* sb;
    float alpha_host;
    // TOK_EPI_BF16
    __nv_bfloat16* out;
    const __nv_bfloat16* bias;
    // TOK_EPI_ROPE
    const __nv_bfloat16* rope;
    __nv_bfloat16* outQ;
    __nv_bfloat16* outK;
    __nv_bfloat16* outV;
    const int* devpos;
    int q_dim, k_dim, v_dim, head_dim;
    // TOK_EPI_GEGLU
    uint8_t* out8;
    const float* out_scale;
    int half;
    // TOK_EPI_RESID: residual (M, N) bf16 in/out, gate (N,), stats_out [tile][TOK_STAT_STRIDE] (may be null)
    __nv_bfloat16* resid;
    const __nv_bfloat16* gate;
    float* stats_out;
    // TOK_PRO_NORM: x (M, K) bf16, stats_in [n_stat][TOK_STAT_STRIDE], style = [scale (K) | shift (K)] one row
    const __nv_bfloat16* x;
    const float* stats_in;
    int n_stat;
    int K;
    const __nv_bfloat16* style;
    float eps;
};

template <int BN>
struct TokCfg {
    static constexpr int A_BYTES = 128 * 128;                 // 128 token rows x 128 K-bytes
    static constexpr int W_BYTES = BN * 128;
    static constexpr int STAGE_BYTES = A_BYTES + W_BYTES;
    static constexpr int MAX_STAGES = BN == 256 ? 4 : BN == 128 ? 6 : 8;
    static constexpr int AUX_BYTES = 2048;                    // barriers, flags, per-token 1 / rms
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static int smem_bytes(int stages, int stage_rows) {
        const int ops = stages * STAGE_BYTES, red = stage_rows * BN * 4;
        return AUX_BYTES + 1024 + (ops > red ? ops : red);
    }
};

__device__ __forceinline__ float4 dsmem_ld_v4(uint32_t cluster_addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(cluster_addr)
                 : "memory");
    return v;
}

// Sum over the S ranks (fixed order) of the 8 staged fp32 values of (row, 8-column group starting at column c8*8).
template <int BN>
__device__ __forceinline__ void tok_reduce8(const uint32_t* rank_base, uint32_t S, int row, int c8, float* a) {
    const uint32_t sw = (uint32_t)(row & 7);
    const uint32_t o0 = (uint32_t)row * (BN * 4) + ((((uint32_t)(2 * c8)) ^ sw) << 4);
    const uint32_t o1 = (uint32_t)row * (BN * 4) + ((((uint32_t)(2 * c8 + 1)) ^ sw) << 4);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = 0.0f;
    // four ranks (eight 16-byte loads) in flight per round trip
#pragma unroll
    for (uint32_t s0 = 0; s0 < 8; s0 += 4) {
        if (s0 < S) {
            float4 x[4], y[4];
#pragma unroll
            for (uint32_t s = 0; s < 4; ++s) {
                if (s0 + s < S) {
                    x[s] = dsmem_ld_v4(rank_base[s0 + s] + o0);
                    y[s] = dsmem_ld_v4(rank_base[s0 + s] + o1);
                }
            }
#pragma unroll
            for (uint32_t s = 0; s < 4; ++s) {
                if (s0 + s < S) {
                    a[0] += x[s].x; a[1] += x[s].y; a[2] += x[s].z; a[3] += x[s].w;
                    a[4] += y[s].x; a[5] += y[s].y; a[6] += y[s].z; a[7] += y[s].w;
                }
            }
        }
    }
}

template <int BN, int PRO, int EPI>
__global__ void __launch_bounds__(256, 2)
gemm_tok_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, TokParams p) {
    static_assert(EPI != TOK_EPI_GEGLU || BN == 256, "GeGLU tiles are 128 gate rows + the 128 matching up rows");
    using Cfg = TokCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* aux = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = aux + Cfg::AUX_BYTES;                       // 1024-aligned
    uint64_t* full = reinterpret_cast<uint64_t*>(aux);          // [8]
    uint64_t* empty = full + 8;                                  // [8]
    uint64_t* accum_bar = empty + 8;
    uint64_t* a_ready = accum_bar + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(a_ready + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;
    volatile int* consumed = abort_flag + 2;
    float* s_rms = reinterpret_cast<float*>(aux + 512);          // [128]
    float* red = reinterpret_cast<float*>(tiles);                // aliases the operand ring after the last MMA

    const uint64_t deadline = tc::global_timer_ns() + FRT_KERNEL_DEADLINE_NS;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tile = blockIdx.x;
    // first weight row of the tile; with GeGLU a tile is 128 gate rows + the 128 matching up rows
    const int n0 = (EPI == TOK_EPI_GEGLU) ? tile * 128 : tile * BN;
    const int m0 = blockIdx.y * 128;
    const int Mt = (p.M - m0) < 128 ? (p.M - m0) : 128;         // tokens of this m-tile
    const uint32_t S = tc::cluster_nctarank();
    const uint32_t rank = tc::cluster_ctarank();
    const int nkb = p.nkb;
    const int kb0 = (int)rank * nkb;
    const int STG = p.stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 8; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        tc::mbar_init(accum_bar, 1);
        tc::mbar_init(a_ready, 256);
        *abort_flag = 0;
        *issued = 0;
        *consumed = 0;
        tc::mbar_fence_init();
        if (PRO == TOK_PRO_TMA) tc::tma_prefetch_desc(&tmA);
        tc::tma_prefetch_desc(&tmW);
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
        // ---------------- TMA producer: the weights do not depend on the producer grid and start streaming now
        const uint32_t tx = (PRO == TOK_PRO_TMA) ? Cfg::STAGE_BYTES : Cfg::W_BYTES;
        auto load_w = [&](int stage, int kb) {
            uint8_t* dst = tiles + stage * Cfg::STAGE_BYTES + Cfg::A_BYTES;
            if (EPI == TOK_EPI_GEGLU) {      // tmW has a 128-row box here
                tc::tma_load_2d(dst, &tmW, &full[stage], kb * 128, n0);
                tc::tma_load_2d(dst + 128 * 128, &tmW, &full[stage], kb * 128, p.half + n0);
            } else {
                tc::tma_load_2d(dst, &tmW, &full[stage], kb * 128, n0);
            }
        };
        const int pre = nkb < STG ? nkb : STG;
        for (int i = 0; i < pre; ++i) {
            tc::mbar_arrive_expect_tx(&full[i], tx);
            load_w(i, kb0 + i);
        }
        pdl_wait();
        if (PRO == TOK_PRO_TMA) {
            for (int i = 0; i < pre; ++i)
                tc::tma_load_2d(tiles + i * Cfg::STAGE_BYTES, &tmA, &full[i], (kb0 + i) * 128, m0);
        }
        *issued = pre;
        for (int i = pre; i < nkb; ++i) {
            const int s = i % STG;
            const uint32_t ph = ((i / STG) - 1) & 1;
            if (!tc::mbar_wait_until(&empty[s], ph, deadline, abort_flag)) {
                *abort_flag = 1;
                atomicCAS(&g_gemm_status, 0, ERR_PRODUCER | (blockIdx.x << 8));
                break;
            }
            tc::mbar_arrive_expect_tx(&full[s], tx);
            load_w(s, kb0 + i);
            if (PRO == TOK_PRO_TMA) tc::tma_load_2d(tiles + s * Cfg::STAGE_BYTES, &tmA, &full[s], (kb0 + i) * 128, m0);
            *issued = i + 1;
        }
    }

    if (PRO == TOK_PRO_NORM) {
        // ---------------- A operand from the residual stream: adaRMS(style) -> FP8, written in the 128-byte-swizzled
        // K-major layout the MMA reads.  Thread = one 16-element chunk of the K-slice, looped over the tokens.
        const int CH = nkb * 8;                       // 16-byte chunks per row of the K-slice (8, 16 or 32)
        const int c16 = threadIdx.x % CH;
        const int rstep = 256 / CH;
        const int r_first = threadIdx.x / CH;
        const int kcol = (kb0 * 128) + c16 * 16;      // first feature of this thread's chunk
        // style row and scale do not depend on the producer grid
        const uint4 sc0 = ld_global_v4(p.style + kcol), sc1 = ld_global_v4(p.style + kcol + 8);
        const uint4 sh0 = ld_global_v4(p.style + p.K + kcol), sh1 = ld_global_v4(p.style + p.K + kcol + 8);
        const float inv_scale = __fdiv_rn(1.0f, p.sa ? *p.sa : 1.0f);
        pdl_wait();
        // per-token 1 / rms from the per-tile partial sums of squares (fixed order)
        if ((int)threadIdx.x < Mt) {
            float tot = 0.0f;
            for (int t = 0; t < p.n_stat; ++t) tot = __fadd_rn(tot, __ldcg(p.stats_in + t * TOK_STAT_STRIDE + m0 + threadIdx.x));
            const float var = __fadd_rn(__fdiv_rn(tot, (float)p.K), p.eps);
            s_rms[threadIdx.x] = __fdiv_rn(1.0f, __fsqrt_rn(var));
        }
        // residual chunks of up to four tokens per pass in flight
        const int passes = (Mt + rstep - 1) / rstep;
        for (int pb = 0; pb < passes; pb += 4) {
            uint4 xa[4], xb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = r_first + (pb + j) * rstep;
                if (pb + j < passes && r < Mt) {
                    const __nv_bfloat16* src = p.x + (size_t)(m0 + r) * p.K + kcol;
                    xa[j] = __ldcg(reinterpret_cast<const uint4*>(src));
                    xb[j] = __ldcg(reinterpret_cast<const uint4*>(src + 8));
                }
            }
            if (pb == 0) __syncthreads();             // s_rms visible (every thread passes here exactly once)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = r_first + (pb + j) * rstep;
                if (pb + j < passes && r < Mt) {
                    const float rms = s_rms[r];
                    const uint32_t xw[8] = {xa[j].x, xa[j].y, xa[j].z, xa[j].w, xb[j].x, xb[j].y, xb[j].z, xb[j].w};
                    const uint32_t scw[8] = {sc0.x, sc0.y, sc0.z, sc0.w, sc1.x, sc1.y, sc1.z, sc1.w};
                    const uint32_t shw[8] = {sh0.x, sh0.y, sh0.z, sh0.w, sh1.x, sh1.y, sh1.z, sh1.w};
                    uint32_t q[4];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        float v[4];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float r0, r1, s0, s1, h0, h1;
                            unpack_bf16x2(xw[i + h], r0, r1);
                            unpack_bf16x2(scw[i + h], s0, s1);
                            unpack_bf16x2(shw[i + h], h0, h1);
                            const float n0v = __fmaf_rn(__fmul_rn(r0, rms), __fadd_rn(1.0f, s0), h0);
                            const float n1v = __fmaf_rn(__fmul_rn(r1, rms), __fadd_rn(1.0f, s1), h1);
                            v[2 * h] = clamp448(__fmul_rn(n0v, inv_scale));
                            v[2 * h + 1] = clamp448(__fmul_rn(n1v, inv_scale));
                        }
                        q[i >> 1] = f32x4_to_e4m3x4(v[0], v[1], v[2], v[3]);
                    }
                    const int kb = c16 >> 3, c = c16 & 7;
                    uint8_t* dst = tiles + kb * Cfg::STAGE_BYTES + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4);
                    *reinterpret_cast<uint4*>(dst) = make_uint4(q[0], q[1], q[2], q[3]);
                }
            }
        }
        if (passes == 0) __syncthreads();
        tc::fence_proxy_async_smem();
        tc::mbar_arrive(a_ready);
    }
    if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        constexpr uint32_t idesc = tc::make_idesc(0, 0, 0, 0, 128, BN);
        bool failed = false;
        if (PRO == TOK_PRO_NORM) {
            if (!tc::mbar_wait_until(a_ready, 0, deadline, abort_flag)) {
                *abort_flag = 1;
                atomicCAS(&g_gemm_status, 0, ERR_MMA | (blockIdx.x << 8));
                failed = true;
            }
        }
        const uint64_t dA0 = tc::make_desc_kmajor_sw128(tc::smem_u32(tiles));
        const uint64_t dW0 = tc::make_desc_kmajor_sw128(tc::smem_u32(tiles + Cfg::A_BYTES));
        for (int i = 0; i < nkb && !failed; ++i) {
            const int s = i % STG;
            const uint32_t ph = (i / STG) & 1;
            if (!tc::mbar_wait_until(&full[s], ph, deadline, abort_flag)) {
                *abort_flag = 1;
                atomicCAS(&g_gemm_status, 0, ERR_MMA | (blockIdx.x << 8));
                failed = true;
                break;
            }
            tc::tc_fence_after_sync();
            const uint64_t so = (uint64_t)((s * Cfg::STAGE_BYTES) >> 4);
#pragma unroll
            for (int k = 0; k < 4; ++k)   // 4 x (K = 32) per 128-byte k-block; +32 bytes = +2 in the address field
                tc::mma_f8(tmem_d, dA0 + so + 2 * k, dW0 + so + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            tc::mma_commit(&empty[s]);
            *consumed = i + 1;
        }
        if (!failed) tc::mma_commit(accum_bar);
    }
    __syncwarp();

    // ---------------- accumulator -> fp32 staging rows (16-byte chunks xor-swizzled by the row)
    pdl_wait();
    const bool acc_seen = tc::mbar_wait_until(accum_bar, 0, deadline, abort_flag);
    const bool have_acc = __all_sync(0xffffffffu, acc_seen);   // tcgen05.ld below is warp-collective
    if (!have_acc && !*abort_flag) {
        *abort_flag = 1;
        atomicCAS(&g_gemm_status, 0, ERR_EPILOGUE | (blockIdx.x << 8));
    }
    __syncwarp();
    tc::tc_fence_after_sync();
    {
        const int quad = warp & 3, chalf = warp >> 2;
        const int row = quad * 32 + lane;
        if (have_acc && quad * 32 < p.stage_rows) {
            const uint32_t trow = tmem_d + ((uint32_t)(quad * 32) << 16);
            const uint32_t sw = (uint32_t)(row & 7);
#pragma unroll 1
            for (int c = chalf * (BN / 2); c < (chalf + 1) * (BN / 2); c += 32) {
                uint32_t v[32];
                tc::tmem_ld32(trow + c, v);
                tc::tmem_ld_wait();
                float4* rrow = reinterpret_cast<float4*>(red + (size_t)row * BN);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    rrow[((uint32_t)((c >> 2) + j)) ^ sw] =
                        make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                    __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
            }
        }
    }
    tc::tc_fence_before_sync();
    if (S > 1) tc::cluster_sync_all(); else __syncthreads();

    // ---------------- finish: rank r sums the S partials of its token range and applies the epilogue
    {
        const uint32_t red_addr = tc::smem_u32(red);
        uint32_t rank_base[8];
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) rank_base[r] = tc::dsmem_map(red_addr, r < S ? r : 0);
        const int per = (Mt + (int)S - 1) / (int)S;
        const int tb = (int)rank * per;
        const int te = tb + per < Mt ? tb + per : Mt;
        constexpr int G = (EPI == TOK_EPI_GEGLU) ? 16 : BN / 8;       // 8-feature groups per token that carry output
        const int items = (te > tb ? te - tb : 0) * G;
        const int items_pad = (items + 31) & ~31;                     // whole warps iterate together (shuffles below)
        const bool live = !*abort_flag;
        float alpha = p.alpha_host;
        if (p.sa) alpha *= *p.sa;
        if (p.sb) alpha *= *p.sb;
        const float inv_os = (EPI == TOK_EPI_GEGLU) ? __fdiv_rn(1.0f, *p.out_scale) : 0.0f;
        const int pos = (EPI == TOK_EPI_ROPE && p.devpos) ? *p.devpos : 0;
        for (int it = threadIdx.x; it < items_pad; it += 256) {
            const bool act = live && it < items;
            const int row = tb + it / G;          // token inside the m-tile
            const int g = it % G;
            const int m = m0 + row;
            float a[8];
            if (act) {
                tok_reduce8<BN>(rank_base, S, row, g, a);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) a[j] = 0.0f;
            }
            if (EPI == TOK_EPI_BF16) {
                const int n = n0 + g * 8;
                if (act && n < p.N) {
                    float f[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        f[j] = a[j] * alpha;
                        if (p.bias && n + j < p.N) f[j] += __bfloat162float(p.bias[n + j]);
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
                }
            } else if (EPI == TOK_EPI_ROPE) {
                // same rounding points as the separate kernels: bf16 GEMM result, fp32 rotation, bf16 store
                const int n = n0 + g * 8;
                if (act && n < p.N) {
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
                }
            } else if (EPI == TOK_EPI_GEGLU) {
                // a = gate columns g*8.. of the tile, b = the matching up columns 128 + g*8..
                const int h = n0 + g * 8;
                if (act && h < p.half) {
                    float b[8];
                    tok_reduce8<BN>(rank_base, S, row, 16 + g, b);
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
            } else {
                // gated residual: x <- bf16(x + bf16(o) * gate); sum of squares of the UNROUNDED update per (tile, token)
                const int n = n0 + g * 8;
                float ssq = 0.0f;
                if (act && n < p.N) {
                    __nv_bfloat16* rp = p.resid + (size_t)m * p.N + n;
                    const uint4 rv = ld_global_v4(rp);
                    const uint4 gv = ld_global_v4(p.gate + n);
                    const uint32_t* rw = &rv.x;
                    const uint32_t* gw = &gv.x;
                    uint4 ob;
                    uint32_t* ow = &ob.x;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float r0, r1, g0, g1;
                        unpack_bf16x2(rw[k], r0, r1);
                        unpack_bf16x2(gw[k], g0, g1);
                        const float o0 = __bfloat162float(__float2bfloat16_rn(a[2 * k] * alpha));
                        const float o1 = __bfloat162float(__float2bfloat16_rn(a[2 * k + 1] * alpha));
                        r0 = __fmaf_rn(o0, g0, r0);
                        r1 = __fmaf_rn(o1, g1, r1);
                        ssq = __fmaf_rn(r0, r0, ssq);
                        ssq = __fmaf_rn(r1, r1, ssq);
                        ow[k] = pack_bf16x2(r0, r1);
                    }
                    st_global_v4(rp, ob);
                }
                // the G lanes of a token are neighbours (G divides 32): butterfly inside the group, fixed order
#pragma unroll
                for (int off = G / 2; off >= 1; off >>= 1) ssq = __fadd_rn(ssq, __shfl_xor_sync(0xffffffffu, ssq, off));
                if (act && g == 0 && p.stats_out) p.stats_out[tile * TOK_STAT_STRIDE + m] = ssq;
            }
        }
    }
    if (S > 1) tc::cluster_sync_all();     // no rank leaves while its staging rows may still be read

    // ---------------- teardown
    tc::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // give copies that were issued but never consumed a bounded chance to land
        for (int i = *consumed; i < *issued; ++i) {
            const int s = i % STG;
            for (int it = 0; it < 4096; ++it) {
                if (tc::mbar_try_wait(&full[s], (i / STG) & 1)) break;
                __nanosleep(256);
            }
        }
    }
    __syncthreads();
    if (warp == 2) tc::tmem_dealloc(tmem_d, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------ host side
struct TokPlan { int BN, S, nkb, stages; };

// Tile width and split-K factor for (M, N, K): as many CTAs as fit one wave of `sms` SMs, at most 4 resident
// k-blocks per CTA where the shape allows it, the smaller cluster on ties.  want_bn / want_s (> 0) pin a choice.
static bool tok_plan(int N, int K, int m_tiles, int epi, int pro, int sms, int want_bn, int want_s, TokPlan* out) {
    if (K % 128) return false;
    const int kbt = K / 128;
    const int bns[3] = {256, 128, 64};
    double best = 1e30;
    bool found = false;
    for (int bi = 0; bi < 3; ++bi) {
        const int BN = bns[bi];
        if (want_bn > 0 && BN != want_bn) continue;
        if (epi == TOK_EPI_GEGLU && BN != 256) continue;
        if (epi == TOK_EPI_RESID && BN == 256) continue;    // the 8-lane / 16-lane row-sum groups
        const int tiles = (epi == TOK_EPI_GEGLU ? (N / 2 + 127) / 128 : (N + BN - 1) / BN) * m_tiles;
        const int max_st = BN == 256 ? 4 : BN == 128 ? 6 : 8;
        for (int S = 1; S <= 8; S *= 2) {
            if (want_s > 0 && S != want_s) continue;
            if (kbt % S) continue;
            const int nkb = kbt / S;
            if (pro == TOK_PRO_NORM && (nkb > max_st || nkb > 4 || (nkb != 1 && nkb != 2 && nkb != 4))) continue;
            const int ctas = tiles * S;
            // serial cost model in us: instruction issue of the K-slice, the cluster exchange, waves beyond the first
            double cost = nkb * 0.33 + (S > 1 ? 0.25 + 0.06 * S : 0.0) + 0.004 * BN;
            if (ctas > sms) cost += 3.0 * ((ctas + sms - 1) / sms - 1);
            if (cost < best) {
                best = cost;
                out->BN = BN; out->S = S; out->nkb = nkb; out->stages = nkb < max_st ? nkb : max_st;
                found = true;
            }
        }
    }
    return found;
}

template <int BN, int PRO, int EPI>
static int launch_gemm_tok(const void* A, const void* W, TokParams p, int K, const TokPlan& pl, bool pdl,
                           cudaStream_t stream) {
    using Cfg = TokCfg<BN>;
    auto kern = gemm_tok_kernel<BN, PRO, EPI>;
    const int m_tiles = (p.M + 127) / 128;
    const int mt = p.M < 128 ? p.M : 128;
    p.nkb = pl.nkb;
    p.stages = pl.stages;
    p.stage_rows = (mt + 31) & ~31;
    p.K = K;
    const int smem = Cfg::smem_bytes(pl.stages, p.stage_rows);
    int dev = 0;
    cudaGetDevice(&dev);
    static int attr_smem[64] = {0};
    if (dev < 0 || dev >= 64) return FRT_ERR_UNSUPPORTED;
    if (attr_smem[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        attr_smem[dev] = smem;
    }
    CUtensorMap tmA, tmW;
    int rc;
    if (PRO == TOK_PRO_TMA) {
        rc = get_tmap_2d_u8(&tmA, A, (uint64_t)p.M, (uint64_t)K, (uint64_t)K, 128);
        if (rc) return rc;
    } else {
        memset(&tmA, 0, sizeof(tmA));
    }
    rc = get_tmap_2d_u8(&tmW, W, (uint64_t)p.N, (uint64_t)K, (uint64_t)K, EPI == TOK_EPI_GEGLU ? 128 : BN);
    if (rc) return rc;
    const int tiles = EPI == TOK_EPI_GEGLU ? (p.half + 127) / 128 : (p.N + BN - 1) / BN;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, m_tiles, pl.S);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = pl.S;
    ++na;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmW, p);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}

static int tok_sm_count() {
    static int sms[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev] > 0 ? sms[dev] : 148;
}

template <int PRO, int EPI>
static int dispatch_gemm_tok(const void* A, const void* W, TokParams p, int K, int want_bn, int want_s, bool pdl,
                             cudaStream_t s) {
    TokPlan pl;
    if (!tok_plan(EPI == TOK_EPI_GEGLU ? 2 * p.half : p.N, K, (p.M + 127) / 128, EPI, PRO, tok_sm_count(), want_bn,
                  want_s, &pl))
        return FRT_ERR_UNSUPPORTED;
    if (pl.BN == 256) return launch_gemm_tok<256, PRO, EPI>(A, W, p, K, pl, pdl, s);
    if constexpr (EPI != TOK_EPI_GEGLU) {
        if (pl.BN == 128) return launch_gemm_tok<128, PRO, EPI>(A, W, p, K, pl, pdl, s);
        return launch_gemm_tok<64, PRO, EPI>(A, W, p, K, pl, pdl, s);
    }
    return FRT_ERR_UNSUPPORTED;
}
