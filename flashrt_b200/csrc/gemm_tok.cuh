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
// Split-K: rank r of the cluster finishes a contiguous range of tokens.  Every rank PUSHES the accumulator rows of a
// token straight from registers into the owner's shared memory (st.async, 16 bytes each, completing bytes on the
// owner's mbarrier); the owner waits for S x tokens x BN x 4 bytes and sums the S slots in fixed order 0, 1, ...
// No cluster barrier and no remote load sits between the last MMA and the result.  Measured on B200: a cluster
// barrier costs 0.75 us and a pull-based exchange needs two of them plus two remote round trips (6.2 us per launch
// of the attention-out projection against 4.3 us with the push); staging the rows and pushing them with
// cp.async.bulk (shared::cta -> shared::cluster) was no faster: either way the cluster network moves about
// 2.2 TB/s over the whole chip (~17 GB/s per SM), so the tile width and the split are chosen to keep the exchanged
// bytes per CTA ((S - 1) / S x tokens x BN x 4) near 10 KB.  No global workspace; deterministic.
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

// Diagnostic build (-DFRT_PHASE_STAMPS): every CTA stamps %globaltimer at the phases of the kernel (start, set-up done,
// dependency wait returned, first / last MMA issued, accumulator seen, rows pushed, slots received, finish done, end)
// into one of 8 launch slots; frt_b200_phase_stamps_read returns them.  Compiled out otherwise.
#ifdef FRT_PHASE_STAMPS
__device__ unsigned long long g_tok_trace[8][160][16];
static int g_tok_trace_slot = 0;
#define TOK_STAMP(i) do { if (threadIdx.x == tstamp_thread) g_tok_trace[p.trace_slot][ (blockIdx.z * gridDim.x + blockIdx.x) % 160][i] = tc::global_timer_ns(); } while (0)
#else
#define TOK_STAMP(i)
#endif

enum { TOK_EPI_BF16 = 0, TOK_EPI_ROPE = 1, TOK_EPI_GEGLU = 2, TOK_EPI_RESID = 3 };
// A token's row in a receive slot is BN + 4 floats long: the finish reads 32 bytes per thread, 8 threads per token, and
// with rows of BN floats (a multiple of 32 banks) the four tokens of a warp hit the same banks (8 wavefronts per 16-byte
// load instead of 4); four floats of padding rotate them apart.
constexpr int TOK_ROW_PAD = 4;
enum { TOK_PRO_TMA = 0, TOK_PRO_NORM = 1 };
enum { TOK_STAT_STRIDE = 128 };          // floats between the per-tile rows of a statistics buffer

struct TokParams {
    int M, N;                  // activation rows (all m-tiles), output features
    int nkb;                   // 128-byte k-blocks per split
    int stages;                // shared-memory ring depth (>= nkb when the A operand is produced in the kernel)
    int per;                   // tokens finished by one rank of the cluster = ceil(tokens of an m-tile / S)
    int row_pad;               // floats of padding behind a token's BN floats in a receive slot (TOK_ROW_PAD, or 0 when
                               // the padded slots would not fit)
    int per_magic;             // ceil(65536 / per): row / per == (row * per_magic) >> 16 for row < 128 (no division on the
                               // path between the last MMA and the first pushed row)
    int ring_bytes;            // bytes of the operand ring / staging area in front of the receive slots
    int m64;                   // one m-tile of at most 64 tokens: M = 64 MMAs over a 64-row A tile (8 KB per k-block), token
                               // 16 i + j on tensor-memory lane 32 i + j; a CTA then leaves room for a neighbour's CTA
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
    int gate_act;              // 0 = GELU(tanh) gate (GeGLU), 1 = SiLU gate (SwiGLU), 2 = GELU(tanh) with the hardware tanh
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
    int w_kn;                  // weights stored (K, N) row-major (the MN-major B operand) instead of (N, K)
    // Deferred row scale (TOK_PRO_TMA with TOK_EPI_ROPE / TOK_EPI_GEGLU, active when stats_in != NULL): the A operand
    // holds e4m3(x * (1 + scale)) WITHOUT the 1 / rms factor; the finish applies it per token and adds the column
    // term:  y[m][n] = bf16(alpha * acc[m][n] * rms[m] + col_term[n]),  rms from stats_in / n_stat / K / eps as above,
    // col_term[n] = sum_k W[n][k] * shift[k] (fp32, N entries).
    const float* col_term;
    // TOK_EPI_RESID, optional (q8_out != NULL): the un-normalised operand of the next projection,
    //   q8_out[m][n] = e4m3(clamp(bf16(residual[m][n]) * (1 + q8_mod[n]) / *q8_scale, +-448))
    uint8_t* q8_out;
    const __nv_bfloat16* q8_mod;
    const float* q8_scale;
#ifdef FRT_PHASE_STAMPS
    int trace_slot;
#endif
};

template <int BN>
struct TokCfg {
    static constexpr int W_BYTES = BN * 128;
    // A tile of a stage: 128 (or, for at most 64 tokens, 64) token rows x 128 K-bytes
    static constexpr int a_bytes(bool m64) { return m64 ? 64 * 128 : 128 * 128; }
    static constexpr int stage_bytes(bool m64) { return a_bytes(m64) + W_BYTES; }
    static constexpr int MAX_STAGES = BN == 256 ? 4 : BN == 128 ? 6 : 8;
    static constexpr int AUX_BYTES = 2048;                    // barriers, flags, per-token 1 / rms
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    // operand ring, then the receive slots [S][per][BN] fp32 of the split-K exchange (never aliased: a fast rank
    // pushes while a slow rank's MMAs still read its operands)
    static int ring_bytes(int stages, bool m64) { return stages * stage_bytes(m64); }
    static int smem_bytes(int stages, int S, int per, bool m64, int pad) {
        return AUX_BYTES + 1024 + ring_bytes(stages, m64) + S * per * (BN + pad) * 4;
    }
};

// 16 bytes from registers into a cluster peer's shared memory; the bytes are counted on the peer's mbarrier
__device__ __forceinline__ void st_async_v4(uint32_t peer_addr, uint32_t peer_bar, uint32_t a, uint32_t b, uint32_t c,
                                            uint32_t d) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(peer_addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(peer_bar)
                 : "memory");
}
__device__ __forceinline__ void cluster_arrive_release() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// column inside a head: a mask for the usual power-of-two head sizes, a division otherwise
__device__ __forceinline__ int rope_col(int n, int head_dim) {
    return (head_dim & (head_dim - 1)) == 0 ? (n & (head_dim - 1)) : n % head_dim;
}

// Sum over the S slots (fixed order) of the 8 received fp32 values of (token t of this rank, columns c8*8 .. +7).
template <int BN>
__device__ __forceinline__ void tok_sum8(const float* recv, int S, int per, int pad, int t, int c8, float* a) {
    const float4* row = reinterpret_cast<const float4*>(recv + (size_t)t * (BN + pad));
    const int c0 = 2 * c8, c1 = 2 * c8 + 1;
    const size_t slot = (size_t)per * (BN + pad) / 4;
    // S is 1, 2, 4 or 8: the loads of four slots in flight at a time, the sums in slot order
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = 0.0f;
#pragma unroll
    for (int s0 = 0; s0 < 8; s0 += 4) {
        if (s0 < S) {
            float4 x[4], y[4];
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                if (s0 + s < S) {
                    x[s] = row[(s0 + s) * slot + c0];
                    y[s] = row[(s0 + s) * slot + c1];
                }
            }
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                if (s0 + s < S) {
                    if (s0 + s == 0) {
                        a[0] = x[s].x; a[1] = x[s].y; a[2] = x[s].z; a[3] = x[s].w;
                        a[4] = y[s].x; a[5] = y[s].y; a[6] = y[s].z; a[7] = y[s].w;
                    } else {
                        a[0] += x[s].x; a[1] += x[s].y; a[2] += x[s].z; a[3] += x[s].w;
                        a[4] += y[s].x; a[5] += y[s].y; a[6] += y[s].z; a[7] += y[s].w;
                    }
                }
            }
        }
    }
}

// ACT (GeGLU epilogue only): the gate activation, 0 exact GELU(tanh), 1 SiLU, 2 GELU through the hardware tanh.  A
// template argument, not a field of the parameters: selected at run time inside the unrolled finish the choice cost
// 0.55 us per gate|up launch of the action-expert loop (0.10 ms per loop), a third of that epilogue's arithmetic.
template <int BN, int PRO, int EPI, int ACT = 0>
__global__ void __launch_bounds__(256, 2)
gemm_tok_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, TokParams p) {
    static_assert(EPI != TOK_EPI_GEGLU || BN >= 128, "GeGLU tiles are BN / 2 gate rows + the matching up rows");
    using Cfg = TokCfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* aux = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = aux + Cfg::AUX_BYTES;                       // 1024-aligned
    uint64_t* full = reinterpret_cast<uint64_t*>(aux);          // [8]
    uint64_t* empty = full + 8;                                  // [8]
    uint64_t* accum_bar = empty + 8;
    uint64_t* a_ready = accum_bar + 1;
    uint64_t* recv_bar = a_ready + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(recv_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;
    volatile int* consumed = abort_flag + 2;
    float* s_rms = reinterpret_cast<float*>(aux + 512);          // [128]
    float* recv = reinterpret_cast<float*>(tiles + p.ring_bytes);   // [S][per][BN + p.row_pad]

    const uint64_t deadline = tc::global_timer_ns() + FRT_KERNEL_DEADLINE_NS;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
#ifdef FRT_PHASE_STAMPS
    int tstamp_thread = 0;
#endif
    TOK_STAMP(0);
    const int tile = blockIdx.x;
    // first weight row of the tile; with GeGLU a tile is BN / 2 gate rows + the BN / 2 matching up rows
    const int n0 = (EPI == TOK_EPI_GEGLU) ? tile * (BN / 2) : tile * BN;
    const int m0 = blockIdx.y * 128;
    const int Mt = (p.M - m0) < 128 ? (p.M - m0) : 128;         // tokens of this m-tile
    const int S = (int)tc::cluster_nctarank();
    const int rank = (int)tc::cluster_ctarank();
    const int nkb = p.nkb;
    const int kb0 = rank * nkb;
    const int STG = p.stages;
    const int per = p.per;
    const bool m64 = p.m64 != 0;
    const int A_BYTES = Cfg::a_bytes(m64), STAGE_BYTES = Cfg::stage_bytes(m64);
    // tokens this rank finishes: [tb, te) inside the m-tile
    const int tb = rank * per < Mt ? rank * per : Mt;
    const int te = tb + per < Mt ? tb + per : Mt;
    const int ntok = te - tb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 8; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        tc::mbar_init(accum_bar, 1);
        tc::mbar_init(a_ready, 256);
        tc::mbar_init(recv_bar, 1);
        *abort_flag = 0;
        *issued = 0;
        *consumed = 0;
        tc::mbar_fence_init();
        // every rank (this one included) sends this rank's tokens: S slots of ntok rows
        tc::mbar_arrive_expect_tx(recv_bar, (uint32_t)(S * ntok * BN * 4));
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
    // the peers may push into this CTA once they have seen this arrival (they wait for it just before their first push)
    cluster_arrive_release();
    TOK_STAMP(1);

    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer: the weights do not depend on the producer grid and start streaming now
        const uint32_t tx = (PRO == TOK_PRO_TMA) ? STAGE_BYTES : Cfg::W_BYTES;
        auto load_w = [&](int stage, int kb) {
            uint8_t* dst = tiles + stage * STAGE_BYTES + A_BYTES;
            if (p.w_kn) {
                // (K, N) weights: boxes of 128 K-rows x 128 N-bytes, one per 128 output features; the tile is then an
                // MN-major operand (128-byte rows along N, 8 K-rows per swizzle atom, 16 KB between the chunks)
#pragma unroll
                for (int j = 0; j < (BN >= 128 ? BN / 128 : 1); ++j) {
                    const int nj = (EPI == TOK_EPI_GEGLU && j == 1) ? p.half + n0 : n0 + j * 128;
                    tc::tma_load_2d(dst + j * 16384, &tmW, &full[stage], nj, kb * 128);
                }
            } else if (EPI == TOK_EPI_GEGLU) {      // tmW has a box of BN / 2 rows here
                tc::tma_load_2d(dst, &tmW, &full[stage], kb * 128, n0);
                tc::tma_load_2d(dst + (BN / 2) * 128, &tmW, &full[stage], kb * 128, p.half + n0);
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
                tc::tma_load_2d(tiles + i * STAGE_BYTES, &tmA, &full[i], (kb0 + i) * 128, m0);
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
            if (PRO == TOK_PRO_TMA) tc::tma_load_2d(tiles + s * STAGE_BYTES, &tmA, &full[s], (kb0 + i) * 128, m0);
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
        float one_sc[16], shf[16];                    // 1 + scale and shift of this thread's 16 features
        {
            const uint4 sc0 = ld_global_v4(p.style + kcol), sc1 = ld_global_v4(p.style + kcol + 8);
            const uint4 sh0 = ld_global_v4(p.style + p.K + kcol), sh1 = ld_global_v4(p.style + p.K + kcol + 8);
            const uint32_t scw[8] = {sc0.x, sc0.y, sc0.z, sc0.w, sc1.x, sc1.y, sc1.z, sc1.w};
            const uint32_t shw[8] = {sh0.x, sh0.y, sh0.z, sh0.w, sh1.x, sh1.y, sh1.z, sh1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float s0, s1;
                unpack_bf16x2(scw[i], s0, s1);
                one_sc[2 * i] = __fadd_rn(1.0f, s0);
                one_sc[2 * i + 1] = __fadd_rn(1.0f, s1);
                unpack_bf16x2(shw[i], shf[2 * i], shf[2 * i + 1]);
            }
        }
        const float inv_scale = __fdiv_rn(1.0f, p.sa ? *p.sa : 1.0f);
        pdl_wait();
        const int passes = (Mt + rstep - 1) / rstep;
        for (int pb = 0; pb < passes; pb += 4) {
            // residual chunks of up to four tokens in flight, and (first batch) the row statistics behind them
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
            if (pb == 0) {
                // per-token 1 / rms from the per-tile partial sums of squares: all partials of a token in flight,
                // summed in order
                if ((int)threadIdx.x < Mt) {
                    float tot = 0.0f;
                    for (int t0 = 0; t0 < p.n_stat; t0 += 16) {
                        float v[16];
#pragma unroll
                        for (int t = 0; t < 16; ++t)
                            v[t] = (t0 + t < p.n_stat)
                                       ? __ldcg(p.stats_in + (t0 + t) * TOK_STAT_STRIDE + m0 + threadIdx.x) : 0.0f;
#pragma unroll
                        for (int t = 0; t < 16; ++t)
                            if (t0 + t < p.n_stat) tot = __fadd_rn(tot, v[t]);
                    }
                    const float var = __fadd_rn(__fdiv_rn(tot, (float)p.K), p.eps);
                    s_rms[threadIdx.x] = __fdiv_rn(1.0f, __fsqrt_rn(var));
                }
                __syncthreads();                      // every thread passes here exactly once (passes >= 1)
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r = r_first + (pb + j) * rstep;
                if (pb + j < passes && r < Mt) {
                    const float rms = s_rms[r];
                    const uint32_t xw[8] = {xa[j].x, xa[j].y, xa[j].z, xa[j].w, xb[j].x, xb[j].y, xb[j].z, xb[j].w};
                    uint32_t q[4];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        float v[4];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float r0, r1;
                            unpack_bf16x2(xw[i + h], r0, r1);
                            const int e = 2 * (i + h);
                            const float n0v = __fmaf_rn(__fmul_rn(r0, rms), one_sc[e], shf[e]);
                            const float n1v = __fmaf_rn(__fmul_rn(r1, rms), one_sc[e + 1], shf[e + 1]);
                            v[2 * h] = clamp448(__fmul_rn(n0v, inv_scale));
                            v[2 * h + 1] = clamp448(__fmul_rn(n1v, inv_scale));
                        }
                        q[i >> 1] = f32x4_to_e4m3x4(v[0], v[1], v[2], v[3]);
                    }
                    const int kb = c16 >> 3, c = c16 & 7;
                    uint8_t* dst = tiles + kb * STAGE_BYTES + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4);
                    *reinterpret_cast<uint4*>(dst) = make_uint4(q[0], q[1], q[2], q[3]);
                }
            }
        }
        tc::fence_proxy_async_smem();
        tc::mbar_arrive(a_ready);
        TOK_STAMP(12);
    }

    if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        const uint32_t idesc = tc::make_idesc(0, 0, 0, 0, m64 ? 64 : 128, BN) | (p.w_kn ? (1u << 16) : 0u);   // bit 16: B MN-major
        bool failed = false;
        if (PRO == TOK_PRO_NORM) {
            if (!tc::mbar_wait_until(a_ready, 0, deadline, abort_flag)) {
                *abort_flag = 1;
                atomicCAS(&g_gemm_status, 0, ERR_MMA | (blockIdx.x << 8));
                failed = true;
            }
        }
        const uint64_t dA0 = tc::make_desc_kmajor_sw128(tc::smem_u32(tiles));
        const uint64_t dW0 = p.w_kn ? tc::make_desc_mnmajor_sw128(tc::smem_u32(tiles + A_BYTES), 16384)
                                    : tc::make_desc_kmajor_sw128(tc::smem_u32(tiles + A_BYTES));
        // one K = 32 step: 32 bytes along a K-major row, or 32 rows of 128 bytes of an MN-major tile
        const uint64_t wstep = p.w_kn ? (uint64_t)((32 * 128) >> 4) : 2u;
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
#ifdef FRT_PHASE_STAMPS
            if (i == 0) g_tok_trace[p.trace_slot][(blockIdx.z * gridDim.x + blockIdx.x) % 160][10] = tc::global_timer_ns();
#endif
            const uint64_t so = (uint64_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
            for (int k = 0; k < 4; ++k)   // 4 x (K = 32) per 128-byte k-block; +32 bytes = +2 in the address field
                tc::mma_f8(tmem_d, dA0 + so + 2 * k, dW0 + so + wstep * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
            tc::mma_commit(&empty[s]);
            *consumed = i + 1;
        }
        if (!failed) tc::mma_commit(accum_bar);
#ifdef FRT_PHASE_STAMPS
        g_tok_trace[p.trace_slot][(blockIdx.z * gridDim.x + blockIdx.x) % 160][11] = tc::global_timer_ns();
#endif
    }
    __syncwarp();

    // ---------------- work items of the finish: (token of this rank, group of 8 output features); what an item needs
    // from global memory besides the accumulator is fetched now, behind the MMAs
    TOK_STAMP(2);
    pdl_wait();
    TOK_STAMP(3);
    constexpr int G = (EPI == TOK_EPI_GEGLU) ? BN / 16 : BN / 8;      // 8-feature groups per token that carry output
    const int items = ntok * G;
    const int items_pad = (items + 31) & ~31;                         // whole warps iterate together (shuffles below)
    float alpha = p.alpha_host;
    if (p.sa) alpha *= *p.sa;
    if (p.sb) alpha *= *p.sb;
    const float inv_os = (EPI == TOK_EPI_GEGLU) ? __fdiv_rn(1.0f, *p.out_scale) : 0.0f;
    const int pos = (EPI == TOK_EPI_ROPE && p.devpos) ? *p.devpos : 0;
    uint4 pre0 = make_uint4(0, 0, 0, 0), pre1 = make_uint4(0, 0, 0, 0);   // first item's operands
    uint4 pre2 = make_uint4(0, 0, 0, 0);
    float4 ct0 = make_float4(0.f, 0.f, 0.f, 0.f), ct1 = ct0, ct2 = ct0, ct3 = ct0;   // first item's column terms
    const bool rowscale = PRO == TOK_PRO_TMA && (EPI == TOK_EPI_ROPE || EPI == TOK_EPI_GEGLU) && p.stats_in != nullptr;
    const bool emit_q8 = EPI == TOK_EPI_RESID && p.q8_out != nullptr;
    const float inv_q8 = emit_q8 ? __fdiv_rn(1.0f, *p.q8_scale) : 0.0f;
    if (rowscale && (int)threadIdx.x < ntok) {
        // 1 / rms of this rank's tokens from the per-tile partial sums of squares (all partials in flight, summed in order)
        const int m = m0 + tb + threadIdx.x;
        float tot = 0.0f;
        for (int t0 = 0; t0 < p.n_stat; t0 += 16) {
            float v[16];
#pragma unroll
            for (int t = 0; t < 16; ++t)
                v[t] = (t0 + t < p.n_stat) ? __ldcg(p.stats_in + (t0 + t) * TOK_STAT_STRIDE + m) : 0.0f;
#pragma unroll
            for (int t = 0; t < 16; ++t)
                if (t0 + t < p.n_stat) tot = __fadd_rn(tot, v[t]);
        }
        const float var = __fadd_rn(__fdiv_rn(tot, (float)p.K), p.eps);
        s_rms[threadIdx.x] = __fdiv_rn(1.0f, __fsqrt_rn(var));
    }
    {
        const int it = threadIdx.x;
        if (it < items) {
            const int m = m0 + tb + it / G, n = n0 + (it % G) * 8;
            if (rowscale) {
                if (EPI == TOK_EPI_GEGLU) {
                    if (n < p.half) {
                        ct0 = ld_global_f4(p.col_term + n);
                        ct1 = ld_global_f4(p.col_term + n + 4);
                        ct2 = ld_global_f4(p.col_term + p.half + n);
                        ct3 = ld_global_f4(p.col_term + p.half + n + 4);
                    }
                } else if (n < p.N) {
                    ct0 = ld_global_f4(p.col_term + n);
                    ct1 = ld_global_f4(p.col_term + n + 4);
                }
            }
            if (EPI == TOK_EPI_RESID && n < p.N) {
                pre0 = ld_global_v4(p.resid + (size_t)m * p.N + n);
                pre1 = ld_global_v4(p.gate + n);
                if (emit_q8) pre2 = ld_global_v4(p.q8_mod + n);
            } else if (EPI == TOK_EPI_ROPE && n < p.q_dim + p.k_dim) {
                const int nr = n < p.q_dim ? n : n - p.q_dim;
                pre0 = ld_global_v4(p.rope + (size_t)m * p.head_dim + rope_col(nr, p.head_dim));
            } else if (EPI == TOK_EPI_BF16 && p.bias && n + 8 <= p.N &&
                       (reinterpret_cast<uintptr_t>(p.bias + n) & 15) == 0) {
                pre0 = ld_global_v4(p.bias + n);
            }
        }
    }

    // ---------------- accumulator rows -> the owning rank's receive slot [this rank][token][BN]
    const bool acc_seen = tc::mbar_wait_until(accum_bar, 0, deadline, abort_flag);
    const bool have_acc = __all_sync(0xffffffffu, acc_seen);   // tcgen05.ld below is warp-collective
    if (!have_acc && !*abort_flag) {
        *abort_flag = 1;
        atomicCAS(&g_gemm_status, 0, ERR_EPILOGUE | (blockIdx.x << 8));
    }
    __syncwarp();
    tc::tc_fence_after_sync();
    TOK_STAMP(4);
    cluster_wait_acquire();          // every peer has initialised its receive barrier (arrived during its set-up)
    {
        const int quad = warp & 3, chalf = warp >> 2;
        const int qrows = m64 ? 16 : 32;                       // accumulator rows per 32-lane quadrant
        const int row = lane < qrows ? quad * qrows + lane : Mt;   // token inside the m-tile (none on the idle lanes)
        if (have_acc && quad * qrows < Mt) {
            const uint32_t trow = tmem_d + ((uint32_t)(quad * 32) << 16);
            const int rq = (row * p.per_magic) >> 16;           // row / per
            const int owner = rq < S ? rq : 0;
            const uint32_t dst_local = tc::smem_u32(recv) + (uint32_t)(((rank * per + (row - rq * per)) * (BN + p.row_pad)) * 4);
            const uint32_t dst = tc::dsmem_map(dst_local, (uint32_t)owner);
            const uint32_t bar = tc::dsmem_map(tc::smem_u32(recv_bar), (uint32_t)owner);
#pragma unroll 1
            for (int c = chalf * (BN / 2); c < (chalf + 1) * (BN / 2); c += 32) {
                uint32_t v[32];
                tc::tmem_ld32(trow + c, v);
                tc::tmem_ld_wait();
                if (row < Mt) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        st_async_v4(dst + (uint32_t)(c + 4 * j) * 4u, bar, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
        }
    }
    TOK_STAMP(5);
    // ---------------- all S slots of this rank's tokens have landed
    const bool got = tc::mbar_wait_until(recv_bar, 0, deadline, abort_flag);
    if (!got && !*abort_flag) {
        *abort_flag = 1;
        atomicCAS(&g_gemm_status, 0, ERR_EPILOGUE | (blockIdx.x << 8));
    }
    __syncwarp();
    if (rowscale) __syncthreads();       // s_rms of this rank's tokens is complete
    TOK_STAMP(6);

    // ---------------- finish: sum the S slots in order and apply the epilogue
    {
        const bool live = !*abort_flag;
        for (int it = threadIdx.x; it < items_pad; it += 256) {
            const bool act = live && it < items;
            const int t = it / G;                 // token of this rank
            const int g = it % G;
            const int m = m0 + tb + t;
            const bool first = it < 256;
            float a[8];
            if (act) {
                tok_sum8<BN>(recv, S, per, p.row_pad, t, g, a);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) a[j] = 0.0f;
            }
            if (EPI == TOK_EPI_BF16) {
                const int n = n0 + g * 8;
                if (act && n < p.N) {
                    float f[8];
                    const bool vec = n + 8 <= p.N && (reinterpret_cast<uintptr_t>(p.out + (size_t)m * p.N + n) & 15) == 0;
                    const bool bvec = p.bias && n + 8 <= p.N && (reinterpret_cast<uintptr_t>(p.bias + n) & 15) == 0;
                    uint4 bv = pre0;
                    if (bvec && !first) bv = ld_global_v4(p.bias + n);
                    const uint32_t* bw = &bv.x;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const bool hb = p.bias && (bvec || n + j < p.N);
                        const float bj = !hb ? 0.0f : bvec ? bf16_bits_to_f32((bw[j >> 1] >> ((j & 1) * 16)) & 0xffffu)
                                                         : __bfloat162float(p.bias[n + j]);
                        f[j] = scale_bias(a[j], alpha, bj, hb);
                    }
                    __nv_bfloat16* dst = p.out + (size_t)m * p.N + n;
                    if (vec) {
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
                    if (rowscale) {
                        float4 c0 = ct0, c1 = ct1;
                        if (!first) {
                            c0 = ld_global_f4(p.col_term + n);
                            c1 = ld_global_f4(p.col_term + n + 4);
                        }
                        const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                        const float rs = s_rms[t];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            v[j] = __bfloat162float(__float2bfloat16_rn(__fadd_rn(__fmul_rn(a[j] * alpha, rs), cc[j])));
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(a[j] * alpha));
                    }
                    const bool is_q = n < p.q_dim;
                    const bool is_k = !is_q && n < p.q_dim + p.k_dim;
                    const int nr = is_q ? n : (is_k ? n - p.q_dim : n - p.q_dim - p.k_dim);
                    uint4 o;
                    if (is_q || is_k) {
                        uint4 tq = pre0;
                        if (!first) tq = ld_global_v4(p.rope + (size_t)m * p.head_dim + rope_col(nr, p.head_dim));
                        const uint32_t* tw = &tq.x;
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
                // a = gate columns g*8.. of the tile, b = the matching up columns BN / 2 + g*8..
                const int h = n0 + g * 8;
                if (act && h < p.half) {
                    float b[8];
                    tok_sum8<BN>(recv, S, per, p.row_pad, t, G + g, b);
                    float q[8];
                    if (rowscale) {
                        float4 c0 = ct0, c1 = ct1, c2 = ct2, c3 = ct3;
                        if (!first) {
                            c0 = ld_global_f4(p.col_term + h);
                            c1 = ld_global_f4(p.col_term + h + 4);
                            c2 = ld_global_f4(p.col_term + p.half + h);
                            c3 = ld_global_f4(p.col_term + p.half + h + 4);
                        }
                        const float cg[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                        const float cu[8] = {c2.x, c2.y, c2.z, c2.w, c3.x, c3.y, c3.z, c3.w};
                        const float rs = s_rms[t];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            a[j] = __fadd_rn(__fmul_rn(a[j] * alpha, rs), cg[j]);
                            b[j] = __fadd_rn(__fmul_rn(b[j] * alpha, rs), cu[j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            a[j] = a[j] * alpha;
                            b[j] = b[j] * alpha;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float gt = __bfloat162float(__float2bfloat16_rn(a[j]));
                        const float up = __bfloat162float(__float2bfloat16_rn(b[j]));
                        const float act = ACT == 2 ? fast_gelu_tanh(gt) : ACT == 1 ? det_silu(gt) : det_gelu_tanh(gt);
                        q[j] = clamp448(__fmul_rn(__fmul_rn(act, up), inv_os));
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
                    uint4 rv = pre0, gv = pre1, mv = pre2;
                    if (!first) {
                        rv = ld_global_v4(rp);
                        gv = ld_global_v4(p.gate + n);
                        if (emit_q8) mv = ld_global_v4(p.q8_mod + n);
                    }
                    const uint32_t* mw = &mv.x;
                    float u[8];
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
                    if (emit_q8) {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float b0, b1, s0, s1;
                            unpack_bf16x2(ow[k], b0, b1);          // what the next reader of the residual sees
                            unpack_bf16x2(mw[k], s0, s1);
                            u[2 * k] = clamp448(__fmul_rn(__fmul_rn(b0, __fadd_rn(1.0f, s0)), inv_q8));
                            u[2 * k + 1] = clamp448(__fmul_rn(__fmul_rn(b1, __fadd_rn(1.0f, s1)), inv_q8));
                        }
                        uint2 o8;
                        o8.x = f32x4_to_e4m3x4(u[0], u[1], u[2], u[3]);
                        o8.y = f32x4_to_e4m3x4(u[4], u[5], u[6], u[7]);
                        st_global_v2(p.q8_out + (size_t)m * p.N + n, o8);
                    }
                }
                // the G lanes of a token are neighbours (G divides 32): butterfly inside the group, fixed order
#pragma unroll
                for (int off = G / 2; off >= 1; off >>= 1) ssq = __fadd_rn(ssq, __shfl_xor_sync(0xffffffffu, ssq, off));
                if (act && g == 0 && p.stats_out) p.stats_out[tile * TOK_STAT_STRIDE + m] = ssq;
            }
        }
    }
    TOK_STAMP(7);

    // ---------------- teardown (nothing of this CTA is read by a peer: no cluster barrier before leaving)
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
    TOK_STAMP(9);
}

// ------------------------------------------------------------------ host side
struct TokPlan { int BN, S, nkb, stages; };

// Tile width and split-K factor for (M, N, K) from a serial cost model in microseconds, fitted to device-timer
// traces of the four decoder projections at 50 tokens: 0.33 per resident k-block (four MMA issues), 0.06 per KB a
// CTA pushes to its cluster peers, 0.05 per rank for the receive wait, 0.6 per k-block of in-kernel norm work, a
// charge for SMs that have to carry two CTAs, and a second wave only when the CTAs cannot all be resident (two per
// SM fit while a CTA stays under ~110 KB of shared memory).  want_bn / want_s (> 0) pin a choice; callers that
// have measured their shapes do so.
static bool tok_plan(int N, int K, int m_tiles, int mt, int epi, int pro, int sms, int want_bn, int want_s,
                     TokPlan* out, bool w_kn = false) {
    if (K % 128) return false;
    const int kbt = K / 128;
    const int bns[3] = {256, 128, 64};
    double best = 1e30;
    bool found = false;
    for (int bi = 0; bi < 3; ++bi) {
        const int BN = bns[bi];
        if (want_bn > 0 && BN != want_bn) continue;
        if (epi == TOK_EPI_GEGLU && (BN == 64 || ((N / 2) % (BN / 2)))) continue;
        if (epi == TOK_EPI_RESID && BN == 256) continue;    // the 8-lane / 16-lane row-sum groups
        if (w_kn && (BN == 64 || (epi == TOK_EPI_GEGLU && BN != 256))) continue;   // 128-feature boxes of (K, N) weights
        const int tiles = (epi == TOK_EPI_GEGLU ? (N / 2 + BN / 2 - 1) / (BN / 2) : (N + BN - 1) / BN) * m_tiles;
        const int max_st = BN == 256 ? 4 : BN == 128 ? 6 : 8;
        const int stage_bytes = (m_tiles == 1 && mt <= 64 ? 8192 : 16384) + BN * 128;
        for (int S = 1; S <= 8; S *= 2) {
            if (want_s > 0 && S != want_s) continue;
            if (kbt % S) continue;
            const int nkb = kbt / S;
            if (pro == TOK_PRO_NORM && (nkb > max_st || nkb > 4 || (nkb != 1 && nkb != 2 && nkb != 4))) continue;
            const int ctas = tiles * S;
            const int stages = nkb < max_st ? nkb : max_st;
            const int per = (mt + S - 1) / S;
            const int smem = 3072 + stages * stage_bytes + S * per * (BN + TOK_ROW_PAD) * 4;
            if (pro == TOK_PRO_NORM && smem - S * per * TOK_ROW_PAD * 4 > 227 * 1024) continue;
            // the launcher shortens the ring down to two stages, not further
            if (3072 + (stages < 2 ? stages : 2) * stage_bytes + S * per * BN * 4 > 227 * 1024) continue;
            const double pushed_kb = (double)(S - 1) / S * mt * BN * 4 / 1024.0;
            double cost = nkb * 0.33 + pushed_kb * 0.06 + (S > 1 ? 0.05 * S : 0.0);
            if (pro == TOK_PRO_NORM) cost += 0.6 * nkb;
            const int resident = smem <= 110 * 1024 ? 2 * sms : sms;
            if (ctas > resident) cost += 3.0 * ((ctas + resident - 1) / resident - 1);
            else if (ctas > sms) cost += 1.0 * (ctas - sms) / sms;   // SMs that carry two CTAs run both slower
            if (cost < best) {
                best = cost;
                out->BN = BN; out->S = S; out->nkb = nkb; out->stages = stages;
                found = true;
            }
        }
    }
    return found;
}

template <int BN, int PRO, int EPI, int ACT = 0>
static int launch_gemm_tok(const void* A, const void* W, TokParams p, int K, const TokPlan& pl, bool pdl,
                           cudaStream_t stream) {
    using Cfg = TokCfg<BN>;
    auto kern = gemm_tok_kernel<BN, PRO, EPI, ACT>;
    const int m_tiles = (p.M + 127) / 128;
    const int mt = p.M < 128 ? p.M : 128;
    p.nkb = pl.nkb;
    p.stages = pl.stages;
    p.per = (mt + pl.S - 1) / pl.S;
    p.per_magic = (65536 + p.per - 1) / p.per;
    p.m64 = (m_tiles == 1 && mt <= 64) ? 1 : 0;
    const bool m64 = p.m64 != 0;
    // padded receive rows unless even a two-stage ring would not fit beside them
    const int need_stages = PRO == TOK_PRO_NORM ? pl.nkb : (p.stages < 2 ? p.stages : 2);   // the ring's lower bound
    p.row_pad = Cfg::smem_bytes(need_stages, pl.S, p.per, m64, TOK_ROW_PAD) > 227 * 1024 ? 0 : TOK_ROW_PAD;
    // the operand ring shrinks until it fits beside the receive slots
    while (p.stages > 2 && Cfg::smem_bytes(p.stages, pl.S, p.per, m64, p.row_pad) > 227 * 1024) --p.stages;
    if (PRO == TOK_PRO_NORM && p.stages < pl.nkb) return FRT_ERR_UNSUPPORTED;
    p.K = K;
#ifdef FRT_PHASE_STAMPS
    p.trace_slot = g_tok_trace_slot;
    g_tok_trace_slot = (g_tok_trace_slot + 1) % 8;
#endif
    const int smem = Cfg::smem_bytes(p.stages, pl.S, p.per, m64, p.row_pad);
    p.ring_bytes = Cfg::ring_bytes(p.stages, m64);
    if (smem > 227 * 1024) return FRT_ERR_UNSUPPORTED;
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
        rc = get_tmap_2d_u8(&tmA, A, (uint64_t)p.M, (uint64_t)K, (uint64_t)K, m64 ? 64 : 128);
        if (rc) return rc;
    } else {
        memset(&tmA, 0, sizeof(tmA));
    }
    rc = p.w_kn ? get_tmap_2d_u8(&tmW, W, (uint64_t)K, (uint64_t)p.N, (uint64_t)p.N, 128)
                : get_tmap_2d_u8(&tmW, W, (uint64_t)p.N, (uint64_t)K, (uint64_t)K, EPI == TOK_EPI_GEGLU ? BN / 2 : BN);
    if (rc) return rc;
    const int tiles = EPI == TOK_EPI_GEGLU ? (p.half + BN / 2 - 1) / (BN / 2) : (p.N + BN - 1) / BN;
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
    if (!tok_plan(EPI == TOK_EPI_GEGLU ? 2 * p.half : p.N, K, (p.M + 127) / 128, p.M < 128 ? p.M : 128, EPI, PRO,
                  tok_sm_count(), want_bn, want_s, &pl, p.w_kn != 0))
        return FRT_ERR_UNSUPPORTED;
    if constexpr (EPI == TOK_EPI_GEGLU) {
        if (pl.BN != 256 && pl.BN != 128) return FRT_ERR_UNSUPPORTED;
        if (p.gate_act == 2)
            return pl.BN == 256 ? launch_gemm_tok<256, PRO, EPI, 2>(A, W, p, K, pl, pdl, s)
                                : launch_gemm_tok<128, PRO, EPI, 2>(A, W, p, K, pl, pdl, s);
        if (p.gate_act == 1)
            return pl.BN == 256 ? launch_gemm_tok<256, PRO, EPI, 1>(A, W, p, K, pl, pdl, s)
                                : launch_gemm_tok<128, PRO, EPI, 1>(A, W, p, K, pl, pdl, s);
    }
    if (pl.BN == 256) return launch_gemm_tok<256, PRO, EPI>(A, W, p, K, pl, pdl, s);
    if (pl.BN == 128) return launch_gemm_tok<128, PRO, EPI>(A, W, p, K, pl, pdl, s);
    if constexpr (EPI != TOK_EPI_GEGLU) return launch_gemm_tok<64, PRO, EPI>(A, W, p, K, pl, pdl, s);
    return FRT_ERR_UNSUPPORTED;
}
