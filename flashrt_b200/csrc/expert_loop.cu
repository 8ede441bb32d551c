// The whole Pi0.5 action-expert denoise loop (N Euler steps x L decoder blocks) as ONE persistent kernel, sm_100a.
//
// Stands in for the reference's captured loop
//   Pi05Pipeline.transformer_decoder / _decoder_layer   flash_rt/models/pi05/pipeline_rtx.py:1451-1749
// (the same arithmetic as the kernel-per-operator composition of this library: FP8 E4M3 projections with static
// per-site activation scales, bf16 residual stream, bf16 attention with fp32 softmax, fp32 Euler state).
//
// Why one kernel: at 50 action tokens every operator moves a few MB and runs for a few microseconds, so the loop of
// 1300 launches is bound by launch and drain latency, not by bandwidth.  Here one CTA per SM stays resident for the
// whole loop and the operators become phases separated by grid-wide barriers:
//
//   A  rows      gated residual of the previous down-projection, adaRMS -> FP8          (CTA r owns token row r)
//   B  GEMM      QKV projection, RoPE + split + KV append in the epilogue              (20 units)
//   C  attention 16 tokens x 8 heads per tile x one chunk of 64 keys -> partials         (4 x chunks units)
//   D  combine   split partials -> FP8 attention output                                 (all CTAs)
//   E  GEMM      output projection, split-K 2 -> fp32 partials                          (16 units)
//   F  rows      gated residual, adaRMS -> FP8
//   G  GEMM      gate|up projection, GeGLU -> FP8 in the epilogue                       (64 units)
//   H  GEMM      down projection, split-K 4 -> fp32 partials                            (32 units)
//
// A GEMM unit is 128 weight rows x 1024 K bytes (128 KB): the weight rows feed the 128 TMEM lanes, the (<= 64) token
// rows are the accumulator columns.  Units are dealt to CTAs round-robin over the whole loop, so every CTA streams
// the same share of the weights.  Weights do not depend on activations: a dedicated warp per CTA walks the CTA's
// static unit list and keeps a ring of TMA stages full ACROSS phase boundaries, so the HBM stream of the next
// phases runs while the CTA waits at a barrier.  Activations (a few hundred KB, L2 resident) are fetched with plain
// loads after each barrier and written into the swizzled operand layout by the worker warps; Q goes to tensor memory
// and is the attention MMA's A operand; the key / value chunks that lie inside the prefix are fetched by TMA at the
// start of phase A (attention CTAs own no QKV unit of the same block, so their operand space is free until phase C).
// Partials (split-K fp32, attention bf16 + log-sum-exp) cross CTAs through L2 scratch and are summed in fixed order:
// replays are bit-reproducible.  The residual row of token r never leaves the registers of CTA r.
//
// Measured (18 blocks x 10 steps, 50 tokens, 768 prefix keys): 10.5 ms per loop against 9.75 ms for the graph of 1300
// operator launches, i.e. a phase costs what a launch costs (barrier 1.1-1.4 us + one L2 round trip for the operand
// 1.5 us + 32 MMAs 2 us + epilogue).
//
// Warps: 0 = weight TMA producer, 1 = MMA issuer (one thread), 2-9 = workers (operand loads, softmax, epilogues,
// row phases, grid barrier).  Every wait is bounded by one wall-clock deadline taken at kernel start; a wait that
// gives up records a status word, raises the CTA's abort flag and every later wait returns at once.
#include "common.cuh"
#include "tc05.cuh"
#include "flashrt_b200.h"

namespace frt {

int get_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t row_bytes, uint64_t pitch,
                   uint32_t box_rows);   // gemm_fp8.cu

__device__ int g_loop_status = 0;   // 0 ok; otherwise first failure code | (blockIdx.x << 8)


namespace el {

constexpr int D = 1024, HID = 4096, NH = 8, HD = 256, NQKV = 2560, QD = 2048, ADIM = 32;
constexpr int MAXS = 64;                       // token rows = accumulator columns
constexpr int RING = 8, STAGE = 16384;         // weight ring: 128 rows x 128 K bytes per stage = one whole unit
constexpr int KB_PER_UNIT = 8;                 // 1024 K bytes
constexpr int OFF_SH = RING * STAGE;           // phase-shared region: token operand | K + V chunk | staging
constexpr int SH_BYTES = 65536;
constexpr int OFF_K = OFF_SH, OFF_V = OFF_K + 32768;
constexpr int OFF_MISC = OFF_SH + SH_BYTES;
constexpr int MISC_BYTES = 256 + 4096 + 256 + 512 + 512;
constexpr int SMEM_BYTES = OFF_MISC + MISC_BYTES + 1024;
constexpr int U_QKV = 20, U_O = 16, U_GU = 64, U_D = 32, U_LAYER = U_QKV + U_O + U_GU + U_D;
constexpr int BKV = 64;
constexpr int TMEM_COLS = 512, O_COL = 128, Q_COL = 384;   // S / P: columns 0-63, O: 128-383, Q: 384-511
constexpr int NWORK = 256;

enum { ERR_PRODUCER = 1, ERR_MMA = 2, ERR_WORKER = 3, ERR_GRID = 4 };

struct LoopParams {
    const float *ws_qkv, *ws_o, *ws_gu, *ws_d, *act_scale;
    const __nv_bfloat16 *style_attn, *style_ffn, *style_final, *rope, *in_w, *in_b, *out_w, *out_b;
    __nv_bfloat16 *k_cache, *v_cache;
    float* noise;
    unsigned* sync;        // [0] barrier arrivals (zeroed before the launch), [1] abort broadcast
    uint8_t* act8;         // (64, 1024)
    __nv_bfloat16* q;      // (64, 2048)
    uint8_t* attn8;        // (64, 2048)
    uint8_t* hid8;         // (64, 4096)
    float* part;           // (4, 64, 1024) split-K partials
    __nv_bfloat16* po;     // (attention units, 128, 256) normalised partial outputs
    float* plse;           // (attention units, 128)
    int steps, layers, S, prefix_len, kv_rows, T, chunks_total, nsplit, att_units, att_tiles;
    float scale_log2;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float bf16r(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
__device__ __forceinline__ void work_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// unit of GEMM phase `ph` (0 QKV, 1 O, 2 gate|up, 3 down) of global layer `gl` that CTA `cta` owns, or -1
__host__ __device__ __forceinline__ int gemm_unit(int G, int cta, int gl, int ph) {
    const int off = ph == 0 ? 0 : ph == 1 ? U_QKV : ph == 2 ? U_QKV + U_O : U_QKV + U_O + U_GU;
    const int n = ph == 0 ? U_QKV : ph == 1 ? U_O : ph == 2 ? U_GU : U_D;
    const long long g0 = (long long)gl * U_LAYER + off;
    const int u = (int)((((long long)cta - g0) % G + G) % G);
    return u < n ? u : -1;
}
__host__ __device__ __forceinline__ int att_unit(int G, int cta, int gl, int units) {
    const long long g0 = (long long)gl * U_LAYER + U_QKV;     // right behind the block's QKV units
    const int u = (int)((((long long)cta - g0) % G + G) % G);
    return u < units ? u : -1;
}

// rows of ROW_BYTES from global memory into K-major 128-byte-swizzled operand blocks: block db holds bytes
// [128 db, 128 db + 128) of every row, rows in groups of 8 (1024 bytes), 16-byte chunk c stored at c ^ (row % 8).
// src(r) returns the row's address or nullptr (row filled with zeros).  All 256 workers take part.
template <int ROW_BYTES, int PER_THREAD, typename Src>
__device__ __forceinline__ void load_tile(uint8_t* dst, int nrows, int wtid, Src src) {
    constexpr int CPR = ROW_BYTES / 16;
    uint4 v[PER_THREAD];                 // nrows * CPR == PER_THREAD * 256: every load of a thread is in flight at once
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int idx = j * NWORK + wtid;
        const int r = idx / CPR, c16 = idx % CPR;
        const uint8_t* s = src(r);
        v[j] = s ? __ldcg(reinterpret_cast<const uint4*>(s + c16 * 16)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int idx = j * NWORK + wtid;
        const int r = idx / CPR, c16 = idx % CPR;
        const int db = c16 >> 3, c = c16 & 7;
        *reinterpret_cast<uint4*>(dst + db * (nrows * 128) + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)) = v[j];
    }
}

__global__ void __launch_bounds__(320, 1)
expert_loop_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmO,
                   const __grid_constant__ CUtensorMap tmGU, const __grid_constant__ CUtensorMap tmD,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, LoopParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = smem;
    uint8_t* sh = smem + OFF_SH;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_MISC);
    uint64_t* full = bars;              // [RING]
    uint64_t* empty = bars + RING;      // [RING]
    uint64_t* b_ready = bars + 2 * RING;      // 256 arrivals: the workers have written the token / Q,K,V operands
    uint64_t* acc_bar = b_ready + 1;          // accumulator (or S = Q.K^T) complete
    uint64_t* p_ready = b_ready + 2;          // 128 arrivals: P is in tensor memory
    uint64_t* o_full = b_ready + 3;           // P.V complete
    uint64_t* kv_full = b_ready + 4;          // prefix K / V chunk fetched ahead of the attention phase has landed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_ready + 5);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;
    volatile int* consumed = abort_flag + 2;
    volatile int* snap = abort_flag + 3;       // abort flag as sampled by one thread inside the grid barrier
    float* s_row = reinterpret_cast<float*>(smem + OFF_MISC + 256);   // 1024
    float* s_small = s_row + 1024;                                    // 64
    float* s_l = s_small + 64;                                        // 128
    float* s_lse = s_l + 128;                                         // 128

    const uint64_t deadline = tc::global_timer_ns() + FRT_KERNEL_DEADLINE_NS;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int G = gridDim.x;
    const int cta = blockIdx.x;
    const int L = p.layers;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RING; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        tc::mbar_init(b_ready, NWORK);
        tc::mbar_init(acc_bar, 1);
        tc::mbar_init(p_ready, 128);
        tc::mbar_init(o_full, 1);
        tc::mbar_init(kv_full, 1);
        *abort_flag = 0;
        *issued = 0;
        *consumed = 0;
        *snap = 0;
        tc::mbar_fence_init();
        tc::tma_prefetch_desc(&tmQKV);
        tc::tma_prefetch_desc(&tmO);
        tc::tma_prefetch_desc(&tmGU);
        tc::tma_prefetch_desc(&tmD);
        tc::tma_prefetch_desc(&tmK);
        tc::tma_prefetch_desc(&tmV);
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    auto fail = [&](int code) {
        if (!*abort_flag) {
            atomicCAS(&g_loop_status, 0, code | (cta << 8));
            atomicExch(p.sync + 1, 1u);
        }
        *abort_flag = 1;
    };

    if (warp == 0) {
        // ================================================================ weight producer
        if (lane == 0) {
            uint32_t pc = 0;
            bool dead = false;
            for (int gl = 0; gl < p.steps * L && !dead; ++gl) {
                const int layer = gl % L;
                for (int ph = 0; ph < 4 && !dead; ++ph) {
                    const int u = gemm_unit(G, cta, gl, ph);
                    if (u < 0) continue;
                    const CUtensorMap* tm;
                    int x0, y0, y1 = -1;
                    if (ph == 0) { tm = &tmQKV; x0 = 0; y0 = layer * NQKV + u * 128; }
                    else if (ph == 1) { tm = &tmO; x0 = (u >> 3) * 1024; y0 = layer * D + (u & 7) * 128; }
                    else if (ph == 2) { tm = &tmGU; x0 = 0; y0 = layer * 2 * HID + u * 64; y1 = y0 + HID; }
                    else { tm = &tmD; x0 = (u >> 3) * 1024; y0 = layer * D + (u & 7) * 128; }
                    for (int kb = 0; kb < KB_PER_UNIT; ++kb) {
                        const int s = pc % RING;
                        if (pc >= RING) {
                            if (!tc::mbar_wait_until(&empty[s], ((pc / RING) - 1) & 1, deadline, abort_flag)) {
                                fail(ERR_PRODUCER);
                                dead = true;
                                break;
                            }
                        }
                        tc::mbar_arrive_expect_tx(&full[s], STAGE);
                        uint8_t* dst = ring + s * STAGE;
                        tc::tma_load_2d(dst, tm, &full[s], x0 + kb * 128, y0);
                        if (y1 >= 0) tc::tma_load_2d(dst + 64 * 128, tm, &full[s], x0 + kb * 128, y1);
                        ++pc;
                        *issued = (int)pc;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_g = tc::make_idesc(0, 0, 0, 0, 128, MAXS);
            constexpr uint32_t idesc_s = tc::make_idesc(1, 1, 0, 0, 128, BKV);
            constexpr uint32_t idesc_o = tc::make_idesc(1, 1, 0, 1, 128, HD);   // A = P from TMEM, B = V MN-major
            const uint32_t sh_addr = tc::smem_u32(sh);
            const uint64_t dk_base = tc::make_desc_kmajor_sw128(tc::smem_u32(smem + OFF_K));
            const uint64_t dv_base = tc::make_desc_mnmajor_sw128(tc::smem_u32(smem + OFF_V), BKV * 128);
            uint32_t cc = 0, nb = 0, np = 0;
            bool dead = false;
            auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
                if (dead) return false;
                if (!tc::mbar_wait_until(bar, parity, deadline, abort_flag)) {
                    fail(ERR_MMA);
                    dead = true;
                    return false;
                }
                return true;
            };
            auto run_gemm = [&](int u, int gl, int tr) {
                (void)gl; (void)tr;
                if (u < 0 || dead) return;
                if (!wait(b_ready, nb & 1)) return;
                ++nb;
                tc::tc_fence_after_sync();
                for (int kb = 0; kb < KB_PER_UNIT; ++kb) {
                    const int s = cc % RING;
                    if (!wait(&full[s], (cc / RING) & 1)) return;
                    tc::tc_fence_after_sync();
                    const uint64_t dW = tc::make_desc_kmajor_sw128(tc::smem_u32(ring + s * STAGE));
                    const uint64_t dX = tc::make_desc_kmajor_sw128(sh_addr + kb * (MAXS * 128));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc::mma_f8(tmem, dW + 2 * k, dX + 2 * k, idesc_g, (kb > 0 || k > 0) ? 1u : 0u);
                    tc::mma_commit(&empty[s]);
                    ++cc;
                    *consumed = (int)cc;
                }
                tc::mma_commit(acc_bar);
            };
            for (int gl = 0; gl < p.steps * L && !dead; ++gl) {
                run_gemm(gemm_unit(G, cta, gl, 0), gl, 40);
                const int au = att_unit(G, cta, gl, p.att_units);
                if (au >= 0 && wait(b_ready, nb & 1)) {
                    ++nb;
                    tc::tc_fence_after_sync();
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k)        // S = Q . K^T, Q from tensor memory (8 columns per K = 16)
                        tc::mma_f16_ts(tmem, tmem + Q_COL + 8 * k,
                                       dk_base + (uint64_t)((k / 4) * ((BKV * 128) >> 4) + 2 * (k % 4)), idesc_s,
                                       k > 0 ? 1u : 0u);
                    tc::mma_commit(acc_bar);
                    if (wait(p_ready, np & 1)) {
                        ++np;
                        tc::tc_fence_after_sync();
#pragma unroll
                        for (int k = 0; k < BKV / 16; ++k)
                            tc::mma_f16_ts(tmem + O_COL, tmem + 8 * k, dv_base + (uint64_t)(k * ((16 * 128) >> 4)),
                                           idesc_o, k > 0 ? 1u : 0u);
                        tc::mma_commit(o_full);
                    }
                }
                run_gemm(gemm_unit(G, cta, gl, 1), gl, 42);
                run_gemm(gemm_unit(G, cta, gl, 2), gl, 44);
                run_gemm(gemm_unit(G, cta, gl, 3), gl, 46);
            }
        }
    } else {
        // ================================================================ workers
        const int wtid = threadIdx.x - 64;          // 0 .. 255
        const int ww = warp - 2;                    // 0 .. 7
        const int quad = warp & 3;                  // TMEM lane quadrant this warp may read
        const int half = ww >> 2;                   // which half of the accumulator columns
        const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
        const int S = p.S;
        const bool row_cta = cta < S;
        const int row = cta;
        const int n0 = wtid * 4;
        uint32_t n_acc = 0, n_o = 0, n_kv = 0, epoch = 0;
        // `dead` is the same for all 256 workers (it is taken from one thread's sample inside the grid barrier), so
        // it may guard code that contains worker barriers; `bad` is per warp and only short-circuits later waits
        bool dead = false, bad = false;
        float xr[4] = {0.f, 0.f, 0.f, 0.f};         // this thread's 4 elements of residual row `row` (bf16 values)

        auto wait = [&](uint64_t* bar, uint32_t parity) -> bool {
            // warp-uniform result: the tensor-memory loads that follow are warp-collective
            bool ok = !bad && tc::mbar_wait_until(bar, parity, deadline, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok && !bad) {
                fail(ERR_WORKER);
                bad = true;
            }
            return ok;
        };
        // this thread's 32 accumulator columns.  (Four independent accumulation chains, one per K = 32 slice, were
        // measured: the MMA issue time of a unit stayed at 2.2 us, so the chain is not what bounds it.)
        auto ld_acc = [&](uint32_t* v) {
            tc::tmem_ld32(tmem + lane_off + half * 32, v);
            tc::tmem_ld_wait();
        };
        // split-K partial of a projection: accumulator -> shared memory [token][128 features] -> rows of 512 bytes
        auto store_partial = [&](bool ok, int ks, int tile) {
            float* stage = reinterpret_cast<float*>(sh);
            if (ok) {
                tc::tc_fence_after_sync();
                uint32_t v[32];
                ld_acc(v);
#pragma unroll
                for (int j = 0; j < 32; ++j) stage[(half * 32 + j) * 128 + quad * 32 + lane] = __uint_as_float(v[j]);
                tc::tc_fence_before_sync();
            }
            work_sync();
            for (int m = ww; m < S; m += 8)
                __stcg(reinterpret_cast<float4*>(p.part + ((size_t)ks * MAXS + m) * D + tile * 128) + lane,
                       *reinterpret_cast<const float4*>(stage + m * 128 + lane * 4));
        };
        auto grid_barrier = [&]() {
            ++epoch;
            work_sync();
            if (wtid == 0 && !*abort_flag) {
                __threadfence();
                atomicAdd(p.sync, 1u);
                const unsigned target = epoch * (unsigned)G;
                bool ok = false;
                for (uint32_t it = 0;; ++it) {
                    unsigned seen;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.sync) : "memory");
                    if (seen >= target) { ok = true; break; }
                    if ((it & 63) == 63) {
                        unsigned ab;
                        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(ab) : "l"(p.sync + 1) : "memory");
                        if (ab || tc::global_timer_ns() > deadline) break;
                    }
                }
                if (!ok) fail(ERR_GRID);
                __threadfence();
            }
            if (wtid == 0) *snap = *abort_flag;
            work_sync();
            if (*snap) dead = true;
        };
        auto block_sum = [&](float v) -> float {
            v = warp_sum_butterfly(v);
            if (lane == 0) s_small[ww] = v;
            work_sync();
            float tot = s_small[0];
#pragma unroll
            for (int w = 1; w < 8; ++w) tot = __fadd_rn(tot, s_small[w]);
            work_sync();
            return tot;
        };
        auto ld4bf = [&](const __nv_bfloat16* ptr, float* o) {
            const uint2 v = *reinterpret_cast<const uint2*>(ptr);
            unpack_bf16x2(v.x, o[0], o[1]);
            unpack_bf16x2(v.y, o[2], o[3]);
        };
        // x <- bf16(x + bf16(alpha * sum of split partials) * gate); returns the sum of squares of the unrounded x
        auto add_delta = [&](int nsp, float alpha, const __nv_bfloat16* gate_row) -> float {
            float4 t[4];
#pragma unroll
            for (int s = 0; s < 4; ++s)
                t[s] = s < nsp ? __ldcg(reinterpret_cast<const float4*>(p.part + ((size_t)s * MAXS + row) * D + n0))
                               : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 a = t[0];
#pragma unroll
            for (int s = 1; s < 4; ++s) { a.x += t[s].x; a.y += t[s].y; a.z += t[s].z; a.w += t[s].w; }
            const float av[4] = {a.x, a.y, a.z, a.w};
            float g[4];
            ld4bf(gate_row + n0, g);
            float ssq = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float o = bf16r(av[i] * alpha);
                const float rf = __fmaf_rn(o, g[i], xr[i]);
                ssq = __fmaf_rn(rf, rf, ssq);
                xr[i] = bf16r(rf);
            }
            return ssq;
        };
        auto rms_of = [&](float ssq) -> float {
            const float tot = block_sum(ssq);
            const float var = __fadd_rn(__fdiv_rn(tot, (float)D), 1e-6f);
            return __fdiv_rn(1.0f, __fsqrt_rn(var));
        };
        // adaRMS with the style row [scale | shift | gate] -> FP8 row of the next projection's input
        auto ada_norm_fp8 = [&](float ssq, const __nv_bfloat16* style_row, float out_scale) {
            const float rms = rms_of(ssq);
            const float inv_os = __fdiv_rn(1.0f, out_scale);
            float sc[4], shf[4], q[4];
            ld4bf(style_row + n0, sc);
            ld4bf(style_row + D + n0, shf);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float nv = __fmaf_rn(__fmul_rn(xr[i], rms), __fadd_rn(1.0f, sc[i]), shf[i]);
                q[i] = clamp448(__fmul_rn(nv, inv_os));
            }
            *reinterpret_cast<uint32_t*>(p.act8 + (size_t)row * D + n0) = f32x4_to_e4m3x4(q[0], q[1], q[2], q[3]);
        };
        // end of Euler step sp: last gated residual, final adaRMS (bf16), out-projection accumulated into the noise
        auto finish_step = [&](int sp) {
            const int gl = sp * L + (L - 1);
            const float alpha = p.act_scale[(size_t)gl * 4 + 3] * p.ws_d[L - 1];
            (void)add_delta(4, alpha, p.style_ffn + (size_t)gl * 3 * D + 2 * D);
            float ssq = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) ssq = __fmaf_rn(xr[i], xr[i], ssq);
            const float rms = rms_of(ssq);
            const __nv_bfloat16* st = p.style_final + (size_t)sp * 3 * D;
            float sc[4], shf[4];
            ld4bf(st + n0, sc);
            ld4bf(st + D + n0, shf);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                s_row[n0 + i] = bf16r(__fmaf_rn(__fmul_rn(xr[i], rms), __fadd_rn(1.0f, sc[i]), shf[i]));
            work_sync();
            float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
            for (int i = 0; i < D / 32; ++i) {
                const int k = lane + 32 * i;
                float w[4];
                ld4bf(p.out_w + (size_t)k * ADIM + 4 * ww, w);
                const float xv = s_row[k];
#pragma unroll
                for (int j = 0; j < 4; ++j) a4[j] = fmaf(xv, w[j], a4[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) a4[j] = warp_sum_butterfly(a4[j]);
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int o = 4 * ww + j;
                    const float nz = p.noise[(size_t)row * ADIM + o] + (a4[j] + __bfloat162float(p.out_b[o]));
                    p.noise[(size_t)row * ADIM + o] = nz;
                    s_small[32 + o] = nz;
                }
            }
            work_sync();
        };

        for (int step = 0; step < p.steps; ++step) {
            for (int layer = 0; layer < L; ++layer) {
                const int gl = step * L + layer;
                const float* asc = p.act_scale + (size_t)gl * 4;
                // The keys / values of the prefix do not change during the loop: the chunk of this CTA's attention unit
                // is fetched by TMA now and lands during phases A and B (an attention CTA owns no QKV unit of the same
                // block, so nothing else uses the operand region until phase C).
                const int au = dead ? -1 : att_unit(G, cta, gl, p.att_units);
                const bool kv_ahead = au >= 0 && (au / p.att_tiles + 1) * BKV <= p.prefix_len;
                if (kv_ahead && wtid == 0) {
                    const int y = layer * p.kv_rows + (au / p.att_tiles) * BKV;
                    tc::mbar_arrive_expect_tx(kv_full, 2 * BKV * HD * 2);
#pragma unroll
                    for (int db = 0; db < 4; ++db) {
                        tc::tma_load_2d(smem + OFF_K + db * (BKV * 128), &tmK, kv_full, db * 128, y);
                        tc::tma_load_2d(smem + OFF_V + db * (BKV * 128), &tmV, kv_full, db * 128, y);
                    }
                }
                // ---------------------------------------------------------------- A: rows
                if (row_cta && !dead) {
                    float ssq = 0.0f;
                    if (layer == 0) {
                        if (step > 0) finish_step(step - 1);
                        else {
                            if (wtid < ADIM) s_small[32 + wtid] = p.noise[(size_t)row * ADIM + wtid];
                            work_sync();
                        }
                        // in-projection: bf16(noise) . in_w + in_b -> bf16 residual row
                        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
                        for (int k = 0; k < ADIM; ++k) {
                            float w[4];
                            ld4bf(p.in_w + (size_t)k * D + n0, w);
                            const float a = bf16r(s_small[32 + k]);
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[i] = fmaf(a, w[i], acc[i]);
                        }
                        float b[4];
                        ld4bf(p.in_b + n0, b);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            xr[i] = bf16r(acc[i] + b[i]);
                            ssq = __fmaf_rn(xr[i], xr[i], ssq);
                        }
                        work_sync();     // s_small[32..] is rewritten by the next finish_step only after this point
                    } else {
                        const float alpha = p.act_scale[(size_t)(gl - 1) * 4 + 3] * p.ws_d[layer - 1];
                        ssq = add_delta(4, alpha, p.style_ffn + (size_t)(gl - 1) * 3 * D + 2 * D);
                    }
                    ada_norm_fp8(ssq, p.style_attn + (size_t)gl * 3 * D, asc[0]);
                }
                grid_barrier();

                // ---------------------------------------------------------------- B: QKV projection + RoPE + split
                {
                    const int u = gemm_unit(G, cta, gl, 0);
                    if (u >= 0 && !dead) {
                        load_tile<D, 16>(sh, MAXS, wtid, [&](int r) -> const uint8_t* {
                            return r < S ? p.act8 + (size_t)r * D : nullptr;
                        });
                        tc::fence_proxy_async_smem();
                        tc::mbar_arrive(b_ready);
                        const int n = u * 128 + quad * 32 + lane;       // feature of the fused q|k|v row
                        const bool is_q = n < QD, is_k = !is_q && n < QD + HD;
                        const int nr = n & (HD - 1);
                        // the RoPE pairs of this thread's feature for its 32 tokens, fetched while the MMAs run
                        uint32_t rp[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int m = half * 32 + j;
                            rp[j] = (m < S && (is_q || is_k))
                                        ? __ldg(reinterpret_cast<const uint32_t*>(p.rope + (size_t)m * HD + (nr & ~1)))
                                        : 0u;
                        }
                        const float alpha = asc[0] * p.ws_qkv[layer];
                        const bool ok = wait(acc_bar, n_acc & 1);
                        ++n_acc;
                        if (ok) {
                            tc::tc_fence_after_sync();
                            uint32_t v[32];
                            ld_acc(v);
                            __nv_bfloat16* dst = is_q ? p.q + n
                                                      : (is_k ? p.k_cache : p.v_cache) +
                                                            ((size_t)layer * p.kv_rows + p.prefix_len) * HD + nr;
                            const size_t dstride = is_q ? QD : HD;
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const int m = half * 32 + j;
                                if (m < S) {                                  // warp-uniform
                                    const float val = bf16r(__uint_as_float(v[j]) * alpha);
                                    const float other = __shfl_xor_sync(0xffffffffu, val, 1);
                                    float out = val;
                                    if (is_q || is_k) {
                                        float cs, sn;
                                        unpack_bf16x2(rp[j], cs, sn);
                                        out = (nr & 1) ? __fmaf_rn(val, cs, __fmul_rn(other, sn))
                                                       : __fmaf_rn(val, cs, -__fmul_rn(other, sn));
                                    }
                                    dst[(size_t)m * dstride] = __float2bfloat16_rn(out);
                                }
                            }
                            tc::tc_fence_before_sync();
                        }
                    }
                }
                grid_barrier();

                // ---------------------------------------------------------------- C: attention partials
                // unit = (tile of 16 tokens x 8 heads, one chunk of 64 keys).  Q goes to tensor memory (each thread
                // = one (token, head) row, bf16 pairs per column) and feeds the MMA as the A operand, K and V sit in
                // the 64 KB operand region, P overlays S.
                {
                    if (au >= 0 && !dead) {
                        const int tile = au % p.att_tiles, c = au / p.att_tiles;
                        const int tok0 = tile * 16, key0 = c * BKV;
                        const __nv_bfloat16* kc = p.k_cache + (size_t)layer * p.kv_rows * HD;
                        const __nv_bfloat16* vc = p.v_cache + (size_t)layer * p.kv_rows * HD;
                        const int arow = quad * 32 + lane;                  // (token, head) row of this thread
                        {
                            const int tok = tok0 + (arow >> 3);
                            const uint4* src = reinterpret_cast<const uint4*>(p.q + (size_t)tok * QD + (arow & 7) * HD + half * 128);
                            uint4 qv[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) qv[i] = tok < S ? __ldcg(src + i) : make_uint4(0, 0, 0, 0);
                            if (!kv_ahead) {       // the chunk holds rows appended in phase B: plain loads
                                load_tile<HD * 2, 8>(smem + OFF_K, BKV, wtid, [&](int r) -> const uint8_t* {
                                    return key0 + r < p.T ? reinterpret_cast<const uint8_t*>(kc + (size_t)(key0 + r) * HD)
                                                          : nullptr;
                                });
                                load_tile<HD * 2, 8>(smem + OFF_V, BKV, wtid, [&](int r) -> const uint8_t* {
                                    return key0 + r < p.T ? reinterpret_cast<const uint8_t*>(vc + (size_t)(key0 + r) * HD)
                                                          : nullptr;
                                });
                            }
                            const uint32_t tq = tmem + Q_COL + lane_off + half * 64;
                            tc::tmem_st32(tq, &qv[0].x);
                            tc::tmem_st32(tq + 32, &qv[8].x);
                            tc::tmem_st_wait();
                        }
                        if (kv_ahead) {
                            (void)wait(kv_full, n_kv & 1);
                            ++n_kv;
                        }
                        tc::fence_proxy_async_smem();
                        tc::tc_fence_before_sync();
                        tc::mbar_arrive(b_ready);
                        bool ok = wait(acc_bar, n_acc & 1);
                        ++n_acc;
                        float m_run = -INFINITY, l_run = 0.0f;
                        if (ok && ww < 4) {
                            // ---- softmax of the chunk: thread = row, P (bf16) overlays S in tensor memory
                            tc::tc_fence_after_sync();
                            const uint32_t tmem_S = tmem + lane_off;
                            const int valid = p.T - key0;
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
                                for (int q4 = 0; q4 < 4; ++q4) mx4[q4] = fmaxf(mx4[q4], __uint_as_float(sv[i + q4]));
                            }
                            m_run = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
                            const float m_use = (m_run == -INFINITY) ? 0.0f : m_run;
                            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                            for (int cb = 0; cb < BKV; cb += 32) {
                                uint32_t uu[16];
#pragma unroll
                                for (int i = 0; i < 16; ++i) {
                                    const float a = ex2(__fmaf_rn(__uint_as_float(sv[cb + 2 * i]), p.scale_log2, -m_use));
                                    const float b = ex2(__fmaf_rn(__uint_as_float(sv[cb + 2 * i + 1]), p.scale_log2, -m_use));
                                    sum4[i & 3] += a + b;
                                    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(uu[i]) : "f"(b), "f"(a));
                                }
                                tc::tmem_st16(tmem_S + (cb >> 1), uu);
                            }
                            tc::tmem_st_wait();
                            l_run = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                            tc::tc_fence_before_sync();
                            tc::mbar_arrive(p_ready);
                            s_l[arow] = l_run > 0.0f ? 1.0f / l_run : 0.0f;
                            s_lse[arow] = l_run > 0.0f ? m_run + log2f(l_run) : -INFINITY;
                        }
                        ok = wait(o_full, n_o & 1);
                        ++n_o;
                        // ---- normalised partial as bf16 -> shared memory (rows of 512 bytes, 16-byte chunks xor-swizzled)
                        // -> global scratch with full-row stores (runs even after a failed wait: everyone must reach
                        // the worker barriers)
                        work_sync();
                        tc::tc_fence_after_sync();
                        const float invl = s_l[arow];
                        {
                            const uint32_t tmem_O = tmem + O_COL + lane_off + half * 128;
#pragma unroll 1
                            for (int cb = 0; cb < 128; cb += 32) {
                                uint32_t ov[32];
                                tc::tmem_ld32(tmem_O + cb, ov);
                                tc::tmem_ld_wait();
#pragma unroll
                                for (int j8 = 0; j8 < 4; ++j8) {
                                    uint4 o;
                                    o.x = pack_bf16x2(__uint_as_float(ov[j8 * 8 + 0]) * invl, __uint_as_float(ov[j8 * 8 + 1]) * invl);
                                    o.y = pack_bf16x2(__uint_as_float(ov[j8 * 8 + 2]) * invl, __uint_as_float(ov[j8 * 8 + 3]) * invl);
                                    o.z = pack_bf16x2(__uint_as_float(ov[j8 * 8 + 4]) * invl, __uint_as_float(ov[j8 * 8 + 5]) * invl);
                                    o.w = pack_bf16x2(__uint_as_float(ov[j8 * 8 + 6]) * invl, __uint_as_float(ov[j8 * 8 + 7]) * invl);
                                    const int ch = ((half * 128 + cb) >> 3) + j8;             // 16-byte chunk of the row, 0..31
                                    *reinterpret_cast<uint4*>(sh + arow * 512 + ((ch ^ (arow & 7)) << 4)) = o;
                                }
                            }
                        }
                        tc::tc_fence_before_sync();
                        work_sync();
                        uint4* dst_unit = reinterpret_cast<uint4*>(p.po + (size_t)au * 128 * HD);
#pragma unroll 4
                        for (int r = ww; r < 128; r += 8)
                            __stcg(dst_unit + r * 32 + lane, *reinterpret_cast<const uint4*>(sh + r * 512 + ((lane ^ (r & 7)) << 4)));
                        if (wtid < 128) __stcg(p.plse + (size_t)au * 128 + wtid, s_lse[wtid]);
                    }
                }
                grid_barrier();

                // ---------------------------------------------------------------- D: combine the chunks -> FP8
                if (!dead) {
                    const float inv_os = __fdiv_rn(1.0f, asc[1]);
                    const int items = S * NH * (HD / 8);
                    for (int it = cta * NWORK + wtid; it < items; it += G * NWORK) {
                        const int ch = it & 31, head = (it >> 5) & 7, tok = it >> 8;
                        const int tile = tok >> 4, r = ((tok & 15) << 3) + head;
                        float M = -INFINITY, Lw = 0.0f, a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                        for (int s0 = 0; s0 < p.nsplit; s0 += 8) {
                            // eight partials in flight together, then folded into the running (max, sum, value)
                            float lse[8];
                            uint4 x[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const bool in = s0 + j < p.nsplit;
                                const size_t ub = (size_t)((in ? s0 + j : 0) * p.att_tiles + tile) * 128 + r;
                                lse[j] = in ? __ldcg(p.plse + ub) : -INFINITY;
                                x[j] = in ? __ldcg(reinterpret_cast<const uint4*>(p.po + ub * HD) + ch) : make_uint4(0, 0, 0, 0);
                            }
                            float Mg = M;
#pragma unroll
                            for (int j = 0; j < 8; ++j) Mg = fmaxf(Mg, lse[j]);
                            const float resc = (M == -INFINITY) ? 0.0f : ex2(M - Mg);
                            Lw *= resc;
#pragma unroll
                            for (int e = 0; e < 8; ++e) a[e] *= resc;
                            M = Mg;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float w = (lse[j] == -INFINITY) ? 0.0f : ex2(lse[j] - M);
                                Lw += w;
                                const uint32_t* xw = &x[j].x;
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    float lo, hi;
                                    unpack_bf16x2(xw[e], lo, hi);
                                    a[2 * e] += w * lo;
                                    a[2 * e + 1] += w * hi;
                                }
                            }
                        }
                        const float invL = Lw > 0.0f ? 1.0f / Lw : 0.0f;
                        // the attention output is a bf16 tensor in the operator composition: keep that rounding point
                        float q8[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) q8[e] = clamp448(__fmul_rn(bf16r(a[e] * invL), inv_os));
                        uint2 o8;
                        o8.x = f32x4_to_e4m3x4(q8[0], q8[1], q8[2], q8[3]);
                        o8.y = f32x4_to_e4m3x4(q8[4], q8[5], q8[6], q8[7]);
                        *reinterpret_cast<uint2*>(p.attn8 + (size_t)tok * QD + head * HD + ch * 8) = o8;
                    }
                }
                grid_barrier();

                // ---------------------------------------------------------------- E: output projection (split-K 2)
                {
                    const int u = gemm_unit(G, cta, gl, 1);
                    if (u >= 0 && !dead) {
                        const int ks = u >> 3, tile = u & 7;
                        load_tile<D, 16>(sh, MAXS, wtid, [&](int r) -> const uint8_t* {
                            return r < S ? p.attn8 + (size_t)r * QD + ks * 1024 : nullptr;
                        });
                        tc::fence_proxy_async_smem();
                        tc::mbar_arrive(b_ready);
                        const bool ok = wait(acc_bar, n_acc & 1);
                        ++n_acc;
                        store_partial(ok, ks, tile);
                    }
                }
                grid_barrier();

                // ---------------------------------------------------------------- F: rows
                if (row_cta && !dead) {
                    const float alpha = asc[1] * p.ws_o[layer];
                    const float ssq = add_delta(2, alpha, p.style_attn + (size_t)gl * 3 * D + 2 * D);
                    ada_norm_fp8(ssq, p.style_ffn + (size_t)gl * 3 * D, asc[2]);
                }
                grid_barrier();

                // ---------------------------------------------------------------- G: gate|up projection + GeGLU
                {
                    const int u = gemm_unit(G, cta, gl, 2);
                    if (u >= 0 && !dead) {
                        load_tile<D, 16>(sh, MAXS, wtid, [&](int r) -> const uint8_t* {
                            return r < S ? p.act8 + (size_t)r * D : nullptr;
                        });
                        tc::fence_proxy_async_smem();
                        tc::mbar_arrive(b_ready);
                        const bool ok = wait(acc_bar, n_acc & 1);
                        ++n_acc;
                        // the token operand is dead once the accumulator is complete: its space carries the exchange
                        float* ex = reinterpret_cast<float*>(sh);                 // [gate | up][token][64]
                        const float alpha = asc[2] * p.ws_gu[layer];
                        const int rr = quad * 32 + lane;                          // < 64: gate row, else up row
                        if (ok) {
                            tc::tc_fence_after_sync();
                            uint32_t v[32];
                            ld_acc(v);
                            float* exr = ex + (rr >> 6) * (MAXS * 64) + (rr & 63);
#pragma unroll
                            for (int j = 0; j < 32; ++j) exr[(half * 32 + j) * 64] = bf16r(__uint_as_float(v[j]) * alpha);
                            tc::tc_fence_before_sync();
                        }
                        work_sync();
                        {
                            // thread = hidden unit h of this tile for tokens tg, tg + 4, ...: all operands first, then
                            // the arithmetic, then the stores (32 consecutive bytes per warp and token)
                            const float inv_os = __fdiv_rn(1.0f, asc[3]);
                            const int h = wtid & 63, tg = wtid >> 6;
                            float gt[16], up[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int m = tg + 4 * i;
                                gt[i] = ex[m * 64 + h];
                                up[i] = ex[MAXS * 64 + m * 64 + h];
                            }
                            uint8_t* dst = p.hid8 + u * 64 + h;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int m = tg + 4 * i;
                                const float qv = clamp448(__fmul_rn(__fmul_rn(det_gelu_tanh(gt[i]), up[i]), inv_os));
                                if (m < S) dst[(size_t)m * HID] = (uint8_t)__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3);
                            }
                        }
                    }
                }
                grid_barrier();

                // ---------------------------------------------------------------- H: down projection (split-K 4)
                {
                    const int u = gemm_unit(G, cta, gl, 3);
                    if (u >= 0 && !dead) {
                        const int ks = u >> 3, tile = u & 7;
                        load_tile<D, 16>(sh, MAXS, wtid, [&](int r) -> const uint8_t* {
                            return r < S ? p.hid8 + (size_t)r * HID + ks * 1024 : nullptr;
                        });
                        tc::fence_proxy_async_smem();
                        tc::mbar_arrive(b_ready);
                        const bool ok = wait(acc_bar, n_acc & 1);
                        ++n_acc;
                        store_partial(ok, ks, tile);
                    }
                }
                grid_barrier();
            }
        }
        if (row_cta && !dead) finish_step(p.steps - 1);
    }

    // ---------------- teardown
    __syncwarp();
    tc::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // copies that were issued but never consumed get a bounded chance to land before the CTA exits
        for (int i = *consumed; i < *issued; ++i) {
            const int s = i % RING;
            for (int it = 0; it < 4096; ++it) {
                if (tc::mbar_try_wait(&full[s], (i / RING) & 1)) break;
                __nanosleep(256);
            }
        }
    }
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace el
}  // namespace frt

using namespace frt;

static inline long long align_up(long long v, long long a) { return (v + a - 1) / a * a; }

struct LoopLayout {
    long long sync, act8, q, attn8, hid8, part, po, plse, total;
    int T, chunks, nsplit, tiles, units;
};
static int loop_layout(int S, int prefix_len, LoopLayout* o) {
    if (S < 1 || S > el::MAXS || prefix_len < 0) return FRT_ERR_UNSUPPORTED;
    o->T = prefix_len + S;
    o->chunks = (o->T + el::BKV - 1) / el::BKV;
    o->nsplit = o->chunks;                 // one attention unit per (tile, chunk of 64 keys)
    o->tiles = (S + 15) / 16;
    o->units = o->tiles * o->nsplit;
    long long off = 0;
    o->sync = off; off += 256;
    o->act8 = off; off += (long long)el::MAXS * el::D;
    o->q = off; off += (long long)el::MAXS * el::QD * 2;
    o->attn8 = off; off += (long long)el::MAXS * el::QD;
    o->hid8 = off; off += (long long)el::MAXS * el::HID;
    o->part = off; off += 4LL * el::MAXS * el::D * 4;
    o->po = off; off += (long long)o->units * 128 * el::HD * 2;
    o->plse = off; off += align_up((long long)o->units * 128 * 4, 256);
    o->total = off;
    return FRT_OK;
}

extern "C" {

int frt_b200_expert_loop_workspace_bytes(int S, int prefix_len, long long* out_bytes) {
    LoopLayout lay;
    if (!out_bytes) return FRT_ERR_INVALID;
    const int rc = loop_layout(S, prefix_len, &lay);
    if (rc) return rc;
    *out_bytes = lay.total;
    return FRT_OK;
}

int frt_b200_expert_loop_fp8(const void* host_args, int args_bytes, void* stream) {
    if (!host_args || args_bytes != (int)sizeof(frt_b200_expert_loop_args)) return FRT_ERR_INVALID;
    const frt_b200_expert_loop_args& a = *reinterpret_cast<const frt_b200_expert_loop_args*>(host_args);
    const void* need[] = {a.w_qkv, a.w_o, a.w_gu, a.w_d, a.ws_qkv, a.ws_o, a.ws_gu, a.ws_d, a.act_scale, a.style_attn,
                          a.style_ffn, a.style_final, a.rope, a.in_w, a.in_b, a.out_w, a.out_b, a.k_cache, a.v_cache,
                          a.noise, a.workspace};
    for (const void* ptr : need)
        if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 3)) return FRT_ERR_INVALID;
    if (a.steps < 1 || a.layers < 1 || a.kv_rows < a.prefix_len + a.S) return FRT_ERR_INVALID;
    if ((reinterpret_cast<uintptr_t>(a.workspace) & 255) || (reinterpret_cast<uintptr_t>(a.k_cache) & 15) ||
        (reinterpret_cast<uintptr_t>(a.v_cache) & 15) || (reinterpret_cast<uintptr_t>(a.rope) & 15) ||
        (reinterpret_cast<uintptr_t>(a.style_attn) & 15) || (reinterpret_cast<uintptr_t>(a.style_ffn) & 15) ||
        (reinterpret_cast<uintptr_t>(a.style_final) & 15) || (reinterpret_cast<uintptr_t>(a.in_w) & 15) ||
        (reinterpret_cast<uintptr_t>(a.out_w) & 15) || (reinterpret_cast<uintptr_t>(a.in_b) & 15))
        return FRT_ERR_INVALID;
    LoopLayout lay;
    int rc = loop_layout(a.S, a.prefix_len, &lay);
    if (rc) return rc;
    if (a.workspace_bytes < lay.total) return FRT_ERR_INVALID;

    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    static frt::PerDeviceOnce attr_once;
    int attr_dev = 0;
    if (attr_once.need(attr_dev)) {
        cudaError_t e = cudaFuncSetAttribute(el::expert_loop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             el::SMEM_BYTES);
        if (e != cudaSuccess) return FRT_CUDA_ERR(e);
        attr_once.set(attr_dev);
    }
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, el::expert_loop_kernel, 320, el::SMEM_BYTES);
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    if (per_sm < 1) return FRT_ERR_UNSUPPORTED;
    const int G = sms;
    // every CTA owns at most one unit per phase and one token row
    if (G < el::U_GU || G < a.S || G < el::U_QKV + lay.units) return FRT_ERR_UNSUPPORTED;

    CUtensorMap tmQKV, tmO, tmGU, tmD;
    rc = get_tmap_2d_u8(&tmQKV, a.w_qkv, (uint64_t)a.layers * el::NQKV, el::D, el::D, 128);
    if (rc) return rc;
    rc = get_tmap_2d_u8(&tmO, a.w_o, (uint64_t)a.layers * el::D, el::QD, el::QD, 128);
    if (rc) return rc;
    rc = get_tmap_2d_u8(&tmGU, a.w_gu, (uint64_t)a.layers * 2 * el::HID, el::D, el::D, 64);
    if (rc) return rc;
    rc = get_tmap_2d_u8(&tmD, a.w_d, (uint64_t)a.layers * el::D, el::HID, el::HID, 128);
    if (rc) return rc;
    CUtensorMap tmK, tmV;      // caches as byte matrices: one row of 512 bytes per key
    rc = get_tmap_2d_u8(&tmK, a.k_cache, (uint64_t)a.layers * a.kv_rows, el::HD * 2, el::HD * 2, el::BKV);
    if (rc) return rc;
    rc = get_tmap_2d_u8(&tmV, a.v_cache, (uint64_t)a.layers * a.kv_rows, el::HD * 2, el::HD * 2, el::BKV);
    if (rc) return rc;

    uint8_t* ws = reinterpret_cast<uint8_t*>(a.workspace);
    el::LoopParams p;
    p.ws_qkv = (const float*)a.ws_qkv; p.ws_o = (const float*)a.ws_o; p.ws_gu = (const float*)a.ws_gu;
    p.ws_d = (const float*)a.ws_d; p.act_scale = (const float*)a.act_scale;
    p.style_attn = (const __nv_bfloat16*)a.style_attn; p.style_ffn = (const __nv_bfloat16*)a.style_ffn;
    p.style_final = (const __nv_bfloat16*)a.style_final; p.rope = (const __nv_bfloat16*)a.rope;
    p.in_w = (const __nv_bfloat16*)a.in_w; p.in_b = (const __nv_bfloat16*)a.in_b;
    p.out_w = (const __nv_bfloat16*)a.out_w; p.out_b = (const __nv_bfloat16*)a.out_b;
    p.k_cache = (__nv_bfloat16*)a.k_cache; p.v_cache = (__nv_bfloat16*)a.v_cache;
    p.noise = (float*)a.noise;
    p.sync = reinterpret_cast<unsigned*>(ws + lay.sync);
    p.act8 = ws + lay.act8;
    p.q = reinterpret_cast<__nv_bfloat16*>(ws + lay.q);
    p.attn8 = ws + lay.attn8;
    p.hid8 = ws + lay.hid8;
    p.part = reinterpret_cast<float*>(ws + lay.part);
    p.po = reinterpret_cast<__nv_bfloat16*>(ws + lay.po);
    p.plse = reinterpret_cast<float*>(ws + lay.plse);
    p.steps = a.steps; p.layers = a.layers; p.S = a.S; p.prefix_len = a.prefix_len; p.kv_rows = a.kv_rows;
    p.T = lay.T; p.chunks_total = lay.chunks; p.nsplit = lay.nsplit; p.att_units = lay.units; p.att_tiles = lay.tiles;
    p.scale_log2 = 0.0625f * 1.4426950408889634f;

    e = cudaMemsetAsync(ws + lay.sync, 0, 256, (cudaStream_t)stream);
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(G);
    cfg.blockDim = dim3(320);
    cfg.dynamicSmemBytes = el::SMEM_BYTES;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident together: they wait for one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, el::expert_loop_kernel, tmQKV, tmO, tmGU, tmD, tmK, tmV, p);
    return e == cudaSuccess ? FRT_OK : FRT_CUDA_ERR(e);
}

// The static schedule of the loop kernel, evaluated on the host (no GPU needed): which unit of `phase` (0 QKV, 1 output
// projection, 2 gate|up, 3 down, 4 attention with `att_units` units) of global block `gl` = step * layers + layer
// the CTA `cta` of a grid of G owns; *unit_out = -1 when it owns none.
int frt_b200_expert_loop_schedule(int G, int cta, int gl, int phase, int att_units, int* unit_out) {
    if (!unit_out || G < 1 || cta < 0 || cta >= G || gl < 0 || phase < 0 || phase > 4) return FRT_ERR_INVALID;
    *unit_out = phase < 4 ? el::gemm_unit(G, cta, gl, phase) : el::att_unit(G, cta, gl, att_units);
    return FRT_OK;
}

}  // extern "C"
namespace frt {
int* expert_loop_status_device_ptr() {
    void* p = nullptr;
    return cudaGetSymbolAddress(&p, g_loop_status) == cudaSuccess ? static_cast<int*>(p) : nullptr;
}
}  // namespace frt
extern "C" {

// device status word of the persistent loop kernel (0 = no bounded wait ever gave up); code 1 weight producer,
// 2 MMA issuer, 3 worker, 4 grid barrier, | CTA index << 8.  Synchronises the device.
int frt_b200_expert_loop_status(int reset) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_loop_status, sizeof(int));
    if (e != cudaSuccess) return FRT_CUDA_ERR(e);
    if (reset && v) {
        int z = 0;
        cudaMemcpyToSymbol(g_loop_status, &z, sizeof(int));
    }
    return v;
}

}  // extern "C"
