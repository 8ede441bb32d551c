/*
 * flashrt_b200 -- C ABI of the sm_100a (B200) denoise-path kernel library.
 *
 * Plain pointers and sizes only: every pointer is a device pointer unless a
 * comment says "host"; `stream` is a cudaStream_t passed as void* (NULL = the
 * default stream).  Nothing here allocates device memory unless its comment
 * says so, nothing synchronises the device, every launch is capturable in a
 * CUDA graph.  The caller owns all buffers.
 *
 * Return value: 0 on success, otherwise
 *   -1  invalid argument (null pointer, negative size, misaligned pointer)
 *   -2  unsupported shape / feature
 *   -3  a bounded device-side wait gave up (see frt_b200_gemm_status)
 *   -4  the request exceeds a built-in fixed-size buffer (entry points that say so)
 *   -(1000 + cudaError_t) for a CUDA runtime failure at launch.
 *
 * `flags` bit 0: launch with programmatic dependent launch (the kernel starts
 * its input-independent prologue before the previous kernel in the stream has
 * finished; only set it when scales / weights / styles are not written by that
 * previous kernel).
 *
 * Citations name the reference entry point each function stands in for, as
 * path:line inside the FlashRT source tree.
 */
#ifndef FLASHRT_B200_H
#define FLASHRT_B200_H

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- fused norm + quantise
 * One kernel family for
 *   rms_norm_fp8                csrc/bindings.cpp:899-907  -> csrc/kernels/norm.cu:286-343
 *   ada_rms_norm_style_fp8      csrc/bindings.cpp:909-921  -> csrc/kernels/norm.cu:392-442
 *   residual_add_rms_norm_fp8   csrc/bindings.cpp:923-935  -> csrc/kernels/norm.cu:445-495
 *   gate_residual_ada_norm_fp8  csrc/bindings.cpp:1144-1162 -> csrc/kernels/fusion.cu:15-81
 *
 *   if x:        residual <- bf16(residual + x * gate_in)      (gate_in NULL: residual + x)
 *   rms        = 1 / sqrt(mean(r^2) + eps)                     (r unrounded when updated)
 *   y          = bf16(residual) * rms * weight                 (weight NULL: ones)
 *   if style:    y = y * (1 + scale) + shift ; gate_out <- gate   (style row = [scale|shift|gate])
 *   out_fp8    = e4m3(clamp(y * (1 / *d_scale), +-448))
 *
 * residual (rows, dim) bf16 in/out; x (rows, dim) bf16 or NULL; gate_in bf16 rows at
 * gate_in + r * gate_in_stride (stride in elements; 0 = one row shared by all);
 * style rows of 3*dim at style + r * style_stride (0 = shared); gate_out (rows, dim) or NULL.
 * dim % 8 == 0, dim <= 8192; pointers 16-byte aligned (out_fp8: 8).
 */
int frt_b200_norm_fp8(void* residual, const void* x, const void* gate_in, long long gate_in_stride,
                      const void* weight, const void* style, long long style_stride, void* out_fp8,
                      void* gate_out, int rows, int dim, float eps, const float* d_scale, int flags,
                      void* stream);

/* Same with a bf16 result instead of FP8:
 *   rms_norm                    csrc/bindings.cpp:854-862
 *   ada_rms_norm_style          csrc/bindings.cpp:887-897  -> csrc/kernels/norm.cu:345-389
 *   residual_add_rms_norm       csrc/bindings.cpp:937-947  -> csrc/kernels/norm.cu:498-539 */
int frt_b200_norm_bf16(void* residual, const void* x, const void* gate_in, long long gate_in_stride,
                       const void* weight, const void* style, long long style_stride, void* out_bf16,
                       void* gate_out, int rows, int dim, float eps, int flags, void* stream);

/* ---------------------------------------------------------------- activation / quantise
 * gate_geglu_merged_fp8        csrc/bindings.cpp:1037-1044 -> csrc/kernels/activation.cu:249-279
 *   merged (rows, 2*half_dim) bf16 = [gate | up];  out (rows, half_dim) e4m3 =
 *   e4m3(clamp(gelu_tanh(gate) * up * (1 / *d_scale), +-448)).  half_dim % 8 == 0.
 *   flags bit 1: SiLU gate, silu(gate) * up with silu(g) = g / (1 + exp(-g)) -- the arithmetic of
 *   silu_mul_split_fp8_kernel (csrc/kernels/activation.cu:291-306; bindings csrc/bindings.cpp:1912-1918) on the merged
 *   [gate | up] layout (SwiGLU). */
int frt_b200_geglu_fp8(const void* merged, void* out_fp8, int rows, int half_dim, const float* d_scale,
                       int flags, void* stream);
/* gate_geglu_merged            csrc/bindings.cpp:1031-1035 (bf16 result; flags bit 1: SiLU gate as above) */
int frt_b200_geglu_bf16(const void* merged, void* out_bf16, int rows, int half_dim, int flags, void* stream);

/* quantize_fp8_static          csrc/bindings.cpp:1191-1196 -> csrc/kernels/quantize.cu:61-75,297-304 */
int frt_b200_quantize_fp8_static(const void* in_bf16, void* out_fp8, const float* d_scale, long long n,
                                 int flags, void* stream);
/* quantize_fp8_device          csrc/bindings.cpp:1198-1204 -> csrc/kernels/quantize.cu:131-156
 *   *d_scale <- max(absmax(in) / 448, 1e-12), then quantise with it (4 stream operations). */
int frt_b200_quantize_fp8_device(const void* in_bf16, void* out_fp8, float* d_scale, long long n, void* stream);
/* fp8_accumulate_scale_max     csrc/bindings.cpp:1205-1211 -> csrc/kernels/quantize.cu:137-146 */
int frt_b200_fp8_accumulate_scale_max(const float* src_scale, float* dst_scale, void* stream);

/* ---------------------------------------------------------------- residual-style adds (bf16, in place)
 * residual_add                 csrc/bindings.cpp:1116-1119 -> csrc/kernels/elementwise.cu:302 */
int frt_b200_residual_add(void* residual, const void* x, long long n, int flags, void* stream);
/* bias_residual                csrc/bindings.cpp:1108-1114 -> csrc/kernels/elementwise.cu:207 */
int frt_b200_bias_residual(void* residual, const void* x, const void* bias, int rows, int dim, int flags,
                           void* stream);
/* gate_mul_residual            csrc/bindings.cpp:1103-1106 -> csrc/kernels/elementwise.cu:34
 *   residual += x * gate; gate rows at gate + r * gate_stride (0 = shared row) */
int frt_b200_gate_mul_residual(void* residual, const void* x, const void* gate, long long gate_stride, int rows,
                               int dim, int flags, void* stream);

/* ---------------------------------------------------------------- RoPE + QKV split + KV-cache append
 * qkv_split_rope               csrc/bindings.cpp:1071-1082 -> csrc/kernels/rope.cu:135-208
 * qkv_split_rope_devpos        csrc/bindings.cpp:1086-1099 -> csrc/kernels/rope.cu:215-277
 *   qkv (seq, q_dim+k_dim+v_dim) bf16; rope (seq, head_dim) bf16 = [cos0,sin0,cos1,sin1,...];
 *   Q (seq, q_dim); K/V rows written at row (*devpos + t) (devpos NULL: row t). */
int frt_b200_qkv_split_rope(const void* qkv, const void* rope, void* Q, void* K, void* V, const int* devpos,
                            int seq, int q_dim, int k_dim, int v_dim, int head_dim, int flags, void* stream);

/* ---------------------------------------------------------------- FP8 GEMM (tcgen05 / TMEM / TMA)
 * GemmRunner::fp8_nt_dev       csrc/bindings.cpp:717-727   -> csrc/gemm/gemm_runner.cu (cuBLASLt)
 * fp8_gemm_descale_bf16out     csrc/bindings.cpp:2062-2069 -> csrc/kernels/decoder_fused.cu:310-468
 * cutlass_fp8_*_bf16out        csrc/bindings.cpp:2388-2422 -> csrc/gemm/cutlass_sm100.cu:75-125
 *   D(M,N) bf16 = alpha_host * (*d_scale_a) * (*d_scale_b) * A(M,K) . W(N,K)^T + bias(N)
 *   A, W: E4M3, row-major, K contiguous, 16-byte aligned, K % 16 == 0.  d_scale_* and bias may be NULL.
 *   splits: 0 = choose; else split-K factor in [1, 16] (reduced inside a thread-block cluster).  At M > 256 the
 *   library never chooses a split itself: a 128 x 256 fp32 tile per rank through distributed shared memory costs
 *   several times what the split saves (measured 2048 x 3072 x 14336: 92 us unsplit, 284 us with splits = 2).
 *   M > 256 runs as a persistent kernel (one CTA per SM walking the tile list, two accumulators in tensor memory so
 *   that the epilogue overlaps the next tile's MMAs); flags bit 1 selects the one-tile-per-CTA kernel instead;
 *   tile lists of at least two waves with K >= 2048 (or flags bit 3; M > 256, N >= 256, no split-K) run a kernel with
 *   one 256 x 256 tile per CTA pair (tcgen05 cta_group::2: each CTA stages its 128 rows of A and 128 of the 256 weight
 *   rows, the leader issues the MMAs for both); flags bit 5 keeps the one-CTA persistent kernel.
 *   M <= 128 (up to 256 with a pinned tile width or split) with K % 128 == 0 and N % 8 == 0 runs the token-major kernel (activation rows on the 128 accumulator
 *   lanes, up to 256 weight rows on the columns, split-K in {1, 2, 4, 8} over a cluster); flags bit 4 keeps the
 *   swapped kernel (weights on the lanes) instead; flags bits 8-9 pin the tile width (1 = 64, 2 = 128, 3 = 256). */
int frt_b200_gemm_fp8_nt(const void* A, const void* W, void* D, int M, int N, int K, const float* d_scale_a,
                         const float* d_scale_b, float alpha_host, const void* bias, int splits, int flags,
                         void* stream);
/* GemmRunner::fp8_nn_dev (csrc/bindings.cpp:706-716 -> csrc/gemm/gemm_runner.cu:67-76), the reference's default weight
 * layout: B stored (K, N) row-major.  D(M,N) bf16 = alpha_host * (*d_scale_a) * (*d_scale_b) * A(M,K) . B(K,N) + bias.
 * The weight tiles are loaded as 128 K-rows x 128 N-bytes and consumed as an MN-major MMA operand; the result equals
 * frt_b200_gemm_fp8_nt on the transposed weights bit for bit.  K % 128 == 0, N % 16 == 0, N >= 128. */
int frt_b200_gemm_fp8_nn(const void* A, const void* B, void* D, int M, int N, int K, const float* d_scale_a,
                         const float* d_scale_b, float alpha_host, const void* bias, int splits, int flags,
                         void* stream);
/* The same GEMM (M <= 256) with the kernel that follows it in the decoder fused into its epilogue.
 *
 * QKV projection + qkv_split_rope[_devpos] (csrc/bindings.cpp:1071-1099 -> csrc/kernels/rope.cu:135-277):
 *   the (M, q_dim+k_dim+v_dim) result is rounded to bf16, q and k parts are rotated pairwise with
 *   rope (M, head_dim) = [cos0, sin0, cos1, sin1, ...]; Q -> (M, q_dim); K / V rows -> row (*devpos + m)
 *   of Kout / Vout (devpos NULL: row m).  Byte-identical to frt_b200_gemm_fp8_nt (same `splits`) followed by
 *   frt_b200_qkv_split_rope. */
int frt_b200_gemm_fp8_nt_rope_split(const void* A, const void* W, int M, int K, const float* d_scale_a,
                                    const float* d_scale_b, const void* rope, void* Q, void* Kout, void* Vout,
                                    const int* devpos, int q_dim, int k_dim, int v_dim, int head_dim, int splits,
                                    int flags, void* stream);
/* gate|up projection + gate_geglu_merged_fp8 (csrc/bindings.cpp:1037-1044 -> csrc/kernels/activation.cu:249-279):
 *   W (2*half, K), rows [0, half) = gate, [half, 2*half) = up; out8 (M, half) e4m3 with scale *d_out_scale.
 *   half % 64 == 0.  Byte-identical to frt_b200_gemm_fp8_nt (same `splits`) followed by frt_b200_geglu_fp8.
 *   flags bit 6: SiLU gate (SwiGLU; M <= 128 and K % 128 == 0 only, else -2), byte-identical to frt_b200_geglu_fp8
 *   with its flags bit 1 behind the same GEMM.
 *   flags bit 7 (here and in the _rowscale / norm_gemm forms): GELU(tanh) through the hardware tanh (tanh.approx.f32,
 *   relative error 2^-11) instead of the explicitly rounded exp + division -- six instructions per value instead of
 *   thirty in a finish that is bound by them; FP8 codes then agree with the exact form except for single last-place
 *   flips (the reference's kernel uses the fast __expf itself); same limits as bit 6. */
int frt_b200_gemm_fp8_nt_geglu_fp8(const void* A, const void* W, void* out8, int M, int half, int K,
                                   const float* d_scale_a, const float* d_scale_b, const float* d_out_scale,
                                   int splits, int flags, void* stream);
/* Reads (and optionally clears) the device status word of the tensor-core kernels.  0 = no bounded wait
 * ever gave up; otherwise (code | blockIdx.x << 8), code 1 = TMA producer, 2 = MMA issuer, 3 = epilogue.
 * Synchronises the device (a cudaMemcpyFromSymbol): do not call inside graph capture. */
int frt_b200_gemm_status(int reset);

/* ---------------------------------------------------------------- flash attention forward (tcgen05 / TMEM / TMA)
 * fa2.fwd_bf16                 csrc/fa2_bindings.cpp:173-183  -> csrc/attention/fa2_wrapper.cu
 * fa2.fwd_bf16_seqused[_splitkv] csrc/fa2_bindings.cpp:142-160
 *   Non-causal softmax(Q K^T * softmax_scale) V, bf16 in / bf16 out, fp32 softmax and accumulation.
 *   Q, O: (batch, seqlen_q, num_heads_q, head_dim); K, V: (batch, seqlen_k, num_heads_kv, head_dim);
 *   *_strides: host arrays of 3 element strides {batch, row, head}; head_dim (128 or 256) contiguous.
 *   num_heads_q / num_heads_kv must divide 128.  O_fp8 + out_scale: optional fused
 *   e4m3(clamp(O * (1 / *out_scale), +-448)) written with O's indexing (NULL to skip).
 *   lse: optional (batch, num_heads_q, seqlen_q) fp32; seqused_k: optional device int (valid keys).
 *   kv_splits: 0 = choose, else 1..8, rounded down to a power of two (combined inside a thread-block cluster;
 *   no scratch buffers).  kv_static_rows: leading K/V rows that the previous kernel in the stream does not
 *   write (with flags bit0 they are fetched before that kernel has finished); pass 0 if unsure.
 *   o_accum, lse_accum, counters: optional split-KV scratch (all three or none): o_accum (splits, batch,
 *   num_heads_q, seqlen_q, head_dim) fp32 and lse_accum (splits, batch, num_heads_q, seqlen_q) fp32 -- the
 *   reference's FA2 split-kv buffers -- and counters = 2 unsigned per (128-row tile, kv head, batch), zeroed once
 *   by the caller.  Given scratch, the head_dim-256 kernel may run more CTAs than (tiles x splits): the grid
 *   (tiles x kv heads x batch x splits) must then fit the device in one wave, else -2 is returned.  When four times
 *   that grid fits as well, every (tile, split) is cut into four head-dim parts, and the kv splits of a part
 *   exchange their partials (a) as one thread-block cluster through distributed shared memory -- scratch and counters
 *   stay untouched -- when the device can hold all those clusters at once (asked from the occupancy API once per
 *   device; with a last tile of at most 32 rows that tile may run in two parts instead to make them fit), else
 *   (b) through the scratch, published with an arrival counter per tile.  (a) and (b) give the same bits.
 *   flags: bit 0 = programmatic dependent launch; bit 1 = keep the single-tile kernel; head_dim 256 with scratch:
 *   bit 2 = one CTA per (tile, split) instead of four head-dim parts, bit 3 = always (b). */
int frt_b200_attention_fwd_bf16(const void* Q, const void* K, const void* V, void* O, void* O_fp8,
                                const float* out_scale, float* lse, const int* seqused_k, int batch, int seqlen_q,
                                int seqlen_k, int num_heads_q, int num_heads_kv, int head_dim,
                                const long long* q_strides, const long long* k_strides, const long long* v_strides,
                                const long long* o_strides, float softmax_scale, int kv_splits, int kv_static_rows,
                                float* o_accum, float* lse_accum, void* counters, int flags, void* stream);
/* Attention with split KV for callers that cannot allocate device memory where they call it (a control loop with a
 * frozen memory map, a plugin inside another runtime's captured or pooled region, a host that only hands out fixed
 * buffers).  This entry point has no counterpart in the reference.  Same operation and arguments as
 * frt_b200_attention_fwd_bf16 minus the scratch pointers: the partials go to a fixed array inside the library
 * (about 4.2 MB of device memory on every GPU that loads it, held until the process exits).
 * Limits: kv_splits <= 8, batch * num_heads_q * seqlen_q <= 512, head_dim <= 256, at most 64 (row tile, kv head,
 * batch) triples; beyond them the call returns -4 and launches nothing.  It allocates and frees nothing.
 * The first call on each device fetches the array's device address and clears its arrival counters with a memset
 * on the caller's stream -- make that call before any stream capture (inside one it is refused with -1).  All calls share the one array and it keeps the last call's
 * contents; calls whose kernels may run at the same time (two streams, parallel graph branches) race on it. */
int frt_b200_attention_fwd_bf16_static_scratch(const void* Q, const void* K, const void* V, void* O, void* O_fp8,
                                               const float* out_scale, float* lse, const int* seqused_k, int batch,
                                               int seqlen_q, int seqlen_k, int num_heads_q, int num_heads_kv,
                                               int head_dim, const long long* q_strides, const long long* k_strides,
                                               const long long* v_strides, const long long* o_strides,
                                               float softmax_scale, int kv_splits, int kv_static_rows, int flags,
                                               void* stream);
/* Status word of the attention kernels (0 = no bounded wait gave up); synchronises the device. */
int frt_b200_attention_status(int reset);
/* The status words of the GEMM, attention and one-launch loop kernels copied to out3[0..2] (device ints) by a kernel in
 * stream order (no counterpart in the reference, whose kernels have no bounded waits): a captured graph can return them
 * with its results instead of the host calling the three blocking status readers after every replay.  reset != 0
 * clears the words after the copy.  flags bit 0: programmatic dependent launch. */
int frt_b200_status_words_async(int* out3, int reset, int flags, void* stream);
/* Diagnostics, no counterpart in the reference: device-timer (%globaltimer, ns) phase stamps of the last 8 launches of
 * the token-major small-M GEMM (gemm_host: 8 launches x 160 CTAs x 16 stamps) and of the head_dim-256 attention kernel
 * (attn_host: 8 x 128 x 16); either pointer may be NULL.  Recorded only by a library built with -DFRT_PHASE_STAMPS
 * (FRT_NVCC_EXTRA=-DFRT_PHASE_STAMPS python -m flashrt_b200._build --force); a regular build returns -2.
 * reset != 0 restarts the launch slots and clears the stamps after copying them out.  Synchronises the device. */
int frt_b200_phase_stamps_read(unsigned long long* gemm_host, unsigned long long* attn_host, int reset);

/* ---------------------------------------------------------------- video-DiT (Wan-shape) fused producers
 * ada_layer_norm_fp8                 csrc/bindings.cpp:3482-3495 -> csrc/quantize/ada_layer_norm_fp8.cu:58-147
 * ada_layer_norm_bf16[_per_token]    csrc/bindings.cpp:2802-2816 -> csrc/kernels/dit_bf16.cu:151-278
 * layer_norm                         csrc/bindings.cpp:879-885   -> csrc/kernels/norm.cu:113-162
 *   y = (x - mean) * inv_std  [* weight + bias]  [* (1 + scale) + shift], statistics over `dim` per row, eps inside
 *   the square root; scale / shift rows at + r * mod_stride (0 = one shared (dim,) row); weight / bias (dim,).
 *   out_fp8 != NULL: e4m3(clamp(bf16(y) * (1 / *d_scale), +-448)) (the value is rounded through bf16 first, as the
 *   reference does); otherwise out_bf16 = bf16(y).  Exactly one of out_fp8 / out_bf16.  dim % 8 == 0, dim <= 8192. */
int frt_b200_layer_norm(const void* x, const void* weight, const void* bias, const void* scale, const void* shift,
                        long long mod_stride, void* out_fp8, void* out_bf16, const float* d_scale, int rows, int dim,
                        float eps, int flags, void* stream);
/* qkv_split_norm_rope_bf16           csrc/bindings.cpp:3574 -> csrc/quantize/qkv_split_norm_rope_bf16.cu:16-140
 *   packed_qkv (B*L, 3*dim) bf16 = [q | k | v], dim = N * D_h.  q, k: RMSNorm over the full width dim with weights
 *   norm_q_w / norm_k_w, then complex pairs (2c, 2c+1) of every head multiplied by freqs_re/im[t, c] (fp32,
 *   (>= seq_len, D_h/2)); rows with t = row % L >= seq_len are normalised but not rotated.  V stays in packed_qkv.
 *   ext_ssq_q / ext_ssq_k (rows,) fp32 + full_dim: optional precomputed sums of squares over the FULL model width
 *   (tensor parallelism: N is then the local head count); NULL = reduce over the N * D_h columns given. */
int frt_b200_qkv_split_norm_rope(const void* packed_qkv, const void* norm_q_w, const void* norm_k_w,
                                 const float* freqs_re, const float* freqs_im, void* q_out, void* k_out, int B, int L,
                                 int N, int D_h, int seq_len, float eps, const float* ext_ssq_q,
                                 const float* ext_ssq_k, int full_dim, int flags, void* stream);
/* Helpers for the same norms under tensor parallelism (they have no counterpart in the reference, which has no
 * multi-GPU path): a rank holds only its heads' columns, so the per-row sums of squares are formed per rank
 * (frt_b200_row_sumsq), summed across ranks by the caller (an all-reduce of one float per row) and handed back
 * through ext_ssq_q / ext_ssq_k + full_dim above, or to frt_b200_rms_norm_ext for a plain RMSNorm of a slice. */
int frt_b200_row_sumsq(const void* x, long long row_stride, int col0, int ncols, float* out, long long rows, int flags,
                       void* stream);
/* RMSNorm of a column slice with the full-width sum of squares supplied (no counterpart in the reference). */
int frt_b200_rms_norm_ext(const void* x, long long x_stride, const void* weight, const float* ssq, void* out,
                          long long out_stride, long long rows, int dim, int full_dim, float eps, int flags,
                          void* stream);
/* bias_gelu_quantize_fp8_static_bf16 csrc/bindings.cpp:3427-3440 -> csrc/quantize/bias_gelu_quantize_fp8.cu:24-49
 *   out (M, N) e4m3 = clamp(gelu_tanh(in + bias) * (1 / *d_scale), +-448); bias (N,) or NULL; N % 8 == 0. */
int frt_b200_bias_gelu_quantize_fp8(const void* in_bf16, const void* bias, void* out_fp8, const float* d_scale,
                                    long long M, int N, int flags, void* stream);
/* bias_gate_mul_residual_bf16        csrc/bindings.cpp:1122-1131 -> csrc/kernels/elementwise.cu:1648-1683
 *   residual (rows, dim) += (x + bias) * gate; gate rows at + r * gate_stride (0 = shared row); bias (dim,) or NULL. */
int frt_b200_bias_gate_mul_residual(void* residual, const void* x, const void* bias, const void* gate,
                                    long long gate_stride, long long rows, int dim, int flags, void* stream);
/* add_bias_bf16                      csrc/bindings.cpp:2818-2826:  x (rows, dim) += bias (dim,) */
int frt_b200_add_bias(void* x, const void* bias, long long rows, int dim, int flags, void* stream);
/* adaln_modulation6_bf16             csrc/bindings.cpp:3705-3726 -> csrc/kernels/elementwise.cu:603-645
 *   out_j (B, S, D) bf16 = adaln_params (B, S, 6, D) fp32 [:, :, j, :] + layer_modulation (6, D) fp32 [j], j = 0..5 */
int frt_b200_adaln_modulation6(const float* adaln_params, const float* layer_modulation, void* out0, void* out1,
                               void* out2, void* out3, void* out4, void* out5, int B, int S, int D, int flags,
                               void* stream);

/* fp8 GEMM (GemmRunner::fp8_nt_dev, csrc/bindings.cpp:717-727) + gate_residual_ada_norm_fp8
 * (csrc/bindings.cpp:1144-1162 -> csrc/kernels/fusion.cu:15-81) in one launch, M <= 64, N = 128 .. 1024 (N % 128 == 0):
 *   o = bf16(sa * sb * A . W^T); residual <- bf16(residual + o * gate); out8 = e4m3 of the adaRMS-modulated row
 *   (unit norm weight; gate (N,), style = [scale (N) | shift (N)] shared by all rows) with scale *d_out_scale.
 * One thread-block cluster holds every 128-column tile of the row (x its split-K halves), so the row's sum of
 * squares is exchanged through distributed shared memory.  Same rounding points as the two separate calls; the sum of
 * squares is accumulated in a different fixed order, so single FP8 codes may differ in the last place. */
int frt_b200_gemm_fp8_nt_gate_res_norm_fp8(const void* A, const void* W, int M, int N, int K, const float* d_scale_a,
                                           const float* d_scale_b, void* residual, const void* gate, const void* style,
                                           void* out8, const float* d_out_scale, float eps, int splits, int flags,
                                           void* stream);
/* The decoder's projections with the norm kernel between them folded in (token-major kernel, M <= 128, K % 128 == 0).
 *
 * Row-parallel projection + first pass of gate_residual_ada_norm_fp8 (csrc/bindings.cpp:1144-1162 ->
 * csrc/kernels/fusion.cu:41-47):  o = bf16(sa * sb * A . W^T); residual (M, N) <- bf16(residual + o * gate), gate (N,)
 * shared by all rows; stats_out[tile][m] (row pitch 128 floats; may be NULL) = sum over the tile's features of the
 * squares of the unrounded updated residual.  *stat_tiles (host, may be NULL) = rows of stats_out written.
 * N % 64 == 0. */
int frt_b200_gemm_fp8_nt_gate_residual(const void* A, const void* W, int M, int N, int K, const float* d_scale_a,
                                       const float* d_scale_b, void* residual, const void* gate, float* stats_out,
                                       int* stat_tiles, int splits, int flags, void* stream);
/* The same launch, also leaving the NEXT projection's FP8 operand without the 1 / rms factor of the norm between them
 * (second pass of gate_residual_ada_norm_fp8, csrc/kernels/fusion.cu:48-81, with the quantisation point moved in front of
 * the row scale):  q8_out[m][n] = e4m3(clamp(bf16(residual[m][n]) * (1 + next_scale[n]) / *d_q8_scale, +-448)),
 * next_scale = scale third of the next norm's style row (N bf16).  q8_out NULL: exactly the entry point above. */
int frt_b200_gemm_fp8_nt_gate_residual_q8(const void* A, const void* W, int M, int N, int K, const float* d_scale_a,
                                          const float* d_scale_b, void* residual, const void* gate, float* stats_out,
                                          int* stat_tiles, const void* next_scale, void* q8_out,
                                          const float* d_q8_scale, int splits, int flags, void* stream);
/* Projections of such an operand (GemmRunner::fp8_nt_dev, csrc/bindings.cpp:717-727, with the row scale and the shift of
 * the norm applied in the finish):  y[m][n] = bf16(sa * sb * (A . W^T)[m][n] * rms[m] + col_term[n]),
 *   rms[m] = 1 / sqrt(sum_t stats_in[t][m] / K + eps), t = 0 .. n_stat-1 in order (the statistics rows written above),
 *   col_term (fp32, one entry per output feature) = W . shift, which the caller computes once per (step, layer);
 * followed by the epilogue of frt_b200_gemm_fp8_nt_rope_split (qkv_split_rope, csrc/kernels/rope.cu:135-277) or of
 * frt_b200_gemm_fp8_nt_geglu_fp8 (gate_geglu_merged_fp8, csrc/kernels/activation.cu:249-279; col_term has 2 * half
 * entries, gate rows first).  M <= 128, K % 128 == 0. */
int frt_b200_gemm_fp8_nt_rope_split_rowscale(const void* A, const void* W, int M, int K, const float* d_scale_a,
                                             const float* d_scale_b, const float* stats_in, int n_stat, float eps,
                                             const float* col_term, const void* rope, void* Q, void* Kout, void* Vout,
                                             const int* devpos, int q_dim, int k_dim, int v_dim, int head_dim,
                                             int splits, int flags, void* stream);
/* gate|up form of the row-scaled projection: gate_geglu_merged_fp8 (csrc/kernels/activation.cu:249-279) behind it. */
int frt_b200_gemm_fp8_nt_geglu_fp8_rowscale(const void* A, const void* W, void* out8, int M, int half, int K,
                                            const float* d_scale_a, const float* d_scale_b, const float* stats_in,
                                            int n_stat, float eps, const float* col_term, const float* d_out_scale,
                                            int splits, int flags, void* stream);
/* Second pass of gate_residual_ada_norm_fp8 (csrc/kernels/fusion.cu:48-81) produced inside the next projection:
 *   rms[m] = 1 / sqrt(sum_t stats_in[t][m] / K + eps), t = 0 .. n_stat-1 in order;
 *   a = e4m3(clamp(((x * rms) * (1 + scale) + shift) / *d_scale_a, +-448)), style = [scale (K) | shift (K)] one bf16 row
 *   (unit norm weight), x (M, K) bf16;
 * then GemmRunner::fp8_nt_dev and the epilogue of frt_b200_gemm_fp8_nt_rope_split / _geglu_fp8.  K / splits must
 * be 128, 256 or 512 bytes (the K-slice stays resident in shared memory). */
int frt_b200_norm_gemm_fp8_nt_rope_split(const void* x, const float* stats_in, int n_stat, const void* style, float eps,
                                         const void* W, int M, int K, const float* d_scale_a, const float* d_scale_b,
                                         const void* rope, void* Q, void* Kout, void* Vout, const int* devpos,
                                         int q_dim, int k_dim, int v_dim, int head_dim, int splits, int flags,
                                         void* stream);
/* The same producer (csrc/kernels/fusion.cu:48-81) in front of the gate|up projection, gate_geglu_merged_fp8
 * (csrc/kernels/activation.cu:249-279) behind it; half % 64 == 0. */
int frt_b200_norm_gemm_fp8_nt_geglu_fp8(const void* x, const float* stats_in, int n_stat, const void* style, float eps,
                                        const void* W, void* out8, int M, int half, int K, const float* d_scale_a,
                                        const float* d_scale_b, const float* d_out_scale, int splits, int flags,
                                        void* stream);
/* fp8 GEMM (GemmRunner::fp8_nt_dev, csrc/bindings.cpp:717-727) + bias_gelu_quantize_fp8_static_bf16
 * (csrc/bindings.cpp:3427-3440 -> csrc/quantize/bias_gelu_quantize_fp8.cu:24-49) in one launch, M > 256, N >= 128:
 *   out8 (M, N) e4m3 = clamp(gelu_tanh(bf16(sa * sb * A . W^T) + bias) * (1 / *d_out_scale), +-448)
 * byte-identical to the two separate calls.  flags bit 7: GELU through the hardware tanh (tanh.approx.f32, 2^-11
 * relative) -- at K = 3072 the exact form (about 36 instructions per value on 8 epilogue warps) takes longer than the
 * MMAs of the tile; codes then differ from the exact form by single last-place flips. */
int frt_b200_gemm_fp8_nt_bias_gelu_fp8(const void* A, const void* W, void* out8, int M, int N, int K,
                                       const float* d_scale_a, const float* d_scale_b, const void* bias,
                                       const float* d_out_scale, int flags, void* stream);

/* ---------------------------------------------------------------- NVFP4 (e2m1 x 16-element blocks x unsigned-E4M3 scales)
 * Packed data: two elements per byte, low nibble = even element, row = K / 2 bytes.
 * Scales: one byte per 16 elements, stored in 512-byte atoms of 128 rows x 4 blocks --
 *   offset(row, blk) = ((row / 128) * ceil(K / 64) + blk / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + blk % 4
 * (csrc/kernels/quantize.cu:476-486; CUTLASS Sm1xxBlockScaledConfig<16> at csrc/quantize/quantize_fp4_sfa.cu:191-206).
 * Scale buffers are zero-filled once by the caller: padding entries are never written (flash_rt/executors/fp4_utils.py:78-86).
 * `family` selects the reference's quantiser convention:
 *   0 = flash_rt_kernels  (scale = smallest UE4M3 >= amax / 6, thresholds '<')   csrc/kernels/nvfp4_convert.cuh:31-105
 *   1 = flash_rt_fp4      (scale = RN-even E4M3 of max(amax / 6, 1e-12), '<=')   csrc/quantize/quantize_fp4_sfa.cu:31-109
 * The reference's quantisers carry no FP32 global scale; here an optional device float g divides the input first
 * and the caller folds g into the GEMM's alpha. */

/* sfa_size_bytes               csrc/fp4_bindings.cpp:349-352  (*out_bytes is a host pointer) */
int frt_b200_nvfp4_sf_bytes(long long rows, int K, long long* out_bytes);
/* quantize_bf16_to_nvfp4_swizzled        csrc/bindings.cpp:1277-1285 -> csrc/kernels/quantize.cu:450-526   (family 0)
 * quantize_fp4_dynamic_sfa_bf16_vec      csrc/fp4_bindings.cpp:1124-1137                                    (family 1)
 * quantize_fp4_dynamic_sfa_fp16[_vec]    csrc/fp4_bindings.cpp:299-333 -> csrc/quantize/quantize_fp4_sfa.cu:63-109
 *   in (rows, D) bf16 -> packed (rows, D / 2), sf.  D % 16 == 0.  The same call quantises weights (is_sfb). */
int frt_b200_quantize_nvfp4(const void* in, void* packed, void* sf, long long rows, int D, int family,
                            const float* d_global_scale, int flags, void* stream);
/* gate_geglu_fp4_sfa[_v2,_vec]_fp16      csrc/fp4_bindings.cpp:711-753 -> csrc/fused_fp4/silu_mul_fp4_sfa_vec.cu:50-107
 *   merged (rows, 2H) bf16 = [gate | up] -> NVFP4 of the fp32 product gelu_tanh(gate) * up.  H % 16 == 0. */
int frt_b200_geglu_nvfp4(const void* merged, void* packed, void* sf, int rows, int H, int family, int flags,
                         void* stream);
/* pi05_adarms_fp4_sfa[_native]_fp16              csrc/fp4_bindings.cpp:547-570,602-625
 * pi05_gate_res_adarms_fp4_sfa[_native]_fp16     csrc/fp4_bindings.cpp:572-600,627-657 -> csrc/fused_fp4/norm_silu_fp4_sfa.cu:147-268
 * rms_norm_fp4_sfa_fp16, residual_add_rms_norm_fp4_sfa[_v2]_fp16   csrc/fp4_bindings.cpp:501-545
 * rms_norm_to_nvfp4_swizzled_bf16, residual_add_rms_norm_to_nvfp4_swizzled_bf16   csrc/bindings.cpp:1475-1590 -> csrc/kernels/quantize.cu:1656-1755,2114-2226
 *   the fused norm of frt_b200_norm_fp8 with an NVFP4 result: the modulated value is rounded to bf16 and then
 *   block-quantised, i.e. byte-identical to frt_b200_norm_bf16 followed by frt_b200_quantize_nvfp4.
 *   Any row count and any dim % 16 == 0 (the reference's pi05 entries accept seq_len 10, dim 1024 only). */
int frt_b200_norm_nvfp4(void* residual, const void* x, const void* gate_in, long long gate_in_stride,
                        const void* weight, const void* style, long long style_stride, void* out_packed,
                        void* out_sf, void* gate_out, int rows, int dim, float eps, int family, int flags,
                        void* stream);
/* cutlass_fp4_gemm_variant, cutlass_fp4_sq_fp16   csrc/fp4_bindings.cpp:85-99,355-370 -> csrc/gemm/fp4/cutlass_fp4_gemm.cu
 * cutlass_fp4_gemm_bias_bf16                       csrc/fp4_bindings.cpp:1139-1155
 *   D(M,N) bf16 = alpha * (*d_alpha) * (A.SFA)(M,K) . (W.SFW)(N,K)^T + bias;  d_alpha, bias optional;  K % 256 == 0;
 *   beta is not supported (the decoder path calls with beta = 0).  One kernel for every variant index. */
int frt_b200_gemm_nvfp4_nt(const void* A, const void* SFA, const void* W, const void* SFW, void* D, int M, int N,
                           int K, float alpha, const float* d_alpha, const void* bias, int splits, int flags,
                           void* stream);
/* cutlass_fp4_gemm_variant (csrc/fp4_bindings.cpp:355-370) + qkv_split_rope_kvcache_fp16[_devpos,_vec] fused, the pair
 * called at flash_rt/models/pi05/pipeline_thor.py:366-385:
 *   the NVFP4 form of frt_b200_gemm_fp8_nt_rope_split. */
int frt_b200_gemm_nvfp4_nt_rope_split(const void* A, const void* SFA, const void* W, const void* SFW, int M, int K,
                                      float alpha, const void* rope, void* Q, void* Kout, void* Vout,
                                      const int* devpos, int q_dim, int k_dim, int v_dim, int head_dim, int splits,
                                      int flags, void* stream);

/* ---------------------------------------------------------------- small bf16 projections, copies, queries
 * GemmRunner::bf16_nn          csrc/bindings.cpp:662-667  (action in/out projections 32 <-> 1024)
 *   D(M,N) = A(M,K) . B(K,N) (+ bias(N)) (+ D when accumulate != 0); B bf16 row-major (K,N).
 *   io bit0: A is fp32 (each element rounded to bf16 on load) instead of bf16; io bit1: D is fp32 instead of
 *   bf16 (lets the Euler state x <- x + dt*v stay in fp32 across the denoise steps). */
int frt_b200_gemm_bf16_nn_small(const void* A, const void* B, void* D, const void* bias, int M, int N, int K,
                                int accumulate, int io, int flags, void* stream);
/* The launches between two Euler steps of Pi05Pipeline.transformer_decoder (flash_rt/models/pi05/pipeline_rtx.py:1451-1504)
 * as one, one CTA per token: final adaRMS (bf16) of the step that ends, action out-projection (GemmRunner::bf16_nn,
 * csrc/bindings.cpp:662-667) accumulated into the fp32 noise, action in-projection of the step that begins, first
 * adaRMS -> FP8 of layer 0 (ada_rms_norm_style_fp8).  x (rows, dim) bf16 in/out; noise (rows, 32) fp32 in/out; style rows
 * = [scale (dim) | shift (dim) | ...] bf16; w_out (dim, 32), w_in (32, dim), biases bf16.  style_prev NULL: second half
 * only (first step); style_next NULL: first half only (last step).  The same bits as the four separate launches.
 * action_dim == 32, dim % 256 == 0, dim <= 2048. */
int frt_b200_step_boundary(void* x, float* noise, const void* style_prev, const void* w_out, const void* b_out,
                           const void* w_in, const void* b_in, const void* style_next, void* act8,
                           const float* d_act_scale, int rows, int dim, int action_dim, float eps, int flags,
                           void* stream);
/* gpu_copy                     csrc/bindings.cpp:2533-2537  (device-to-device, async on stream) */
int frt_b200_copy(void* dst, const void* src, long long nbytes, void* stream);
/* get_sm_version               csrc/bindings.cpp:2447-2453  (returns major*10+minor, 100 on B200) */
int frt_b200_sm_version(void);

/* cfg_combine_into_residual    csrc/bindings.cpp:1133-1141 -> csrc/kernels/elementwise.cu:2299-2338
 *   residual[i] += v_uncond[i] + beta * (v_cond[i] - v_uncond[i]), i < n (classifier-free guidance, Eq. 13 of the
 *   reference's flash_rt/refs/pi05_cfg_reference.py:8-15).  f32 = 0: bf16 arrays as in the reference; f32 = 1: fp32
 *   arrays (the Euler state of this library).  n % 2 == 0. */
int frt_b200_cfg_combine_into_residual(void* residual, const void* v_cond, const void* v_uncond, float beta,
                                       long long n, int f32, int flags, void* stream);

/* ---------------------------------------------------------------- the whole denoise loop as one persistent kernel
 * Pi05Pipeline.transformer_decoder / _decoder_layer   flash_rt/models/pi05/pipeline_rtx.py:1451-1749
 * (the reference runs this loop as ~2000 launches inside one CUDA graph; its kernel library has no counterpart in the
 * reference for a single-launch form: no counterpart in the reference).  Same arithmetic as the operator-by-operator
 * composition of this library (FP8 E4M3 projections with static per-site activation scales, bf16 residual stream and
 * attention, fp32 Euler state), batch 1, S <= 64 action tokens, decoder width 1024 / hidden 4096 / 8 x 256 query
 * heads over one KV head.  One cooperative launch of one CTA per SM; phases are separated by grid-wide barriers with
 * bounded waits (see frt_b200_expert_loop_status).
 *
 * All members are device pointers except `workspace_bytes` and the ints.  Weights are E4M3 bytes, (layers, N, K) with
 * K contiguous: w_qkv N = 2560 (Q rows and K rows interleaved for adjacent-pair RoPE), w_o N = 1024 K = 2048,
 * w_gu N = 8192 (gate rows, then up rows), w_d N = 1024 K = 4096; ws_* (layers,) fp32 weight scales;
 * act_scale (steps, layers, 4) fp32, sites qkv / o / gate-up / down; style_attn, style_ffn (steps, layers, 3072) and
 * style_final (steps, 3072) bf16 rows [scale | shift | gate]; rope (S, 256) bf16 [cos0, sin0, cos1, sin1, ...];
 * in_w (32, 1024), in_b (1024), out_w (1024, 32) and out_b (32) bf16, the out-projection pre-scaled by -1 / steps;
 * k_cache / v_cache (layers, kv_rows, 256) bf16 holding the prefix in rows [0, prefix_len) -- rows
 * [prefix_len, prefix_len + S) are overwritten; noise (S, 32) fp32 in/out.  workspace: frt_b200_expert_loop_workspace_bytes
 * bytes, 256-byte aligned, contents arbitrary. */
typedef struct frt_b200_expert_loop_args {
    const void *w_qkv, *w_o, *w_gu, *w_d;
    const void *ws_qkv, *ws_o, *ws_gu, *ws_d;
    const void *act_scale;
    const void *style_attn, *style_ffn, *style_final;
    const void *rope;
    const void *in_w, *in_b, *out_w, *out_b;
    void *k_cache, *v_cache;
    void *noise;
    void *workspace;
    long long workspace_bytes;
    int steps, layers, S, prefix_len, kv_rows;
} frt_b200_expert_loop_args;
/* host_args: HOST pointer to a frt_b200_expert_loop_args, args_bytes = sizeof of it (checked). */
int frt_b200_expert_loop_fp8(const void* host_args, int args_bytes, void* stream);
/* no counterpart in the reference: size of the loop kernel's scratch for S action tokens behind prefix_len keys */
int frt_b200_expert_loop_workspace_bytes(int S, int prefix_len, long long* out_bytes);
/* no counterpart in the reference: the loop kernel's static work assignment, evaluated on the HOST (no GPU needed).
 * Every unit of a phase (0 QKV: 20 units, 1 output projection: 16, 2 gate|up: 64, 3 down: 32, 4 attention:
 * att_units) of block gl = step * layers + layer belongs to exactly one CTA of the grid of G; *unit_out (host) = the
 * unit of CTA `cta`, or -1.  The CTAs of a block's attention units own none of its QKV units (their operand space
 * receives the prefetched K/V chunk while the QKV phase runs). */
int frt_b200_expert_loop_schedule(int G, int cta, int gl, int phase, int att_units, int* unit_out);
/* Status word of the loop kernel (0 = no bounded wait gave up; else code | CTA << 8, code 1 weight producer, 2 MMA
 * issuer, 3 worker, 4 grid barrier); synchronises the device. */
int frt_b200_expert_loop_status(int reset);

/* number of SMs of the current device (grid sizing) */
int frt_b200_device_sm_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FLASHRT_B200_H */
