/*
 * antares_b200 — C ABI of the B200 (sm_100a) kernel library that stands in for what the
 * Antares/AutoRT CUDA backend would generate for the Llama-2-7B int4 operator path.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the parameter name ends in `_host`;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - fp16 tensors are IEEE binary16; `dtype` is AB200_F16 or AB200_F32 and names the dtype
 *     of activations, scales and results together (the reference declares them together,
 *     samples/05_llama2_7b_int4.py:133,139);
 *   - functions return AB200_OK (0) or an error code; ab200_last_error() gives the text.
 *     Nothing calls exit() (the reference's CHECK_OK does, graph_evaluator/execute_module.hpp:40);
 *   - no function allocates device memory or synchronises the device unless it says so;
 *     all are legal inside CUDA stream capture unless they say otherwise.
 *
 * Each entry point names the reference interface it replaces (paths relative to the
 * reference project root).
 */
#ifndef ANTARES_B200_H_
#define ANTARES_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  AB200_OK = 0,
  AB200_EINVAL = 1,       /* bad shape / alignment / null pointer */
  AB200_ECUDA = 2,        /* a CUDA runtime call failed */
  AB200_EUNSUPPORTED = 3, /* valid request outside the built kernel family */
  AB200_ETIMEOUT = 4      /* a bounded device-side wait ran out */
};

enum { AB200_F16 = 0, AB200_F32 = 1 };

/* Text of the last error on the calling thread ("" if none). */
const char *ab200_last_error(void);
int ab200_abi_version(void);

/* Reads and clears the device-side status word.  Kernels that wait on barriers bound every
 * wait; a wait that ran out leaves a site code here instead of hanging (the reference has a
 * host watchdog that exits the process, graph_evaluator/run_graph.cpp:59-73).  Returns
 * AB200_ETIMEOUT if the word was set.  Synchronises the device; not legal during capture. */
int ab200_kernel_status(int *status_host);

/* Tuning knobs, the counterpart of the `config=` hints of autort.export
 * (samples/05_llama2_7b_int4.py:139).  Names: "gemv_cluster" (0 = auto, 1/2/4/8 K-slices per
 * column tile), "gemv_impl" (0 auto, 1 scalar pipes only, 2 cluster warp-MMA, 3 persistent warp-MMA,
 * 4 TMA ring + warp-MMA, 5 bulk-copy ring for batch 1, 6 TMA ring with streamed activations for batch 5-16,
 * 7 tcgen05 MMA with the dequantised weights written to tensor memory),
 * "gemv_depth" (0 auto, 2..6 units of prefetch per warp in the cluster warp-MMA kernel),
 * "ring_depth" (0 auto, even 2..16: 8 KiB stages per CTA in the bulk-copy ring kernel).
 * "comm_wait_polls": polls after which the push all-reduce gives up waiting for a peer.
 * "pdl" (0 off, 1 default, 2): launch kernels with programmatic dependent launch so that a
 * kernel's weight prefetch overlaps the tail of its predecessor in the stream; every such kernel
 * executes griddepcontrol.wait before it touches anything an earlier kernel wrote.  1 releases
 * the dependent kernel at kernel start, 2 after the GEMV's streaming loop.  Process-wide; host call. */
int ab200_set_option(const char *name, int value);

/* Device property probe; replaces engine/cuda_properties.cc:35-52 (which prints
 * key/value pairs for the code generator).  Fills 8 ints:
 * [0] SM count, [1] max shared memory per block (opt-in, bytes), [2] L2 bytes,
 * [3] SM clock kHz, [4] memory clock kHz, [5] memory bus width bits,
 * [6] compute capability major*10+minor, [7] max threads per block.
 * Host call; touches no stream. */
int ab200_device_info(int device, int *out8_host);

/* ---- int4 packing ------------------------------------------------------------------------
 * Layout (GPTQ, as loaded by samples/05_llama2_7b_int4.py:24-28): qweight int32 [K/8, N],
 * N contiguous; word (r, n) holds the eight 4-bit values of rows 8r..8r+7 of column n,
 * lowest nibble = lowest row. */

/* q_out u8 [K, N] = (qweight[S/8, N] >> (S%8*4)) & 15  — IR statement 1,
 * samples/05_llama2_7b_int4.py:136. */
int ab200_w4_unpack(const int32_t *qweight, int K, int N, uint8_t *q_out, void *stream);

/* Inverse of ab200_w4_unpack (no reference counterpart: the sample loads packed weights). */
int ab200_w4_pack(const uint8_t *q, int K, int N, int32_t *qweight_out, void *stream);

/* w_out [K, N] = scales[S/group, N] * (q - 8) in `dtype` — IR statements 1-2,
 * samples/05_llama2_7b_int4.py:136-137.  Bit-exact with the reference's CPU backend. */
int ab200_w4_dequant(const int32_t *qweight, const void *scales, int K, int N, int group,
                     int dtype, void *w_out, void *stream);

/* ---- W4A16 contraction --------------------------------------------------------------------
 * out[M, N] = sum_S x[M, S] * (scales[S/group, N] * (q[S, N] - 8)), fp32 accumulation —
 * the exported op `my_custom_fn` of samples/05_llama2_7b_int4.py:135-144 (`matmul_dequat`).
 * This is the decode path (M <= 16): weights are streamed once from HBM.
 * Constraints: K % 32 == 0, group % 32 == 0, K % group == 0, N % 4 == 0, 1 <= M <= 16,
 * pointers 16-byte aligned. */
int ab200_w4a16_gemv(const void *x, const int32_t *qweight, const void *scales, void *out, int M,
                     int K, int N, int group, int dtype, void *stream);

/* Same contraction with the decode step's residual update fused into the epilogue:
 *   resid_f32[M, N] += fp16_round(out[M, N])        (x, scales fp16)
 * replaces `xb = matmul_dequat(...); x = x + xb`, samples/05_llama2_7b_int4.py:167-168,172-173. */
int ab200_w4a16_gemv_residual(const void *x, const int32_t *qweight, const void *scales,
                              float *resid_f32, int M, int K, int N, int group, void *stream);

/* Same contraction, fp16 inputs, unrounded fp32 result: the per-rank partial sum of a
 * row-parallel projection, to be all-reduced and then added with ab200_residual_add.
 * (Tensor-parallel decode has no counterpart in the reference: its samples are single-device.) */
int ab200_w4a16_gemv_f32out(const void *x, const int32_t *qweight, const void *scales,
                            float *out_f32, int M, int K, int N, int group, void *stream);

/* The decode step's fused form of the same contraction (fp16 weights path), one launch:
 *   prologue  0: x is fp16 [M, K]
 *             1: x is the fp32 residual stream [M, K]; the kernel applies RMSNorm with
 *                norm_weight_f16 [K] and eps (replaces rmsnorm + matmul_dequat, lines 150-152,169-171)
 *             2: x is fp16 [M, 2K] = gate | up; the kernel feeds silu(gate) * up (lines 171-172)
 *   epilogue  0: out fp16 [M, N];  1: out fp32 [M, N] += fp16_round(result);  2: out fp32 [M, N]
 * workspace: device scratch of at least ab200_w4a16_gemv_workspace_bytes(M, K, N) bytes, 16-byte
 * aligned, whose first 64 KiB are zero before the first use (the kernel leaves them zero); NULL =
 * use the library's own per-device scratch.  Calls sharing a workspace must not overlap on the
 * GPU.  Two kernels use scratch: the persistent kernel (option gemv_impl=3) and the kernel that
 * streams the activations through the TMA ring (the default for 9-16 rows at N >= 8192 and for
 * 5-8 rows at N >= 16384, which stages the re-ordered activations there).  The library scratch is
 * allocated (cudaMalloc, for the persistent kernel also a device synchronise) by the first call
 * that needs it on a device, also from ab200_w4a16_gemv / _residual / _f32out: make that first
 * call outside stream capture, and do not let two such calls overlap on different streams. */
int ab200_w4a16_gemv_fused(const void *x, int prologue, const void *norm_weight_f16, float eps,
                           const int32_t *qweight, const void *scales, void *out, int epilogue,
                           int M, int K, int N, int group, void *workspace, size_t workspace_bytes,
                           void *stream);
size_t ab200_w4a16_gemv_workspace_bytes(int M, int K, int N);

/* ab200_w4a16_gemv_fused on weights stored TILE-MAJOR, the layout this library prefers in HBM:
 *   qweight_tiled int32 [N/128][K/8][128]   (tile t, packed row r, column c  <-  qweight[r][128 t + c])
 *   scales_tiled  fp16  [N/128][K/group][128]
 * so that the weights one CTA streams are one contiguous range (the reference layout [K/8, N]
 * gives it 512-byte pieces 4 N bytes apart).  Same arithmetic, same results bit for bit.  N must
 * be a multiple of 128, batch 1..4, fp16.  antares_b200.packing.tile_weights() produces the
 * layout from the reference's.  No counterpart in the reference (its layout is fixed by the
 * checkpoint format, samples/05_llama2_7b_int4.py:22-29). */
int ab200_w4a16_gemv_tiled(const void *x, int prologue, const void *norm_weight_f16, float eps,
                           const int32_t *qweight_tiled, const void *scales_tiled, void *out,
                           int epilogue, int M, int K, int N, int group, void *stream);

/* ab200_w4a16_gemv for callers that may not allocate device memory.  No counterpart in the
 * reference.  Some hosts hand a plugin no way to allocate: an inference server that reserves the
 * whole device for its own memory pool at start-up and forbids driver allocations afterwards
 * (they would fail, or stall every stream while the driver synchronises), or a real-time loop
 * that must never block in the driver.  This entry point computes the same fp16 contraction
 * with the split-K kernel, whose partial sums and tile counters live in a fixed 2 MiB + 64 KiB
 * array inside the library image (each GPU that loads the library holds it until the process
 * exits).  It calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - Limits: fp16 only, K % 128 == 0, x must fit the kernel's shared memory, and the K-slice
 *     partials (slices * M * N * 4 bytes, as ab200_w4a16_gemv_workspace_bytes reports) must fit
 *     the 2 MiB; larger requests return AB200_EINVAL with the sizes in the message.  All four
 *     Llama-2-7B projections fit at batch 1, the three with K = 4096 up to batch 4.
 *   - The first call on each device looks up the array's device address (that device must be
 *     current); make that first call before any stream capture.
 *   - Every call uses the same array, which keeps what the last call left; the counters are
 *     cleared on `stream` before the launch.  Two calls that overlap on the GPU (different
 *     streams, or this and another process-wide user of the array) race: serialise them. */
int ab200_w4a16_gemv_static(const void *x, const int32_t *qweight, const void *scales, void *out,
                            int M, int K, int N, int group, void *stream);

/* x_f32[i] += fp16_round(partial_f32[i]) — the residual update of lines 168,173 applied to an
 * all-reduced partial. */
int ab200_residual_add(float *x_f32, const float *partial_f32, int n, void *stream);

/* Prefill contraction on tensor cores (tcgen05 + TMEM): same arithmetic, any M >= 1 (fp16, K a
 * multiple of 64, group a multiple of 64 dividing K, N a multiple of 8).  Replaces the same
 * exported op called with a leading M axis.  When the problem has fewer 256 x 256 output tiles
 * than half the SMs, K is split over the idle SMs and the partial sums pass through a
 * library-owned per-device scratch (at most 37 MiB), allocated by the first such call on a
 * device: make that call outside stream capture, and do not let two such calls overlap on
 * different streams. */
int ab200_w4a16_gemm(const void *x, const int32_t *qweight, const void *scales, void *out, int M,
                     int K, int N, int group, int dtype, void *stream);

/* ---- elementwise / reduction operators ---------------------------------------------------- */

/* out[i] = 1 - 1 / (1 + exp(x[i])) — README.md:66 (`sigmoid_f32`); dtype F32 or F16. */
int ab200_sigmoid(const void *x, void *out, size_t n, int dtype, void *stream);

/* autort.ops.rmsnorm_f32(x, vsum, weight, extra=[inv_n]) — call site
 * samples/05_llama2_7b_int4.py:128-131: out[i] = x[i] * rsqrt(vsum[0]*inv_n + eps) * weight[i]. */
int ab200_rmsnorm_vsum(const void *x, const float *vsum, const void *weight, void *out, size_t n,
                       float inv_n, float eps, int dtype, void *stream);

/* Row-wise RMSNorm that computes the sum of squares itself (replaces the torch reduction plus
 * the op above, samples/05_llama2_7b_int4.py:128-131).  x [rows, cols] in x_dtype (F16 or
 * F32), weight fp16 [cols], out fp16 [rows, cols]; cols % 8 == 0, cols <= 16384. */
int ab200_rmsnorm(const void *x, int x_dtype, const void *weight_f16, void *out_f16, int rows,
                  int cols, float eps, void *stream);

/* autort.ops.rotary_f32(x.view(H,2,D/2), inv_freq[D], out[H,D], extra=[pos]) — call site
 * samples/05_llama2_7b_int4.py:157-158, batched: x, out [rows, H, D] in dtype; row r is rotated by
 * position pos[r] (int32 device array); inv_freq fp32 [D/2 or D]. Rotate-half convention. */
int ab200_rope(const void *x, const float *inv_freq, const int32_t *pos, void *out, int rows,
               int H, int D, int dtype, void *stream);

/* Row softmax — AntaresIR.md:226.  x, out [rows, cols] in dtype. */
int ab200_softmax(const void *x, void *out, int rows, int cols, int dtype, void *stream);

/* autort.ops.attention_f32(q[H,D], K[S,H,D], V[S,H,D], att_f[1]) — call site
 * samples/05_llama2_7b_int4.py:161-165.  q/K/V/out in dtype (F16 or F32), fp32 math.  The number of cache rows
 * attended is S = *seq_len_dev + seq_len_add (a device int, so a captured graph can be replayed as the
 * sequence grows); kv_stride = elements between consecutive cache rows; D == 128. */
int ab200_attention_decode(const void *q, const void *k_cache, const void *v_cache, void *out,
                           const int32_t *seq_len_dev, int seq_len_add, int max_seq, int H, int D,
                           long kv_stride, float scale, int dtype, void *stream);

/* ---- decode-step glue (replaces torch eager ops in samples/05_llama2_7b_int4.py:146-177) -- */

/* x_f32[d] = embed_f16[token, d], token = *token_dev  (line 147). */
int ab200_embed_lookup(const void *embed_f16, const int32_t *token_dev, float *x_f32, int dim,
                       int vocab, void *stream);

/* Splits the fused projection output vqk[3*Hl*D] (order V, Q, K as in line 27), rotates Q and
 * K at position *pos_dev, writes q_out[Hl*D], and stores K and V into cache row *pos_dev
 * (lines 151-158). */
int ab200_rope_kv_store(const void *vqk_f16, const float *inv_freq, const int32_t *pos_dev,
                        void *q_out_f16, void *k_cache_f16, void *v_cache_f16, int H, int D,
                        long kv_stride, int max_seq, void *stream);

/* The three calls above in one launch: splits vqk (V | Q | K), rotates Q and K at position
 * *pos_dev, stores K and V into cache row *pos_dev and attends over rows 0..*pos_dev (lines
 * 151-165).  Heads are split over several CTAs that merge through distributed shared memory.
 * With programmatic dependent launch on (the default), *pos_dev and the cache rows below it are
 * read before the preceding kernel in the stream has finished: they must come from earlier work
 * (in a decode step they date from earlier steps), not from that kernel. */
int ab200_attention_fused(const void *vqk_f16, const float *inv_freq, const int32_t *pos_dev,
                          void *k_cache_f16, void *v_cache_f16, void *out_f16, int H, int D,
                          long kv_stride, int max_seq, float scale, void *stream);

/* Paged KV cache (the reference keeps one contiguous [seq_len, 4096] cache per layer,
 * samples/05_llama2_7b_int4.py:119-120; a serving host hands out cache rows in pages).  The _paged
 * forms of the three calls that touch the cache take a device table int32[ceil(max_seq /
 * page_rows)], page_rows a power of two: logical cache row s lives in physical row
 * page_table[s / page_rows] * page_rows + s % page_rows of k_cache / v_cache.  max_seq stays the
 * logical length.  The table entries of rows at or below the current position must be in place
 * before the call (the fused decode form reads them before the preceding kernel has finished). */
int ab200_attention_fused_paged(const void *vqk_f16, const float *inv_freq, const int32_t *pos_dev,
                                void *k_cache_f16, void *v_cache_f16, void *out_f16, int H, int D,
                                long kv_stride, int max_seq, float scale, const int32_t *page_table,
                                int page_rows, void *stream);
int ab200_rope_kv_store_rows_paged(const void *vqk_f16, const float *inv_freq, const int32_t *pos0_dev,
                                   void *q_out_f16, void *k_cache_f16, void *v_cache_f16, int rows,
                                   int H, int D, long kv_stride, int max_seq,
                                   const int32_t *page_table, int page_rows, void *stream);
int ab200_attention_prefill_paged(const void *q_f16, const void *k_cache_f16, const void *v_cache_f16,
                                  void *out_f16, const int32_t *pos0_dev, int rows, int max_seq, int H,
                                  int D, long kv_stride, float scale, const int32_t *page_table,
                                  int page_rows, void *stream);

/* out[i] = silu(gate_up[i]) * gate_up[n + i], fp32 math (line 171). */
int ab200_silu_mul(const void *gate_up_f16, void *out_f16, int n, void *stream);

/* logits_f32[N] = W[N, K] . x[K]; W fp16 row-major (line 176: classifier matmul). */
int ab200_dense_gemv(const void *x_f16, const void *w_f16, float *logits_f32, int K, int N,
                     void *stream);

/* Greedy sampling and loop bookkeeping on the device (lines 197-207): next = argmax(logits)
 * (first maximum) unless *pos_dev + 1 < n_prompt, in which case next = prompt[*pos_dev + 1];
 * writes next to *token_dev and to out_tokens[*pos_dev + 1] (if non-null); *pos_dev += 1.
 * out_tokens holds out_cap ids: once *pos_dev + 1 reaches out_cap nothing is stored and the
 * position no longer advances (a step too many cannot write past the log).
 * Tensor-parallel vocabulary shards: ab200_greedy_next_tp. */
int ab200_greedy_next(const float *logits_f32, int n, const int32_t *prompt, int n_prompt,
                      int32_t *token_dev, int32_t *pos_dev, int32_t *out_tokens, int out_cap, void *stream);

/* Generic element-wise operator: interprets a stack program compiled from an Antares-IR statement
 * `out[axes] = expr` whose tensors are all indexed by the output's axes (antares_b200/ir.py::
 * compile_elementwise; the reference generates one kernel per such expression,
 * lang/einstein_v2.py:297-578).  ops/args: n_ops byte codes with their operand (input or constant
 * index); operation codes: 0 input, 1 constant, 2 add, 3 sub, 4 mul, 5 div, 6 neg, 7 exp, 8 log,
 * 9 sqrt, 10 rsqrt, 11 tanh, 12 erf, 13 sin, 14 cos, 15 abs, 16 floor, 17 ceil, 18 max, 19 min,
 * 20 pow, 21 sigmoid.  At most 48 operations, 16 constants, 8 inputs, stack depth 8; inputs and
 * output hold n elements of AB200_F16 or AB200_F32; arithmetic in fp32.  The program is
 * validated on the host (AB200_EINVAL on a malformed one). */
int ab200_eltwise_vm(const unsigned char *ops_host, const unsigned char *args_host, int n_ops,
                     const float *consts_host, int n_consts, const void *const *inputs_host,
                     const int *in_dtypes_host, int n_inputs, void *out, int out_dtype, size_t n,
                     void *stream);

/* Row-reduction template: a chain of row reductions closed by one map statement over one [rows, cols]
 * index space, e.g. the softmax and layernorm programs of AntaresIR.md:226,232
 *   t0[N] >=! f0(x[N, C]);  t1[N] +=! f1(x[N, C], t0[N]);  out[N, C] = g(x[N, C], t0[N], t1[N], w[C], C.val())
 * (the reference generates one kernel per statement, lang/einstein_v2.py:297-578).  Each of the
 * n_stages (<= 4) statements is a stack program; ops/args hold them back to back, stage_len their
 * lengths (<= 48 each), stage_reduce their kind (1 sum, 2 max, 3 min; 0 = the final map, which must be
 * last).  Operation codes as for ab200_eltwise_vm (0 = a [rows, cols] input), plus 22 = row result of
 * an earlier stage (operand: its index), 23 = a [cols] vector input, 24 = cols as a number.  Inputs and
 * output AB200_F16 or AB200_F32, arithmetic in fp32, reductions in a fixed order.  Validated on the host. */
int ab200_rowreduce_vm(const unsigned char *ops_host, const unsigned char *args_host,
                       const int *stage_len_host, const int *stage_reduce_host, int n_stages,
                       const float *consts_host, int n_consts, const void *const *mat_inputs_host,
                       const int *mat_dtypes_host, int n_mat, const void *const *col_inputs_host,
                       const int *col_dtypes_host, int n_col, void *out, int out_dtype, int rows,
                       int cols, void *stream);

/* ---- batched (prefill) forms of the glue above: one row per prompt token.  The reference feeds the
 * prompt token by token through the decode step (samples/05_llama2_7b_int4.py:194-200); these let
 * the whole prompt go through ab200_w4a16_gemm instead. ---- */

/* x_f32[r, :] = embed_f16[tokens_dev[r], :]. */
int ab200_embed_rows(const void *embed_f16, const int32_t *tokens_dev, float *x_f32, int rows,
                     int dim, int vocab, void *stream);
/* ab200_rope_kv_store for rows consecutive tokens: vqk [rows, 3*H*D], positions *pos0_dev + r. */
int ab200_rope_kv_store_rows(const void *vqk_f16, const float *inv_freq, const int32_t *pos0_dev,
                             void *q_out_f16, void *k_cache_f16, void *v_cache_f16, int rows, int H,
                             int D, long kv_stride, int max_seq, void *stream);
/* Causal attention: query row r (position *pos0_dev + r) attends cache rows 0 .. *pos0_dev + r. */
int ab200_attention_prefill(const void *q_f16, const void *k_cache_f16, const void *v_cache_f16,
                            void *out_f16, const int32_t *pos0_dev, int rows, int max_seq, int H,
                            int D, long kv_stride, float scale, void *stream);
/* out[r, i] = silu(gate_up[r, i]) * gate_up[r, n + i]. */
int ab200_silu_mul_rows(const void *gate_up_f16, void *out_f16, int rows, int n, void *stream);
/* x_f32[i] += y_f16[i] (residual update after a prefill GEMM). */
int ab200_residual_add_f16(float *x_f32, const void *y_f16, size_t n, void *stream);

/* One-shot hint for the calling thread's NEXT fp16 ab200_w4a16_gemv* call: while that kernel
 * streams its own weights, one thread per CTA also asks for the two byte ranges (normally the
 * following projection's qweight and scales) to be pulled into L2, so HBM stays busy across the
 * kernel boundary (measured neutral on B200 for the decode step; off by default there).  Results are unaffected.  Either pointer may be NULL.  No reference counterpart. */
int ab200_w4a16_gemv_prefetch_hint(const void *p0, size_t bytes0, const void *p1, size_t bytes1);

/* ---- tensor-parallel exchange over NVLink peer memory -----------------------------------------
 * The reference's only collectives are NCCL calls inside its TensorFlow plugin
 * (frameworks/tensorflow/communicate_ops.cc:65-99 bootstrap, :191 ncclAllReduce); its Llama
 * samples are single-device.  These entry points give the tensor-parallel decode step a one-shot
 * push all-reduce: one process per GPU, each rank owns a receive buffer, peers map it through
 * CUDA IPC and store into it directly.  No multicast objects are used. */

/* Bytes of one rank's receive buffer for `world` ranks and messages of up to n_max floats. */
size_t ab200_comm_buffer_bytes(int world, int n_max);
/* Allocates (cudaMalloc) and zeroes this rank's receive buffer on the current device and, if
 * ipc_handle64_host is not NULL, writes its 64-byte CUDA IPC handle there.  Set-up call:
 * allocates and synchronises. */
int ab200_comm_alloc(int world, int n_max, void **buf_out, void *ipc_handle64_host);
/* Maps a peer's receive buffer from its IPC handle (peer access is enabled on demand). */
int ab200_comm_open(const void *ipc_handle64_host, void **peer_buf_out);
int ab200_comm_close(void *peer_buf);
int ab200_comm_free(void *buf);

/* x_f32[0..n) += fp16_round(sum over ranks of partial_f32[0..n)) in one kernel per rank:
 * peer stores of the partial into every rank's buffer, epoch flags, a bounded wait for all
 * ranks, summation in rank order (bit-identical on all ranks).  bufs_host[r] = rank r's buffer as
 * mapped in this process (own entry = the local allocation).  Replaces
 * `all_reduce(partial); x = x + partial` after the row-parallel projections.  A wait that runs out
 * (a peer never arrived) is reported by ab200_kernel_status as site 100 + peer, and is sticky: while
 * the status word is set, later exchanges poll once instead of waiting, so read (and thereby
 * clear) the status after a step before trusting its result. */
int ab200_allreduce_residual(float *x_f32, const float *partial_f32, int n, void *const *bufs_host,
                             int rank, int world, int n_max, void *stream);

/* The row-parallel projection of a tensor-parallel decode step with the sum over ranks fused into
 * its epilogue, one kernel per rank:
 *   resid_f32[N] += fp16_round( sum over ranks r of  x_r[K_r] . dequant(W_r) )
 * x is fp16 [K] (prologue 0) or fp16 [2K] = gate | up fed as silu(gate) * up (prologue 2); weights
 * tile-major (see ab200_w4a16_gemv_tiled), group 128, K % 128 == 0, N % 128 == 0, N <= n_max.
 * Every thread that owns an output column stores its rank's fp32 sum as a (value, epoch) pair
 * into slot `rank` of each peer's receive buffer (plain peer stores over NVLink), polls its own
 * buffer for the other ranks' pairs (bounded, reported like ab200_allreduce_residual), adds in rank
 * order (bit-identical on every rank) and updates the residual.  bufs_host as for
 * ab200_allreduce_residual; exchanges through one buffer set must be issued in the same order on
 * every rank.  Replaces `xb = matmul_dequat(...); all_reduce(xb); x = x + xb`
 * (samples/05_llama2_7b_int4.py:167-168,172-173 are the single-device form; the reference has no
 * tensor-parallel path).  world == 1 degenerates to ab200_w4a16_gemv_tiled with the residual epilogue. */
int ab200_w4a16_gemv_tiled_allreduce(const void *x, int prologue, const int32_t *qweight_tiled,
                                     const void *scales_tiled, float *resid_f32, int K, int N,
                                     int group, void *const *bufs_host, int rank, int world, int n_max,
                                     void *stream);
/* The same kernel with all `world` ranks as consecutive CTA ranges of ONE cooperative launch on one
 * GPU (per-rank host arrays of device pointers; K_host[r] = rank r's rows, they may differ): the
 * protocol check for machines with fewer GPUs than ranks.  emu_scratch_dev:
 * ab200_w4a16_gemv_emulation_scratch_bytes() bytes.  Synchronises the stream once while setting up. */
int ab200_w4a16_gemv_tiled_allreduce_emulated(const void *const *x_host, int prologue,
                                              const int32_t *const *qweight_tiled_host,
                                              const void *const *scales_tiled_host,
                                              float *const *resid_host, const int *K_host, int N,
                                              void *const *bufs_host, int world, int n_max,
                                              void *emu_scratch_dev, void *stream);
size_t ab200_w4a16_gemv_emulation_scratch_bytes(void);

/* Vocabulary-parallel greedy step over the same kind of exchange buffer (its own one, n_max >= 4):
 * argmax of this rank's logits shard, exchange of the per-rank (value, global index) candidates by
 * peer stores, same winner on every rank (highest value, lowest index on ties), then the
 * bookkeeping of ab200_greedy_next.  Replaces the logits all-gather of the reference's
 * classifier step (samples/05_llama2_7b_int4.py:176-178) in tensor-parallel runs. */
int ab200_greedy_next_tp(const float *logits_local_f32, int n_local, int vocab_offset,
                         void *const *bufs_host, int rank, int world, int n_max,
                         const int32_t *prompt, int n_prompt, int32_t *token_dev, int32_t *pos_dev,
                         int32_t *out_tokens, int out_cap, void *stream);

/* The same protocol with all `world` ranks run as the blocks of ONE cooperative launch on one
 * GPU (x_host[r], partial_host[r], bufs_host[r] = rank r's device pointers): lets the exchange
 * be tested on fewer GPUs than ranks.  emu_scratch_dev: ab200_comm_emulation_scratch_bytes()
 * bytes of device memory.  Synchronises the stream once while setting up. */
int ab200_allreduce_residual_emulated(float *const *x_host, const float *const *partial_host, int n,
                                      void *const *bufs_host, int world, int n_max,
                                      void *emu_scratch_dev, void *stream);
size_t ab200_comm_emulation_scratch_bytes(void);
/* ab200_greedy_next_tp with all ranks as the blocks of one cooperative launch on one GPU (per-rank
 * host arrays of device pointers): the protocol check for machines with fewer GPUs than ranks. */
int ab200_greedy_next_tp_emulated(const float *const *logits_host, const int *n_local_host,
                                  const int *offset_host, void *const *bufs_host, int world, int n_max,
                                  const int32_t *prompt, int n_prompt, int32_t *const *token_host,
                                  int32_t *const *pos_host, int32_t *const *out_tokens_host, int out_cap,
                                  void *emu_scratch_dev, void *stream);

/* ---- the reference's native plugin boundary ---------------------------------------------------
 * frameworks/pytorch/main_ops.cc:17-54 binds two calls over kernel-source text:
 *   int  inject(const std::string &source)            -> key
 *   void forward(int key, std::vector<Tensor> tensors)   tensors = inputs (sorted by name) ++ outputs
 * and graph_evaluator/execute_module.hpp:274-283 reads the text's header.  The same pair here: */

/* Accepts kernel-source text in the reference's wire format
 *   // GLOBALS: name:dtype[d0, d1], ... -> name:dtype[...]        (antares/antares_compiler.py:183-199)
 *   // BACKEND: c-b200 (device)
 *   // COMPUTE_V1: - einstein_v2(input_dict={...}, extra_outputs=[...], exprss="<Antares IR>")
 * (statements of the IR separated by ';', frameworks/pytorch/custom_op.py:20-32), recognises the
 * operator natively and binds it to its hand-written kernel: W4A16 dequantise-and-multiply
 * (samples/05_llama2_7b_int4.py:136-138; 16 rows or fewer run the decode kernel, more the tensor-core
 * kernel), sigmoid (README.md:66 and AntaresIR.md:241), row softmax (AntaresIR.md:226).  Any other IR,
 * or another backend name, is AB200_EUNSUPPORTED: nothing is compiled and nothing falls back.
 * Host call, thread-safe; keys stay valid for the life of the process. */
int ab200_inject(const char *source, int *key_out);

/* Launches the module on `stream`.  args_host[i] = device pointer of the i-th tensor of the GLOBALS
 * line, inputs first, then outputs (main_ops.cc:38-42).  Shapes are the ones the text declared.
 * Nothing is allocated, looked up by name or synchronised on this path. */
int ab200_forward(int key, void *const *args_host, int n_args, void *stream);

/* What a binding needs to allocate outputs (custom_op.py:81-116 parses the same from the text):
 * counts and the exported op's name, then name, dtype, shape (at most 8 extents) per argument slot. */
int ab200_module_info(int key, int *n_inputs_host, int *n_outputs_host, char *op_name_host, int op_name_cap);
int ab200_module_tensor(int key, int slot, char *name_host, int name_cap, char *dtype_host, int dtype_cap,
                        long *shape8_host, int *rank_host);

/* Host cost of the call path: `iters` ab200_forward calls back to back on `stream`, wall time per
 * call in nanoseconds (the reference's per-call cost is the map rebuilding of
 * graph_evaluator/execute_module.hpp:322-333 plus cuLaunchKernel).  Synchronises nothing. */
int ab200_forward_host_ns(int key, void *const *args_host, int n_args, void *stream, int iters,
                          double *ns_per_call_host);

/* ---- device memory, copies and timing for hosts that do not link the CUDA runtime -------------------
 * What the reference's HAL offers its runtime next to module loading and launching:
 * ab::alloc / memcpyHtoD / memcpyDtoH / memcpyDtoD / synchronize / recordTime / convertToElapsedTime
 * (backends/c-rocm/include/backend.hpp:92-114,221-252).  include/c-b200/backend.hpp maps `namespace ab`
 * onto these and onto ab200_inject / ab200_forward, so that the reference's evaluator
 * (graph_evaluator/run_graph.cpp) can drive this library.  All are host calls; the allocating ones
 * say so in their names. */
int ab200_hal_set_device(int device);
int ab200_hal_malloc(void **ptr_out_host, size_t bytes);             /* cudaMalloc */
int ab200_hal_free(void *ptr);
/* kind: 0 host->device, 1 device->host, 2 device->device; asynchronous on `stream`. */
int ab200_hal_memcpy(void *dst, const void *src, size_t bytes, int kind, void *stream);
int ab200_hal_synchronize(void *stream);
/* Creates an event and records it on `stream`; ab200_hal_event_elapsed waits for the stop event,
 * returns the seconds between the two and destroys both. */
int ab200_hal_event_record(void **event_out_host, void *stream);
int ab200_hal_event_elapsed(void *start_event, void *stop_event, double *seconds_host);

#ifdef __cplusplus
}
#endif
#endif /* ANTARES_B200_H_ */
