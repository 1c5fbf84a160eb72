/* libh3b200: C ABI of the B200 (sm_100a) implementation of h3metal's W8A8 Hadamard-rotated linear.
 *
 * It stands where the reference's Metal launcher stands (src/capi.h of audenvenn/h3metal): a small C library that
 * a Python (ctypes) host drives. The reference's library is a generic kernel launcher for run-time compiled Metal
 * shaders; here the two kernels of the quantised-linear path are compiled ahead of time for sm_100a and exposed
 * as typed entry points, while the context / error / commit / wait / profile conventions are kept:
 *
 *   - pointer-returning calls return NULL on failure, int-returning calls return 0 on success (src/capi.h:59-63);
 *   - the message of the last failed call on this thread is read with h3b_last_error() (src/capi.h:26-27);
 *   - launches are asynchronous and ordered on the context's stream; results are valid after h3b_wait(), which
 *     returns the GPU seconds of the work since the previous wait, or a negative value on failure
 *     (src/capi.h:64-70);
 *   - a context is not thread-safe: one context per host thread / rank.
 *
 * Memory stays with the caller: every tensor argument is a plain device pointer plus sizes and strides in
 * ELEMENTS. Nothing in these signatures is a PyTorch type.
 */
#ifndef H3B200_H
#define H3B200_H

#include <stdint.h>

#if defined(__GNUC__)
#define H3B_API __attribute__((visibility("default")))
#else
#define H3B_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct h3b_ctx h3b_ctx;

/* element types of tensor arguments */
enum { H3B_F32 = 0, H3B_F16 = 1, H3B_BF16 = 2, H3B_I8 = 3, H3B_I32 = 4 };

/* Message of the last failed call on this thread (empty if none). Replaces h3_last_error (src/capi.h:27). */
H3B_API const char *h3b_last_error(void);

/* Opens CUDA device `device`, which must be compute capability 10.0 (the int8 tensor-core instruction used here
 * exists only there), creates the context's stream and raises the kernels' shared-memory limits.
 * Replaces h3_open (src/capi.h:29), whose argument was the shader directory. NULL on failure. */
H3B_API h3b_ctx *h3b_open(int device);
/* Waits for the context's work, then frees it. Replaces h3_close (src/capi.h:30). */
H3B_API void h3b_close(h3b_ctx *ctx);
/* Replaces h3_device_name (src/capi.h:31). */
H3B_API const char *h3b_device_name(h3b_ctx *ctx);
/* Device memory a working set may use (total device memory) and the largest single allocation.
 * Replace h3_recommended_working_set / h3_max_buffer_length (src/capi.h:32-33). */
H3B_API uint64_t h3b_recommended_working_set(h3b_ctx *ctx);
H3B_API uint64_t h3b_max_buffer_length(h3b_ctx *ctx);
/* Number of SMs of the device (grid sizing of the persistent product kernel). No reference counterpart. */
H3B_API int h3b_sm_count(h3b_ctx *ctx);

/* Makes later launches go to `cuda_stream` (a cudaStream_t, taken as is: NULL is CUDA's legacy default stream,
 * which is also PyTorch's default stream), so that a host that owns the tensors can order the kernels with its
 * other work. h3b_use_own_stream returns to the non-blocking stream the context created at h3b_open, which is
 * where launches go until h3b_set_stream is called. No reference counterpart (Metal command queues are owned by
 * the reference's context, src/metal_rt.h:16-45). Both return 0. */
H3B_API int h3b_set_stream(h3b_ctx *ctx, void *cuda_stream);
H3B_API int h3b_use_own_stream(h3b_ctx *ctx);

/* Launch overlap (on by default; on = 0 turns it off): the product kernels and the TMA-fed rotate+quantise kernels are
 * launched with CUDA's programmatic stream serialization, so a kernel's set-up (barriers, tensor memory, descriptor
 * prefetch) runs while the kernel before it in the stream drains; each kernel waits for its predecessor's completion
 * before it touches global memory, so results and ordering are unchanged (every other kernel of the library is launched
 * the ordinary way). Measured on B200 on whole blocks: -4 % on one 3072 x 3072 linear over 4096 tokens, -2 % on the
 * FLUX.2-shaped block with LoRA terms, -3 % on the 33B block with rank-64 terms at 66 560 tokens, neutral on the plain
 * 33B block. Off in profile mode. No reference counterpart (Metal encodes one command buffer, src/capi.mm:51-64).
 * Returns 0. */
H3B_API int h3b_set_launch_overlap(h3b_ctx *ctx, int on);

/* Rotate + per-token int8 quantise. Replaces the dispatch of the Metal kernel rot_q8
 * (kernels/ops.metal:274-334; parameter block RotQParams kernels/params.h:25-29; launcher h3metal/ops.py:214-222).
 *   x        [M][x_stride] of x_dtype (H3B_BF16 / H3B_F16 / H3B_F32); with mode 1 columns D..2D-1 hold the gates
 *   out      int8 [M][D] contiguous; with out_hr != 0, fp16 [M][D] (rotated rows, not quantised)
 *   sa       fp32 [M] row scales (ignored with out_hr)
 *   block    rotation block: 64, 128 or 256 (the reference kernel has 256); D % block == 0
 *   mode     0: rotate x; 1: rotate x[:, :D] * silu(x[:, D:2D])
 * x must be 16-byte aligned with x_stride * sizeof(x_dtype) a multiple of 16; out 16-byte aligned. */
H3B_API int h3b_rot_q8(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, void *out, float *sa, int M, int D,
               int block, int mode, int out_hr);

/* RMSNorm (or LayerNorm without affine) + modulation + the same rotate + quantise tail, in one pass over the fp32
 * residual stream. Replaces the dispatch of the Metal kernel norm_mod_q8 (kernels/ops.metal:111-268; parameter block
 * NormQParams kernels/params.h:18-23; launcher h3metal/ops.py:200-211; buffers x, mod, rtype, out, sa, params, y, post).
 *   x      fp32 [M][x_stride]; with post it is updated in place: x[m] += post * rmsnorm(y[m])
 *   mod    fp32, per row type D scale' values then D shift values; rows mod_stride (>= 2 D) apart
 *   rtype  one byte per row: the row's type
 *   out    out_kind 0: int8 [M][D] with row scales in sa; 1: fp32 [M][D] = norm(x) * scale' + shift (no rotation);
 *          2: the same as fp16; 3: the rotated row as fp16
 *   ln     non-zero: subtract the row mean first (LayerNorm); excludes post
 *   y, post  both or neither: fp32 [M][D] and fp32 [D]
 * D must be a multiple of block (64, 128, 256). All tensors 16-byte aligned, strides multiples of 16 bytes. */
H3B_API int h3b_norm_mod_q8(h3b_ctx *ctx, float *x, int64_t x_stride, const float *mod, int64_t mod_stride,
                            const uint8_t *rtype, void *out, float *sa, int M, int D, int block, float eps, int ln,
                            int out_kind, const float *y, const float *post);

/* The two halves of h3b_rot_q8 for a row whose channels are sharded over several GPUs (a K-sharded, "row-parallel"
 * layer): the reference quantises with ONE scale per token taken over the whole row (kernels/ops.metal:315-317), so
 * each GPU first reports the largest rotated magnitude of its shard, the host reduces those with MAX over the GPUs,
 * and each GPU then quantises its shard with the reduced value. No reference counterpart (single GPU).
 *   h3b_rot_amax           amax[m] = max_c |rot(x)[m][c]| over this shard's D channels; writes no codes
 *   h3b_rot_q8_given_amax  reads amax_to_scale[m] (the reduced maximum), writes the int8 codes of this shard and
 *                          overwrites amax_to_scale[m] with the scale (amax / 127, or 1 for an all-zero row)
 * Other arguments as h3b_rot_q8. With one shard the pair gives bit for bit what h3b_rot_q8 gives. */
H3B_API int h3b_rot_amax(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, float *amax, int M, int D,
                         int block, int mode);
H3B_API int h3b_rot_q8_given_amax(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, void *out,
                                  float *amax_to_scale, int M, int D, int block, int mode);

/* The same pair with the maxima exchanged through peer-mapped memory (h3b_peer_*) instead of a collective: every GPU
 * has a table of `world` slots of M maxima. h3b_rot_amax_push stores this shard's maxima into dst[q][m], q < world -
 * this GPU's slot in GPU q's table, one address per GPU (plain stores through the peer mappings). After
 * h3b_peer_sync, h3b_rot_q8_given_amax_slots takes, for row m, the largest of slots[s * slot_stride + m], s < world
 * (this GPU's own table), quantises the shard with it and writes the scale to scale[m]. 16-bit inputs of at most
 * 16384 channels. Same codes and scales as the all-reduce variant. No reference counterpart. */
H3B_API int h3b_rot_amax_push(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, float *const *dst, int world,
                              int M, int D, int block, int mode);
H3B_API int h3b_rot_q8_given_amax_slots(h3b_ctx *ctx, const void *x, int x_dtype, int64_t x_stride, void *out,
                                        const float *slots, int64_t slot_stride, int world, float *scale, int M, int D,
                                        int block, int mode);

/* The product's epilogue on its own: C[m][n] = c_dtype(float(acc[m][n]) * sa[m] * sw[n] + bias[n]) for int32
 * accumulators [M][acc_stride] produced by h3b_gemm_w8a8 with H3B_I32 and summed over the GPUs of a K-sharded layer.
 * Same operation order as the fused epilogue (kernels/gemm.metal:238-255), so the result equals the single-GPU
 * product bit for bit. No reference counterpart. */
H3B_API int h3b_dequant_i32(h3b_ctx *ctx, const int32_t *acc, int64_t acc_stride, const float *sa, const float *sw,
                            const float *bias, void *C, int c_dtype, int64_t c_stride, int M, int N);

/* int8 x int8 product with the dequantising epilogue. Replaces the dispatch of the Metal kernel gemm with weight
 * format 1 and epilogue 0 (kernels/gemm.metal:117-261; parameter block GemmParams kernels/params.h:7-16; launcher
 * h3metal/ops.py:124-174; buffer order a, w, sw, sa, out, bias, ..., lt, lb, lr).
 *   C[m][n] = c_dtype(float(acc) * sa[m] * sw[n] + bias[n] + sum_{k0<=j<k1} T[m][j] * B[n][j]),
 *   acc[m][n] = sum_k A[m][k] * W[n][k]  (exact, int32)
 *   A     int8 [M][a_stride], K-contiguous        W   int8 [N][w_stride], K-contiguous
 *   sw    fp32 [N]    sa  fp32 [M]    bias  fp32 [N] or NULL
 *   C     [M][c_stride] of c_dtype: H3B_BF16 / H3B_F16 / H3B_F32, or H3B_I32 for the raw accumulators (scales,
 *         bias and the low-rank term are then ignored)
 *   lora_T  fp16 [M][t_stride] or NULL    lora_B  fp16 [N][b_stride]    R  ranks used (multiple of 32, <= 128)
 *   lora_ranges  int32 [2 * ceil(N / h3b_gemm_tile_n(..))] = (k0, k1) per column tile, multiples of 16, or NULL for
 *         the whole range 0..R (the reference's table `lr` without its two leading strides)
 * All M rows are computed and stored (the caller passes its padded row count, as h3metal/ops.py:165 does).
 * A, W, T, B must be 16-byte aligned with row strides that are multiples of 16 bytes. */
H3B_API int h3b_gemm_w8a8(h3b_ctx *ctx, const int8_t *A, int64_t a_stride, const int8_t *W, int64_t w_stride,
                  const float *sw, const float *sa, const float *bias, void *C, int c_dtype, int64_t c_stride,
                  int M, int N, int K, const void *lora_T, int64_t t_stride, const void *lora_B, int64_t b_stride,
                  int R, const int32_t *lora_ranges);

/* The same product with the reference's second epilogue (EPI 1, kernels/gemm.metal:18-20,256-259; launcher
 * h3metal/ops.py:124-174 with epi=1): instead of storing, it accumulates into the fp32 residual stream,
 *   X[m][n] += gate[rtype[m]][n] * (float(acc) * sa[m] * sw[n] + bias[n] + low[m][n])
 * X fp32 [M][c_stride]; rtype one byte per row; gate fp32 [types][g_stride]. Other arguments as h3b_gemm_w8a8.
 * K may be split by the caller into consecutive slices accumulated by successive calls (the reference's ksplit). */
H3B_API int h3b_gemm_w8a8_gated(h3b_ctx *ctx, const int8_t *A, int64_t a_stride, const int8_t *W, int64_t w_stride,
                                const float *sw, const float *sa, const float *bias, float *X, int64_t c_stride, int M,
                                int N, int K, const uint8_t *rtype, const float *gate, int64_t g_stride,
                                const void *lora_T, int64_t t_stride, const void *lora_B, int64_t b_stride, int R,
                                const int32_t *lora_ranges);

/* ---- Row-parallel (K-sharded) layers over the GPUs of one node, data path without a communication library --------
 * No counterpart in the reference (single GPU). One process and one context per GPU. Every GPU computes a partial
 * product of ALL M rows over its K shard; GPU o owns rows [o * rows_per_gpu, (o + 1) * rows_per_gpu) of the result.
 * h3b_gemm_w8a8_push stores each finished tile of the partial product straight into the owner's staging memory
 * (plain stores through a CUDA IPC peer mapping, overlapping the rest of the product); after h3b_peer_sync the owner
 * runs h3b_reduce_dequant over its rows, which sums the slots, applies the epilogue and can store the finished rows
 * into every GPU's output (an all-gather by peer stores; a second h3b_peer_sync then makes them readable everywhere).
 *
 *   h3b_peer_alloc    zero-filled device memory that can be shared (cudaMalloc); NULL on failure. Setup only.
 *   h3b_peer_export   64-byte IPC handle of a h3b_peer_alloc'd block, to be sent to the other processes
 *   h3b_peer_import   maps another process's block into this one (peer access over NVLink is enabled on first use);
 *                     returns the local address of the mapping, NULL on failure. Not for a handle of this process.
 *   h3b_peer_unmap / h3b_peer_free   undo import / alloc
 *   h3b_peer_sync     flags[q] is (this process's mapping of) GPU q's array of `world` 32-bit words, zero at start.
 *                     mode 0: store `epoch` into word `rank` of every array, then wait until every word of this
 *                     GPU's own array has reached `epoch`; mode 1: only the stores; mode 2: only the wait. Epochs
 *                     must grow from call to call (1, 2, ...). The wait is bounded (about a second); if it runs out
 *                     the kernel returns and the next h3b_wait fails with a message - the device is not left hanging.
 *                     Every rank must make the same sequence of calls; the kernels of different ranks run on
 *                     different GPUs (never use mode 0 between contexts that share one GPU).
 *   h3b_gemm_w8a8_push  slots[o] = where this GPU's partial of owner o's rows goes: [rows_per_gpu][stage_stride] of
 *                     stage_dtype inside o's staging block (this GPU's slot there). stage_dtype H3B_I32: raw int32
 *                     accumulators (sw, sa unused; the sum over GPUs is exact, the result bit-identical to one GPU);
 *                     H3B_BF16: float(acc) * sa[m] * sw[n] rounded to bf16 (half the traffic; 1e-3-level agreement).
 *                     M = world * rows_per_gpu, rows_per_gpu % 128 == 0, N % 32 == 0. sa holds the WHOLE-row scales
 *                     (h3b_rot_amax, MAX over the GPUs, h3b_rot_q8_given_amax).
 *   h3b_reduce_dequant  stage: this GPU's staging block, `world` slots slot_stride elements apart, each
 *                     [rows][stage_stride]. int32: out = c_dtype(float(sum) * sa[m] * sw[n] + bias[n]), the operation
 *                     order of h3b_gemm_w8a8's epilogue; bf16: out = c_dtype(fp32 sum in slot order + bias[n]). The
 *                     rows are stored at rows row0 .. row0 + rows - 1 of each of the n_out buffers outs[i]
 *                     ([..][c_stride] of c_dtype; local or peer-mapped). sa points at the owner's first row.
 * Staging is reused safely when callers alternate between two staging blocks from one layer call to the next: a GPU
 * passes the rendezvous of call c + 1 only after every owner has finished reading the block of call c. */
H3B_API void *h3b_peer_alloc(h3b_ctx *ctx, uint64_t bytes);
H3B_API int h3b_peer_free(h3b_ctx *ctx, void *ptr);
H3B_API int h3b_peer_export(h3b_ctx *ctx, void *ptr, unsigned char handle[64]);
H3B_API void *h3b_peer_import(h3b_ctx *ctx, const unsigned char handle[64]);
H3B_API int h3b_peer_unmap(h3b_ctx *ctx, void *ptr);
H3B_API int h3b_peer_sync(h3b_ctx *ctx, void *const *flags, int rank, int world, uint32_t epoch, int mode);
H3B_API int h3b_gemm_w8a8_push(h3b_ctx *ctx, const int8_t *A, int64_t a_stride, const int8_t *W, int64_t w_stride,
                               const float *sw, const float *sa, void *const *slots, int world, int rows_per_gpu,
                               int stage_dtype, int64_t stage_stride, int M, int N, int K);
H3B_API int h3b_reduce_dequant(h3b_ctx *ctx, const void *stage, int64_t slot_stride, int64_t stage_stride,
                               int stage_dtype, int world, const float *sa, const float *sw, const float *bias,
                               void *const *outs, int n_out, int c_dtype, int64_t c_stride, int rows, int N, int row0);
/* The owner's reduction for a row-parallel layer that carries a low-rank term: as h3b_reduce_dequant (gate == NULL) or
 * h3b_reduce_dequant_gated (gate != NULL; c_dtype is then ignored and outs[0] is X), with low[m][n] - fp32
 * [rows][low_stride], the owner's rows of T B'^T - added after the bias, where the product's own epilogue adds the
 * term (kernels/gemm.metal:251-253). The owner obtains T for its rows from the K shards' int32 partial sums of the
 * term's input-side product, pushed and reduced like the main product's, and the term itself from one call of
 * h3b_gemm_w8a8 on an all-zero int8 product with that T (the epilogue then stores 0 * sa * sw + low). No reference
 * counterpart (single GPU). */
H3B_API int h3b_reduce_dequant_low(h3b_ctx *ctx, const void *stage, int64_t slot_stride, int64_t stage_stride,
                                   int stage_dtype, int world, const float *sa, const float *sw, const float *bias,
                                   const float *low, int64_t low_stride, void *const *outs, int n_out, int c_dtype,
                                   int64_t c_stride, int rows, int N, int row0, const uint8_t *rtype, const float *gate,
                                   int64_t g_stride);
/* The owner's reduction with the reference's second epilogue (EPI 1, kernels/gemm.metal:18-20,256-259), for the
 * attention-out and FFN-down projections of models that accumulate into an fp32 residual stream: with v the value
 * h3b_reduce_dequant would store,  X[row0 + m][n] += gate[rtype[m]][n] * v  for the owner's rows; X fp32
 * [..][c_stride] local to the owner (every GPU keeps its own rows of the stream), rtype one byte per owned row, gate
 * fp32 [types][g_stride]. Bit-identical to h3b_gemm_w8a8_gated on one GPU for int32 staging. */
H3B_API int h3b_reduce_dequant_gated(h3b_ctx *ctx, const void *stage, int64_t slot_stride, int64_t stage_stride,
                                     int stage_dtype, int world, const float *sa, const float *sw, const float *bias,
                                     float *X, int64_t c_stride, int rows, int N, int row0, const uint8_t *rtype,
                                     const float *gate, int64_t g_stride);

/* The product with a LoRA term for callers that cannot allocate device memory. It has no counterpart in the
 * reference (whose Scratch object, h3metal/ops.py:37-47, simply grows a buffer on demand).
 *
 * Who needs it: a host that was handed a fixed set of buffers and owns none of the device's memory itself. Two
 * examples are an inference server whose allocator reserved the whole of HBM at start-up, so that a cudaMalloc
 * from a plug-in fails or fights that allocator, and a serving loop with a latency bound, where cudaMalloc /
 * cudaFree would synchronise the whole device in the middle of a step. h3b_gemm_w8a8 asks such a caller for a T
 * buffer of M x R fp16 values; this entry point brings its own: T lives in a static device array inside the library
 * image, H3B_NOALLOC_MAX_T_VALUES fp16 values (8 MiB), which every GPU that loads the library holds until the
 * process exits. The call performs no cudaMalloc, cudaFree or other allocating call, and its TMA descriptors are
 * built on the stack. h3b_open() looks the array up on its device (which also makes the CUDA runtime load this
 * library's device code and place the 8 MiB there, at set-up, where the context allocates anyway), so a caller that
 * opened its context before handing HBM to its own allocator meets no implicit allocation later. One caveat remains
 * outside the library's control: with CUDA's default lazy loading the two product kernels are loaded on their first
 * launch, so the FIRST call per device may still load code; run one warm-up call at set-up (or set
 * CUDA_MODULE_LOADING=EAGER) and the guarantee holds from the second call on.
 *
 * Size limit in practice: M x R <= 4 Mi values, e.g. 32768 rows at rank 128 or 65536 rows at rank 64. The largest
 * benchmark configuration (66560 rows, rank 64 = 4.06 Mi values) is just above it: feed it as two row slices
 * (any split into multiples of 128 rows; rows are independent).
 *
 * It computes T = fp16((A x lora_A^T) * sa[m] * lora_sw[j]) into that array and then the same product as
 * h3b_gemm_w8a8 with lora_T pointing at it; arguments as there, except that the term's input side is passed as its
 * int8 codes lora_A [R][la_stride] and fp32 scales lora_sw [R] (what ops.low_rank() stores) instead of a finished T.
 * Returns non-zero with a message if M x R exceeds H3B_NOALLOC_MAX_T_VALUES.
 *
 * The array's device address is looked up (cudaGetSymbolAddress) in h3b_open(); should a context ever reach this
 * call without it, the first call on that device does the look-up itself, so make that first call outside any
 * stream capture. Every argument of both products is checked before the first launch: a refused call launches
 * nothing and leaves the array as it was. All calls on a device share the one array and each overwrites the part it uses in
 * full: calls that overlap on the GPU (two streams, two contexts on the same device) race on it - keep them on one
 * stream or order them yourself. */
#define H3B_NOALLOC_MAX_T_VALUES (4u << 20)
H3B_API int h3b_gemm_w8a8_lora_noalloc(h3b_ctx *ctx, const int8_t *A, int64_t a_stride, const int8_t *W,
                                       int64_t w_stride, const float *sw, const float *sa, const float *bias, void *C,
                                       int c_dtype, int64_t c_stride, int M, int N, int K, const int8_t *lora_A,
                                       int64_t la_stride, const float *lora_sw, const void *lora_B, int64_t b_stride,
                                       int R, const int32_t *lora_ranges);

/* Column-tile width the product uses for N outputs with (lora != 0) or without a low-rank term: the granularity
 * of lora_ranges. Plays the part of the TN macro the reference compiles into its kernel (kernels/gemm.metal:48-50). */
H3B_API int h3b_gemm_tile_n(h3b_ctx *ctx, int N, int lora);
/* Overrides the product's choices: tile_n (0 = automatic; 32, 64, 128, 256: single-CTA tiles of that width), band
 * (row tiles swept per column tile, 0 = automatic) and pair (CTA pairs computing 256 x 256 tiles with
 * tcgen05.mma cta_group::2: 0 = automatic - pairs for products of at least 256 x 256 outputs without a low-rank term
 * -, 1 = whenever no low-rank term is attached, -1 = never: 128-row single-CTA tiles). The
 * counterpart of the tile= and swz= arguments of h3metal/ops.py:124-126. Returns 0. */
H3B_API int h3b_gemm_set_policy(h3b_ctx *ctx, int tile_n, int band, int pair);
/* How the CTA-pair product writes 16-bit outputs: 1 = staged - the epilogue converts a tile into shared memory,
 * frees the accumulator at once and TMA stores the tile while the next one is being multiplied - whenever the output
 * is bf16 / f16, not gated and 16-byte aligned; -1 = always with direct stores from registers; 0 = automatic
 * (staged for launches of at most three tiles per CTA pair with K <= 4096, where the last, exposed epilogue counts,
 * and for very tall products, M >= 49152, whose output no longer fits L2; everything else gains more from the two
 * ring stages that staging costs).
 * No reference counterpart. Returns 0. */
H3B_API int h3b_gemm_set_store_mode(h3b_ctx *ctx, int mode);
/* Tuning of the rotate+quantise kernel. tma_stages: rows a CTA keeps in flight in shared memory (1..4), 0 =
 * automatic, -1 = do not use the TMA-fed kernel. threads_target: CTA size target of the register-fed kernel that
 * serves fp32 inputs, rows over 16384 channels and tma_stages = -1 (0 = automatic). chunk: channels a thread of the
 * TMA-fed kernel owns, 32 or 64 (0 = automatic). The counterpart of the NSG/MAXB geometry of
 * h3metal/ops.py:193-197. Returns 0. */
H3B_API int h3b_rot_set_policy(h3b_ctx *ctx, int threads_target, int tma_stages, int chunk);

/* Self-test of the error path the kernels share. Every device-side wait in this library is bounded: when one runs
 * out the kernel records a code in the context's status word, winds down and returns, and the next h3b_wait reports
 * it (negative return, message in h3b_last_error) with the context still usable. This call launches a one-CTA kernel
 * that waits about a millisecond on a barrier nothing signals, so that exactly that happens. The counterpart of a
 * failed command buffer surfacing from h3_wait (src/capi.h:66-70, src/capi.mm:235-243). Returns 0 (the launch). */
H3B_API int h3b_selftest_expire_wait(h3b_ctx *ctx);

/* Issue-rate probe of the int8 tensor pipe: the measured ceiling the product's fractions are quoted against.
 * Counterpart of the reference's register-fed matrix-unit probe (bench/hw/mma_rate.py:9-24, bench/hw/mma_rate.metal),
 * whose figure is the "peak" of every percentage the reference publishes (README.md:271-273). One CTA per SM issues
 * `iters` x 4 tcgen05.mma kind::i8 instructions of 128 x 256 x 32 (pair = 0) or, per CTA pair, 256 x 256 x 32 with
 * cta_group::2 (pair = 1) on operand tiles that stay in shared memory, alternating between two int32 accumulators in
 * tensor memory; no TMA, no epilogue; one bounded wait at the end. Blocking (it synchronises the context's stream and
 * allocates a small result buffer). out[0] = seconds of the launch (CUDA events), out[1] = cycles of the slowest CTA
 * (clock64), out[2] = multiply-add operations (2 per MAC) per clock and SM, out[3] = TOP/s over the CTAs that ran,
 * out[4] = CTAs that ran. Returns 0 on success. */
H3B_API int h3b_mma_rate_probe(h3b_ctx *ctx, int pair, int iters, double out[5]);

/* Nothing is deferred on CUDA, so commit only exists for interface parity. Replaces h3_commit (src/capi.h:65). */
H3B_API void h3b_commit(h3b_ctx *ctx);
/* Blocks until the work launched through this context is done. Returns the GPU seconds between the first launch
 * since the previous wait and the end of the last one, 0 if nothing was launched, or a negative value if a kernel
 * failed or reported a device-side timeout (see h3b_last_error). Replaces h3_wait (src/capi.h:66-70). */
H3B_API double h3b_wait(h3b_ctx *ctx);
/* With profiling on every launch is timed on its own (and the host waits for it); h3b_profile_take returns the
 * seconds recorded since the last call. Replace h3_set_profile / h3_profile_take (src/capi.h:71-74). */
H3B_API void h3b_set_profile(h3b_ctx *ctx, int on);
H3B_API int h3b_profile_take(h3b_ctx *ctx, double *seconds, int max);
/* Kernels launched through this context since it was opened (the benchmark's launch count). No counterpart. */
H3B_API uint64_t h3b_launch_count(h3b_ctx *ctx);

#ifdef __cplusplus
}
#endif

#endif /* H3B200_H */
