// Internal (C++) interface between the C ABI (capi.cu) and the kernel translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace h3b {

// Element types as the C ABI numbers them (include/h3b200.h).
enum Dtype : int { kDtypeF32 = 0, kDtypeF16 = 1, kDtypeBf16 = 2, kDtypeI8 = 3, kDtypeI32 = 4 };
constexpr int kMaxPeers = 8;  // GPUs of one node that may share a row-parallel layer

void rot_q8_geometry(int D, int threads_target, int *ch, int *threads);
cudaError_t launch_rot_q8(const void *x, int x_dtype, long long x_stride, void *out, float *sa, int M, int D,
                          int block, int mode, int out_hr, int scale_mode, int threads_target, int sms,
                          cudaStream_t stream);

// Norm + modulation in front of the same tail. out_kind: 0 int8 codes + scales, 1 modulated fp32, 2 modulated fp16,
// 3 rotated fp16. post != null selects the fused residual update (needs y); ln selects LayerNorm.
cudaError_t launch_norm_mod_q8(float *x, long long x_stride, const float *mod, long long mod_stride,
                               const unsigned char *rtype, void *out, float *sa, int M, int D, int block, float eps,
                               int ln, int out_kind, const float *y, const float *post, cudaStream_t stream);

// TMA-fed variant for bf16 / fp16 inputs of up to 16384 channels. `map` describes the input as
// {64, cols / 64, M} with box {64, D / 64, 1} and 128-byte swizzle (built by the caller).
bool rot_q8_tma_supported(int x_dtype, int D);
// Row maxima of a K-sharded row exchanged through peer-mapped memory instead of a collective. With scale_mode 1 the
// shard's maximum of row m is stored to amax_dst[q][m] for q < n_dst (one destination per GPU: this GPU's slot in
// every GPU's table). With scale_mode 2 the row's maximum is the largest of sa[s * amax_slot_stride + m], s <
// amax_slots (this GPU's table, one slot per GPU), and the scale goes to scale_out[m].
struct RotShardArgs {
  float *amax_dst[kMaxPeers];
  int n_dst;
  int amax_slots;
  long long amax_slot_stride;
  float *scale_out;
};
// chunk_wanted: channels per thread, 32 or 64 (anything else: the default). shard: null for the plain behaviour
// (scale_mode 1 writes sa[m]; scale_mode 2 reads sa[m] and overwrites it with the scale).
cudaError_t launch_rot_q8_tma(const CUtensorMap &map, int x_dtype, void *out, float *sa, int M, int D, int block,
                              int mode, int out_hr, int scale_mode, int stages_wanted, int chunk_wanted, int sms,
                              int *status, cudaStream_t stream, bool overlap = false,
                              const RotShardArgs *shard = nullptr);
// The norm + modulation front end on the same TMA-fed kernel: fp32 rows of up to 8192 channels, no fused residual
// update. `map` describes x as {32 floats, D / 32, M} and `map_mod` the modulation table as
// {32 floats, mod_stride / 32, types}, both with box {32, D / 32, 1} and 128-byte swizzle.
bool norm_mod_q8_tma_supported(int D);
cudaError_t launch_norm_mod_q8_tma(const CUtensorMap &map, const CUtensorMap &map_mod, const float *mod,
                                   long long mod_stride, const unsigned char *rtype, void *out, float *sa, int M, int D,
                                   int block, float eps, int ln, int out_kind, int stages_wanted, int chunk_wanted, int sms,
                                   int *status, cudaStream_t stream);

// out[m][n] = c_dtype(float(acc[m][n]) * sa[m] * sw[n] + bias[n]): the product's epilogue applied to accumulators
// that were summed elsewhere (row-parallel layers reduce their int32 partial accumulators over the GPUs first).
cudaError_t launch_dequant_i32(const int32_t *acc, long long acc_stride, const float *sa, const float *sw,
                               const float *bias, void *out, int c_dtype, long long c_stride, int M, int N, int sms,
                               cudaStream_t stream);

// Owner's side of the row-parallel push: out[m][n] = epilogue(sum over the `world` slots of stage[slot][m][n]) for
// the owner's `rows` rows. stage_dtype kDtypeI32: int32 partial accumulators, summed exactly, then the product's
// epilogue (* sa[m] * sw[n] + bias[n]). kDtypeBf16: dequantised bf16 partials, summed in fp32 in slot order, plus bias.
// out_peers (or null): the finished rows are also stored into every GPU's copy of the output at row `row0` on (an
// all-gather by peer stores); out_peers[rank] may be the local buffer.
struct ReduceLaunch {
  const void *stage;        // [world][rows][stage_stride] of stage_dtype
  long long slot_stride;    // elements between slots
  long long stage_stride;   // elements between rows
  int stage_dtype, world;
  const float *sa, *sw, *bias;
  // A low-rank term of a row-parallel layer: fp32 [rows][low_stride], added after the bias, where the product's own
  // epilogue adds it (the owner computes it for its rows from the reduced T; see h3b_reduce_dequant_low). Or null.
  const float *low;
  long long low_stride;
  void *out[kMaxPeers];     // out[0] only, or one base per GPU (each [..][c_stride], rows written at row0 + m)
  int n_out;
  long long c_stride;
  int c_dtype, rows, N, row0;
  // Gated-residual epilogue (the reference's epilogue 1, kernels/gemm.metal:18-20,256-259) on the owner's rows:
  // out[0] is the fp32 residual stream X and X[row0 + m][n] += gate[rtype[m]][n] * v. rtype points at the owner's
  // first row. gate == null: plain store.
  const unsigned char *rtype;
  const float *gate;
  long long g_stride;
  // The context's device status word (or null). A kernel earlier in the stream that gave up a bounded wait - the
  // rendezvous before this reduction, above all - leaves a code there; the reduction then stores nothing, so that
  // sums over staging memory a late GPU has not filled never reach anybody's output.
  const int *status;
};
cudaError_t launch_reduce_dequant(const ReduceLaunch &r, int sms, cudaStream_t stream);

// Cross-GPU rendezvous on flag words in peer-mapped memory. flags[q] points at GPU q's array of `world` 32-bit words;
// this GPU (index `rank`) stores `epoch` into word `rank` of every GPU's array (mode 0 or 1) and then waits, for at
// most about a second, until every word of its own array has reached `epoch` (mode 0 or 2). A wait that runs out
// leaves kStatusPeerTimeout in the status word and the kernel returns; nothing spins for ever.
struct PeerSync {
  unsigned int *flags[kMaxPeers];
  int rank, world, mode;
  unsigned int epoch;
  int *status;
  long long limit_cycles;
};
cudaError_t launch_peer_sync(const PeerSync &p, cudaStream_t stream);

// Issue-rate probe of the int8 tensor pipe (mma_probe.cu). *ctas: CTAs wanted in, CTAs launched out (CTA pairs are
// limited to what can be resident at once). cycles[cta] receives each CTA's clock64 span, 0 if its wait ran out.
cudaError_t launch_mma_probe(int pair, int iters, int *ctas, int *status, unsigned long long *cycles,
                             cudaStream_t stream);

// Self-test: a kernel whose bounded wait must expire after `limit_cycles` and report through the status word.
cudaError_t launch_expire_wait(int *status, long long limit_cycles, cudaStream_t stream);

// Everything one launch of the int8 product needs. Tensor maps are built by the caller (capi.cu) because they
// need the driver entry point and are cached per context.
struct GemmLaunch {
  CUtensorMap map_a;   // int8 [M][K], box 128 x 128 (rows x bytes), 128-byte swizzle
  CUtensorMap map_w;   // int8 [N][K], box BN x 128
  CUtensorMap map_t;   // fp16 [M][R], box 128 x 32 halves, 64-byte swizzle (LoRA only)
  CUtensorMap map_b;   // fp16 [N][R], box BN x 32 halves (LoRA only)
  CUtensorMap map_c;   // 16-bit output [M][N] rows c_stride apart, box 32 rows x 64 columns, 128-byte swizzle (tma_store only)
  const float *sw;     // [N]
  const float *sa;     // [M]
  const float *bias;   // [N] or null
  void *c;             // [M][c_stride] of c_dtype
  const int *ranges;   // (k0, k1) per BN-wide column tile, or null for the whole rank range
  const unsigned char *rtype;  // gated-residual epilogue: one type byte per row, else null
  const float *gate;   // gated-residual epilogue: fp32 [types][g_stride]
  long long g_stride;
  long long c_stride;
  int c_dtype;         // kDtypeBf16 / kDtypeF16 / kDtypeF32, or kDtypeI32 for the raw accumulators
  int M, N, K;
  int R;               // LoRA rank (multiple of 32), 0 = no low-rank term
  int bn;              // tile width: 32, 64, 128 or 256
  int acc_stages;      // accumulator buffers in tensor memory: 1 or 2
  int band;            // row tiles swept per column tile before moving on (L2 reuse)
  int grid;            // CTAs (persistent)
  int *status;         // device status word of the context
  // Row-parallel push (K-sharded layers over several GPUs): rows [o * peer_rows, (o + 1) * peer_rows) of the result
  // belong to GPU o, and this GPU's partial product of those rows is stored straight into peer_c[o], its slot
  // [peer_rows][c_stride] in o's staging memory (a peer mapping; o == this GPU for its own rows). c_dtype is then
  // kDtypeI32 (raw partial accumulators, summed exactly by the owner) or kDtypeBf16 (dequantised partials without
  // bias). peer_rows == 0: no push, `c` is used.
  void *peer_c[kMaxPeers];
  int peer_rows;
  int overlap;         // host side: launch with programmatic stream serialization (prologue overlaps the previous kernel's tail)
  int tma_store;       // CTA pairs: the epilogue stages 16-bit outputs in shared memory and TMA stores them (map_c)
};

// Shared memory a launch with this tile width and rank needs for `stages` operand stages; 0 if unsupported.
size_t gemm_smem_bytes(int bn, int R, int stages);
// Largest stage count (<= 8) that fits the device's opt-in shared memory, or 0. push: the row-parallel push's
// transposition buffers are part of the launch.
int gemm_pick_stages(int bn, int R, size_t smem_optin, bool push = false);
cudaError_t gemm_configure(int device);  // raises the dynamic shared-memory limit of every instantiation
cudaError_t launch_gemm_w8a8(const GemmLaunch &g, int stages, cudaStream_t stream);

// CTA-pair variant (256 x 256 tile per cluster of two CTAs). map_w and map_b must have boxes of 128 rows (each CTA
// stages half of the W tile and of the low-rank term's B' rows); g.band counts 256-row tiles; g.bn is ignored;
// g.ranges, if given, holds one (k0, k1) per 256-column tile.
size_t gemm_pair_smem_bytes(int stages, bool staged_stores);
int gemm_pair_pick_stages(size_t smem_optin, bool staged_stores);
cudaError_t gemm_pair_configure();
int gemm_pair_max_clusters(int stages);
cudaError_t launch_gemm_w8a8_pair(const GemmLaunch &g, int stages, int clusters, cudaStream_t stream);

}  // namespace h3b
