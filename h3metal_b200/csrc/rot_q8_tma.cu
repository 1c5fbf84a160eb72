// Rotate + per-token int8 quantise, TMA-fed: the normal case of the path (16-bit activations, rows of up to 16384
// channels) and the norm + modulation front end on the fp32 residual stream (rows of up to 8192 channels; the
// scale' and shift vectors of the current row type stay in shared memory and are re-fetched only when the type of a
// CTA's next row differs).
//
// Same arithmetic as rot_q8.cu / norm_mod_q8.cu (the reference's kernels rot_q8, kernels/ops.metal:274-334, and
// norm_mod_q8, :111-268, operation by operation); what differs is how rows reach the registers. Rows are fetched by
// TMA into a ring of shared-memory stages ahead of the arithmetic, so the kernel has tens of kilobytes per SM in
// flight without spending registers or load instructions on it, and the warps only compute:
//   * the input [M][stride] is described to TMA as a 3-D tensor {128 bytes of channels, chunks, M rows}; one
//     cp.async.bulk.tensor copy brings a whole row into a stage, 128-byte swizzled;
//   * thread t owns CH = 64 consecutive channels: one 128-byte shared-memory line for 16-bit inputs (eight 16-byte
//     loads), two lines for fp32. The swizzle places piece k of line r at column k ^ (r & 7), so the eight threads
//     of a quarter-warp hit different bank groups although their lines lie 128 (or 256) bytes apart. With CH = 32
//     (16-bit inputs only) a thread owns half a line: half the registers per thread, so twice the threads per SM
//     hide the latencies of the arithmetic, at the price of one more cross-lane butterfly stage;
//   * after the first CTA barrier of a row (the exchange of the row statistic: the sum of squares with the norm
//     front end, else the row maximum) every thread has finished reading the stage, and thread 0 re-arms it with
//     the row `stages` rows ahead; no separate "empty" barrier is needed.
// One warp per 32 CH channels; CTAs are persistent over rows m = blockIdx.x, += gridDim.x. Only one thread polls a
// stage's barrier; the CTA barrier that follows releases everybody with a uniform go / stop decision. Waits are
// bounded: on a timeout the CTA sets the context's status word, stops taking rows, waits (bounded) for its copies
// in flight and returns.
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "kernels.h"
#include "ptx.cuh"
#include "rot_common.cuh"

namespace h3b {
namespace {

using namespace rot;

constexpr int kMaxStages = 4;
enum Front : int { kPlain = 0, kSwiglu = 1, kNorm = 2 };           // what happens before the rotation
enum OutKind : int { kOutQ8 = 0, kOutF32 = 1, kOutF16 = 2, kOutHr = 3 };  // codes+scales, modulated fp32 / fp16, rotated fp16

struct RotTmaArgs {
  CUtensorMap map;     // {128 bytes of channels, cols * esize / 128, M}, box {., D * esize / 128, 1}, 128-byte swizzle
  CUtensorMap map_mod; // norm front end: the modulation table as {32 floats, mod_stride / 32, types}, same box
  void *out;
  float *sa;
  int *status;
  const float *mod;            // norm front end: per row type D scale' then D shift values
  const unsigned char *rtype;  // norm front end: row types
  long long mod_stride;
  int M, D;
  int stages;          // ring depth
  int stage_bytes;     // bytes per stage (value row, then gate row; each padded to 1024)
  int gate_offset;     // offset of the gate row in a stage; norm front end: distance from the scale' to the shift vector
  int mod_bytes;       // norm front end: bytes behind the stages that hold the current row type's scale' and shift vectors
  float normaliser;
  float eps;
  int scale_mode;      // 0: scale from this row's maximum; 1: only write the maximum to sa; 2: sa holds the maximum to use
  int overlap;         // host side: launch with programmatic stream serialization
  RotShardArgs shard;  // where scale_mode 1 stores the maxima and scale_mode 2 finds them (see kernels.h)
};

// CH consecutive values of the thread's chunk `t`, widened to fp32. IN: 0 bf16, 1 fp16 (a line, or half a line with
// CH = 32), 2 fp32 (two lines, or one with CH = 32).
template <int IN, int CH>
__device__ __forceinline__ void read_chunk(const uint8_t *stage, int t, float (&v)[CH]) {
  if constexpr (IN == 2) {
    static_assert(CH == 64 || CH == 32, "fp32 rows are read one or two lines per thread");
#pragma unroll
    for (int half = 0; half < CH / 32; ++half) {
      const int line = (CH / 32) * t + half;
      const uint8_t *row = stage + line * 128;
      const int sw = line & 7;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float4 q = *reinterpret_cast<const float4 *>(row + ((k ^ sw) << 4));
        v[32 * half + 4 * k] = q.x; v[32 * half + 4 * k + 1] = q.y;
        v[32 * half + 4 * k + 2] = q.z; v[32 * half + 4 * k + 3] = q.w;
      }
    }
  } else {
    constexpr int kPieces = CH / 8;                       // 16-byte pieces per thread: 8 (a whole line) or 4
    const int line = CH == 64 ? t : t >> 1;
    const int first = CH == 64 ? 0 : (t & 1) * 4;
    const uint8_t *row = stage + line * 128;
    const int sw = line & 7;
#pragma unroll
    for (int k = 0; k < kPieces; ++k) {
      const uint4 q = *reinterpret_cast<const uint4 *>(row + (((first + k) ^ sw) << 4));
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (IN == 1) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
          v[8 * k + 2 * j] = f.x;
          v[8 * k + 2 * j + 1] = f.y;
        } else {
          v[8 * k + 2 * j] = __uint_as_float(w[j] << 16);
          v[8 * k + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
      }
    }
  }
}

// Sum of the thread's 64 values: four interleaved partial sums, combined pairwise. With the lane tree and the
// sequential pass over the warps below this fixes the (fp32) summation order of the row statistics.
template <int N>
__device__ __forceinline__ float sum64(const float (&v)[N], bool squares) {
  float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
  for (int i = 0; i < N; ++i) s[i & 3] = __fadd_rn(s[i & 3], squares ? __fmul_rn(v[i], v[i]) : v[i]);
  return __fadd_rn(__fadd_rn(s[0], s[1]), __fadd_rn(s[2], s[3]));
}

template <int IN, int BLOCK, int FRONT, bool LN, int OUT, int CH = kChunk>
__global__ void __launch_bounds__(CH == 32 ? 512 : 256) rot_q8_tma_kernel(const __grid_constant__ RotTmaArgs p) {
  static_assert(CH == 64 || CH == 32, "a thread owns 64 or 32 channels");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw_addr);
  const uint32_t mod_off = p.stages * p.stage_bytes;                       // norm front end: scale' | shift of one row type
  const uint32_t tail = mod_off + p.mod_bytes;
  const uint32_t bars = base + tail;                                       // full[kMaxStages], then the vectors' barrier
  const uint32_t mod_bar = bars + 8u * kMaxStages;
  float *exchange = reinterpret_cast<float *>(base_ptr + tail + 64);       // [4][16]: row statistics, rotating buffers
  volatile int *cta_abort = reinterpret_cast<volatile int *>(base_ptr + tail + 320);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
  const int n_chunks = p.D / CH;
  const bool active = tid < n_chunks;
  const float2 norm2 = make_float2(p.normaliser, p.normaliser);
  constexpr int kEsize = IN == 2 ? 4 : 2;
  const uint32_t row_bytes = static_cast<uint32_t>(p.D) * kEsize;
  const int lines = p.D * kEsize / 128;  // 128-byte lines per row

  auto issue = [&](int s, int m) {  // thread 0 only
    const uint32_t bar = bars + 8u * s;
    mbar_arrive_expect_tx(bar, FRONT == kSwiglu ? 2u * row_bytes : row_bytes);
    tma_load_3d(base + s * p.stage_bytes, &p.map, bar, 0, 0, m);
    if (FRONT == kSwiglu) tma_load_3d(base + s * p.stage_bytes + p.gate_offset, &p.map, bar, 0, lines, m);
  };
  // Norm front end: the scale' and shift vectors of ONE row type live in shared memory behind the stages (so that
  // the modulation reads shared memory instead of waiting on dependent global loads) and are fetched by TMA, from
  // L2 where the small table lives, only when a row's type differs from the row before it in this CTA.
  int cur_type = -1;        // thread 0 only
  int next_type = 0;        // thread 0 only: type of the row this CTA takes next, read one row ahead of its use
  uint32_t mod_loads = 0;   // thread 0 only: completed fetches (the barrier's phase)
  bool mod_pending = false;

  if (tid == 0) {
    tma_prefetch_descriptor(&p.map);
    if (FRONT == kNorm) tma_prefetch_descriptor(&p.map_mod);
    for (int s = 0; s < p.stages; ++s) mbar_init(bars + 8u * s, 1);
    mbar_init(mod_bar, 1);
    *cta_abort = 0;
    fence_barrier_init();
  }
  __syncthreads();
  // so far only this CTA's shared memory was touched; global memory must wait for the previous kernel in the stream
  grid_dep_launch();
  grid_dep_wait();
  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      const int m = blockIdx.x + s * gridDim.x;
      if (m < p.M) issue(s, m);
    }
    if (FRONT == kNorm && static_cast<int>(blockIdx.x) < p.M) next_type = p.rtype[blockIdx.x];
  }

  int it = 0;
  unsigned xbuf = 0;  // which exchange buffer the next CTA-wide reduction uses
  // CTA-wide reduction of one value per thread: lane tree, then the warps in order. One barrier per call.
  auto cta_reduce = [&](float v, bool is_max) {
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) {
      const float o = __shfl_xor_sync(0xFFFFFFFFu, v, sft);
      v = is_max ? fmaxf(v, o) : __fadd_rn(v, o);
    }
    float *buf = exchange + (xbuf++ & 3u) * 16;
    if (lane == 0) buf[warp] = v;
    __syncthreads();
    float r = buf[0];
    for (int w = 1; w < n_warps; ++w) r = is_max ? fmaxf(r, buf[w]) : __fadd_rn(r, buf[w]);
    return r;
  };

  for (int m = blockIdx.x; m < p.M; m += gridDim.x, ++it) {
    const int s = it % p.stages;
    const uint32_t ph = (it / p.stages) & 1u;
    bool arrived = true;
    if (tid == 0) {
      if (FRONT == kNorm) {
        // every thread is past the last barrier of the row before, and the vectors are read before that barrier:
        // they may be replaced now
        const int type = next_type;
        if (m + static_cast<int>(gridDim.x) < p.M) next_type = p.rtype[m + gridDim.x];  // used one row from now
        if (type != cur_type) {
          mbar_arrive_expect_tx(mod_bar, 2u * row_bytes);
          tma_load_3d(base + mod_off, &p.map_mod, mod_bar, 0, 0, type);
          tma_load_3d(base + mod_off + p.gate_offset, &p.map_mod, mod_bar, 0, lines, type);
          mod_pending = true;
          arrived = mbar_wait(mod_bar, mod_loads & 1u, cta_abort, p.status, kStatusRotTimeout);
          if (arrived) {
            mod_pending = false;
            ++mod_loads;
            cur_type = type;
          }
        }
      }
      arrived = arrived && mbar_wait(bars + 8u * s, ph, cta_abort, p.status, kStatusRotTimeout);
    }
    if (!__syncthreads_and(arrived)) break;

    const uint8_t *stage = base_ptr + s * p.stage_bytes;
    float v[CH];
    if (active) {
      read_chunk<IN, CH>(stage, tid, v);
      if (FRONT == kSwiglu) {
        float g[CH];
        read_chunk<IN, CH>(stage + p.gate_offset, tid, g);
#pragma unroll
        for (int i = 0; i < CH; ++i) v[i] = __fmul_rn(v[i], silu(g[i]));
      }
    } else {
#pragma unroll
      for (int i = 0; i < CH; ++i) v[i] = 0.0f;
    }
    bool refilled = false;
    auto refill = [&]() {  // after a CTA barrier that follows the reads: the stage may be overwritten
      if (!refilled && tid == 0) {
        const int m_next = m + p.stages * static_cast<int>(gridDim.x);
        if (m_next < p.M) issue(s, m_next);
      }
      refilled = true;
    };

    if constexpr (FRONT == kNorm) {
      // RMSNorm (LayerNorm: mean removed first), then v * inv * scale'[type] + shift[type]
      const float fd = static_cast<float>(p.D);
      if (LN) {
        const float mean = __fdiv_rn(cta_reduce(sum64(v, false), false), fd);
        refill();  // the row is in registers and everybody has passed a barrier since: its stage is free
        if (active) {
#pragma unroll
          for (int i = 0; i < CH; ++i) v[i] = __fsub_rn(v[i], mean);
        }
      }
      const float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(cta_reduce(sum64(v, true), false), fd), p.eps));
      refill();
      if (active) {
        float sc[CH], sh[CH];
        read_chunk<2, CH>(base_ptr + mod_off, tid, sc);
        read_chunk<2, CH>(base_ptr + mod_off + p.gate_offset, tid, sh);
        const float2 inv2 = make_float2(inv, inv);
#pragma unroll
        for (int i = 0; i < CH; i += 2) {
          float2 x = __fmul2_rn(__fmul2_rn(make_float2(v[i], v[i + 1]), inv2), make_float2(sc[i], sc[i + 1]));
          x = __fadd2_rn(x, make_float2(sh[i], sh[i + 1]));
          v[i] = x.x; v[i + 1] = x.y;
        }
      }
      if (OUT == kOutF32 || OUT == kOutF16) {
        // no further exchange follows: a barrier of its own before the next row may replace the vectors
        __syncthreads();
      }
    }

    if constexpr (OUT == kOutF32) {
      if (active) {
        float4 *o = reinterpret_cast<float4 *>(static_cast<float *>(p.out) + static_cast<size_t>(m) * p.D + tid * CH);
#pragma unroll
        for (int q = 0; q < CH / 4; ++q) o[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      }
      continue;
    }
    if constexpr (OUT != kOutF16) {  // rotation
      chunk_butterflies(v);
      lane_butterflies<BLOCK>(v, lane);
#pragma unroll
      for (int i = 0; i < CH; i += 2) {
        const float2 r = __fmul2_rn(make_float2(v[i], v[i + 1]), norm2);
        v[i] = r.x; v[i + 1] = r.y;
      }
    }
    if constexpr (OUT == kOutF16 || OUT == kOutHr) {
      if (!(FRONT == kNorm && OUT == kOutF16)) {  // no exchange follows the last read: a barrier of its own frees the stage
        __syncthreads();
        refill();
      }
      if (active) {
        __half *dst = static_cast<__half *>(p.out) + static_cast<size_t>(m) * p.D + tid * CH;
#pragma unroll
        for (int q = 0; q < CH / 8; ++q) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __half2 h = __floats2half2_rn(v[8 * q + 2 * j], v[8 * q + 2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t *>(&h);
          }
          reinterpret_cast<uint4 *>(dst)[q] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      continue;
    }
    if constexpr (OUT == kOutQ8) {
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < CH; i += 2) amax = fmaxf(amax, fmaxf(fabsf(v[i]), fabsf(v[i + 1])));
      float row_max = cta_reduce(amax, true);
      refill();
      if (p.scale_mode == 1) {  // a shard of a longer row: hand the local maximum to the caller (or to every GPU)
        if (tid < p.shard.n_dst) p.shard.amax_dst[tid][m] = row_max;
        continue;
      }
      if (p.scale_mode == 2) {  // the whole row's maximum: already reduced over the shards, or one slot per shard
        row_max = p.sa[m];
        for (int sl = 1; sl < p.shard.amax_slots; ++sl) row_max = fmaxf(row_max, p.sa[sl * p.shard.amax_slot_stride + m]);
      }
      const float scale = row_max > 0.0f ? __fdiv_rn(row_max, 127.0f) : 1.0f;
      const float rs = __fdiv_rn(1.0f, scale);
      const float2 rs2 = make_float2(rs, rs);
      if (active) {
        uint32_t w[CH / 4];
#pragma unroll
        for (int j = 0; j < CH / 4; ++j) {
          const float2 y0 = __fmul2_rn(make_float2(v[4 * j], v[4 * j + 1]), rs2);
          const float2 y1 = __fmul2_rn(make_float2(v[4 * j + 2], v[4 * j + 3]), rs2);
          w[j] = pack4_s8(__float2int_rn(y0.x), __float2int_rn(y0.y), __float2int_rn(y1.x), __float2int_rn(y1.y));
        }
        uint4 *d4 = reinterpret_cast<uint4 *>(static_cast<int8_t *>(p.out) + static_cast<size_t>(m) * p.D + tid * CH);
#pragma unroll
        for (int j = 0; j < CH / 16; ++j) d4[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
      }
      if (tid == 0) p.shard.scale_out[m] = scale;
    }
  }

  if (*cta_abort && tid == 0) {
    if (FRONT == kNorm && mod_pending) {
      int ignore = 0;
      mbar_wait(mod_bar, mod_loads & 1u, &ignore, p.status, kStatusDrainTimeout, kDrainLimitCycles);
    }
    // wind-down after a timeout: rows it .. it + stages - 1 may still be landing in shared memory
    for (int j = it; j < it + p.stages; ++j) {
      if (blockIdx.x + static_cast<long long>(j) * gridDim.x >= p.M) break;
      int ignore = 0;
      mbar_wait(bars + 8u * (j % p.stages), (j / p.stages) & 1u, &ignore, p.status, kStatusDrainTimeout,
                kDrainLimitCycles);
    }
  }
  __syncthreads();
}

int resident_ctas(const void *fn, int threads, size_t smem) {
  static std::mutex mu;
  static std::map<std::tuple<const void *, int, size_t>, int> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple(fn, threads, smem);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  int n = 0;
  cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, threads, smem) != cudaSuccess || n < 1) n = 1;
  cache[key] = n;
  return n;
}

template <int IN, int BLOCK, int FRONT, bool LN, int OUT, int CH = kChunk>
cudaError_t launch_final(const RotTmaArgs &a, int threads, size_t smem, int sms, cudaStream_t stream) {
  auto *fn = rot_q8_tma_kernel<IN, BLOCK, FRONT, LN, OUT, CH>;
  const long long resident = static_cast<long long>(sms) * resident_ctas(reinterpret_cast<const void *>(fn), threads, smem);
  const int grid = static_cast<int>(a.M < resident ? a.M : resident);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, fn, a);
}

template <int IN, int BLOCK, int CH>
cudaError_t launch_rot(const RotTmaArgs &a, int threads, size_t smem, int sms, int mode, int out_hr, cudaStream_t stream) {
  if (out_hr) {
    return mode == 1 ? launch_final<IN, BLOCK, kSwiglu, false, kOutHr, CH>(a, threads, smem, sms, stream)
                     : launch_final<IN, BLOCK, kPlain, false, kOutHr, CH>(a, threads, smem, sms, stream);
  }
  return mode == 1 ? launch_final<IN, BLOCK, kSwiglu, false, kOutQ8, CH>(a, threads, smem, sms, stream)
                   : launch_final<IN, BLOCK, kPlain, false, kOutQ8, CH>(a, threads, smem, sms, stream);
}

template <int BLOCK, bool LN, int CH>
cudaError_t launch_norm_ch(const RotTmaArgs &a, int threads, size_t smem, int sms, int out_kind, cudaStream_t stream) {
  switch (out_kind) {
    case kOutQ8: return launch_final<2, BLOCK, kNorm, LN, kOutQ8, CH>(a, threads, smem, sms, stream);
    case kOutF32: return launch_final<2, BLOCK, kNorm, LN, kOutF32, CH>(a, threads, smem, sms, stream);
    case kOutF16: return launch_final<2, BLOCK, kNorm, LN, kOutF16, CH>(a, threads, smem, sms, stream);
    default: return launch_final<2, BLOCK, kNorm, LN, kOutHr, CH>(a, threads, smem, sms, stream);
  }
}
template <int BLOCK, bool LN>
cudaError_t launch_norm(const RotTmaArgs &a, int chunk, int threads, size_t smem, int sms, int out_kind, cudaStream_t stream) {
  return chunk == 32 ? launch_norm_ch<BLOCK, LN, 32>(a, threads, smem, sms, out_kind, stream)
                     : launch_norm_ch<BLOCK, LN, 64>(a, threads, smem, sms, out_kind, stream);
}

void plan(int D, int esize, bool gates, int stages_wanted, int chunk, RotTmaArgs *a, int *threads, size_t *smem) {
  const int row = (D * esize + 1023) / 1024 * 1024;
  a->gate_offset = row;
  a->stage_bytes = gates ? 2 * row : row;
  a->mod_bytes = esize == 4 ? 2 * row : 0;  // norm front end: one row type's scale' and shift vectors
  // measured: one row ahead (2 stages) is best for plain 16-bit rows; with gates, or with fp32 rows and their
  // vectors, a CTA's footprint is large and a single stage, which lets more CTAs share an SM, wins
  int s = stages_wanted > 0 ? stages_wanted : ((gates || esize == 4) ? 1 : 2);
  if (s > kMaxStages) s = kMaxStages;
  while (s > 1 && static_cast<size_t>(s) * a->stage_bytes + a->mod_bytes + 2048 > 232448) --s;
  a->stages = s;
  *threads = (D / chunk + 31) / 32 * 32;
  *smem = 1024 + static_cast<size_t>(s) * a->stage_bytes + a->mod_bytes + 512;
}

}  // namespace

bool rot_q8_tma_supported(int x_dtype, int D) {
  return (x_dtype == kDtypeBf16 || x_dtype == kDtypeF16) && D % kChunk == 0 && D / kChunk <= 256;
}
bool norm_mod_q8_tma_supported(int D) { return D % kChunk == 0 && D / 32 <= 256; }  // the box holds D / 32 lines

cudaError_t launch_rot_q8_tma(const CUtensorMap &map, int x_dtype, void *out, float *sa, int M, int D, int block,
                              int mode, int out_hr, int scale_mode, int stages_wanted, int chunk_wanted, int sms,
                              int *status, cudaStream_t stream, bool overlap, const RotShardArgs *shard) {
  RotTmaArgs a = {};
  a.map = map; a.out = out; a.sa = sa; a.status = status; a.M = M; a.D = D; a.scale_mode = scale_mode;
  a.overlap = overlap ? 1 : 0;
  if (shard) {
    a.shard = *shard;
  } else {
    a.shard.amax_dst[0] = sa; a.shard.n_dst = 1; a.shard.amax_slots = 1; a.shard.amax_slot_stride = 0; a.shard.scale_out = sa;
  }
  a.normaliser = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
  int threads;
  size_t smem;
  // measured: half-line chunks (twice the threads) win for short rows, whole lines from about 3840 channels on
  const int chunk = chunk_wanted == 32 || chunk_wanted == 64 ? chunk_wanted : (D <= 3072 ? 32 : kChunk);
  plan(D, 2, mode == 1, stages_wanted, chunk, &a, &threads, &smem);
  if (threads > (chunk == 32 ? 512 : 256) || smem > 232448) return cudaErrorInvalidConfiguration;
#define H3B_ROT(IN, CH)                                                                    \
  switch (block) {                                                                         \
    case 64: return launch_rot<IN, 64, CH>(a, threads, smem, sms, mode, out_hr, stream);   \
    case 128: return launch_rot<IN, 128, CH>(a, threads, smem, sms, mode, out_hr, stream); \
    default: return launch_rot<IN, 256, CH>(a, threads, smem, sms, mode, out_hr, stream);  \
  }
  if (chunk == 32) {
    if (x_dtype == kDtypeF16) { H3B_ROT(1, 32) }
    H3B_ROT(0, 32)
  }
  if (x_dtype == kDtypeF16) { H3B_ROT(1, 64) }
  H3B_ROT(0, 64)
#undef H3B_ROT
}

cudaError_t launch_norm_mod_q8_tma(const CUtensorMap &map, const CUtensorMap &map_mod, const float *mod,
                                   long long mod_stride, const unsigned char *rtype, void *out, float *sa, int M, int D,
                                   int block, float eps, int ln, int out_kind, int stages_wanted, int chunk_wanted, int sms,
                                   int *status, cudaStream_t stream) {
  RotTmaArgs a = {};
  a.map = map; a.map_mod = map_mod; a.out = out; a.sa = sa; a.status = status; a.M = M; a.D = D; a.scale_mode = 0;
  a.shard.amax_dst[0] = sa; a.shard.n_dst = 1; a.shard.amax_slots = 1; a.shard.scale_out = sa;
  a.mod = mod; a.mod_stride = mod_stride; a.rtype = rtype; a.eps = eps;
  a.normaliser = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
  int threads;
  size_t smem;
  // measured: 32 channels (one 128-byte line) per thread, twice the warps per SM for the same shared memory, is
  // 12-29 % faster than 64 on this latency-bound kernel
  const int chunk = chunk_wanted == 64 ? kChunk : 32;
  plan(D, 4, false, stages_wanted, chunk, &a, &threads, &smem);
  if (threads > (chunk == 32 ? 512 : 256) || smem > 232448) return cudaErrorInvalidConfiguration;
  switch (block) {
    case 64: return ln ? launch_norm<64, true>(a, chunk, threads, smem, sms, out_kind, stream) : launch_norm<64, false>(a, chunk, threads, smem, sms, out_kind, stream);
    case 128: return ln ? launch_norm<128, true>(a, chunk, threads, smem, sms, out_kind, stream) : launch_norm<128, false>(a, chunk, threads, smem, sms, out_kind, stream);
    default: return ln ? launch_norm<256, true>(a, chunk, threads, smem, sms, out_kind, stream) : launch_norm<256, false>(a, chunk, threads, smem, sms, out_kind, stream);
  }
}

}  // namespace h3b
