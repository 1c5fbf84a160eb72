// Rotate + per-token int8 quantise, TMA-fed variant for 16-bit inputs (the path's normal case).
//
// Same arithmetic as rot_q8.cu (the reference's kernel rot_q8, kernels/ops.metal:274-334, operation by operation);
// what differs is how rows reach the registers. Rows are fetched by TMA into a ring of shared-memory stages a few
// rows ahead of the arithmetic, so the kernel has tens of kilobytes per SM in flight without spending registers or
// load instructions on it, and the warps only compute:
//   * the input [M][x_stride] is described to TMA as a 3-D tensor {64 channels, cols / 64 chunks, M rows}; one
//     cp.async.bulk.tensor copy brings a whole row (D / 64 chunks of 128 bytes) into a stage, 128-byte swizzled;
//   * thread t owns chunk t: it reads its 128 bytes with eight 16-byte shared-memory loads; the swizzle places
//     piece k of chunk t at column k ^ (t & 7), so the eight threads of a quarter-warp hit eight different bank
//     groups although their chunks lie 128 bytes apart;
//   * after the row maximum has been exchanged (the one CTA barrier per row) every thread has finished reading the
//     stage, and thread 0 re-arms it with the row `stages` rows ahead; no separate "empty" barrier is needed.
// A CTA has one warp per 2048 channels (D <= 16384); CTAs are persistent over rows m = blockIdx.x, += gridDim.x.
// Waits on the stage barriers are bounded: on a timeout the CTA sets the context's status word, stops taking rows,
// waits (bounded) for its copies in flight and returns.
#include <cuda.h>

#include <map>
#include <mutex>

#include "kernels.h"
#include "ptx.cuh"
#include "rot_common.cuh"

namespace h3b {
namespace {

using namespace rot;

constexpr int kMaxStages = 4;

struct RotTmaArgs {
  CUtensorMap map;     // {64, cols / 64, M} of the 16-bit input, box {64, D / 64, 1}, 128-byte swizzle
  void *out;
  float *sa;
  int *status;
  int M, D;
  int stages;          // ring depth
  int stage_bytes;     // bytes per stage (value row, then gate row; each padded to 1024)
  int gate_offset;     // offset of the gate row inside a stage
  float normaliser;
  int scale_mode;      // 0: scale from this row's maximum; 1: only write the maximum to sa; 2: sa holds the maximum to use
};

// 64 consecutive 16-bit values of chunk `t` of a stage, widened to fp32.
template <bool IS_HALF>
__device__ __forceinline__ void read_chunk(const uint8_t *stage, int t, float (&v)[kChunk]) {
  const uint8_t *row = stage + t * 128;
  const int sw = t & 7;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint4 q = *reinterpret_cast<const uint4 *>(row + ((k ^ sw) << 4));
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (IS_HALF) {
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

template <bool IS_HALF, int BLOCK, bool SWIGLU, bool OUT_HR>
__global__ void __launch_bounds__(256) rot_q8_tma_kernel(const __grid_constant__ RotTmaArgs p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw_addr);
  const uint32_t tail = p.stages * p.stage_bytes;
  const uint32_t bars = base + tail;                                       // full[kMaxStages]
  float *warp_max = reinterpret_cast<float *>(base_ptr + tail + 64);       // [2][8]
  volatile int *cta_abort = reinterpret_cast<volatile int *>(base_ptr + tail + 128);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
  const int n_chunks = p.D / kChunk;
  const bool active = tid < n_chunks;
  const float2 norm2 = make_float2(p.normaliser, p.normaliser);
  const uint32_t row_bytes = static_cast<uint32_t>(p.D) * 2u;

  auto issue = [&](int s, int m) {  // thread 0 only
    const uint32_t bar = bars + 8u * s;
    mbar_arrive_expect_tx(bar, SWIGLU ? 2u * row_bytes : row_bytes);
    tma_load_3d(base + s * p.stage_bytes, &p.map, bar, 0, 0, m);
    if (SWIGLU) tma_load_3d(base + s * p.stage_bytes + p.gate_offset, &p.map, bar, 0, n_chunks, m);
  };

  if (tid == 0) {
    tma_prefetch_descriptor(&p.map);
    for (int s = 0; s < p.stages; ++s) mbar_init(bars + 8u * s, 1);
    *cta_abort = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      const int m = blockIdx.x + s * gridDim.x;
      if (m < p.M) issue(s, m);
    }
  }

  int it = 0;
  for (int m = blockIdx.x; m < p.M; m += gridDim.x, ++it) {
    const int s = it % p.stages;
    const uint32_t ph = (it / p.stages) & 1u;
    // One thread polls the stage's barrier (a whole CTA spinning on it would eat the issue slots the arithmetic
    // needs); the CTA barrier then releases everybody with a uniform decision: all threads go on or none does.
    const bool arrived = tid != 0 || mbar_wait(bars + 8u * s, ph, cta_abort, p.status, kStatusRotTimeout);
    if (!__syncthreads_and(arrived)) break;

    const uint8_t *stage = base_ptr + s * p.stage_bytes;
    float v[kChunk];
    if (active) {
      read_chunk<IS_HALF>(stage, tid, v);
      if (SWIGLU) {
        float g[kChunk];
        read_chunk<IS_HALF>(stage + p.gate_offset, tid, g);
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[i] = __fmul_rn(v[i], silu(g[i]));
      }
    } else {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[i] = 0.0f;
    }
    chunk_butterflies(v);
    lane_butterflies<BLOCK>(v, lane);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < kChunk; i += 2) {
      const float2 r = __fmul2_rn(make_float2(v[i], v[i + 1]), norm2);
      v[i] = r.x; v[i + 1] = r.y;
      amax = fmaxf(amax, fmaxf(fabsf(r.x), fabsf(r.y)));
    }
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, sft));
    float *wm = warp_max + (it & 1) * 8;
    if (lane == 0) wm[warp] = amax;
    __syncthreads();  // row maximum exchanged; also: every thread is done reading this stage
    if (tid == 0) {
      const int m_next = m + p.stages * static_cast<int>(gridDim.x);
      if (m_next < p.M) issue(s, m_next);
    }
    float row_max = wm[0];
    for (int w = 1; w < n_warps; ++w) row_max = fmaxf(row_max, wm[w]);
    if (!OUT_HR && p.scale_mode == 1) {  // a shard of a longer row: hand the local maximum to the caller
      if (tid == 0) p.sa[m] = row_max;
      continue;
    }
    if (!OUT_HR && p.scale_mode == 2) row_max = p.sa[m];  // the whole row's maximum, reduced over the shards

    if constexpr (OUT_HR) {
      if (active) {
        __half *dst = static_cast<__half *>(p.out) + static_cast<size_t>(m) * p.D + tid * kChunk;
#pragma unroll
        for (int q = 0; q < kChunk / 8; ++q) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __half2 h = __floats2half2_rn(v[8 * q + 2 * j], v[8 * q + 2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t *>(&h);
          }
          reinterpret_cast<uint4 *>(dst)[q] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    } else {
      const float scale = row_max > 0.0f ? __fdiv_rn(row_max, 127.0f) : 1.0f;
      const float rs = __fdiv_rn(1.0f, scale);
      const float2 rs2 = make_float2(rs, rs);
      if (active) {
        uint32_t w[kChunk / 4];
#pragma unroll
        for (int j = 0; j < kChunk / 4; ++j) {
          const float2 y0 = __fmul2_rn(make_float2(v[4 * j], v[4 * j + 1]), rs2);
          const float2 y1 = __fmul2_rn(make_float2(v[4 * j + 2], v[4 * j + 3]), rs2);
          w[j] = pack4_s8(__float2int_rn(y0.x), __float2int_rn(y0.y), __float2int_rn(y1.x), __float2int_rn(y1.y));
        }
        uint4 *d4 = reinterpret_cast<uint4 *>(static_cast<int8_t *>(p.out) + static_cast<size_t>(m) * p.D + tid * kChunk);
#pragma unroll
        for (int j = 0; j < kChunk / 16; ++j) d4[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
      }
      if (tid == 0) p.sa[m] = scale;
    }
  }

  if (*cta_abort && tid == 0) {
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

template <bool IS_HALF, int BLOCK, bool SWIGLU, bool OUT_HR>
cudaError_t launch_final(const RotTmaArgs &a, int threads, size_t smem, int sms, cudaStream_t stream) {
  auto *fn = rot_q8_tma_kernel<IS_HALF, BLOCK, SWIGLU, OUT_HR>;
  const long long resident = static_cast<long long>(sms) * resident_ctas(reinterpret_cast<const void *>(fn), threads, smem);
  const int grid = static_cast<int>(a.M < resident ? a.M : resident);
  fn<<<grid, threads, smem, stream>>>(a);
  return cudaGetLastError();
}

template <bool IS_HALF, int BLOCK>
cudaError_t launch_mode(const RotTmaArgs &a, int threads, size_t smem, int sms, int mode, int out_hr, cudaStream_t stream) {
  if (out_hr) {
    return mode == 1 ? launch_final<IS_HALF, BLOCK, true, true>(a, threads, smem, sms, stream)
                     : launch_final<IS_HALF, BLOCK, false, true>(a, threads, smem, sms, stream);
  }
  return mode == 1 ? launch_final<IS_HALF, BLOCK, true, false>(a, threads, smem, sms, stream)
                   : launch_final<IS_HALF, BLOCK, false, false>(a, threads, smem, sms, stream);
}

template <bool IS_HALF>
cudaError_t launch_block(const RotTmaArgs &a, int block, int threads, size_t smem, int sms, int mode, int out_hr,
                         cudaStream_t stream) {
  switch (block) {
    case 64: return launch_mode<IS_HALF, 64>(a, threads, smem, sms, mode, out_hr, stream);
    case 128: return launch_mode<IS_HALF, 128>(a, threads, smem, sms, mode, out_hr, stream);
    default: return launch_mode<IS_HALF, 256>(a, threads, smem, sms, mode, out_hr, stream);
  }
}

}  // namespace

bool rot_q8_tma_supported(int x_dtype, int D) {
  return (x_dtype == kDtypeBf16 || x_dtype == kDtypeF16) && D % kChunk == 0 && D / kChunk <= 256;
}

void rot_q8_tma_plan(int D, int mode, int stages_wanted, int *threads, int *stages, int *stage_bytes, int *gate_offset,
                     size_t *smem) {
  const int row = (D * 2 + 1023) / 1024 * 1024;
  *gate_offset = row;
  *stage_bytes = mode == 1 ? 2 * row : row;
  // measured: one row ahead (2 stages) is best for plain rows; with gates a stage is twice as large and a single
  // stage, which lets more CTAs share an SM, wins
  int s = stages_wanted > 0 ? stages_wanted : (mode == 1 ? 1 : 2);
  if (s > kMaxStages) s = kMaxStages;
  while (s > 1 && static_cast<size_t>(s) * *stage_bytes + 2048 > 232448) --s;
  *stages = s;
  *threads = (D / kChunk + 31) / 32 * 32;
  *smem = 1024 + static_cast<size_t>(s) * *stage_bytes + 256;
}

cudaError_t launch_rot_q8_tma(const CUtensorMap &map, int x_dtype, void *out, float *sa, int M, int D, int block,
                              int mode, int out_hr, int scale_mode, int stages_wanted, int sms, int *status,
                              cudaStream_t stream) {
  RotTmaArgs a;
  a.map = map; a.out = out; a.sa = sa; a.status = status; a.M = M; a.D = D; a.scale_mode = scale_mode;
  a.normaliser = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
  int threads;
  size_t smem;
  rot_q8_tma_plan(D, mode, stages_wanted, &threads, &a.stages, &a.stage_bytes, &a.gate_offset, &smem);
  if (threads > 256 || smem > 232448) return cudaErrorInvalidConfiguration;
  return x_dtype == kDtypeF16 ? launch_block<true>(a, block, threads, smem, sms, mode, out_hr, stream)
                              : launch_block<false>(a, block, threads, smem, sms, mode, out_hr, stream);
}

}  // namespace h3b
