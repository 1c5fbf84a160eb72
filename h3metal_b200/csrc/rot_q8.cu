// Rotate + per-token int8 quantise: one fused, HBM-bound pass over the activations.
//
// For every row m of the input: the D values (bf16, fp16 or fp32; optionally value * silu(gate) with the gates in
// columns D..2D-1) are rotated by a block Walsh-Hadamard transform of `block` channels, normalised by
// 1/sqrt(block); the row's largest magnitude gives the scale (amax / 127, or 1 for an all-zero row); the int8
// codes rint(v * (1 / scale)) and the fp32 scale are written out. With out_hr the rotated row is written as fp16
// and nothing is quantised.
//
// This replaces the reference's Metal kernel rot_q8 (kernels/ops.metal:274-334, helpers :19-47 and :62-72). The
// int8 codes are defined by that kernel's sequence of fp32 operations, which is kept: butterfly stages by
// increasing stride, each pair (a, b) becoming (a + b, a - b); ONE multiply by the normaliser after the last
// stage; rs = 1 / scale; rint(v * rs), ties to even, no clamp. Nothing here may be contracted into a fused
// multiply-add or reassociated, so the arithmetic is written with the _rn intrinsics.
//
// Mapping to the GPU. The kernel is bound by HBM traffic only if it also stays under the SM's instruction issue
// rate (at full bandwidth an SM has about 16 issue slots per channel), so the layout minimises instructions:
//   * a thread owns `CH` chunks of 64 consecutive channels (eight 128-bit loads per bf16/fp16 chunk, four 128-bit
//     stores of int8 codes); the six butterfly stages of stride 1..32 run in its registers, the last five of them
//     as packed two-wide fp32 operations (add.f32x2 / fma.f32x2, each lane rounded like the scalar operation);
//   * only the stages of stride 64 and up cross lanes (shuffles are the scarcest resource here): none for a block
//     of 64, one for 128, two for 256, between 2 or 4 neighbouring lanes, written as o + sign * v (the product is
//     exact, so the fma rounds once, like the add or subtract it stands for);
//   * CTAs are persistent: a CTA walks rows m = blockIdx.x, += gridDim.x and issues the loads of its next row
//     before it transforms the current one, so every thread always has CH x 128 bytes in flight;
//   * a CTA is as many warps as the row needs (one warp covers 2048 channels per chunk); the row maximum is a
//     warp shuffle reduction plus, only when the row spans several warps, one shared-memory exchange per row.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <map>
#include <mutex>

#include "kernels.h"
#include "rot_common.cuh"

namespace h3b {
namespace {

using namespace rot;

struct RotQArgs {
  const void *x;
  void *out;
  float *sa;
  long long x_stride;  // elements between input rows
  int M, D;
  float normaliser;    // fp32(1 / sqrt(block))
  int scale_mode;      // 0: scale from this row's maximum; 1: only write the maximum to sa; 2: sa holds the maximum to use
};

template <typename IN_T, int BLOCK, int CH, bool SWIGLU, bool OUT_HR>
__global__ void __launch_bounds__(256) rot_q8_kernel(const RotQArgs p) {
  __shared__ float warp_max[2][8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
  const int n_chunks = p.D / kChunk;
  const float2 norm2 = make_float2(p.normaliser, p.normaliser);

  RawChunk<IN_T> next[CH];
  RawChunk<IN_T> next_gate[SWIGLU ? CH : 1];
  auto fetch = [&](int m) {
    const IN_T *row = static_cast<const IN_T *>(p.x) + static_cast<size_t>(m) * p.x_stride;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int chunk = tid + c * blockDim.x;
      if (chunk < n_chunks) {
        next[c].load(row + chunk * kChunk);
        if (SWIGLU) next_gate[SWIGLU ? c : 0].load(row + p.D + chunk * kChunk);
      } else {
        next[c].zero();
        if (SWIGLU) next_gate[SWIGLU ? c : 0].zero();
      }
    }
  };

  int m = blockIdx.x;
  if (m < p.M) fetch(m);
  for (int it = 0; m < p.M; m += gridDim.x, ++it) {
    float v[CH][kChunk];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      widen(next[c], v[c]);
      if (SWIGLU) {
        float g[kChunk];
        widen(next_gate[SWIGLU ? c : 0], g);
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[c][i] = __fmul_rn(v[c][i], silu(g[i]));
      }
    }
    if (m + static_cast<int>(gridDim.x) < p.M) fetch(m + gridDim.x);  // next row's loads fly during this row's math

    float amax = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      chunk_butterflies(v[c]);
      lane_butterflies<BLOCK>(v[c], lane);
#pragma unroll
      for (int i = 0; i < kChunk; i += 2) {
        const float2 r = __fmul2_rn(make_float2(v[c][i], v[c][i + 1]), norm2);
        v[c][i] = r.x; v[c][i + 1] = r.y;
        amax = fmaxf(amax, fmaxf(fabsf(r.x), fabsf(r.y)));
      }
    }

    if constexpr (OUT_HR) {
      __half *dst = static_cast<__half *>(p.out) + static_cast<size_t>(m) * p.D;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int chunk = tid + c * blockDim.x;
        if (chunk < n_chunks) {
#pragma unroll
          for (int q = 0; q < kChunk / 8; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __half2 h = __floats2half2_rn(v[c][8 * q + 2 * j], v[c][8 * q + 2 * j + 1]);
              w[j] = *reinterpret_cast<const uint32_t *>(&h);
            }
            reinterpret_cast<uint4 *>(dst + chunk * kChunk)[q] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    } else {
      // row maximum: lanes, then warps (buffers alternate between rows so one barrier per row is enough)
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, s));
      float row_max = amax;
      if (n_warps > 1) {
        float *wm = warp_max[it & 1];
        if (lane == 0) wm[warp] = amax;
        __syncthreads();
        row_max = wm[0];
        for (int w = 1; w < n_warps; ++w) row_max = fmaxf(row_max, wm[w]);
      }

      if (p.scale_mode == 1) {  // a shard of a longer row: hand the local maximum to the caller
        if (tid == 0) p.sa[m] = row_max;
        continue;
      }
      if (p.scale_mode == 2) row_max = p.sa[m];  // the whole row's maximum, reduced over the shards
      const float scale = row_max > 0.0f ? __fdiv_rn(row_max, 127.0f) : 1.0f;
      const float rs = __fdiv_rn(1.0f, scale);
      const float2 rs2 = make_float2(rs, rs);
      int8_t *dst = static_cast<int8_t *>(p.out) + static_cast<size_t>(m) * p.D;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int chunk = tid + c * blockDim.x;
        if (chunk < n_chunks) {
          uint32_t w[kChunk / 4];
#pragma unroll
          for (int j = 0; j < kChunk / 4; ++j) {
            const float2 y0 = __fmul2_rn(make_float2(v[c][4 * j], v[c][4 * j + 1]), rs2);
            const float2 y1 = __fmul2_rn(make_float2(v[c][4 * j + 2], v[c][4 * j + 3]), rs2);
            // round to nearest, ties to even; |y| <= 127 up to rounding, so the saturating pack never clips
            w[j] = pack4_s8(__float2int_rn(y0.x), __float2int_rn(y0.y), __float2int_rn(y1.x), __float2int_rn(y1.y));
          }
          uint4 *d4 = reinterpret_cast<uint4 *>(dst + chunk * kChunk);
#pragma unroll
          for (int j = 0; j < kChunk / 16; ++j) d4[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        }
      }
      if (tid == 0) p.sa[m] = scale;
    }
  }
}

// CTAs per SM of one instantiation at one CTA size (occupancy query, cached).
int resident_ctas(const void *fn, int threads) {
  static std::mutex mu;
  static std::map<std::pair<const void *, int>, int> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_pair(fn, threads);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, threads, 0) != cudaSuccess || n < 1) n = 1;
  cache[key] = n;
  return n;
}

template <typename IN_T, int BLOCK, int CH, bool SWIGLU, bool OUT_HR>
cudaError_t launch_final(const RotQArgs &a, int threads, int sms, cudaStream_t stream) {
  auto *fn = rot_q8_kernel<IN_T, BLOCK, CH, SWIGLU, OUT_HR>;
  const long long resident = static_cast<long long>(sms) * resident_ctas(reinterpret_cast<const void *>(fn), threads);
  const int grid = static_cast<int>(a.M < resident ? a.M : resident);
  fn<<<grid, threads, 0, stream>>>(a);
  return cudaGetLastError();
}

template <typename IN_T, int BLOCK, int CH>
cudaError_t launch_mode(const RotQArgs &a, int threads, int sms, int mode, int out_hr, cudaStream_t stream) {
  if (out_hr) {
    return mode == 1 ? launch_final<IN_T, BLOCK, CH, true, true>(a, threads, sms, stream)
                     : launch_final<IN_T, BLOCK, CH, false, true>(a, threads, sms, stream);
  }
  return mode == 1 ? launch_final<IN_T, BLOCK, CH, true, false>(a, threads, sms, stream)
                   : launch_final<IN_T, BLOCK, CH, false, false>(a, threads, sms, stream);
}

template <typename IN_T, int BLOCK>
cudaError_t launch_ch(const RotQArgs &a, int ch, int threads, int sms, int mode, int out_hr, cudaStream_t stream) {
  switch (ch) {
    case 1: return launch_mode<IN_T, BLOCK, 1>(a, threads, sms, mode, out_hr, stream);
    default: return launch_mode<IN_T, BLOCK, 2>(a, threads, sms, mode, out_hr, stream);
  }
}

template <typename IN_T>
cudaError_t launch_block(const RotQArgs &a, int block, int ch, int threads, int sms, int mode, int out_hr,
                         cudaStream_t stream) {
  switch (block) {
    case 64: return launch_ch<IN_T, 64>(a, ch, threads, sms, mode, out_hr, stream);
    case 128: return launch_ch<IN_T, 128>(a, ch, threads, sms, mode, out_hr, stream);
    default: return launch_ch<IN_T, 256>(a, ch, threads, sms, mode, out_hr, stream);
  }
}

}  // namespace

// Chunks per thread (1 or 2) and CTA size for a row of D channels: the fewest chunks per thread that keep the
// CTA at or under `threads_target` threads (CTAs are limited to 256 threads, 8 warps, by the row-maximum exchange).
void rot_q8_geometry(int D, int threads_target, int *ch, int *threads) {
  const int n_chunks = (D + kChunk - 1) / kChunk;
  int c = 1;
  while (c < 2 && (n_chunks + c - 1) / c > threads_target) c <<= 1;
  int t = (n_chunks + c - 1) / c;
  t = (t + 31) / 32 * 32;
  *ch = c;
  *threads = t;
}

cudaError_t launch_rot_q8(const void *x, int x_dtype, long long x_stride, void *out, float *sa, int M, int D,
                          int block, int mode, int out_hr, int scale_mode, int threads_target, int sms,
                          cudaStream_t stream) {
  RotQArgs a;
  a.x = x; a.out = out; a.sa = sa; a.x_stride = x_stride; a.M = M; a.D = D; a.scale_mode = scale_mode;
  a.normaliser = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
  int ch, threads;
  rot_q8_geometry(D, threads_target, &ch, &threads);
  if (threads > 256) return cudaErrorInvalidConfiguration;
  switch (x_dtype) {
    case kDtypeBf16: return launch_block<__nv_bfloat16>(a, block, ch, threads, sms, mode, out_hr, stream);
    case kDtypeF16: return launch_block<__half>(a, block, ch, threads, sms, mode, out_hr, stream);
    case kDtypeF32: return launch_block<float>(a, block, ch, threads, sms, mode, out_hr, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace h3b
