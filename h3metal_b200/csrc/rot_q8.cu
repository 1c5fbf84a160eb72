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
//   * a thread owns `CH` chunks of 32 consecutive channels (four 128-bit loads per bf16/fp16 chunk, two 128-bit
//     stores of int8 codes); the five butterfly stages of stride 1..16 run in its registers, the last four of them
//     as packed two-wide fp32 operations (add.f32x2 / fma.f32x2, each lane rounded like the scalar operation);
//   * only the stages of stride 32 and up cross lanes: one shuffle stage for a block of 64, two for 128, three
//     for 256, inside groups of 2, 4 or 8 neighbouring lanes, written as o + sign * v (exact product, one rounding);
//   * CTAs are persistent: a CTA walks rows m = blockIdx.x, += gridDim.x and issues the loads of its next row
//     before it transforms the current one, so every thread always has CH x 64 bytes in flight;
//   * the row maximum goes through a warp shuffle reduction and one shared-memory exchange per row.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include <map>
#include <mutex>

#include "kernels.h"

namespace h3b {
namespace {

constexpr int kChunk = 32;  // consecutive channels a thread owns per chunk

struct RotQArgs {
  const void *x;
  void *out;
  float *sa;
  long long x_stride;  // elements between input rows
  int M, D;
  float normaliser;    // fp32(1 / sqrt(block))
};

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Raw (still packed) input of one chunk: 64 bytes for 16-bit inputs, 128 bytes for fp32.
template <typename IN_T>
struct RawChunk {
  static constexpr int kVec = kChunk * sizeof(IN_T) / 16;
  uint4 q[kVec];
  __device__ __forceinline__ void load(const IN_T *p) {
#pragma unroll
    for (int i = 0; i < kVec; ++i) q[i] = ld_stream16(reinterpret_cast<const uint4 *>(p) + i);
  }
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < kVec; ++i) q[i] = make_uint4(0u, 0u, 0u, 0u);
  }
};

__device__ __forceinline__ void widen(const RawChunk<__nv_bfloat16> &r, float (&v)[kChunk]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w[4] = {r.q[i].x, r.q[i].y, r.q[i].z, r.q[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
      v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
  }
}
__device__ __forceinline__ void widen(const RawChunk<__half> &r, float (&v)[kChunk]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t w[4] = {r.q[i].x, r.q[i].y, r.q[i].z, r.q[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
      v[8 * i + 2 * j] = f.x;
      v[8 * i + 2 * j + 1] = f.y;
    }
  }
}
__device__ __forceinline__ void widen(const RawChunk<float> &r, float (&v)[kChunk]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[4 * i] = __uint_as_float(r.q[i].x);
    v[4 * i + 1] = __uint_as_float(r.q[i].y);
    v[4 * i + 2] = __uint_as_float(r.q[i].z);
    v[4 * i + 3] = __uint_as_float(r.q[i].w);
  }
}

// x / (1 + exp(-x)): accurate expf, then one correctly rounded division.
__device__ __forceinline__ float silu(float g) { return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g))); }

// In-thread butterfly stages of stride 1, 2, 4, 8, 16 over the chunk's 32 values. Stride 1 pairs the two halves of
// a float2 and stays scalar; the others combine whole float2 registers: a + b and fma(b, -1, a) = a - b.
__device__ __forceinline__ void chunk_butterflies(float (&v)[kChunk]) {
#pragma unroll
  for (int i = 0; i < kChunk; i += 2) {
    const float a = v[i], b = v[i + 1];
    v[i] = __fadd_rn(a, b);
    v[i + 1] = __fsub_rn(a, b);
  }
  const float2 minus_one = make_float2(-1.0f, -1.0f);
#pragma unroll
  for (int s = 2; s < kChunk; s <<= 1) {
#pragma unroll
    for (int i = 0; i < kChunk; i += 2) {
      if ((i & s) == 0) {
        const float2 a = make_float2(v[i], v[i + 1]), b = make_float2(v[i + s], v[i + s + 1]);
        const float2 sum = __fadd2_rn(a, b), dif = __ffma2_rn(b, minus_one, a);
        v[i] = sum.x; v[i + 1] = sum.y;
        v[i + s] = dif.x; v[i + s + 1] = dif.y;
      }
    }
  }
}

// Stages of stride 32 .. BLOCK/2: the partner value lives in lane ^ (stride / 32). The lower lane keeps v + o, the
// upper lane o - v; both are o + sign * v with sign = +-1 (the product is exact, so the fma rounds once).
template <int BLOCK>
__device__ __forceinline__ void lane_butterflies(float (&v)[kChunk], int lane) {
#pragma unroll
  for (int s = 1; s < BLOCK / kChunk; s <<= 1) {
    const float sg = (lane & s) ? -1.0f : 1.0f;
    const float2 sign = make_float2(sg, sg);
#pragma unroll
    for (int i = 0; i < kChunk; i += 2) {
      const float2 o = make_float2(__shfl_xor_sync(0xFFFFFFFFu, v[i], s), __shfl_xor_sync(0xFFFFFFFFu, v[i + 1], s));
      const float2 r = __ffma2_rn(make_float2(v[i], v[i + 1]), sign, o);
      v[i] = r.x; v[i + 1] = r.y;
    }
  }
}

__device__ __forceinline__ uint32_t pack4_s8(int a, int b, int c, int d) {
  // two saturating s32 -> s8 packs: {c, d} into the low half of a temporary, then {a, b} below it... the
  // instruction puts its first source in byte 1 and its second in byte 0 and shifts the third operand up.
  uint32_t hi, r;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(d), "r"(c));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(b), "r"(a), "r"(hi));
  return r;
}

template <typename IN_T, int BLOCK, int CH, bool SWIGLU, bool OUT_HR>
__global__ void __launch_bounds__(256) rot_q8_kernel(const RotQArgs p) {
  __shared__ float warp_max[2][32];
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
          for (int q = 0; q < 4; ++q) {
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
      float *wm = warp_max[it & 1];
      if (lane == 0) wm[warp] = amax;
      __syncthreads();
      float row_max = lane < n_warps ? wm[lane] : 0.0f;
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xFFFFFFFFu, row_max, s));

      const float scale = row_max > 0.0f ? __fdiv_rn(row_max, 127.0f) : 1.0f;
      const float rs = __fdiv_rn(1.0f, scale);
      const float2 rs2 = make_float2(rs, rs);
      int8_t *dst = static_cast<int8_t *>(p.out) + static_cast<size_t>(m) * p.D;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const int chunk = tid + c * blockDim.x;
        if (chunk < n_chunks) {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float2 y0 = __fmul2_rn(make_float2(v[c][4 * j], v[c][4 * j + 1]), rs2);
            const float2 y1 = __fmul2_rn(make_float2(v[c][4 * j + 2], v[c][4 * j + 3]), rs2);
            // round to nearest, ties to even; |y| <= 127 up to rounding, so the saturating pack never clips
            w[j] = pack4_s8(__float2int_rn(y0.x), __float2int_rn(y0.y), __float2int_rn(y1.x), __float2int_rn(y1.y));
          }
          uint4 *d4 = reinterpret_cast<uint4 *>(dst + chunk * kChunk);
          d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
          d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
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
    case 2: return launch_mode<IN_T, BLOCK, 2>(a, threads, sms, mode, out_hr, stream);
    default: return launch_mode<IN_T, BLOCK, 4>(a, threads, sms, mode, out_hr, stream);
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

// Chunks per thread (1, 2 or 4) and CTA size for a row of D channels: the fewest chunks per thread that keep the
// CTA at or under `threads_target` threads (CTAs are limited to 256 threads by register use).
void rot_q8_geometry(int D, int threads_target, int *ch, int *threads) {
  const int n_chunks = D / kChunk;
  int c = 1;
  while (c < 4 && (n_chunks + c - 1) / c > threads_target) c <<= 1;
  int t = (n_chunks + c - 1) / c;
  t = (t + 31) / 32 * 32;
  *ch = c;
  *threads = t;
}

cudaError_t launch_rot_q8(const void *x, int x_dtype, long long x_stride, void *out, float *sa, int M, int D,
                          int block, int mode, int out_hr, int threads_target, int sms, cudaStream_t stream) {
  RotQArgs a;
  a.x = x; a.out = out; a.sa = sa; a.x_stride = x_stride; a.M = M; a.D = D;
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
