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
// Mapping to the GPU: one CTA per row. A thread owns `CH` chunks of eight consecutive channels (one 128-bit load
// per bf16/fp16 chunk); the three low butterfly stages run in the thread's registers, the rest across the lanes
// of its warp with shuffles (32 lanes x 8 channels = 256 channels, so a rotation block of 64, 128 or 256 never
// leaves the warp). The row maximum goes through a warp shuffle reduction and one shared-memory exchange. All
// loads of a row are issued before the first butterfly so that each thread keeps CH x 16 bytes in flight.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "kernels.h"

namespace h3b {
namespace {

constexpr int kLane = 8;  // channels per chunk

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

// Eight consecutive input values starting at element `col` of `row`, widened to fp32.
template <typename IN_T>
__device__ __forceinline__ void load8(const IN_T *row, int col, float (&v)[kLane]);

template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16 *row, int col, float (&v)[kLane]) {
  const uint4 raw = ld_stream16(row + col);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half *row, int col, float (&v)[kLane]) {
  const uint4 raw = ld_stream16(row + col);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
    v[2 * i] = __low2float(h);
    v[2 * i + 1] = __high2float(h);
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float *row, int col, float (&v)[kLane]) {
  const uint4 a = ld_stream16(row + col), b = ld_stream16(row + col + 4);
  v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
  v[4] = __uint_as_float(b.x); v[5] = __uint_as_float(b.y); v[6] = __uint_as_float(b.z); v[7] = __uint_as_float(b.w);
}

__device__ __forceinline__ float silu(float g) {
  // x / (1 + exp(-x)) in fp32 with IEEE division
  return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
}

// Butterfly stages of stride 1, 2, 4 inside the thread, then stride 8 .. BLOCK/2 across lanes.
template <int BLOCK>
__device__ __forceinline__ void block_wht(float (&v)[kLane], int lane) {
#pragma unroll
  for (int s = 1; s < kLane; s <<= 1) {
#pragma unroll
    for (int i = 0; i < kLane; ++i) {
      if ((i & s) == 0) {
        const float a = v[i], b = v[i + s];
        v[i] = __fadd_rn(a, b);
        v[i + s] = __fsub_rn(a, b);
      }
    }
  }
#pragma unroll
  for (int s = 1; s < BLOCK / kLane; s <<= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int i = 0; i < kLane; ++i) {
      const float o = __shfl_xor_sync(0xFFFFFFFFu, v[i], s);
      v[i] = upper ? __fsub_rn(o, v[i]) : __fadd_rn(v[i], o);
    }
  }
}

template <typename IN_T, int BLOCK, int CH, bool SWIGLU, bool OUT_HR>
__global__ void __launch_bounds__(CH == 4 ? 512 : 1024) rot_q8_kernel(const RotQArgs p) {
  __shared__ float warp_max[32];
  const int m = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_chunks = p.D / kLane;
  const IN_T *row = static_cast<const IN_T *>(p.x) + static_cast<size_t>(m) * p.x_stride;

  float v[CH][kLane];
  float g[SWIGLU ? CH : 1][kLane];
  // every load first: CH (x2 with gates) independent 16-byte requests per thread
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int chunk = tid + c * blockDim.x;
    if (chunk < n_chunks) {
      load8<IN_T>(row, chunk * kLane, v[c]);
      if (SWIGLU) load8<IN_T>(row, p.D + chunk * kLane, g[SWIGLU ? c : 0]);
    } else {
#pragma unroll
      for (int i = 0; i < kLane; ++i) v[c][i] = 0.0f;
      if (SWIGLU) {
#pragma unroll
        for (int i = 0; i < kLane; ++i) g[SWIGLU ? c : 0][i] = 0.0f;
      }
    }
  }
  float amax = 0.0f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    if (SWIGLU) {
#pragma unroll
      for (int i = 0; i < kLane; ++i) v[c][i] = __fmul_rn(v[c][i], silu(g[SWIGLU ? c : 0][i]));
    }
    block_wht<BLOCK>(v[c], lane);
#pragma unroll
    for (int i = 0; i < kLane; ++i) {
      v[c][i] = __fmul_rn(v[c][i], p.normaliser);
      amax = fmaxf(amax, fabsf(v[c][i]));
    }
  }

  if constexpr (OUT_HR) {
    __half *dst = static_cast<__half *>(p.out) + static_cast<size_t>(m) * p.D;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int chunk = tid + c * blockDim.x;
      if (chunk < n_chunks) {
        uint4 pk;
        uint32_t *w = reinterpret_cast<uint32_t *>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __half2 h = __halves2half2(__float2half_rn(v[c][2 * i]), __float2half_rn(v[c][2 * i + 1]));
          w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(dst + chunk * kLane) = pk;
      }
    }
    return;
  } else {
  // row maximum: lanes, then warps
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, s));
  if (lane == 0) warp_max[warp] = amax;
  __syncthreads();
  const int n_warps = blockDim.x >> 5;
  float row_max = lane < n_warps ? warp_max[lane] : 0.0f;
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xFFFFFFFFu, row_max, s));

  const float scale = row_max > 0.0f ? __fdiv_rn(row_max, 127.0f) : 1.0f;
  const float rs = __fdiv_rn(1.0f, scale);
  int8_t *dst = static_cast<int8_t *>(p.out) + static_cast<size_t>(m) * p.D;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int chunk = tid + c * blockDim.x;
    if (chunk < n_chunks) {
      uint32_t w[2] = {0u, 0u};
#pragma unroll
      for (int i = 0; i < kLane; ++i) {
        const int q = __float2int_rn(__fmul_rn(v[c][i], rs));  // round to nearest, ties to even
        w[i >> 2] |= (static_cast<uint32_t>(q) & 0xFFu) << (8 * (i & 3));
      }
      *reinterpret_cast<uint2 *>(dst + chunk * kLane) = make_uint2(w[0], w[1]);
    }
  }
  if (tid == 0) p.sa[m] = scale;
  }
}

template <typename IN_T, int BLOCK, int CH>
cudaError_t launch_mode(const RotQArgs &a, int threads, int mode, int out_hr, cudaStream_t stream) {
  const dim3 grid(a.M), blk(threads);
  if (out_hr) {
    if (mode == 1) rot_q8_kernel<IN_T, BLOCK, CH, true, true><<<grid, blk, 0, stream>>>(a);
    else rot_q8_kernel<IN_T, BLOCK, CH, false, true><<<grid, blk, 0, stream>>>(a);
  } else {
    if (mode == 1) rot_q8_kernel<IN_T, BLOCK, CH, true, false><<<grid, blk, 0, stream>>>(a);
    else rot_q8_kernel<IN_T, BLOCK, CH, false, false><<<grid, blk, 0, stream>>>(a);
  }
  return cudaGetLastError();
}

template <typename IN_T, int BLOCK>
cudaError_t launch_ch(const RotQArgs &a, int ch, int threads, int mode, int out_hr, cudaStream_t stream) {
  switch (ch) {
    case 1: return launch_mode<IN_T, BLOCK, 1>(a, threads, mode, out_hr, stream);
    case 2: return launch_mode<IN_T, BLOCK, 2>(a, threads, mode, out_hr, stream);
    case 4: return launch_mode<IN_T, BLOCK, 4>(a, threads, mode, out_hr, stream);
    default: return launch_mode<IN_T, BLOCK, 8>(a, threads, mode, out_hr, stream);
  }
}

template <typename IN_T>
cudaError_t launch_block(const RotQArgs &a, int block, int ch, int threads, int mode, int out_hr,
                         cudaStream_t stream) {
  switch (block) {
    case 64: return launch_ch<IN_T, 64>(a, ch, threads, mode, out_hr, stream);
    case 128: return launch_ch<IN_T, 128>(a, ch, threads, mode, out_hr, stream);
    default: return launch_ch<IN_T, 256>(a, ch, threads, mode, out_hr, stream);
  }
}

}  // namespace

// Chunks per thread and CTA size for a row of D channels. `threads_target` bounds the CTA (more, smaller CTAs per
// SM hide the row-maximum barrier better than one huge CTA).
void rot_q8_geometry(int D, int threads_target, int *ch, int *threads) {
  const int n_chunks = D / kLane;
  int c = 1;
  while (c < 8 && (n_chunks + c - 1) / c > threads_target) c <<= 1;
  int t = (n_chunks + c - 1) / c;
  t = (t + 31) / 32 * 32;
  *ch = c;
  *threads = t;
}

cudaError_t launch_rot_q8(const void *x, int x_dtype, long long x_stride, void *out, float *sa, int M, int D,
                          int block, int mode, int out_hr, int threads_target, cudaStream_t stream) {
  RotQArgs a;
  a.x = x; a.out = out; a.sa = sa; a.x_stride = x_stride; a.M = M; a.D = D;
  a.normaliser = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
  int ch, threads;
  rot_q8_geometry(D, threads_target, &ch, &threads);
  if (threads > 1024) return cudaErrorInvalidConfiguration;
  switch (x_dtype) {
    case kDtypeBf16: return launch_block<__nv_bfloat16>(a, block, ch, threads, mode, out_hr, stream);
    case kDtypeF16: return launch_block<__half>(a, block, ch, threads, mode, out_hr, stream);
    case kDtypeF32: return launch_block<float>(a, block, ch, threads, mode, out_hr, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace h3b
