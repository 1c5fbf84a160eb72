// RMSNorm / LayerNorm + modulation fused in front of the rotate + per-token int8 quantise tail.
//
//   a[m] = int8(rot(norm(x[m]) * scale'[type[m]] + shift[type[m]]))   with the row scale in sa[m]
//
// Replaces the reference's Metal kernel norm_mod_q8 (kernels/ops.metal:111-268; parameter block NormQParams
// kernels/params.h:18-23; launcher h3metal/ops.py:200-211). x is the fp32 residual stream [M][x_stride]; mod holds,
// per row type, D scale' values followed by D shift values (rows mod_stride apart); rtype is one byte per row.
//   LN      LayerNorm without affine: the row mean is subtracted first (two passes over the registers, :146-160)
//   POST    first x[m] += post * rmsnorm(y[m]) and the sum is written back (:161-198)
//   OUT_F / OUT_H   write the modulated row as fp32 / fp16 and stop (no rotation, no quantisation, :203-219)
//   OUT_HR  write the rotated row as fp16 (:236-245)
// Element arithmetic keeps the kernel's order: v * inv * scale' + shift with separate multiplies and add; the
// rotation and quantisation tail is the one of rot_q8.cu (same helpers). Row sums (sum of squares, mean) are fp32
// sums whose order is this kernel's own: per thread over its 64 channels, then a shuffle tree, then over the warps;
// the reference leaves that order to its SIMD-group reductions, so codes are compared with the one-step-on-1e-4
// allowance rather than bit for bit.
//
// One CTA per row; a thread owns `CH` chunks of 64 consecutive channels (sixteen 128-bit loads each). HBM-bound:
// 4 bytes in and 1 byte out per channel (POST: 8 more in and 4 more out).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "kernels.h"
#include "rot_common.cuh"

namespace h3b {
namespace {

using namespace rot;

struct NormQArgs {
  float *x;
  const float *mod;
  const unsigned char *rtype;
  void *out;
  float *sa;
  const float *y;
  const float *post;
  long long x_stride, mod_stride;
  int M, D;
  float eps, normaliser;
};

__device__ __forceinline__ float block_sum(float v, float *tmp, int lane, int warp, int n_warps) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, s));
  if (n_warps == 1) return v;
  if (lane == 0) tmp[warp] = v;
  __syncthreads();
  float r = tmp[0];
  for (int w = 1; w < n_warps; ++w) r = __fadd_rn(r, tmp[w]);
  __syncthreads();
  return r;
}

template <int BLOCK, int CH, bool LN, bool POST, int OUT>  // OUT: 0 int8 codes, 1 fp32, 2 fp16, 3 rotated fp16
__global__ void __launch_bounds__(256) norm_mod_q8_kernel(const NormQArgs p) {
  __shared__ float tmp[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_warps = blockDim.x >> 5;
  const int n_chunks = p.D / kChunk;
  const int m = blockIdx.x;
  float *row = p.x + static_cast<size_t>(m) * p.x_stride;
  const float fd = static_cast<float>(p.D);  // row statistics are divided by D, as the reference kernel does

  float v[CH][kChunk];
  bool have[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int chunk = tid + c * blockDim.x;
    have[c] = chunk < n_chunks;
    if (have[c]) {
      RawChunk<float> r;
      r.load(row + chunk * kChunk);
      widen(r, v[c]);
    } else {
#pragma unroll
      for (int i = 0; i < kChunk; ++i) v[c][i] = 0.0f;
    }
  }

  if (LN) {
    float sm = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < kChunk; ++i) sm = __fadd_rn(sm, v[c][i]);
    const float mean = __fdiv_rn(block_sum(sm, tmp, lane, warp, n_warps), fd);
#pragma unroll
    for (int c = 0; c < CH; ++c)
      if (have[c]) {
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[c][i] = __fsub_rn(v[c][i], mean);
      }
  }
  if (POST) {
    float yv[CH][kChunk];
    float ssy = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int chunk = tid + c * blockDim.x;
      if (have[c]) {
        RawChunk<float> r;
        r.load(p.y + static_cast<size_t>(m) * p.D + chunk * kChunk);
        widen(r, yv[c]);
      } else {
#pragma unroll
        for (int i = 0; i < kChunk; ++i) yv[c][i] = 0.0f;
      }
#pragma unroll
      for (int i = 0; i < kChunk; ++i) ssy = __fadd_rn(ssy, __fmul_rn(yv[c][i], yv[c][i]));
    }
    const float iy = __frsqrt_rn(__fadd_rn(__fdiv_rn(block_sum(ssy, tmp, lane, warp, n_warps), fd), p.eps));
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int chunk = tid + c * blockDim.x;
      if (have[c]) {
        const float4 *pw = reinterpret_cast<const float4 *>(p.post + chunk * kChunk);
#pragma unroll
        for (int q = 0; q < kChunk / 4; ++q) {
          const float4 w = __ldg(pw + q);
          const float ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[c][4 * q + j] = __fadd_rn(v[c][4 * q + j], __fmul_rn(__fmul_rn(ww[j], yv[c][4 * q + j]), iy));
          reinterpret_cast<float4 *>(row + chunk * kChunk)[q] =
              make_float4(v[c][4 * q], v[c][4 * q + 1], v[c][4 * q + 2], v[c][4 * q + 3]);
        }
      }
    }
  }

  float ss = 0.0f;
#pragma unroll
  for (int c = 0; c < CH; ++c)
#pragma unroll
    for (int i = 0; i < kChunk; ++i) ss = __fadd_rn(ss, __fmul_rn(v[c][i], v[c][i]));
  const float inv = __frsqrt_rn(__fadd_rn(__fdiv_rn(block_sum(ss, tmp, lane, warp, n_warps), fd), p.eps));
  const float *md = p.mod + static_cast<size_t>(p.rtype[m]) * p.mod_stride;

#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int chunk = tid + c * blockDim.x;
    if (have[c]) {
      const float4 *ps = reinterpret_cast<const float4 *>(md + chunk * kChunk);
      const float4 *pb = reinterpret_cast<const float4 *>(md + p.D + chunk * kChunk);
#pragma unroll
      for (int q = 0; q < kChunk / 4; ++q) {
        const float4 s4 = __ldg(ps + q), b4 = __ldg(pb + q);
        const float sc[4] = {s4.x, s4.y, s4.z, s4.w}, sh[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          v[c][4 * q + j] = __fadd_rn(__fmul_rn(__fmul_rn(v[c][4 * q + j], inv), sc[j]), sh[j]);
      }
    }
  }

  if constexpr (OUT == 1) {
    float *o = static_cast<float *>(p.out) + static_cast<size_t>(m) * p.D;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int chunk = tid + c * blockDim.x;
      if (have[c]) {
#pragma unroll
        for (int q = 0; q < kChunk / 4; ++q)
          reinterpret_cast<float4 *>(o + chunk * kChunk)[q] =
              make_float4(v[c][4 * q], v[c][4 * q + 1], v[c][4 * q + 2], v[c][4 * q + 3]);
      }
    }
    return;
  }
  if constexpr (OUT == 0 || OUT == 3) {  // rotation tail, as in rot_q8
    const float2 norm2 = make_float2(p.normaliser, p.normaliser);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      chunk_butterflies(v[c]);
      lane_butterflies<BLOCK>(v[c], lane);
#pragma unroll
      for (int i = 0; i < kChunk; i += 2) {
        const float2 r = __fmul2_rn(make_float2(v[c][i], v[c][i + 1]), norm2);
        v[c][i] = r.x; v[c][i + 1] = r.y;
      }
    }
  }
  if constexpr (OUT == 2 || OUT == 3) {
    __half *o = static_cast<__half *>(p.out) + static_cast<size_t>(m) * p.D;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int chunk = tid + c * blockDim.x;
      if (have[c]) {
#pragma unroll
        for (int q = 0; q < kChunk / 8; ++q) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __half2 h = __floats2half2_rn(v[c][8 * q + 2 * j], v[c][8 * q + 2 * j + 1]);
            w[j] = *reinterpret_cast<const uint32_t *>(&h);
          }
          reinterpret_cast<uint4 *>(o + chunk * kChunk)[q] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    return;
  }
  if constexpr (OUT == 0) {
    float amax = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int i = 0; i < kChunk; ++i) amax = fmaxf(amax, fabsf(v[c][i]));
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, s));
    float row_max = amax;
    if (n_warps > 1) {
      if (lane == 0) tmp[warp] = amax;
      __syncthreads();
      row_max = tmp[0];
      for (int w = 1; w < n_warps; ++w) row_max = fmaxf(row_max, tmp[w]);
    }
    const float scale = row_max > 0.0f ? __fdiv_rn(row_max, 127.0f) : 1.0f;
    const float rs = __fdiv_rn(1.0f, scale);
    const float2 rs2 = make_float2(rs, rs);
    int8_t *dst = static_cast<int8_t *>(p.out) + static_cast<size_t>(m) * p.D;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int chunk = tid + c * blockDim.x;
      if (have[c]) {
        uint32_t w[kChunk / 4];
#pragma unroll
        for (int j = 0; j < kChunk / 4; ++j) {
          const float2 y0 = __fmul2_rn(make_float2(v[c][4 * j], v[c][4 * j + 1]), rs2);
          const float2 y1 = __fmul2_rn(make_float2(v[c][4 * j + 2], v[c][4 * j + 3]), rs2);
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

template <int BLOCK, int CH, bool LN, bool POST>
cudaError_t launch_out(const NormQArgs &a, int threads, int out, cudaStream_t stream) {
  const dim3 grid(a.M), blk(threads);
  switch (out) {
    case 0: norm_mod_q8_kernel<BLOCK, CH, LN, POST, 0><<<grid, blk, 0, stream>>>(a); break;
    case 1: norm_mod_q8_kernel<BLOCK, CH, LN, POST, 1><<<grid, blk, 0, stream>>>(a); break;
    case 2: norm_mod_q8_kernel<BLOCK, CH, LN, POST, 2><<<grid, blk, 0, stream>>>(a); break;
    default: norm_mod_q8_kernel<BLOCK, CH, LN, POST, 3><<<grid, blk, 0, stream>>>(a); break;
  }
  return cudaGetLastError();
}

template <int BLOCK, int CH>
cudaError_t launch_flags(const NormQArgs &a, int threads, bool ln, bool post, int out, cudaStream_t stream) {
  if (ln) return launch_out<BLOCK, CH, true, false>(a, threads, out, stream);
  if (post) return launch_out<BLOCK, CH, false, true>(a, threads, out, stream);
  return launch_out<BLOCK, CH, false, false>(a, threads, out, stream);
}

template <int BLOCK>
cudaError_t launch_ch(const NormQArgs &a, int ch, int threads, bool ln, bool post, int out, cudaStream_t stream) {
  return ch == 1 ? launch_flags<BLOCK, 1>(a, threads, ln, post, out, stream)
                 : launch_flags<BLOCK, 2>(a, threads, ln, post, out, stream);
}

}  // namespace

cudaError_t launch_norm_mod_q8(float *x, long long x_stride, const float *mod, long long mod_stride,
                               const unsigned char *rtype, void *out, float *sa, int M, int D, int block, float eps,
                               int ln, int out_kind, const float *y, const float *post, cudaStream_t stream) {
  NormQArgs a;
  a.x = x; a.mod = mod; a.rtype = rtype; a.out = out; a.sa = sa; a.y = y; a.post = post;
  a.x_stride = x_stride; a.mod_stride = mod_stride; a.M = M; a.D = D; a.eps = eps;
  a.normaliser = static_cast<float>(1.0 / sqrt(static_cast<double>(block)));
  const int n_chunks = D / kChunk;
  const bool is_post = post != nullptr;
  // POST keeps two rows in registers: one chunk per thread only
  int ch = (n_chunks > 256 && !is_post) ? 2 : 1;
  int threads = ((n_chunks + ch - 1) / ch + 31) / 32 * 32;
  if (threads > 256) return cudaErrorInvalidConfiguration;
  switch (block) {
    case 64: return launch_ch<64>(a, ch, threads, ln != 0, is_post, out_kind, stream);
    case 128: return launch_ch<128>(a, ch, threads, ln != 0, is_post, out_kind, stream);
    default: return launch_ch<256>(a, ch, threads, ln != 0, is_post, out_kind, stream);
  }
}

}  // namespace h3b
