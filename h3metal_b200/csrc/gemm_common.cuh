// Pieces shared by the single-CTA and the CTA-pair product kernels: tile constants, the persistent tile order, the
// conversion and packing of output values, and the per-chunk epilogue in the reference's operation order
// (kernels/gemm.metal:238-255 of the reference).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace h3b {
namespace gemm {

constexpr int kBM = 128;            // rows per tile = MMA M
constexpr int kBKBytes = 128;       // K bytes per stage row = one 128-byte swizzle span
constexpr int kABytes = kBM * kBKBytes;
constexpr int kMaxStages = 8;
constexpr int kLoraChunk = 32;      // ranks per LoRA shared-memory chunk: 32 halves = one 64-byte swizzle span
constexpr int kLoraTBytes = kBM * kLoraChunk * 2;
constexpr int kTmemCols = 512;
constexpr int kLowBase = 256;       // first TMEM column of the LoRA accumulators
constexpr int kThreads = 192;
constexpr int kBarrierBytes = 256;
// Row-parallel push: the transposition buffers of the four epilogue warps. int32 partials need 8 KB per warp and use
// the (then idle) column staging as well; bf16 partials need 4 KB per warp behind the column staging.
constexpr int kColStageWarps = 4;  // epilogue warps, each with its own copy of the tile's column scales and biases
__host__ __device__ constexpr int push_bytes(int bn) {
  return 32768 - kColStageWarps * 2 * bn * 4 > 16384 ? 32768 - kColStageWarps * 2 * bn * 4 : 16384;
}

__host__ __device__ constexpr int stage_bytes(int bn) { return kABytes + bn * kBKBytes; }

// Position in the ring of operand stages: the stage index and the phase (parity) of its barriers' current use.
// Stepped by hand so that the per-K-block loops of the single issuing threads need no division.
struct RingPos {
  uint32_t s = 0, ph = 0;
  __device__ __forceinline__ void advance(int stages) {
    if (++s == static_cast<uint32_t>(stages)) {
      s = 0;
      ph ^= 1u;
    }
  }
  __device__ __forceinline__ void retreat(int stages) {
    if (s == 0) {
      s = static_cast<uint32_t>(stages);
      ph ^= 1u;
    }
    --s;
  }
};

struct TileCoord {
  int m_blk, n_blk;
};

// Tile t of the persistent schedule: bands of `band` row tiles; inside a band row tiles vary fastest.
__device__ __forceinline__ TileCoord tile_coord(int t, int m_tiles, int n_tiles, int band) {
  const int per_band = band * n_tiles;
  const int b = t / per_band;
  const int rows = min(band, m_tiles - b * band);
  const int r = t - b * per_band;
  TileCoord c;
  c.m_blk = b * band + r % rows;
  c.n_blk = r / rows;
  return c;
}

template <typename OUT_T>
__device__ __forceinline__ OUT_T to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 32 consecutive values of one row, converted to OUT_T and packed into 32-bit words (16 words for 2-byte types).
template <typename OUT_T>
struct Packed;
template <>
struct Packed<float> {
  static constexpr int kWords = 32;
  static __device__ __forceinline__ void pack(const float (&v)[32], uint32_t (&w)[32]) {
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(v[j]);
  }
};
template <>
struct Packed<__half> {
  static constexpr int kWords = 16;
  static __device__ __forceinline__ void pack(const float (&v)[32], uint32_t (&w)[32]) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t *>(&h);
    }
  }
};
template <>
struct Packed<__nv_bfloat16> {
  static constexpr int kWords = 16;
  static __device__ __forceinline__ void pack(const float (&v)[32], uint32_t (&w)[32]) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t *>(&h);
    }
  }
};

// Stores 32 consecutive output values of one row; 16-byte vector stores when the segment is aligned and whole.
template <typename OUT_T>
__device__ __forceinline__ void store_segment(OUT_T *dst, const float (&v)[32], int n_valid, bool vec_ok) {
  if (vec_ok && n_valid >= 32) {
    uint32_t w[32];
    Packed<OUT_T>::pack(v, w);
#pragma unroll
    for (int j = 0; j < Packed<OUT_T>::kWords / 4; ++j)
      reinterpret_cast<uint4 *>(dst)[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < n_valid) dst[j] = to_out<OUT_T>(v[j]);
    }
  }
}

// float(acc) * sa * sw (+ bias) (+ low) for 32 columns, two at a time with the packed fp32 instructions (each half is
// rounded exactly like the scalar operation): convert, times the row scale, times the column scale, plus bias,
// plus the low-rank term.
__device__ __forceinline__ void dequant32(const GemmLaunch &g, const uint32_t (&acc)[32], const uint32_t (&low)[32],
                                          bool has_low, float sa_m, const float *sw_s, const float *bias_s,
                                          float (&v)[32]) {
  const bool has_bias = g.bias != nullptr;
  const float2 sa2 = make_float2(sa_m, sa_m);
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 w4 = *reinterpret_cast<const float4 *>(sw_s + j);
    const float4 b4 = *reinterpret_cast<const float4 *>(bias_s + j);
    float2 x0 = make_float2(__int2float_rn(static_cast<int32_t>(acc[j])), __int2float_rn(static_cast<int32_t>(acc[j + 1])));
    float2 x1 = make_float2(__int2float_rn(static_cast<int32_t>(acc[j + 2])), __int2float_rn(static_cast<int32_t>(acc[j + 3])));
    x0 = __fmul2_rn(__fmul2_rn(x0, sa2), make_float2(w4.x, w4.y));
    x1 = __fmul2_rn(__fmul2_rn(x1, sa2), make_float2(w4.z, w4.w));
    if (has_bias) {
      x0 = __fadd2_rn(x0, make_float2(b4.x, b4.y));
      x1 = __fadd2_rn(x1, make_float2(b4.z, b4.w));
    }
    if (has_low) {
      x0 = __fadd2_rn(x0, make_float2(__uint_as_float(low[j]), __uint_as_float(low[j + 1])));
      x1 = __fadd2_rn(x1, make_float2(__uint_as_float(low[j + 2]), __uint_as_float(low[j + 3])));
    }
    v[j] = x0.x; v[j + 1] = x0.y; v[j + 2] = x1.x; v[j + 3] = x1.y;
  }
}

__device__ __forceinline__ void store_values32(const GemmLaunch &g, const float (&v)[32], int m, int n, bool vec_ok);

// Finishes 32 accumulator columns [n, n + 32) of row m: either the raw int32 values, or the dequantising
// epilogue float(acc) * sa * sw (+ bias) (+ low) in the reference's operation order, converted to the output type
// or, with a gate table, accumulated into the fp32 residual stream (the reference's epilogue 1,
// kernels/gemm.metal:18-20,256-259).
// sw_s / bias_s point at the tile's staged column scales and biases for these 32 columns.
__device__ __forceinline__ void finish_chunk(const GemmLaunch &g, const uint32_t (&acc)[32], const uint32_t (&low)[32],
                                             bool has_low, int m, int n, float sa_m, const float *sw_s,
                                             const float *bias_s, bool vec_ok) {
  const int n_valid = g.N - n;
  if (m >= g.M || n_valid <= 0) return;
  if (g.c_dtype == kDtypeI32) {
    int32_t *dst = static_cast<int32_t *>(g.c) + static_cast<size_t>(m) * g.c_stride + n;
    if (vec_ok && n_valid >= 32) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        reinterpret_cast<uint4 *>(dst)[j] = make_uint4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < n_valid) dst[j] = static_cast<int32_t>(acc[j]);
      }
    }
    return;
  }
  float v[32];
  dequant32(g, acc, low, has_low, sa_m, sw_s, bias_s, v);
  store_values32(g, v, m, n, vec_ok);
}

// Stores 32 finished values of row m, columns [n, n + 32): converted to the output type, or accumulated into the fp32
// residual stream with a gate table (the reference's epilogue 1).
__device__ __forceinline__ void store_values32(const GemmLaunch &g, const float (&v)[32], int m, int n, bool vec_ok) {
  const int n_valid = g.N - n;
  if (m >= g.M || n_valid <= 0) return;
  const size_t off = static_cast<size_t>(m) * g.c_stride + n;
  if (g.gate != nullptr) {
    // gated-residual epilogue: X[m][n] += gate[type[m]][n] * v, X the fp32 residual stream (one multiply, one add)
    float *x = static_cast<float *>(g.c) + off;
    const float *gr = g.gate + static_cast<size_t>(g.rtype[m]) * g.g_stride + n;
    if (vec_ok && n_valid >= 32 && (reinterpret_cast<uintptr_t>(gr) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 x4 = *reinterpret_cast<const float4 *>(x + j);
        const float4 g4 = __ldg(reinterpret_cast<const float4 *>(gr + j));
        *reinterpret_cast<float4 *>(x + j) =
            make_float4(__fadd_rn(x4.x, __fmul_rn(g4.x, v[j])), __fadd_rn(x4.y, __fmul_rn(g4.y, v[j + 1])),
                        __fadd_rn(x4.z, __fmul_rn(g4.z, v[j + 2])), __fadd_rn(x4.w, __fmul_rn(g4.w, v[j + 3])));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < n_valid) x[j] = __fadd_rn(x[j], __fmul_rn(__ldg(gr + j), v[j]));
      }
    }
    return;
  }
  if (g.c_dtype == kDtypeBf16) store_segment(static_cast<__nv_bfloat16 *>(g.c) + off, v, n_valid, vec_ok);
  else if (g.c_dtype == kDtypeF16) store_segment(static_cast<__half *>(g.c) + off, v, n_valid, vec_ok);
  else store_segment(static_cast<float *>(g.c) + off, v, n_valid, vec_ok);
}

// Row-parallel push: the warp's 32 rows x 64 columns [n, n + 64) of this GPU's partial product (two TMEM chunks)
// go to the staging slot of the rows' owner, which may be another GPU (plain stores through a peer mapping). A lane
// holds one ROW of a chunk, so a direct store would touch 32 rows with 16 bytes each; over NVLink that is 32 small
// packets. The two chunks are therefore transposed through shared memory first: afterwards sixteen (int32) or
// eight (bf16) neighbouring lanes hold one row's 256 or 128 contiguous bytes and every store instruction writes
// whole lines. `xpose` is the warp's own buffer, [32 rows][16 or 8 pieces of 16 bytes]; piece p of row r sits at
// p ^ (r & 7), so that both the row-wise writes and the line-wise reads spread over the banks.
//
// push_stage: chunk `half` (0 or 1) of the pair into the buffer. push_flush: the buffer's first `cols` (32 or 64)
// columns to dst_rows (row 0 of the tile's 128 rows in the slot) at column n.
__device__ __forceinline__ void push_stage(const GemmLaunch &g, const uint32_t (&acc)[32], int half, int lane, float sa_m,
                                           const float *sw_s, const float *bias_s, uint4 *xpose) {
  if (g.c_dtype == kDtypeI32) {
#pragma unroll
    for (int k = 0; k < 8; ++k)
      xpose[lane * 16 + ((half * 8 + k) ^ (lane & 7))] = make_uint4(acc[4 * k], acc[4 * k + 1], acc[4 * k + 2], acc[4 * k + 3]);
  } else {  // bf16 partials: float(acc) * sa * sw, no bias (the owner adds it once)
    const uint32_t no_low[32] = {};
    float v[32];
    dequant32(g, acc, no_low, false, sa_m, sw_s, bias_s, v);
    uint32_t w[32];
    Packed<__nv_bfloat16>::pack(v, w);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      xpose[lane * 8 + ((half * 4 + k) ^ (lane & 7))] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
  }
}

__device__ __forceinline__ void push_flush(const GemmLaunch &g, int quarter, int lane, int n, int cols, const uint4 *xpose,
                                           uint8_t *dst_rows) {
  __syncwarp();
  if (g.c_dtype == kDtypeI32) {
    const int p = lane & 15;
    if (4 * p < cols) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {  // two rows per instruction, sixteen lanes (256 bytes) per row
        const int r = 2 * i + (lane >> 4);
        uint8_t *row = dst_rows + static_cast<size_t>(quarter * 32 + r) * g.c_stride * 4;
        *reinterpret_cast<uint4 *>(row + static_cast<size_t>(n) * 4 + p * 16) = xpose[r * 16 + (p ^ (r & 7))];
      }
    }
  } else {
    const int p = lane & 7;
    if (8 * p < cols) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {  // four rows per instruction, eight lanes (128 bytes) per row
        const int r = 4 * i + (lane >> 3);
        uint8_t *row = dst_rows + static_cast<size_t>(quarter * 32 + r) * g.c_stride * 2;
        *reinterpret_cast<uint4 *>(row + static_cast<size_t>(n) * 2 + p * 16) = xpose[r * 8 + (p ^ (r & 7))];
      }
    }
  }
  __syncwarp();  // the buffer may be overwritten by the next pair
}

// Stages the column scales and biases of columns [n0, n0 + bn) in a warp's own slice of shared memory.
__device__ __forceinline__ void stage_columns(const GemmLaunch &g, int n0, int bn, int lane, float *sw_s, float *bias_s) {
  __syncwarp();
  if (g.c_dtype != kDtypeI32) {
    for (int j = lane; j < bn; j += 32) {
      const int n = n0 + j;
      sw_s[j] = n < g.N ? __ldg(g.sw + n) : 0.0f;
      bias_s[j] = (g.bias != nullptr && n < g.N) ? __ldg(g.bias + n) : 0.0f;
    }
  }
  __syncwarp();
}

}  // namespace gemm
}  // namespace h3b
