// Device helpers shared by the rotate+quantise kernels: widening of packed inputs, the in-thread and cross-lane
// butterfly stages in the reference kernel's operation order (kernels/ops.metal:19-47 of the reference: stages by
// increasing stride, (a, b) -> (a + b, a - b), every operation rounded on its own), silu, and int8 packing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace h3b {
namespace rot {

constexpr int kChunk = 64;  // consecutive channels a thread owns per chunk


__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Raw (still packed) input of one chunk: 128 bytes for 16-bit inputs, 256 bytes for fp32.
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
  for (int i = 0; i < kChunk / 8; ++i) {
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
  for (int i = 0; i < kChunk / 8; ++i) {
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
  for (int i = 0; i < kChunk / 4; ++i) {
    v[4 * i] = __uint_as_float(r.q[i].x);
    v[4 * i + 1] = __uint_as_float(r.q[i].y);
    v[4 * i + 2] = __uint_as_float(r.q[i].z);
    v[4 * i + 3] = __uint_as_float(r.q[i].w);
  }
}

// x / (1 + exp(-x)): accurate expf (the result feeds a rounding to int8, so its last places matter), then the
// fast division (reciprocal and multiply, 2 ulp, no slow path): together within the few-ulp spread that exp
// itself has between math libraries, which is what the one-step-on-1e-4-of-codes allowance of this mode is for.
__device__ __forceinline__ float silu(float g) { return __fdividef(g, __fadd_rn(1.0f, expf(-g))); }

// In-thread butterfly stages of stride 1, 2, ... N / 2 over a thread's N (64 or 32) values. Stride 1 pairs the two
// halves of a float2 and stays scalar; the others combine whole float2 registers: a + b and fma(b, -1, a) = a - b.
template <int N>
__device__ __forceinline__ void chunk_butterflies(float (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N; i += 2) {
    const float a = v[i], b = v[i + 1];
    v[i] = __fadd_rn(a, b);
    v[i + 1] = __fsub_rn(a, b);
  }
  const float2 minus_one = make_float2(-1.0f, -1.0f);
#pragma unroll
  for (int s = 2; s < N; s <<= 1) {
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      if ((i & s) == 0) {
        const float2 a = make_float2(v[i], v[i + 1]), b = make_float2(v[i + s], v[i + s + 1]);
        const float2 sum = __fadd2_rn(a, b), dif = __ffma2_rn(b, minus_one, a);
        v[i] = sum.x; v[i + 1] = sum.y;
        v[i + s] = dif.x; v[i + s + 1] = dif.y;
      }
    }
  }
}

// Stages of stride N .. BLOCK/2: the partner value lives in lane ^ (stride / N). The lower lane keeps v + o, the
// upper lane o - v; both are o + sign * v with sign = +-1 (the product is exact, so the fma rounds once).
template <int BLOCK, int N>
__device__ __forceinline__ void lane_butterflies(float (&v)[N], int lane) {
#pragma unroll
  for (int s = 1; s < BLOCK / N; s <<= 1) {
    const float sg = (lane & s) ? -1.0f : 1.0f;
    const float2 sign = make_float2(sg, sg);
#pragma unroll
    for (int i = 0; i < N; i += 2) {
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

}  // namespace rot
}  // namespace h3b
