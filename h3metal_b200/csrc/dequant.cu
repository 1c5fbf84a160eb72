// Stand-alone dequantising epilogue: out[m][n] = OUT_T(float(acc[m][n]) * sa[m] * sw[n] + bias[n]).
//
// The same fp32 operation order as the product kernel's epilogue (the reference's kernels/gemm.metal:238-255): int32
// to fp32 conversion (rounds above 2^24), times the row scale, times the column scale, plus the bias, convert.
// Used when the int32 accumulators of a K-sharded (row-parallel) layer were summed over the GPUs first; the result
// is then bit-identical to the single-GPU product. HBM-bound: 4 bytes read and 2 (bf16) written per element.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace h3b {
namespace {

// Self-test of the bounded-wait machinery: one CTA initialises an mbarrier that nothing will ever signal and waits
// on it with a short limit. The wait must run out, leave its code in the status word and let the kernel return
// normally (nothing traps, nothing hangs, the context stays usable).
__global__ void expire_wait_kernel(int *status, long long limit_cycles) {
  __shared__ unsigned long long bar;
  __shared__ int cta_abort;
  if (threadIdx.x == 0) {
    cta_abort = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, &cta_abort, status, kStatusSelfTest, limit_cycles);
  __syncthreads();
}

template <typename OUT_T> __device__ __forceinline__ OUT_T cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half cvt_out<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float dequant_one(int acc, float sa, float sw, float bias, bool has_bias) {
  float v = __fmul_rn(__fmul_rn(__int2float_rn(acc), sa), sw);
  return has_bias ? __fadd_rn(v, bias) : v;
}

// One thread per group of 8 consecutive columns (N % 8 == 0, 16-byte aligned rows).
template <typename OUT_T>
__global__ void __launch_bounds__(256) dequant_vec_kernel(const int32_t *acc, long long acc_stride, const float *sa,
                                                          const float *sw, const float *bias, OUT_T *out,
                                                          long long c_stride, int M, int N) {
  const long long groups_per_row = N / 8;
  const long long total = static_cast<long long>(M) * groups_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / groups_per_row);
    const int n = static_cast<int>(i - m * groups_per_row) * 8;
    const int4 a0 = *reinterpret_cast<const int4 *>(acc + m * acc_stride + n);
    const int4 a1 = *reinterpret_cast<const int4 *>(acc + m * acc_stride + n + 4);
    const float4 w0 = *reinterpret_cast<const float4 *>(sw + n), w1 = *reinterpret_cast<const float4 *>(sw + n + 4);
    float4 b0 = make_float4(0, 0, 0, 0), b1 = b0;
    const bool hb = bias != nullptr;
    if (hb) {
      b0 = *reinterpret_cast<const float4 *>(bias + n);
      b1 = *reinterpret_cast<const float4 *>(bias + n + 4);
    }
    const float s = sa[m];
    const float v[8] = {dequant_one(a0.x, s, w0.x, b0.x, hb), dequant_one(a0.y, s, w0.y, b0.y, hb),
                        dequant_one(a0.z, s, w0.z, b0.z, hb), dequant_one(a0.w, s, w0.w, b0.w, hb),
                        dequant_one(a1.x, s, w1.x, b1.x, hb), dequant_one(a1.y, s, w1.y, b1.y, hb),
                        dequant_one(a1.z, s, w1.z, b1.z, hb), dequant_one(a1.w, s, w1.w, b1.w, hb)};
    OUT_T *dst = out + m * c_stride + n;
#pragma unroll
    for (int j = 0; j < 8; ++j) dst[j] = cvt_out<OUT_T>(v[j]);  // the compiler merges these into 16-byte stores
  }
}

template <typename OUT_T>
__global__ void __launch_bounds__(256) dequant_scalar_kernel(const int32_t *acc, long long acc_stride, const float *sa,
                                                             const float *sw, const float *bias, OUT_T *out,
                                                             long long c_stride, int M, int N) {
  const long long total = static_cast<long long>(M) * N;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / N), n = static_cast<int>(i - static_cast<long long>(m) * N);
    out[m * c_stride + n] = cvt_out<OUT_T>(dequant_one(acc[m * acc_stride + n], sa[m], sw[n], bias ? bias[n] : 0.0f, bias != nullptr));
  }
}

template <typename OUT_T>
cudaError_t launch_typed(const int32_t *acc, long long acc_stride, const float *sa, const float *sw, const float *bias,
                         void *out, long long c_stride, int M, int N, int sms, cudaStream_t stream) {
  const bool vec = N % 8 == 0 && acc_stride % 4 == 0 && (c_stride * sizeof(OUT_T)) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(acc) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(sw) % 16 == 0 && (bias == nullptr || reinterpret_cast<uintptr_t>(bias) % 16 == 0);
  const long long work = vec ? static_cast<long long>(M) * (N / 8) : static_cast<long long>(M) * N;
  long long blocks = (work + 255) / 256;
  const long long cap = static_cast<long long>(sms) * 8;  // a multiple of the SM count; grid-stride covers the rest
  if (blocks > cap) blocks = cap;
  if (vec) dequant_vec_kernel<OUT_T><<<static_cast<int>(blocks), 256, 0, stream>>>(acc, acc_stride, sa, sw, bias, static_cast<OUT_T *>(out), c_stride, M, N);
  else dequant_scalar_kernel<OUT_T><<<static_cast<int>(blocks), 256, 0, stream>>>(acc, acc_stride, sa, sw, bias, static_cast<OUT_T *>(out), c_stride, M, N);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_expire_wait(int *status, long long limit_cycles, cudaStream_t stream) {
  expire_wait_kernel<<<1, 32, 0, stream>>>(status, limit_cycles);
  return cudaGetLastError();
}

cudaError_t launch_dequant_i32(const int32_t *acc, long long acc_stride, const float *sa, const float *sw,
                               const float *bias, void *out, int c_dtype, long long c_stride, int M, int N, int sms,
                               cudaStream_t stream) {
  switch (c_dtype) {
    case kDtypeBf16: return launch_typed<__nv_bfloat16>(acc, acc_stride, sa, sw, bias, out, c_stride, M, N, sms, stream);
    case kDtypeF16: return launch_typed<__half>(acc, acc_stride, sa, sw, bias, out, c_stride, M, N, sms, stream);
    case kDtypeF32: return launch_typed<float>(acc, acc_stride, sa, sw, bias, out, c_stride, M, N, sms, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace h3b
