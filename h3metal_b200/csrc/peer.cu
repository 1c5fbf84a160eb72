// Row-parallel layers over the GPUs of one node, without a communication library on the data path.
//
// A K-sharded linear produces, on every GPU, a partial product of ALL rows. The product kernel (gemm_w8a8.cu, PUSH)
// stores each finished tile of it straight into the staging memory of the GPU that owns those rows (plain stores
// through a peer mapping, tile by tile while the tensor cores work on the next tile). What remains is here:
//
//   peer_sync_kernel        the rendezvous "everybody's partials have landed": one flag word per (receiver, sender)
//                           pair in peer-mapped memory, written with release semantics at system scope after the
//                           sender's product kernel, polled with acquire semantics by the receiver. The poll is
//                           bounded (about a second): a GPU that never signals makes the wait give up with
//                           kStatusPeerTimeout in the context's status word instead of hanging the device.
//   reduce_dequant_kernel   the owner's pass over its rows: sum the slots (int32: exact in any order, so the result
//                           is bit-identical to the single-GPU product; bf16 partials: fp32 sum in slot order), apply
//                           the product's epilogue in the reference's operation order (kernels/gemm.metal:238-255
//                           of the reference) and store the rows, optionally into every GPU's output (all-gather by
//                           peer stores). HBM-bound: world x 4 (or 2) bytes read per element, 2 written per copy.
//                           If a kernel before it in the stream gave up a bounded wait (the rendezvous, above all),
//                           it stores nothing: partial sums never reach an output.
//
// The reference is single-GPU; nothing here has a counterpart in it.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace h3b {
namespace {

__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void peer_sync_kernel(const PeerSync p) {
  const int q = threadIdx.x;
  if (q >= p.world) return;
  if (p.mode != 2) {
    // the product kernel that ran before this one on the stream has completed; the fence orders its peer stores
    // (already performed) before the flag for whoever acquires the flag
    __threadfence_system();
    st_release_sys(p.flags[q] + p.rank, p.epoch);
  }
  if (p.mode != 1) {
    const unsigned int *mine = p.flags[p.rank] + q;
    const long long t0 = clock64();
    // epochs only grow; the signed difference keeps the comparison right across a wrap of the counter
    while (static_cast<int>(ld_acquire_sys(mine) - p.epoch) < 0) {
      if (clock64() - t0 > p.limit_cycles) {
        atomicCAS(p.status, kStatusOk, kStatusPeerTimeout);
        return;
      }
      __nanosleep(200);
    }
  }
}

template <typename OUT_T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t *>(&h);
}

template <typename OUT_T>
__device__ __forceinline__ void store8(OUT_T *dst, const float (&v)[8]) {
  if constexpr (sizeof(OUT_T) == 4) {
    reinterpret_cast<float4 *>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4 *>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    *reinterpret_cast<uint4 *>(dst) = make_uint4(pack2<OUT_T>(v[0], v[1]), pack2<OUT_T>(v[2], v[3]),
                                                 pack2<OUT_T>(v[4], v[5]), pack2<OUT_T>(v[6], v[7]));
  }
}

// One thread per group of 8 consecutive columns. STAGE_I32: slots hold int32 partial accumulators, else bf16 partials.
template <typename OUT_T, bool STAGE_I32>
__global__ void __launch_bounds__(256) reduce_dequant_kernel(const __grid_constant__ ReduceLaunch r) {
  if (r.status != nullptr && *reinterpret_cast<const volatile int *>(r.status) != kStatusOk) return;
  const long long groups_per_row = r.N / 8;
  const long long total = static_cast<long long>(r.rows) * groups_per_row;
  const bool has_bias = r.bias != nullptr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int m = static_cast<int>(i / groups_per_row);
    const int n = static_cast<int>(i - m * groups_per_row) * 8;
    const long long at = m * r.stage_stride + n;
    float v[8];
    if constexpr (STAGE_I32) {
      const int32_t *base = static_cast<const int32_t *>(r.stage) + at;
      int4 part[kMaxPeers][2];
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s) {  // all loads first: world x 32 bytes in flight per thread
        if (s < r.world) {
          part[s][0] = *reinterpret_cast<const int4 *>(base + s * r.slot_stride);
          part[s][1] = *reinterpret_cast<const int4 *>(base + s * r.slot_stride + 4);
        }
      }
      int acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s) {
        if (s < r.world) {
          acc[0] += part[s][0].x; acc[1] += part[s][0].y; acc[2] += part[s][0].z; acc[3] += part[s][0].w;
          acc[4] += part[s][1].x; acc[5] += part[s][1].y; acc[6] += part[s][1].z; acc[7] += part[s][1].w;
        }
      }
      const float sa = r.sa[m];
      const float4 w0 = *reinterpret_cast<const float4 *>(r.sw + n), w1 = *reinterpret_cast<const float4 *>(r.sw + n + 4);
      const float sw[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(__fmul_rn(__int2float_rn(acc[j]), sa), sw[j]);
    } else {
      const __nv_bfloat16 *base = static_cast<const __nv_bfloat16 *>(r.stage) + at;
      uint4 part[kMaxPeers];
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s) {
        if (s < r.world) part[s] = *reinterpret_cast<const uint4 *>(base + s * r.slot_stride);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.0f;
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s) {
        if (s < r.world) {
          const uint32_t w[4] = {part[s].x, part[s].y, part[s].z, part[s].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[2 * j] = __fadd_rn(v[2 * j], __uint_as_float(w[j] << 16));
            v[2 * j + 1] = __fadd_rn(v[2 * j + 1], __uint_as_float(w[j] & 0xFFFF0000u));
          }
        }
      }
    }
    if (has_bias) {
      const float4 b0 = *reinterpret_cast<const float4 *>(r.bias + n), b1 = *reinterpret_cast<const float4 *>(r.bias + n + 4);
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __fadd_rn(v[j], b[j]);
    }
    if (r.low != nullptr) {  // the low-rank term joins after the bias, as in the product's epilogue
      const float *lp = r.low + m * r.low_stride + n;
      const float4 l0 = *reinterpret_cast<const float4 *>(lp), l1 = *reinterpret_cast<const float4 *>(lp + 4);
      const float l[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = __fadd_rn(v[j], l[j]);
    }
    const long long dst = (static_cast<long long>(r.row0) + m) * r.c_stride + n;
    if constexpr (sizeof(OUT_T) == 4) {
      if (r.gate != nullptr) {  // X += gate[type] * v: one multiply, one add, like the product's own epilogue 1
        float *x = static_cast<float *>(r.out[0]) + dst;
        const float *gr = r.gate + static_cast<long long>(r.rtype[m]) * r.g_stride + n;
        const float4 x0 = *reinterpret_cast<const float4 *>(x), x1 = *reinterpret_cast<const float4 *>(x + 4);
        const float4 g0 = *reinterpret_cast<const float4 *>(gr), g1 = *reinterpret_cast<const float4 *>(gr + 4);
        reinterpret_cast<float4 *>(x)[0] = make_float4(__fadd_rn(x0.x, __fmul_rn(g0.x, v[0])), __fadd_rn(x0.y, __fmul_rn(g0.y, v[1])),
                                                       __fadd_rn(x0.z, __fmul_rn(g0.z, v[2])), __fadd_rn(x0.w, __fmul_rn(g0.w, v[3])));
        reinterpret_cast<float4 *>(x)[1] = make_float4(__fadd_rn(x1.x, __fmul_rn(g1.x, v[4])), __fadd_rn(x1.y, __fmul_rn(g1.y, v[5])),
                                                       __fadd_rn(x1.z, __fmul_rn(g1.z, v[6])), __fadd_rn(x1.w, __fmul_rn(g1.w, v[7])));
        continue;
      }
    }
#pragma unroll
    for (int o = 0; o < kMaxPeers; ++o) {
      if (o < r.n_out) store8(static_cast<OUT_T *>(r.out[o]) + dst, v);
    }
  }
}

template <typename OUT_T>
cudaError_t launch_typed(const ReduceLaunch &r, int sms, cudaStream_t stream) {
  const long long work = static_cast<long long>(r.rows) * (r.N / 8);
  long long blocks = (work + 255) / 256;
  const long long cap = static_cast<long long>(sms) * 8;  // a multiple of the SM count; grid-stride covers the rest
  if (blocks > cap) blocks = cap;
  if (r.stage_dtype == kDtypeI32) reduce_dequant_kernel<OUT_T, true><<<static_cast<int>(blocks), 256, 0, stream>>>(r);
  else reduce_dequant_kernel<OUT_T, false><<<static_cast<int>(blocks), 256, 0, stream>>>(r);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_peer_sync(const PeerSync &p, cudaStream_t stream) {
  peer_sync_kernel<<<1, 32, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_reduce_dequant(const ReduceLaunch &r, int sms, cudaStream_t stream) {
  if (r.stage_dtype != kDtypeI32 && r.stage_dtype != kDtypeBf16) return cudaErrorInvalidValue;
  if (r.gate != nullptr && (r.c_dtype != kDtypeF32 || r.n_out != 1 || r.rtype == nullptr)) return cudaErrorInvalidValue;
  switch (r.c_dtype) {
    case kDtypeBf16: return launch_typed<__nv_bfloat16>(r, sms, stream);
    case kDtypeF16: return launch_typed<__half>(r, sms, stream);
    case kDtypeF32: return launch_typed<float>(r, sms, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace h3b
