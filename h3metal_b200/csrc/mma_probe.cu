// Issue-rate probe of the int8 tensor pipe: the ceiling the product kernels' fractions are quoted against.
//
// The reference measures the matrix-unit peak it compares its products with by a kernel that only multiplies
// fragments already in registers (bench/hw/mma_rate.py:9-24 and bench/hw/mma_rate.metal of the reference). The
// analogue here: one CTA per SM, both operand tiles resident in shared memory (written once by the CTA itself, no
// TMA inside the loop, no epilogue), and ONE thread issuing a fixed number of
// tcgen05.mma kind::i8 instructions of the product kernels' shape (M 128 or 256 over a CTA pair, N 256, K 32) that
// alternate between two int32 accumulators in tensor memory. One commit and one bounded wait end the run. The CTA
// reports the clock64 cycles between the first issue and the completion of the last instruction.
#include "kernels.h"
#include "ptx.cuh"

namespace h3b {
namespace {

constexpr int kProbeThreads = 128;
constexpr int kProbeABytes = 128 * 128;  // 128 rows x 128 bytes of K (one 128-byte swizzle span per row)
constexpr int kProbeN = 256;

template <bool PAIR>
__global__ void __launch_bounds__(kProbeThreads, 1) mma_probe_kernel(const int iters, int *status,
                                                                     unsigned long long *cycles) {
  // PAIR: each CTA of the pair holds its own 128 rows of A and half (128 rows) of the 256-row B operand
  constexpr int kBRows = PAIR ? kProbeN / 2 : kProbeN;
  constexpr int kBBytes = kBRows * 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *tiles = smem_raw + (base - raw_addr);
  const uint32_t bar = base + kProbeABytes + kBBytes;
  volatile uint32_t *tmem_holder = reinterpret_cast<volatile uint32_t *>(tiles + kProbeABytes + kBBytes + 8);
  volatile int *cta_abort = reinterpret_cast<volatile int *>(tiles + kProbeABytes + kBBytes + 12);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // operands: a fixed pseudo-random byte pattern (values matter only for the power the multipliers draw)
  uint32_t *words = reinterpret_cast<uint32_t *>(tiles);
  for (int i = threadIdx.x; i < (kProbeABytes + kBBytes) / 4; i += kProbeThreads) {
    uint32_t v = (static_cast<uint32_t>(i) + 0x9E3779B9u * (blockIdx.x + 1u)) * 0x85EBCA6Bu;
    v ^= v >> 13;
    v *= 0xC2B2AE35u;
    words[i] = v ^ (v >> 16);
  }
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *cta_abort = 0;
    fence_barrier_init();
  }
  fence_proxy_async_smem();  // the tensor core reads shared memory through the asynchronous proxy
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(smem_u32(const_cast<uint32_t *>(tmem_holder)), 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_holder)), 512);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  if (PAIR) cluster_sync_all();
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  const bool issuer = warp == 0 && lane == 0 && (!PAIR || cluster_cta_rank() == 0);
  const bool waiter = warp == 0 && lane == 0;

  long long t0 = 0;
  if (issuer) {
    constexpr uint32_t idesc = umma_instr_desc(2, 1, PAIR ? 256 : 128, kProbeN);  // s32 accumulate, s8 x s8
    const uint64_t ad = umma_smem_desc(base, 1024, 2);
    const uint64_t bd = umma_smem_desc(base + kProbeABytes, 1024, 2);
    t0 = clock64();
#pragma unroll 1
    for (int i = 0; i < iters; ++i) {
      const uint32_t d = tmem_base + (i & 1) * kProbeN;
#pragma unroll
      for (int k = 0; k < 4; ++k) {  // the four 32-byte K steps of the 128-byte span
        if (PAIR) umma_i8_pair(d, ad + 2u * k, bd + 2u * k, idesc, (i > 1 || k > 0) ? 1u : 0u);
        else umma_i8(d, ad + 2u * k, bd + 2u * k, idesc, (i > 1 || k > 0) ? 1u : 0u);
      }
    }
    if (PAIR) umma_commit_pair(bar, 3);
    else umma_commit(bar);
  } else if (waiter) {
    t0 = clock64();
  }
  if (waiter) {
    // the only wait of the kernel, bounded: the whole run is tens of milliseconds
    const bool ok = mbar_wait(bar, 0, cta_abort, status, kStatusMmaTimeout, 4 * kWaitLimitCycles);
    cycles[blockIdx.x] = ok ? static_cast<unsigned long long>(clock64() - t0) : 0ull;
  }
  tc_fence_before_sync();
  if (PAIR) cluster_sync_all();
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, 512);
    else tmem_dealloc(tmem_base, 512);
  }
}

// More than half of an SM's shared memory, so that no two CTAs share an SM (and its tensor memory).
constexpr size_t probe_smem(bool) { return 120 * 1024; }
static_assert(1024 + kProbeABytes + kProbeN * 128 + 64 <= 120 * 1024, "tiles fit the request");

}  // namespace

cudaError_t launch_mma_probe(int pair, int iters, int *ctas, int *status, unsigned long long *cycles,
                             cudaStream_t stream) {
  cudaError_t e;
  if (pair) {
    if ((e = cudaFuncSetAttribute(mma_probe_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(probe_smem(true)))) != cudaSuccess)
      return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2);
    cfg.blockDim = dim3(kProbeThreads);
    cfg.dynamicSmemBytes = probe_smem(true);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    // only as many pairs as can be resident at once: a second wave would double the time
    int fit = 0;
    if ((e = cudaOccupancyMaxActiveClusters(&fit, mma_probe_kernel<true>, &cfg)) != cudaSuccess) return e;
    if (fit < 1) return cudaErrorLaunchOutOfResources;
    if (2 * fit < *ctas) *ctas = 2 * fit;
    *ctas &= ~1;
    cfg.gridDim = dim3(*ctas);
    return cudaLaunchKernelEx(&cfg, mma_probe_kernel<true>, iters, status, cycles);
  }
  if ((e = cudaFuncSetAttribute(mma_probe_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(probe_smem(false)))) != cudaSuccess)
    return e;
  mma_probe_kernel<false><<<*ctas, kProbeThreads, probe_smem(false), stream>>>(iters, status, cycles);
  return cudaGetLastError();
}

}  // namespace h3b
