// W8A8 product on CTA pairs: C tile 256 x 256 per cluster of two CTAs, tcgen05.mma cta_group::2.
//
// Same arithmetic and epilogue as gemm_w8a8.cu (the reference's kernels/gemm.metal:117-153,201-260, int8 format,
// storing epilogue; no low-rank term here). Why pairs: with one CTA per 128 x 256 tile every MMA (128 cycles)
// makes the tensor core read 12 KB of shared memory while TMA writes another 12 KB, which together saturate the
// SM's 128 B/clk shared-memory path at about two thirds of the tensor rate. A pair shares the B operand: each CTA
// stages its own 128 rows of A and only HALF of the 256 W rows (32 KB per stage instead of 48), the hardware feeds
// both tensor cores from both halves, and the per-SM shared-memory traffic per MMA drops by a third.
//
// Roles per CTA (rank 0 = leader, rank 1 = peer):
//   warp 0   TMA producer: own A rows and own half of W into this CTA's ring; completion bytes of BOTH CTAs are
//            counted on the LEADER's full barrier (the leader's producer arms it with the pair's total).
//   warp 1   leader only: issues the 256-row MMAs, releases a stage to both producers with a commit that arrives
//            on both CTAs' empty barriers, and hands the accumulator to both epilogues the same way.
//   warps 2-5 epilogue of this CTA's 128 rows (TMEM lanes of this SM); they free the accumulator stage by arriving
//            on the LEADER's accumulator-empty barrier (the peer through the cluster address).
// Tensor memory is allocated for the pair (512 columns each: two 256-column int32 accumulators, double-buffered).
// All waits are bounded as in the single-CTA kernel. No load uses multicast.
#include <cuda.h>

#include "gemm_common.cuh"

namespace h3b {
namespace {

using namespace gemm;

constexpr int kPairBN = 256;                       // columns per pair tile
constexpr int kHalfWBytes = 128 * kBKBytes;        // this CTA's half of the W tile
constexpr int kPairStage = kABytes + kHalfWBytes;  // 32 KB
constexpr int kPairMaxStages = 6;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_w8a8_pair_kernel(const __grid_constant__ GemmLaunch g, const int stages) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw_addr);
  const uint32_t bars_off = stages * kPairStage;
  const uint32_t bars = base + bars_off;
  auto full_bar = [&](int i) { return bars + 8u * i; };
  auto empty_bar = [&](int i) { return bars + 64u + 8u * i; };
  auto acc_full_bar = [&](int i) { return bars + 128u + 8u * i; };
  auto acc_empty_bar = [&](int i) { return bars + 144u + 8u * i; };
  volatile uint32_t *tmem_holder = reinterpret_cast<volatile uint32_t *>(base_ptr + bars_off + 176);
  volatile int *cta_abort = reinterpret_cast<volatile int *>(base_ptr + bars_off + 180);
  float *col_stage = reinterpret_cast<float *>(base_ptr + bars_off + kBarrierBytes);  // [4 warps][2][256]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const int m_tiles = (g.M + 255) / 256, n_tiles = (g.N + kPairBN - 1) / kPairBN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (g.K + kBKBytes - 1) / kBKBytes;
  const int first_tile = cluster_id_x(), tile_step = cluster_count_x();

  if (warp == 0 && lane == 0) {
    tma_prefetch_descriptor(&g.map_a);
    tma_prefetch_descriptor(&g.map_w);
    for (int i = 0; i < stages; ++i) {
      mbar_init(full_bar(i), 1);   // the leader's producer arms it; bytes arrive from both CTAs
      mbar_init(empty_bar(i), 1);  // one commit arrival per use
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full_bar(i), 1);
      mbar_init(acc_empty_bar(i), 8);  // four epilogue warps in each CTA of the pair
    }
    *cta_abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t *>(tmem_holder)), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();  // barriers of both CTAs exist before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ---------------------------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      // ring position stepped by hand: the loop runs once per K block (512 cycles at full tensor rate) in one thread
      RingPos pos;
      const uint32_t leader_full0 = map_to_cta(full_bar(0), 0);  // the leader's full barriers, 8 bytes apart
      bool ok = true;
      for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step) {
        const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, g.band);
        const int m0 = tc.m_blk * 256 + static_cast<int>(rank) * 128;
        const int n0 = tc.n_blk * kPairBN + static_cast<int>(rank) * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          const uint32_t s = pos.s;
          ok = mbar_wait(empty_bar(s), pos.ph ^ 1u, cta_abort, g.status, kStatusProducerTimeout);
          if (!ok) break;
          if (leader) mbar_arrive_expect_tx(full_bar(s), 2u * kPairStage);
          const uint32_t leader_full = leader_full0 + 8u * s;
          const uint32_t dst = base + s * kPairStage;
          tma_load_2d_pair(dst, &g.map_a, leader_full, kb * kBKBytes, m0);
          tma_load_2d_pair(dst + kABytes, &g.map_w, leader_full, kb * kBKBytes, n0);
          pos.advance(stages);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------------------------- MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_instr_desc(2, 1, 256, kPairBN);  // s32 accumulate, s8 x s8, M 256 over the pair
      uint32_t at = 0;
      RingPos pos;
      bool ok = true;
      const uint64_t ad0 = umma_smem_desc(base, 1024, 2);
      const uint64_t bd0 = umma_smem_desc(base + kABytes, 1024, 2);
      for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++at) {
        const int as = at & 1;
        const uint32_t aph = (at >> 1) & 1u;
        ok = mbar_wait(acc_empty_bar(as), aph ^ 1u, cta_abort, g.status, kStatusMmaTimeout);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_acc = tmem_base + as * kPairBN;
        uint32_t accumulate = 0;  // the tile's first instruction overwrites the accumulator
        for (int kb = 0; kb < num_kb; ++kb) {
          const uint32_t s = pos.s;
          ok = mbar_wait(full_bar(s), pos.ph, cta_abort, g.status, kStatusMmaTimeout);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t ad = ad0 + static_cast<uint64_t>(s * (kPairStage >> 4));
          const uint64_t bd = bd0 + static_cast<uint64_t>(s * (kPairStage >> 4));
          umma_i8_pair(d_acc, ad, bd, idesc, accumulate);
          accumulate = 1;
#pragma unroll
          for (int k = 1; k < kBKBytes / 32; ++k) umma_i8_pair(d_acc, ad + 2u * k, bd + 2u * k, idesc, 1u);
          umma_commit_pair(empty_bar(s), 3);  // both producers may refill this stage once the MMAs have read it
          pos.advance(stages);
        }
        if (!ok) break;
        umma_commit_pair(acc_full_bar(as), 3);  // both epilogues
      }
    }
  } else {
    // ---------------------------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const bool raw = g.c_dtype == kDtypeI32;
    const size_t esize = (g.c_dtype == kDtypeF32 || raw) ? 4 : 2;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(g.c) % 16 == 0) && ((g.c_stride * esize) % 16 == 0);
    const uint32_t no_low[32] = {};
    uint32_t at = 0;
    bool ok = true;
    for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++at) {
      const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, g.band);
      const int m0 = tc.m_blk * 256 + static_cast<int>(rank) * 128, n0 = tc.n_blk * kPairBN;
      const int as = at & 1;
      const uint32_t aph = (at >> 1) & 1u;
      float *sw_s = col_stage + quarter * 2 * kPairBN, *bias_s = sw_s + kPairBN;
      stage_columns(g, n0, kPairBN, lane, sw_s, bias_s);
      const int m = m0 + row;
      const float sa_m = (!raw && m < g.M) ? __ldg(g.sa + m) : 0.0f;
      ok = mbar_wait(acc_full_bar(as), aph, cta_abort, g.status, kStatusEpilogueTimeout);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * kPairBN;
      // two register sets: the TMEM loads of the next 32 columns are in flight while this chunk is finished
      uint32_t acc_a[32], acc_b[32];
      tmem_ld_32x32b_x32(t_acc, acc_a);
#pragma unroll 1
      for (int c = 0; c < kPairBN / 32; c += 2) {
        tmem_ld_wait();
        tmem_ld_32x32b_x32(t_acc + (c + 1) * 32, acc_b);
        finish_chunk(g, acc_a, no_low, false, m, n0 + c * 32, sa_m, sw_s + c * 32, bias_s + c * 32, vec_ok);
        tmem_ld_wait();
        if (c + 2 < kPairBN / 32) tmem_ld_32x32b_x32(t_acc + (c + 2) * 32, acc_a);
        finish_chunk(g, acc_b, no_low, false, m, n0 + (c + 1) * 32, sa_m, sw_s + (c + 1) * 32, bias_s + (c + 1) * 32, vec_ok);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty_bar(as), 0));  // the leader's MMA thread waits for all 8
    }
  }

  // ------------------------------------------------------------------------------------ wind-down
  // Neither CTA may leave while the other can still read its shared memory, signal its barriers or write its TMEM.
  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace

size_t gemm_pair_smem_bytes(int stages) {
  return 1024 + static_cast<size_t>(stages) * kPairStage + kBarrierBytes + 8 * static_cast<size_t>(kPairBN) * sizeof(float);
}

int gemm_pair_pick_stages(size_t smem_optin) {
  for (int s = kPairMaxStages; s >= 2; --s)
    if (gemm_pair_smem_bytes(s) <= smem_optin) return s;
  return 0;
}

cudaError_t gemm_pair_configure() {
  return cudaFuncSetAttribute(gemm_w8a8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
}

// Largest number of CTA pairs that can be resident at once (a persistent kernel must not launch more).
int gemm_pair_max_clusters(int stages) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = gemm_pair_smem_bytes(stages);
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_w8a8_pair_kernel, &cfg) != cudaSuccess) return 0;
  return n;
}

cudaError_t launch_gemm_w8a8_pair(const GemmLaunch &g, int stages, int clusters, cudaStream_t stream) {
  gemm_w8a8_pair_kernel<<<2 * clusters, kThreads, gemm_pair_smem_bytes(stages), stream>>>(g, stages);
  return cudaGetLastError();
}

}  // namespace h3b
