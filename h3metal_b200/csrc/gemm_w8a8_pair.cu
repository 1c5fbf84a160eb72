// W8A8 product on CTA pairs: C tile 256 x 256 per cluster of two CTAs, tcgen05.mma cta_group::2.
//
// Same arithmetic and epilogue as gemm_w8a8.cu (the reference's kernels/gemm.metal:117-153,201-260, int8 format,
// storing or gated epilogue, optional low-rank term :211-229). Why pairs: a pair shares the W operand. Each CTA
// stages its own 128 rows of A and only HALF of the 256 W rows (32 KB per K block instead of 48), the hardware feeds
// both tensor cores from both halves, and the bytes that travel from L2 into shared memory and from shared memory
// into the tensor core per multiply drop by a third. On a power-capped board that saved data movement is throughput.
//
// Roles per CTA (rank 0 = leader, rank 1 = peer):
//   warp 0   TMA producer: own A rows and own half of W into this CTA's ring; completion bytes of BOTH CTAs are
//            counted on the LEADER's full barrier (the leader's producer arms it with the pair's total). With a
//            low-rank term the tile's T rows and this CTA's half of the B' rows travel through the same ring after
//            the K blocks, 64 ranks per stage.
//   warp 1   leader only: issues the 256-row MMAs (kind::i8 into the int32 accumulator, then kind::f16 for the
//            low-rank term into a second, fp32 accumulator), releases a stage to both producers with a commit that
//            arrives on both CTAs' empty barriers, and hands the accumulators to both epilogues the same way.
//   warps 2.. epilogue of this CTA's 128 rows (TMEM lanes of this SM): four warps, one per lane quarter, or - with
//            a low-rank term - sixteen, four per quarter with 64 columns each; they free the accumulator stage by
//            arriving on the LEADER's accumulator-empty barrier (the peer through the cluster address).
// Tensor memory is allocated for the pair (512 columns each): two 256-column int32 accumulators, so that the
// epilogue of one tile overlaps the main loop of the next. With a low-rank term there is room for one int32 and one
// fp32 accumulator only, and the hand-over is split in two: an epilogue warp copies its int32 values to registers
// and frees that accumulator before any arithmetic (the next tile's main loop starts after one TMEM read), and
// gives the fp32 accumulator back on a barrier of its own, which the leader waits for only before the next tile's
// LAST instructions - the term's.
//
// Staged stores (16-bit outputs, no gate): an epilogue warp converts its 32 rows of the tile into 128-byte-swizzled
// panels of 64 columns in shared memory (16 KB per lane quarter), gives the accumulator back as soon as its last
// tcgen05.ld has landed in registers, and lets TMA write the panels to global memory (cp.async.bulk.tensor, store
// form, this GPU's memory only) while the tensor cores already work on the next tile.
// Launched with programmatic stream serialization when the context asks for it: the set-up above the first global
// access overlaps the previous kernel's tail.
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
constexpr int kHalfBBytes = 128 * kLoraChunk * 2;  // this CTA's half of a 32-rank chunk of B': 8 KB
constexpr int kOutPanel = 32 * 128;                // 32 rows x 64 two-byte columns
constexpr int kOutWarp = 4 * kOutPanel;            // a warp's 32 rows x 256 columns
constexpr int kOutBytes = 4 * kOutWarp;            // 64 KB per CTA

// 32 consecutive output values of row `lane` of the warp, packed to 16-bit, into the warp's staging panel that
// holds columns [64 * (c / 2), +64): piece p of row r sits at p ^ (r & 7) (the 128-byte swizzle TMA expects).
template <typename OUT_T>
__device__ __forceinline__ void stage_out32(uint8_t *warp_buf, int c, int lane, const float (&v)[32]) {
  uint32_t w[32];
  Packed<OUT_T>::pack(v, w);
  uint8_t *row = warp_buf + (c >> 1) * kOutPanel + lane * 128;
  const int first = (c & 1) * 4;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4 *>(row + (((first + j) ^ (lane & 7)) << 4)) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}

template <bool LORA, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(64 + 32 * EPI, 1)
gemm_w8a8_pair_kernel(const __grid_constant__ GemmLaunch g, const int stages) {
  static_assert((!LORA && EPI == 4) || (LORA && EPI == 16), "four epilogue warps, or sixteen with a low-rank term");
  constexpr int kAccStages = LORA ? 1 : 2;
  constexpr int kWarpCols = kPairBN / (EPI / 4);  // columns of the tile one epilogue warp finishes
  constexpr int kWarpChunks = kWarpCols / 32;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw_addr);
  // [ring: stages x 32 KB][staged stores: 64 KB, optional][barriers 256 B][column scales and biases 8 KB]
  const uint32_t out_off = stages * kPairStage;
  const uint32_t bars_off = out_off + (g.tma_store ? kOutBytes : 0);
  const uint32_t bars = base + bars_off;
  auto full_bar = [&](int i) { return bars + 8u * i; };
  auto empty_bar = [&](int i) { return bars + 64u + 8u * i; };
  auto acc_full_bar = [&](int i) { return bars + 128u + 8u * i; };
  auto acc_empty_bar = [&](int i) { return bars + 144u + 8u * i; };
  const uint32_t low_empty_bar = bars + 160u;  // low-rank accumulator free (LORA): its own hand-over, see the epilogue
  volatile uint32_t *tmem_holder = reinterpret_cast<volatile uint32_t *>(base_ptr + bars_off + 176);
  volatile int *cta_abort = reinterpret_cast<volatile int *>(base_ptr + bars_off + 180);
  float *col_stage = reinterpret_cast<float *>(base_ptr + bars_off + kBarrierBytes);  // [EPI warps][2][kWarpCols]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();
  const bool leader = rank == 0;
  const int m_tiles = (g.M + 255) / 256, n_tiles = (g.N + kPairBN - 1) / kPairBN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (g.K + kBKBytes - 1) / kBKBytes;
  const int first_tile = cluster_id_x(), tile_step = cluster_count_x();
  const int chunks = LORA ? g.R / kLoraChunk : 0;   // 32-rank chunks of the low-rank term
  const int lora_blocks = (chunks + 1) / 2;         // ring stages they take per tile (two chunks per stage)

  if (warp == 0 && lane == 0) {
    tma_prefetch_descriptor(&g.map_a);
    tma_prefetch_descriptor(&g.map_w);
    if (LORA) {
      tma_prefetch_descriptor(&g.map_t);
      tma_prefetch_descriptor(&g.map_b);
    }
    if (g.tma_store) tma_prefetch_descriptor(&g.map_c);
    for (int i = 0; i < stages; ++i) {
      mbar_init(full_bar(i), 1);   // the leader's producer arms it; bytes arrive from both CTAs
      mbar_init(empty_bar(i), 1);  // one commit arrival per use
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full_bar(i), 1);
      mbar_init(acc_empty_bar(i), 2 * EPI);  // the epilogue warps of both CTAs of the pair
    }
    mbar_init(low_empty_bar, 2 * EPI);
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
  // everything above touched only the pair's shared and tensor memory; from here on global memory is read and written,
  // which must wait for the kernel before this one in the stream (a no-op unless launched with programmatic stream
  // serialization)
  grid_dep_launch();
  grid_dep_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------------------------- TMA producer (both CTAs)
    if (lane == 0) {
      // ring position stepped by hand: the loop runs once per K block (512 cycles at full tensor rate) in one thread
      RingPos pos;
      uint32_t filled = 0;  // stages this thread has filled so far, saturating at `stages` (for the wind-down)
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
          filled += filled < static_cast<uint32_t>(stages);
        }
        if (!ok) break;
        if (LORA) {  // the term's operands follow the tile's K blocks (its MMAs are the tile's last)
          for (int j = 0; ok && j < lora_blocks; ++j) {
            const uint32_t s = pos.s;
            ok = mbar_wait(empty_bar(s), pos.ph ^ 1u, cta_abort, g.status, kStatusProducerTimeout);
            if (!ok) break;
            const int n_here = min(2, chunks - 2 * j);
            if (leader) mbar_arrive_expect_tx(full_bar(s), 2u * n_here * (kLoraTBytes + kHalfBBytes));
            const uint32_t leader_full = leader_full0 + 8u * s;
            const uint32_t dst = base + s * kPairStage;
            for (int c = 0; c < n_here; ++c) {
              tma_load_2d_pair(dst + c * kLoraTBytes, &g.map_t, leader_full, (2 * j + c) * kLoraChunk, m0);
              tma_load_2d_pair(dst + kABytes + c * kHalfBBytes, &g.map_b, leader_full, (2 * j + c) * kLoraChunk, n0);
            }
            pos.advance(stages);
            filled += filled < static_cast<uint32_t>(stages);
          }
        }
      }
      if (*cta_abort && leader) {
        // wind-down after a timeout: the pair's copies into the last stages filled are counted on the leader's full
        // barriers; wait (bounded) for them so that neither CTA leaves with copies still landing in its shared memory
        for (uint32_t j = 0; j < filled; ++j) {
          pos.retreat(stages);
          int dummy_abort = 0;
          mbar_wait(full_bar(pos.s), pos.ph, &dummy_abort, g.status, kStatusDrainTimeout, kDrainLimitCycles);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------------------------- MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_instr_desc(2, 1, 256, kPairBN);      // s32 accumulate, s8 x s8, M 256 over the pair
      constexpr uint32_t idesc_f16 = umma_instr_desc(1, 0, 256, kPairBN);  // f32 accumulate, f16 x f16
      uint32_t at = 0;
      RingPos pos;
      bool ok = true;
      const uint64_t ad0 = umma_smem_desc(base, 1024, 2);
      const uint64_t bd0 = umma_smem_desc(base + kABytes, 1024, 2);
      for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++at) {
        const int as = at % kAccStages;
        const uint32_t aph = (at / kAccStages) & 1u;
        ok = mbar_wait(acc_empty_bar(as), aph ^ 1u, cta_abort, g.status, kStatusMmaTimeout);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_acc = tmem_base + as * kPairBN;
        // the tile's rank range is needed after the main loop only: its two loads are issued here, off the critical path
        int k0 = 0, k1 = g.R;
        if (LORA && g.ranges != nullptr) {
          const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, g.band);
          k0 = ld_nc_s32_here(g.ranges + 2 * tc.n_blk);
          k1 = ld_nc_s32_here(g.ranges + 2 * tc.n_blk + 1);
        }
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
        if (LORA) {
          // The low-rank MMAs are the tile's last: the fp32 accumulator they write is handed back by the epilogue of
          // the tile before on a barrier of its own, long after that epilogue has freed the int32 accumulator - so the
          // main loop above already ran while the epilogue was still finishing.
          ok = mbar_wait(low_empty_bar, aph ^ 1u, cta_abort, g.status, kStatusMmaTimeout);
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t d_low = tmem_base + kLowBase;
          for (int j = 0; ok && j < lora_blocks; ++j) {
            const uint32_t s = pos.s;
            ok = mbar_wait(full_bar(s), pos.ph, cta_abort, g.status, kStatusMmaTimeout);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t a_addr = base + s * kPairStage;
            const int lo = max(k0, 2 * j * kLoraChunk), hi = min(k1, (2 * j + 2) * kLoraChunk);
            for (int kk = lo; kk < hi; kk += 16) {  // one kind::f16 instruction covers 16 ranks = 32 bytes
              const int c = kk / kLoraChunk - 2 * j;
              const uint32_t koff = ((kk % kLoraChunk) * 2) >> 4;
              const uint64_t td = umma_smem_desc(a_addr + c * kLoraTBytes, 512, 4) + koff;
              const uint64_t bd = umma_smem_desc(a_addr + kABytes + c * kHalfBBytes, 512, 4) + koff;
              umma_f16_pair(d_low, td, bd, idesc_f16, kk != k0 ? 1u : 0u);
            }
            umma_commit_pair(empty_bar(s), 3);
            pos.advance(stages);
          }
          if (!ok) break;
        }
        umma_commit_pair(acc_full_bar(as), 3);  // both epilogues
      }
    }
  } else {
    // ---------------------------------------------------------------------------------- epilogue (both CTAs)
    // A warp reads the TMEM lanes of its quarter (warp index mod 4); the EPI / 4 warps of a quarter split the columns.
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    const int c_begin = part * kWarpChunks;
    const int row = quarter * 32 + lane;
    const bool raw = g.c_dtype == kDtypeI32;
    const size_t esize = (g.c_dtype == kDtypeF32 || raw) ? 4 : 2;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(g.c) % 16 == 0) && ((g.c_stride * esize) % 16 == 0);
    const bool staged = g.tma_store != 0;
    uint8_t *out_buf = base_ptr + out_off + quarter * kOutWarp;  // this warp's staging (staged stores only)
    const uint32_t out_addr = base + out_off + quarter * kOutWarp;
    const uint32_t leader_acc_empty0 = map_to_cta(acc_empty_bar(0), 0);
    const uint32_t leader_low_empty = map_to_cta(low_empty_bar, 0);
    uint32_t at = 0;
    bool ok = true;
    for (int tile = first_tile; ok && tile < num_tiles; tile += tile_step, ++at) {
      const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, g.band);
      const int m0 = tc.m_blk * 256 + static_cast<int>(rank) * 128, n0 = tc.n_blk * kPairBN;
      const int as = at % kAccStages;
      const uint32_t aph = (at / kAccStages) & 1u;
      float *sw_s = col_stage + (warp - 2) * 2 * kWarpCols, *bias_s = sw_s + kWarpCols;  // this warp's columns only
      stage_columns(g, n0 + part * kWarpCols, kWarpCols, lane, sw_s, bias_s);
      const int m = m0 + row;
      const float sa_m = (!raw && m < g.M) ? __ldg(g.sa + m) : 0.0f;
      bool has_low = false;
      if (LORA) {
        int k0 = 0, k1 = g.R;
        if (g.ranges != nullptr) {
          k0 = g.ranges[2 * tc.n_blk];
          k1 = g.ranges[2 * tc.n_blk + 1];
        }
        has_low = k1 > k0;
      }
      if (staged) {
        // the panels of the tile before this one must have been read out of shared memory before they are rewritten
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
      }
      ok = mbar_wait(acc_full_bar(as), aph, cta_abort, g.status, kStatusEpilogueTimeout);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * kPairBN;
      const uint32_t t_low = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kLowBase;
      auto release = [&]() {  // every value of the accumulator is in registers: the leader may overwrite it
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_acc_empty0 + 8u * as);
      };
      if constexpr (LORA) {
        // Split hand-over. The warp reads both of its 32-column chunks of the int32 accumulator into registers and frees
        // that accumulator at once: the leader starts the next tile's main loop while the arithmetic below runs. The
        // low-rank accumulator is written by the LAST instructions of a tile, so it is handed back on a barrier of its
        // own after it has been read, long before the leader needs it. The exposed part of the epilogue is one TMEM
        // read; the values are identical to the joint order (the term is the last addend either way).
        uint32_t a0[32], a1[32];
        const uint32_t no_low[32] = {};
        tmem_ld_32x32b_x32(t_acc + c_begin * 32, a0);
        tmem_ld_32x32b_x32(t_acc + (c_begin + 1) * 32, a1);
        tmem_ld_wait();
        release();
        auto put = [&](const float (&v)[32], int c) {
          if (staged) {
            if (g.c_dtype == kDtypeBf16) stage_out32<__nv_bfloat16>(out_buf, c, lane, v);
            else stage_out32<__half>(out_buf, c, lane, v);
          } else {
            store_values32(g, v, m, n0 + c * 32, vec_ok);
          }
        };
        // the term's 64 columns come in pieces of 16: with both int32 chunks held, registers are the limit
        auto add_low = [&](float (&v)[32], int c, int half) {
          uint32_t low[16];
          tmem_ld_32x32b_x16(t_low + c * 32 + half * 16, low);
          tmem_ld_wait();
          if (c == c_begin + 1 && half == 1) {  // the warp's last values of the low-rank accumulator are in registers
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_low_empty);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) v[half * 16 + j] = __fadd_rn(v[half * 16 + j], __uint_as_float(low[j]));
        };
        float v[32];
        dequant32(g, a0, no_low, false, sa_m, sw_s, bias_s, v);
        if (has_low) {
          add_low(v, c_begin, 0);
          add_low(v, c_begin, 1);
        }
        put(v, c_begin);
        dequant32(g, a1, no_low, false, sa_m, sw_s + 32, bias_s + 32, v);
        if (has_low) {
          add_low(v, c_begin + 1, 0);
          add_low(v, c_begin + 1, 1);
        } else {
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(leader_low_empty);  // nothing to read: hand it back unread
        }
        put(v, c_begin + 1);
      } else {
        // two register sets: the TMEM loads of the next 32 columns are in flight while this chunk is finished
        uint32_t acc_a[32], acc_b[32];
        const uint32_t no_low[32] = {};
        auto finish = [&](const uint32_t (&acc)[32], int c) {  // c: chunk of the tile
          const float *sw_c = sw_s + (c - c_begin) * 32, *bias_c = bias_s + (c - c_begin) * 32;
          if (staged) {
            float v[32];
            dequant32(g, acc, no_low, false, sa_m, sw_c, bias_c, v);
            if (g.c_dtype == kDtypeBf16) stage_out32<__nv_bfloat16>(out_buf, c, lane, v);
            else stage_out32<__half>(out_buf, c, lane, v);
          } else {
            finish_chunk(g, acc, no_low, false, m, n0 + c * 32, sa_m, sw_c, bias_c, vec_ok);
          }
        };
        tmem_ld_32x32b_x32(t_acc + c_begin * 32, acc_a);
#pragma unroll 1
        for (int c = c_begin; c < c_begin + kWarpChunks; c += 2) {
          tmem_ld_wait();
          tmem_ld_32x32b_x32(t_acc + (c + 1) * 32, acc_b);
          finish(acc_a, c);
          tmem_ld_wait();
          if (c + 2 < c_begin + kWarpChunks) tmem_ld_32x32b_x32(t_acc + (c + 2) * 32, acc_a);
          else release();  // the warp's last values have left tensor memory
          finish(acc_b, c + 1);
        }
      }
      if (staged) {
        // generic-proxy writes -> visible to the asynchronous proxy, then one thread hands the warp's panels to TMA
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int y = m0 + quarter * 32;
          if (y < g.M) {
            constexpr int kPanels = kWarpCols >= 64 ? kWarpCols / 64 : 1;
#pragma unroll
            for (int i = 0; i < kPanels; ++i) {
              const int pnl = (c_begin >> 1) + i;
              if (n0 + pnl * 64 < g.N) tma_store_2d(&g.map_c, out_addr + pnl * kOutPanel, n0 + pnl * 64, y);
            }
          }
          tma_store_commit();
        }
      }
    }
    if (staged && lane == 0) tma_store_wait_all();  // the last panels have left shared memory and reached global memory
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

size_t gemm_pair_smem_bytes(int stages, bool staged_stores) {
  return 1024 + static_cast<size_t>(stages) * kPairStage + (staged_stores ? kOutBytes : 0) + kBarrierBytes +
         8 * static_cast<size_t>(kPairBN) * sizeof(float);
}

int gemm_pair_pick_stages(size_t smem_optin, bool staged_stores) {
  for (int s = kPairMaxStages; s >= 2; --s)
    if (gemm_pair_smem_bytes(s, staged_stores) <= smem_optin) return s;
  return 0;
}

cudaError_t gemm_pair_configure() {
  cudaError_t e;
#define H3B_PAIR_CFG(L, E)                                                                                             \
  if ((e = cudaFuncSetAttribute(gemm_w8a8_pair_kernel<L, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448)) != \
      cudaSuccess)                                                                                                     \
    return e;
  H3B_PAIR_CFG(false, 4) H3B_PAIR_CFG(true, 16)
#undef H3B_PAIR_CFG
  return cudaSuccess;
}

// Largest number of CTA pairs that can be resident at once (a persistent kernel must not launch more).
int gemm_pair_max_clusters(int stages) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(64 + 32 * 4, 1, 1);
  cfg.dynamicSmemBytes = gemm_pair_smem_bytes(stages, false);
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0, n_low = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_w8a8_pair_kernel<false, 4>, &cfg) != cudaSuccess) return 0;
  cfg.blockDim = dim3(64 + 32 * 16, 1, 1);
  if (cudaOccupancyMaxActiveClusters(&n_low, gemm_w8a8_pair_kernel<true, 16>, &cfg) != cudaSuccess) return 0;
  return n < n_low ? n : n_low;
}

template <bool LORA, int EPI>
cudaError_t launch_pair(const GemmLaunch &g, int stages, int clusters, size_t smem, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);  // the cluster shape (2, 1, 1) is part of the kernel's declaration
  cfg.blockDim = dim3(64 + 32 * EPI);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g.overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemm_w8a8_pair_kernel<LORA, EPI>, g, stages);
}

cudaError_t launch_gemm_w8a8_pair(const GemmLaunch &g, int stages, int clusters, cudaStream_t stream) {
  const size_t smem = gemm_pair_smem_bytes(stages, g.tma_store != 0);
  // with a low-rank term: one int32 accumulator, so its hand-over is exposed and sixteen warps share the epilogue
  if (g.R > 0) return launch_pair<true, 16>(g, stages, clusters, smem, stream);
  return launch_pair<false, 4>(g, stages, clusters, smem, stream);
}

}  // namespace h3b
