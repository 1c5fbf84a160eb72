// W8A8 product with fused dequantising epilogue:  C[m][n] = OUT_T(float(acc) * sa[m] * sw[n] + bias[n] + low[m][n])
// with acc[m][n] = sum_k A[m][k] * W[n][k] exact in int32 and, optionally, low = T B'^T the rank-R LoRA term.
//
// This replaces the Q8 path of the reference's Metal kernel `gemm` (kernels/gemm.metal:117-153,201-260; weight
// format 1, epilogue 0, low-rank term :211-229). A is int8 [M][K] and W int8 [N][K], both K-contiguous, so the
// product is A W^T with both operands K-major. The epilogue keeps the reference's operation order in fp32:
// convert the int32 accumulator (rounds above 2^24), multiply by the row scale, multiply by the column scale, add
// the bias, add the low-rank term, convert to the output type.
//
// Blackwell mapping (sm_100a, one CTA per SM, persistent over output tiles of 128 x BN):
//   warp 0  TMA producer: one thread issues cp.async.bulk.tensor loads of the A tile (128 rows x 128 bytes of K)
//           and the W tile (BN rows x 128 bytes) into a ring of 128-byte-swizzled shared-memory stages, each
//           guarded by a full/empty mbarrier pair. Rows or K beyond the tensor are zero-filled by TMA.
//   warp 1  MMA issuer: one thread issues tcgen05.mma kind::i8 (M 128, N BN, K 32 per instruction, four per
//           stage) accumulating int32 in tensor memory; tcgen05.commit releases the stage to the producer and,
//           after the last K block, hands the accumulator to the epilogue. With a LoRA term the tile's T and B'
//           slices come through the same ring ahead of the K blocks (one stage holds 64 ranks) and the same thread
//           issues kind::f16 MMAs (fp16 x fp16 -> fp32) on them into a second TMEM region.
//   warps 2-5  epilogue: each warp owns 32 accumulator rows (its TMEM lane quarter), reads 32 columns at a time
//           with tcgen05.ld, applies scales, bias and the low-rank term and stores 64-byte row segments.
// Accumulators are double-buffered in TMEM (2 x BN columns of the 512) so the epilogue of one tile overlaps the
// main loop of the next. Tiles are visited in bands of `band` row tiles per column tile so that the A band stays
// in L2 while W streams through once per band.
//
// Every mbarrier wait is bounded (ptx.cuh): on a timeout the CTA sets the context's status word, stops taking
// tiles, waits for its own TMA copies, frees its tensor memory and returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_common.cuh"

namespace h3b {
namespace {

using namespace gemm;

template <int BN, int ACC_STAGES, bool LORA, int EPI_WARPS, bool PUSH = false>
__global__ void __launch_bounds__(64 + 32 * EPI_WARPS, 1) gemm_w8a8_kernel(const __grid_constant__ GemmLaunch g,
                                                                           const int stages) {
  static_assert(EPI_WARPS == 4, "one epilogue warp per TMEM lane quarter");
  static_assert(!(PUSH && (LORA || EPI_WARPS != 4)), "the row-parallel push has no low-rank term");
  static_assert(ACC_STAGES * BN <= (LORA ? kLowBase : kTmemCols), "accumulators do not fit tensor memory");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw_addr);

  constexpr uint32_t kWBytes = BN * kBKBytes;
  constexpr uint32_t kStage = kABytes + kWBytes;
  constexpr uint32_t kLoraBBytes = BN * kLoraChunk * 2;
  // The low-rank term's operands travel through the same ring as the main operands: before a tile's K blocks come
  // `lora_blocks` stages that hold up to two 32-rank chunks each, T in the A part and B' in the W part of the stage.
  const int chunks = LORA ? g.R / kLoraChunk : 0;
  const int lora_blocks = (chunks + 1) / 2;
  const uint32_t bars_off = stages * kStage;
  const uint32_t bars = base + bars_off;
  auto full_bar = [&](int i) { return bars + 8u * i; };
  auto empty_bar = [&](int i) { return bars + 64u + 8u * i; };
  auto acc_full_bar = [&](int i) { return bars + 128u + 8u * i; };
  auto acc_empty_bar = [&](int i) { return bars + 144u + 8u * i; };
  volatile uint32_t *tmem_holder = reinterpret_cast<volatile uint32_t *>(base_ptr + bars_off + 176);
  volatile int *cta_abort = reinterpret_cast<volatile int *>(base_ptr + bars_off + 180);
  float *col_stage = reinterpret_cast<float *>(base_ptr + bars_off + kBarrierBytes);  // [EPI_WARPS][2][BN]: sw, bias
  // PUSH: transposition buffers of outgoing chunk pairs. int32 partials: 8 KB per epilogue warp from the start of the
  // column staging (which raw accumulators do not use); bf16 partials: 4 KB per warp behind the column staging.
  uint4 *xpose_raw = reinterpret_cast<uint4 *>(col_stage);
  uint4 *xpose_bf16 = reinterpret_cast<uint4 *>(base_ptr + bars_off + kBarrierBytes + kColStageWarps * 2 * BN * sizeof(float));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (g.M + kBM - 1) / kBM, n_tiles = (g.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (g.K + kBKBytes - 1) / kBKBytes;

  if (warp == 0 && lane == 0) {
    tma_prefetch_descriptor(&g.map_a);
    tma_prefetch_descriptor(&g.map_w);
    if (LORA) {
      tma_prefetch_descriptor(&g.map_t);
      tma_prefetch_descriptor(&g.map_b);
    }
    for (int i = 0; i < stages; ++i) {
      mbar_init(full_bar(i), 1);
      mbar_init(empty_bar(i), 1);
    }
    for (int i = 0; i < ACC_STAGES; ++i) {
      mbar_init(acc_full_bar(i), 1);
      mbar_init(acc_empty_bar(i), EPI_WARPS);  // one arrival per epilogue warp
    }
    *cta_abort = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_holder)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;
  // everything above touched only this CTA's shared and tensor memory; from here on global memory is read and
  // written, which must wait for the kernel before this one in the stream
  grid_dep_launch();
  grid_dep_wait();

  if (warp == 0) {
    // ---------------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      // The ring position is a (stage, phase) pair stepped by hand: one thread issues every copy of the CTA, and at
      // full tensor rate a K block lasts 512 cycles, so the loop must stay a few dozen instructions long (a division
      // of a running count by the run-time stage count per K block alone costs a third of that).
      RingPos pos;
      uint32_t filled = 0;  // stages armed so far, saturating at `stages` (for the wind-down)
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, g.band);
        const int m0 = tc.m_blk * kBM, n0 = tc.n_blk * BN;
        if (LORA) {
          for (int j = 0; ok && j < lora_blocks; ++j) {
            ok = mbar_wait(empty_bar(pos.s), pos.ph ^ 1u, cta_abort, g.status, kStatusProducerTimeout);
            if (!ok) break;
            const int n_here = min(2, chunks - 2 * j);
            const uint32_t full = full_bar(pos.s);
            mbar_arrive_expect_tx(full, n_here * (kLoraTBytes + kLoraBBytes));
            const uint32_t dst = base + pos.s * kStage;
            for (int c = 0; c < n_here; ++c) {
              tma_load_2d(dst + c * kLoraTBytes, &g.map_t, full, (2 * j + c) * kLoraChunk, m0);
              tma_load_2d(dst + kABytes + c * kLoraBBytes, &g.map_b, full, (2 * j + c) * kLoraChunk, n0);
            }
            pos.advance(stages);
            filled += filled < static_cast<uint32_t>(stages);
          }
          if (!ok) break;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(empty_bar(pos.s), pos.ph ^ 1u, cta_abort, g.status, kStatusProducerTimeout);
          if (!ok) break;
          const uint32_t full = full_bar(pos.s);
          mbar_arrive_expect_tx(full, kStage);
          const uint32_t dst = base + pos.s * kStage;
          tma_load_2d(dst, &g.map_a, full, kb * kBKBytes, m0);
          tma_load_2d(dst + kABytes, &g.map_w, full, kb * kBKBytes, n0);
          pos.advance(stages);
          filled += filled < static_cast<uint32_t>(stages);
        }
      }
      if (*cta_abort) {
        // wind-down: wait (bounded) for the copies this thread still has in flight - the last `filled` stages armed,
        // walking back from the ring position
        for (uint32_t j = 0; j < filled; ++j) {
          pos.retreat(stages);
          int dummy_abort = 0;
          mbar_wait(full_bar(pos.s), pos.ph, &dummy_abort, g.status, kStatusDrainTimeout, kDrainLimitCycles);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_i8 = umma_instr_desc(2, 1, kBM, BN);   // s32 accumulate, s8 x s8
      constexpr uint32_t idesc_f16 = umma_instr_desc(1, 0, kBM, BN);  // f32 accumulate, f16 x f16
      uint32_t at = 0;
      RingPos pos;
      bool ok = true;
      // operand descriptors of stage 0; stage s adds s * kStage bytes (in 16-byte units) to the address field
      const uint64_t ad0 = umma_smem_desc(base, 1024, 2);
      const uint64_t bd0 = umma_smem_desc(base + kABytes, 1024, 2);
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++at) {
        const int as = at % ACC_STAGES;
        const uint32_t aph = (at / ACC_STAGES) & 1u;
        ok = mbar_wait(acc_empty_bar(as), aph ^ 1u, cta_abort, g.status, kStatusMmaTimeout);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_acc = tmem_base + as * BN;
        if (LORA) {
          const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, g.band);
          int k0 = 0, k1 = g.R;
          if (g.ranges != nullptr) {
            k0 = g.ranges[2 * tc.n_blk];
            k1 = g.ranges[2 * tc.n_blk + 1];
          }
          const uint32_t d_low = tmem_base + kLowBase + as * BN;
          for (int j = 0; ok && j < lora_blocks; ++j) {
            const int s = pos.s;
            ok = mbar_wait(full_bar(s), pos.ph, cta_abort, g.status, kStatusMmaTimeout);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t a_addr = base + s * kStage;
            const int lo = max(k0, 2 * j * kLoraChunk), hi = min(k1, (2 * j + 2) * kLoraChunk);
            for (int kk = lo; kk < hi; kk += 16) {  // one kind::f16 instruction covers 16 ranks = 32 bytes
              const int c = kk / kLoraChunk - 2 * j;
              const uint32_t koff = ((kk % kLoraChunk) * 2) >> 4;
              const uint64_t td = umma_smem_desc(a_addr + c * kLoraTBytes, 512, 4) + koff;
              const uint64_t bd = umma_smem_desc(a_addr + kABytes + c * kLoraBBytes, 512, 4) + koff;
              umma_f16(d_low, td, bd, idesc_f16, kk != k0 ? 1u : 0u);
            }
            umma_commit(empty_bar(s));  // the stage may be refilled once these MMAs have read it
            pos.advance(stages);
          }
          if (!ok) break;
        }
        // The issue loop is kept to a few dozen instructions per K block (no division, descriptors by one multiply
        // of the stage index): one thread feeds the tensor core, and four MMAs last only 512 cycles.
        uint32_t accumulate = 0;  // the tile's first instruction overwrites the accumulator
        for (int kb = 0; kb < num_kb; ++kb) {
          const uint32_t s = pos.s;
          ok = mbar_wait(full_bar(s), pos.ph, cta_abort, g.status, kStatusMmaTimeout);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t ad = ad0 + static_cast<uint64_t>(s * (kStage >> 4));
          const uint64_t bd = bd0 + static_cast<uint64_t>(s * (kStage >> 4));
          umma_i8(d_acc, ad, bd, idesc_i8, accumulate);
          accumulate = 1;
#pragma unroll
          for (int k = 1; k < kBKBytes / 32; ++k) {  // 32 int8 of K per instruction = 32 bytes = 2 descriptor units
            umma_i8_acc(d_acc, ad + 2u * k, bd + 2u * k, idesc_i8);
          }
          umma_commit(empty_bar(s));
          pos.advance(stages);
        }
        if (!ok) break;
        umma_commit(acc_full_bar(as));
      }
    }
  } else {
    // ---------------------------------------------------------------------------------- epilogue (warps 2 ..)
    // A warp may only read the TMEM lanes of its quarter (warp index mod 4).
    const int quarter = warp & 3;
    constexpr int c_begin = 0, c_end = BN / 32;
    const int row = quarter * 32 + lane;
    const bool raw = g.c_dtype == kDtypeI32;
    const size_t esize = (g.c_dtype == kDtypeF32 || raw) ? 4 : 2;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(g.c) % 16 == 0) && ((g.c_stride * esize) % 16 == 0);
    uint32_t at = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++at) {
      const TileCoord tc = tile_coord(tile, m_tiles, n_tiles, g.band);
      const int m0 = tc.m_blk * kBM, n0 = tc.n_blk * BN;
      const int as = at % ACC_STAGES;
      const uint32_t aph = (at / ACC_STAGES) & 1u;
      // per-column scale and bias of this tile -> this warp's own slice of shared memory (no cross-warp barrier)
      float *sw_s = col_stage + (warp - 2) * 2 * BN, *bias_s = sw_s + BN;
      stage_columns(g, n0, BN, lane, sw_s, bias_s);
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
      uint4 *xpose = nullptr;
      uint8_t *push_rows = nullptr;  // PUSH: row 0 of this tile in the owner's staging slot
      if constexpr (PUSH) {
        const int owner = m0 / g.peer_rows;
        xpose = raw ? xpose_raw + (warp - 2) * 512 : xpose_bf16 + (warp - 2) * 256;
        push_rows = static_cast<uint8_t *>(g.peer_c[owner]) +
                    static_cast<size_t>(m0 - owner * g.peer_rows) * g.c_stride * (raw ? 4 : 2);
      }
      auto finish = [&](const uint32_t (&acc)[32], const uint32_t (&low)[32], int c) {
        if constexpr (PUSH) push_stage(g, acc, (c - c_begin) & 1, lane, sa_m, sw_s + c * 32, bias_s + c * 32, xpose);
        else finish_chunk(g, acc, low, LORA && has_low, m, n0 + c * 32, sa_m, sw_s + c * 32, bias_s + c * 32, vec_ok);
      };
      ok = mbar_wait(acc_full_bar(as), aph, cta_abort, g.status, kStatusEpilogueTimeout);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + as * BN;
      const uint32_t t_low = t_acc + kLowBase;
      auto fetch = [&](int c, uint32_t (&acc)[32], uint32_t (&low)[32]) {
        tmem_ld_32x32b_x32(t_acc + c * 32, acc);
        if (LORA && has_low) tmem_ld_32x32b_x32(t_low + c * 32, low);
      };
      // two register sets: the TMEM loads of the next 32 columns are in flight while this chunk is finished
      uint32_t acc_a[32], low_a[32], acc_b[32], low_b[32];
      if (c_begin < c_end) fetch(c_begin, acc_a, low_a);
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 2) {
        tmem_ld_wait();
        if (c + 1 < c_end) fetch(c + 1, acc_b, low_b);
        finish(acc_a, low_a, c);
        if (c + 1 < c_end) {
          tmem_ld_wait();
          if (c + 2 < c_end) fetch(c + 2, acc_a, low_a);
          finish(acc_b, low_b, c + 1);
        }
        if constexpr (PUSH) {  // the pair's columns, as far as they lie inside N (a multiple of 32)
          const int n = n0 + c * 32;
          const int have = c + 1 < c_end ? 64 : 32;
          if (n < g.N) push_flush(g, quarter, lane, n, min(have, g.N - n), xpose, push_rows);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(as));
    }
  }

  // ------------------------------------------------------------------------------------ wind-down
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int BN, int ACC_STAGES, bool LORA, int EPI, bool PUSH = false>
cudaError_t launch_one(const GemmLaunch &g, int stages, cudaStream_t stream) {
  const size_t smem = gemm_smem_bytes(BN, LORA ? g.R : 0, stages) + (PUSH ? push_bytes(BN) : 0);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(g.grid);
  cfg.blockDim = dim3(64 + 32 * EPI);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g.overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, gemm_w8a8_kernel<BN, ACC_STAGES, LORA, EPI, PUSH>, g, stages);
}

template <int BN, int ACC_STAGES, bool LORA, int EPI, bool PUSH = false>
cudaError_t configure_one() {
  return cudaFuncSetAttribute(gemm_w8a8_kernel<BN, ACC_STAGES, LORA, EPI, PUSH>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
}

}  // namespace

size_t gemm_smem_bytes(int bn, int R, int stages) {
  if (bn != 32 && bn != 64 && bn != 128 && bn != 256) return 0;
  if (R % kLoraChunk) return 0;
  return 1024 + static_cast<size_t>(stages) * stage_bytes(bn) + kBarrierBytes +
         static_cast<size_t>(kColStageWarps) * 2 * bn * sizeof(float);  // column scales and biases, per epilogue warp
}

int gemm_pick_stages(int bn, int R, size_t smem_optin, bool push) {
  for (int s = kMaxStages; s >= 2; --s) {
    const size_t need = gemm_smem_bytes(bn, R, s) + (push ? push_bytes(bn) : 0);
    if (need != 0 && need <= smem_optin) return s;
  }
  return 0;
}

cudaError_t gemm_configure(int /*device*/) {
  cudaError_t e;
#define H3B_CFG(BN, AS, L, E) \
  if ((e = configure_one<BN, AS, L, E>()) != cudaSuccess) return e;
  H3B_CFG(32, 2, false, 4) H3B_CFG(64, 2, false, 4) H3B_CFG(128, 2, false, 4) H3B_CFG(256, 2, false, 4)
  H3B_CFG(32, 2, true, 4) H3B_CFG(64, 2, true, 4) H3B_CFG(128, 2, true, 4) H3B_CFG(256, 1, true, 4)
#undef H3B_CFG
#define H3B_CFG_PUSH(BN) \
  if ((e = configure_one<BN, 2, false, 4, true>()) != cudaSuccess) return e;
  H3B_CFG_PUSH(32) H3B_CFG_PUSH(64) H3B_CFG_PUSH(128) H3B_CFG_PUSH(256)
#undef H3B_CFG_PUSH
  return cudaSuccess;
}

cudaError_t launch_gemm_w8a8(const GemmLaunch &g, int stages, cudaStream_t stream) {
  const bool lora = g.R > 0;
  if (g.peer_rows > 0) {
    if (lora) return cudaErrorInvalidValue;
    switch (g.bn) {
      case 32: return launch_one<32, 2, false, 4, true>(g, stages, stream);
      case 64: return launch_one<64, 2, false, 4, true>(g, stages, stream);
      case 128: return launch_one<128, 2, false, 4, true>(g, stages, stream);
      case 256: return launch_one<256, 2, false, 4, true>(g, stages, stream);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (g.bn) {
    case 32: return lora ? launch_one<32, 2, true, 4>(g, stages, stream) : launch_one<32, 2, false, 4>(g, stages, stream);
    case 64: return lora ? launch_one<64, 2, true, 4>(g, stages, stream) : launch_one<64, 2, false, 4>(g, stages, stream);
    case 128: return lora ? launch_one<128, 2, true, 4>(g, stages, stream) : launch_one<128, 2, false, 4>(g, stages, stream);
    case 256:
      // A low-rank term on 256-column tiles leaves room for ONE accumulator pair in tensor memory, so its epilogue
      // does not overlap the next tile's main loop. Measured alternatives: a second epilogue warp per lane quarter
      // changes nothing (the exposed time is the hand-over and the stores, not instruction issue); 128-column tiles
      // with two accumulator pairs are 25 % slower, and 160-column tiles with two main accumulators and one shared
      // low-rank accumulator (480 columns) 15-20 % slower: the narrower the MMA, the more operand bytes it reads from
      // shared memory per multiply (96 bytes per clock at 256 columns, 115 at 160, 128 - the limit - at 128).
      return lora ? launch_one<256, 1, true, 4>(g, stages, stream) : launch_one<256, 2, false, 4>(g, stages, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace h3b
