// CTA-pair variant of the contraction kernel: two CTAs of one cluster (two SMs) compute one 256 x 256
// output tile with tcgen05.mma.cta_group::2.
//
// Each CTA loads ITS 128 rows of A and ITS 128 columns of B (every CTA fetches its own boxes; nothing is
// multicast): a third less shared-memory fill traffic per SM and per unit of work than a single-CTA 128 x 256
// tile.  A ring stage holds two 64-element K boxes of each operand (64 KB per CTA, three stages): the fixed cost
// of a stage hand-over is paid once per 128 K.  The leader CTA (cluster rank 0) issues the MMAs; the
// tensor cores of both SMs read A from their own shared memory and the two halves of B from both, and
// each accumulates its 128 rows x 256 columns in its own tensor memory.
//
// Signalling (all waits are on barriers of the waiting CTA, all are bounded):
//   full[s]       lives in the leader; armed by the leader's producer with the bytes of BOTH CTAs; the
//                 peer's TMA loads count their bytes on it (cp.async.bulk.tensor ... cta_group::2).
//   empty[s]      one per CTA; tcgen05.commit from the leader arrives on both (an arrival, no data).
//   tmem_full[a]  one per CTA; same commit-to-both.
//   tmem_empty[a] lives in the leader; every epilogue warp of both CTAs arrives on it.
//
// Used when both operands can be loaded with TMA, K >= 256 and the tile cost model of the launcher prices pairs
// below single-CTA tiles; everything else runs the single-CTA kernel of gemm_kernel.cuh.
#pragma once
#include "gemm_kernel.cuh"

namespace nova {

static constexpr int kPairBlockM = 256;  // rows per pair tile (128 per CTA)
static constexpr int kPairBlockN = 256;  // columns per pair tile (each CTA loads 128 of them)
static constexpr int kPairSubK = 2;     // 64-element K sub-blocks per ring stage: one barrier round trip per 128 K
static constexpr int kPairStages = 3;
static constexpr int kPairEpilogueWarps = 4;  // 8 (one staging box each) measured the same on every shape

// kEpiWarps epilogue warps per CTA (4 or 8).  The staging area is the same 32 KB either way: two boxes per
// warp for four warps, one box per warp for eight.
template <int kEpiWarps>
struct PairSmemLayout {
  static constexpr int kBoxesPerWarp = 8 / kEpiWarps;
  static constexpr int kATile = kBlockM * kSwizzleBytes;             // 16 KB: this CTA's 128 rows
  static constexpr int kBTile = (kPairBlockN / 2) * kSwizzleBytes;   // 16 KB: this CTA's 128 columns
  static constexpr int kStageBytes = kPairSubK * (kATile + kBTile);
  static constexpr int kRingBytes = kPairStages * kStageBytes;
  static constexpr int kNumBarriers = 2 * kPairStages + 4;
  static constexpr int kStageOutBox = 32 * kSwizzleBytes;
  static constexpr int kStagingOffset = kRingBytes;
  static constexpr int kStagingBytes = kEpiWarps * kBoxesPerWarp * kStageOutBox;
  static constexpr int kBarrierOffset = kStagingOffset + kStagingBytes;
  static constexpr int kMiscOffset = kBarrierOffset + 8 * kNumBarriers;
  static constexpr int kTotalBytes = kMiscOffset + 16;
  static constexpr int kDynamicBytes = kTotalBytes + 1024;
};

// kElemBytes: 2 (f16/bf16) or 4 (f32 as single-pass tf32).  kAMn / kBMn as in the single-CTA kernel.
// p.m_blocks counts 256-row blocks, p.n_blocks 256-column blocks.
template <int kElemBytes, bool kAMn, bool kBMn, int kEpiWarps>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(32 * (kFirstEpilogueWarp + kEpiWarps), 1)
nova_gemm_sm100_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                            const __grid_constant__ CUtensorMap tmap_c, const GemmKernelParams p) {
  using L = PairSmemLayout<kEpiWarps>;
  static_assert(kEpiWarps == 4 || kEpiWarps == 8, "one or two epilogue warps per tensor-memory lane quarter");
  constexpr int kStages = kPairStages;
  constexpr int kElemsPerRow = kSwizzleBytes / kElemBytes;
  constexpr int kSubBlockK = kElemsPerRow;           // K elements per 128-byte row
  constexpr int kBlockK = kPairSubK * kSubBlockK;    // K elements per ring stage
  constexpr int kUmmaK = 32 / kElemBytes;
  constexpr int kKSteps = kSubBlockK / kUmmaK;
  constexpr int kHalfN = kPairBlockN / 2;
  constexpr uint32_t kTmemCols = 2 * kPairBlockN;  // two 128-lane x 256-column accumulators per CTA
  static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory budget");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::kBarrierOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kPairStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kPairStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kPairStages + 2 + a); };
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOffset);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOffset + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  if (threadIdx.x == 0) trace_mark(p.trace, 0, kTraceKernel);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);   // used in the leader only: its producer's arrive + both CTAs' bytes
      mbar_init(empty_bar(s), 1);  // one commit arrival per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 2 * kEpiWarps);  // used in the leader only
    }
    *abort_flag = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  // both CTAs' barriers exist before either CTA signals the other
  cluster_sync_all();
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  if (threadIdx.x == 0) trace_mark(p.trace, 1, kTraceKernel);
  // everything above touched only the pair's shared and tensor memory: it may overlap the previous kernel's tail
  griddep_launch_dependents();
  griddep_wait();

  if (warp == 0) {
    // ============================================================ TMA producer (one per CTA)
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      // Optional L2 prefetch cursor, p.prefetch_dist ring stages ahead of the loads (it runs on into the pair's
      // next tile): pays when operands come cold from HBM and few tiles share a panel; costs L2 request slots
      // when the panels are already L2-resident, so the launcher decides.
      int32_t pf_tile = pair;
      int pf_kb = 0;
      auto pf_advance = [&]() {
        if (++pf_kb == p.k_blocks) { pf_kb = 0; pf_tile += num_pairs; }
      };
      auto pf_issue = [&]() {
        if (pf_tile >= p.tiles) return;
        const TileCoord t = decode_tile(p, pf_tile);
        const int m0 = t.m_blk * kPairBlockM + static_cast<int>(rank) * kBlockM;
        const int n0 = t.n_blk * kPairBlockN + static_cast<int>(rank) * kHalfN;
        const int za = t.batch * p.a_batch_mul, zb = t.batch * p.b_batch_mul;
#pragma unroll
        for (int sub = 0; sub < kPairSubK; ++sub) {
          const int k0 = pf_kb * kBlockK + sub * kSubBlockK;
          if (k0 >= p.K) break;
          if (!kAMn) {
            tma_prefetch_3d(&tmap_a, k0, m0, za);
          } else {
#pragma unroll
            for (int c = 0; c < kBlockM / kElemsPerRow; ++c) tma_prefetch_3d(&tmap_a, m0 + c * kElemsPerRow, k0, za);
          }
          if (!kBMn) {
            tma_prefetch_3d(&tmap_b, k0, n0, zb);
          } else {
#pragma unroll
            for (int c = 0; c < kHalfN / kElemsPerRow; ++c) tma_prefetch_3d(&tmap_b, n0 + c * kElemsPerRow, k0, zb);
          }
        }
      };
      const bool prefetch = p.prefetch_dist > 0;
      if (prefetch)
        for (int i = 0; i < p.prefetch_dist; ++i) pf_advance();
      for (int32_t tile = pair; ok && tile < p.tiles; tile += num_pairs, ++tile_iter) {
        const TileCoord t = decode_tile(p, tile);
        const int m0 = t.m_blk * kPairBlockM + static_cast<int>(rank) * kBlockM;
        const int n0 = t.n_blk * kPairBlockN + static_cast<int>(rank) * kHalfN;
        const int za = t.batch * p.a_batch_mul, zb = t.batch * p.b_batch_mul;
        long long waited = 0;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          if (prefetch) { pf_issue(); pf_advance(); }
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          const long long w0 = (kTraceEnabled && p.trace) ? clock64() : 0;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, kStatusProducerEmptyWait)) { ok = false; break; }
          if (kTraceEnabled && p.trace) waited += clock64() - w0;
          if (kb == 0) trace_mark(p.trace, tile_iter, kTraceProducerFirst);
          const uint32_t stage = smem_base + s * L::kStageBytes;
          if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2u * L::kStageBytes);
          const uint32_t bar = map_to_cta(full_bar(s), 0u);  // the leader's barrier counts both CTAs' bytes
#pragma unroll
          for (int sub = 0; sub < kPairSubK; ++sub) {
            const int k0 = kb * kBlockK + sub * kSubBlockK;  // past K: the box is all zeros
            const uint32_t adst = stage + sub * (L::kATile + L::kBTile);
            if (!kAMn) {
              tma_load_3d_pair(adst, &tmap_a, bar, k0, m0, za);
            } else {
#pragma unroll
              for (int c = 0; c < kBlockM / kElemsPerRow; ++c)
                tma_load_3d_pair(adst + c * (kSubBlockK * kSwizzleBytes), &tmap_a, bar, m0 + c * kElemsPerRow, k0, za);
            }
            const uint32_t bdst = adst + L::kATile;
            if (!kBMn) {
              tma_load_3d_pair(bdst, &tmap_b, bar, k0, n0, zb);
            } else {
#pragma unroll
              for (int c = 0; c < kHalfN / kElemsPerRow; ++c)
                tma_load_3d_pair(bdst + c * (kSubBlockK * kSwizzleBytes), &tmap_b, bar, n0 + c * kElemsPerRow, k0, zb);
            }
          }
        }
        trace_mark(p.trace, tile_iter, kTraceProducerLast);
        trace_value(p.trace, tile_iter, kTraceProducerWait, waited);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ============================================================ MMA issuer (leader CTA only)
    if (rank == 0 && lane == 0) {
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int32_t tile = pair; ok && tile < p.tiles; tile += num_pairs, ++tile_iter) {
        const uint32_t acc = tile_iter & 1u;
        const uint32_t acc_ph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(tmem_empty_bar(acc), acc_ph ^ 1u, abort_flag, p.status, kStatusMmaTmemEmptyWait)) break;
        tc_fence_after_sync();
        trace_mark(p.trace, tile_iter, kTraceMmaStart);
        const uint32_t d_tmem = tmem_base + acc * kPairBlockN;
        long long waited = 0;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          const long long w0 = (kTraceEnabled && p.trace) ? clock64() : 0;
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, kStatusMmaFullWait)) { ok = false; break; }
          if (kTraceEnabled && p.trace) {
            const long long w = clock64() - w0;
            waited += w;
            if (kb < 8) trace_value(p.trace, tile_iter, kTraceEpiWarpStart + kb, w);
          }
          if (kb == 0) trace_mark(p.trace, tile_iter, kTraceMmaFirstFull);
          tc_fence_after_sync();
#pragma unroll
          for (int sub = 0; sub < kPairSubK; ++sub) {
            const uint32_t a_stage = smem_base + s * L::kStageBytes + sub * (L::kATile + L::kBTile);
            const uint32_t b_stage = a_stage + L::kATile;
#pragma unroll
            for (int k = 0; k < kKSteps; ++k) {
              const uint32_t accumulate = (kb | sub | k) == 0 ? 0u : 1u;
              const uint64_t a_desc = make_smem_desc(a_stage + k * p.a_kstep, p.a_desc_lbo, p.a_desc_hi);
              const uint64_t b_desc = make_smem_desc(b_stage + k * p.b_kstep, p.b_desc_lbo, p.b_desc_hi);
              if (kElemBytes == 2) umma_f16_pair(d_tmem, a_desc, b_desc, p.idesc, accumulate);
              else umma_tf32_pair(d_tmem, a_desc, b_desc, p.idesc, accumulate);
            }
          }
          umma_commit_pair(empty_bar(s), 3);  // both CTAs may refill their halves of this stage
        }
        if (ok) umma_commit_pair(tmem_full_bar(acc), 3);  // both CTAs' epilogues may drain
        trace_mark(p.trace, tile_iter, kTraceMmaCommit);
        trace_value(p.trace, tile_iter, kTraceMmaFullWait, waited);
      }
    }
    __syncwarp();
  } else {
    // ============================================================ epilogue (both CTAs)
    const int q = warp & 3;
    constexpr int kColsPerWarp = kPairBlockN / (kEpiWarps / 4);
    const int cg = (warp - kFirstEpilogueWarp) >> 2;  // which column group of the CTA's 256 columns this warp drains
    uint8_t* staging = smem_gen + L::kStagingOffset + (warp - kFirstEpilogueWarp) * (L::kBoxesPerWarp * L::kStageOutBox);
    if (p.vec_store && lane == 0) tma_prefetch_desc(&tmap_c);
    uint32_t tile_iter = 0;
    uint32_t box_iter = 0;
    for (int32_t tile = pair; tile < p.tiles; tile += num_pairs, ++tile_iter) {
      const TileCoord t = decode_tile(p, tile);
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(tmem_full_bar(acc), acc_ph, abort_flag, p.status, kStatusEpilogueTmemFullWait)) break;
      if (warp == kFirstEpilogueWarp && lane == 0) trace_mark(p.trace, tile_iter, kTraceEpiStart);
      tc_fence_after_sync();
      if (warp == kFirstEpilogueWarp && lane == 0) trace_mark(p.trace, tile_iter, 35);
      const int32_t row0 = t.m_blk * kPairBlockM + static_cast<int>(rank) * kBlockM + q * 32;
      const int32_t n0 = t.n_blk * kPairBlockN + cg * kColsPerWarp;
      const uint32_t taddr = tmem_base + acc * kPairBlockN + cg * kColsPerWarp + (static_cast<uint32_t>(q * 32) << 16);
      long long waits[5] = {0, 0, 0, 0, 0};
      long long* wp = (kTraceEnabled && p.trace != nullptr && warp == kFirstEpilogueWarp) ? waits : nullptr;
      if (p.out_dtype == NOVA_B200_BF16)
        epilogue_tile<__nv_bfloat16, kColsPerWarp, L::kBoxesPerWarp>(p, &tmap_c, taddr, staging, box_iter, lane, t.batch, row0, n0, wp);
      else if (p.out_dtype == NOVA_B200_F16)
        epilogue_tile<__half, kColsPerWarp, L::kBoxesPerWarp>(p, &tmap_c, taddr, staging, box_iter, lane, t.batch, row0, n0, wp);
      else
        epilogue_tile<float, kColsPerWarp, L::kBoxesPerWarp>(p, &tmap_c, taddr, staging, box_iter, lane, t.batch, row0, n0, wp);
      if (warp == kFirstEpilogueWarp && lane == 0) trace_mark(p.trace, tile_iter, 32);
      tc_fence_before_sync();
      if (warp == kFirstEpilogueWarp && lane == 0) trace_mark(p.trace, tile_iter, 33);
      __syncwarp();
      if (warp == kFirstEpilogueWarp && lane == 0) trace_mark(p.trace, tile_iter, 34);
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tmem_empty_bar(acc), 0u));
      if (lane == 0) trace_mark(p.trace, tile_iter, kTraceEpiWarpEnd + warp - kFirstEpilogueWarp);
      if (warp == kFirstEpilogueWarp && lane == 0) {
        trace_mark(p.trace, tile_iter, kTraceEpiEnd);
        trace_value(p.trace, tile_iter, kTraceEpiStoreWait, waits[0]);
        trace_value(p.trace, tile_iter, kTraceEpiTmemWait, waits[1]);
        trace_value(p.trace, tile_iter, kTraceEpiMath, waits[2]);
        trace_value(p.trace, tile_iter, kTraceEpiFence, waits[3]);
        trace_value(p.trace, tile_iter, kTraceEpiIssue, waits[4]);
      }
    }
    if (p.vec_store && lane == 0) tma_store_wait_read<0>();  // staged boxes read out before shared memory goes away
    __syncwarp();
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) trace_mark(p.trace, 2, kTraceKernel);
  if (*abort_flag != 0u && threadIdx.x == 0) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);  // let in-flight bulk copies land
  }
  // neither CTA may leave (or free tensor memory) while the other can still signal it or read its shared memory
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace nova
