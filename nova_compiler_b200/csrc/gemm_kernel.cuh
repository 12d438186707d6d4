// The contraction kernel of libnova_b200: a persistent, warp-specialised sm_100a GEMM.
//
//   warp 0      TMA producer: one lane streams 128-byte-swizzled operand boxes into a
//               kStages-deep shared-memory ring (mbarrier full/empty pairs).
//   warp 1      owns tensor memory (alloc/dealloc) and issues tcgen05.mma from one lane;
//               tcgen05.commit releases ring stages and publishes finished accumulators.
//   warps 2..5  epilogue: tcgen05.ld the fp32 accumulator (TMEM lane == output row),
//               add bias / residual, apply ReLU / GELU, cast, stage 32x128-byte boxes in shared
//               memory and write them with TMA stores (element stores when C is not 16-byte
//               aligned).  Two accumulator
//               buffers in TMEM let the epilogue of tile i overlap the mainloop of tile i+1.
//   warps 6..13 (only launched when an operand cannot use TMA) predicated ld.global
//               loader for operands whose base or pitch is not a multiple of 16 bytes.
//
// One CTA per SM; tiles are handed out round-robin in a grouped raster order so that
// the CTAs of one wave share A row-panels and B column-panels in L2.
//
// Ragged extents need no padded copies: TMA zero-fills out-of-bounds box elements
// (zeros add nothing along K) and the epilogue predicates its stores on row < M, col < N.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"
#include "runtime.h"

namespace nova {

static constexpr int kBlockM = 128;          // UMMA M (cta_group::1): TMEM lane i holds output row i
static constexpr int kSwizzleBytes = 128;    // operand rows in shared memory are 128 bytes
static constexpr int kNumEpilogueWarps = 4;
static constexpr int kNumLoaderWarps = 8;
static constexpr int kLoaderGroups = 4;  // loader warps split into groups that fill different ring stages concurrently
static constexpr int kLoaderWarpsPerGroup = kNumLoaderWarps / kLoaderGroups;
static constexpr int kFirstEpilogueWarp = 2;
static constexpr int kFirstLoaderWarp = kFirstEpilogueWarp + kNumEpilogueWarps;
static constexpr int kThreadsTma = 32 * kFirstLoaderWarp;                      // 192
static constexpr int kThreadsWithLoader = 32 * (kFirstLoaderWarp + kNumLoaderWarps);  // 448
static constexpr int kMaxPushPeers = 7;      // the other GPUs of an 8-GPU box

struct GemmKernelParams {
  int32_t M, N, K, batch;
  int32_t m_blocks, n_blocks, k_blocks;
  int32_t group_m;    // raster: tiles walk group_m row-blocks of one column-block before the next column
  int32_t tiles;      // batch * m_blocks * n_blocks
  int32_t a_batch_mul, b_batch_mul;  // 0 when the operand is shared by every batch, else 1
  uint32_t idesc;     // tcgen05 instruction descriptor
  uint32_t a_desc_hi, b_desc_hi;      // shared-memory matrix descriptor, bits 32..63
  uint32_t a_desc_lbo, b_desc_lbo;    // leading-byte-offset field, already shifted into bits 16..29
  uint32_t a_kstep, b_kstep;          // bytes the descriptor start address advances per UMMA K step
  int32_t loader_a, loader_b;         // 0 = TMA, 1 = ld.global loader warps
  // optional timeline (null unless the host asked for one): kTraceSlots clock64 samples per tile for the
  // first kTraceTiles tiles of every CTA
  long long* trace;
  // raw operand views for the ld.global loader
  const void* A; const void* B;
  int64_t lda, ldb, stride_a, stride_b;
  // epilogue
  void* C;
  const void* bias;
  const void* residual;
  int64_t ldc, stride_c, ldr, stride_r;
  int32_t act, init, out_dtype, vec_store;
  int32_t prefetch_dist;  // pair kernel: ring stages the L2 prefetch cursor runs ahead of the loads (0 = none)
  // Split K: launch batch b * split_k_ranges + s is the K range [s * split_k_len, (s + 1) * split_k_len) of operand
  // batch b; a range that runs past K reads zeros from the tensor maps.  split_k_ranges <= 1 = not split.
  int32_t split_k_len, split_k_ranges;
  uint32_t* status;
  // multi-GPU push: every finished output box is also stored into these peers' matrices (same pitch and batch
  // stride as C), with plain 16-byte stores over NVLink
  int32_t n_peers;
  void* peer_c[kMaxPushPeers];
};

// kOpTerms: operand copies per stage (2 = hi and lo halves of the 3xTF32 split, else 1)
template <int kBlockN, int kOpTerms, int kStages, int kEpiWarps = kNumEpilogueWarps>
struct GemmSmemLayout {
  static constexpr int kATile = kBlockM * kSwizzleBytes;  // one operand term of A per stage
  static constexpr int kBTile = kBlockN * kSwizzleBytes;
  static constexpr int kStageBytes = kOpTerms * (kATile + kBTile);
  static constexpr int kRingBytes = kStages * kStageBytes;
  // barriers: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]; then tmem base + abort flag
  static constexpr int kNumBarriers = 2 * kStages + 4;
  // epilogue staging for TMA stores: per epilogue warp two 32-row x 128-byte boxes (double buffered)
  static constexpr int kStageOutBox = 32 * kSwizzleBytes;
  static constexpr int kStagingOffset = kRingBytes;
  static constexpr int kStagingBytes = kEpiWarps * 2 * kStageOutBox;
  static constexpr int kBarrierOffset = kStagingOffset + kStagingBytes;
  static constexpr int kMiscOffset = kBarrierOffset + 8 * kNumBarriers;
  static constexpr int kTotalBytes = kMiscOffset + 16;
  static constexpr int kDynamicBytes = kTotalBytes + 1024;  // slack to align the ring to 1024 bytes
};

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_field, uint32_t hi) {
  return (static_cast<uint64_t>(hi) << 32) | static_cast<uint64_t>(lbo_field | ((addr >> 4) & 0x3fffu));
}

// Role timelines are compiled in only by a diagnostic build (-DNOVA_B200_TRACE_BUILD): even a never-taken
// branch around a clock read in the producer and MMA loops costs a few percent of the tensor rate.
#ifdef NOVA_B200_TRACE_BUILD
static constexpr bool kTraceEnabled = true;
#else
static constexpr bool kTraceEnabled = false;
#endif
static constexpr int kTraceTiles = 16;
static constexpr int kTraceSlots = 40;
enum TraceSlot : int {
  kTraceProducerFirst = 0,  // producer: first stage of the tile may be refilled
  kTraceProducerLast = 1,   // producer: last load of the tile issued
  kTraceMmaStart = 2,       // MMA issuer: accumulator free
  kTraceMmaFirstFull = 3,   // MMA issuer: first stage of the tile has landed
  kTraceMmaCommit = 4,      // MMA issuer: accumulator commit issued
  kTraceEpiStart = 5,       // first epilogue warp: accumulator complete
  kTraceEpiEnd = 6,         // first epilogue warp: accumulator released
  kTraceKernel = 7,         // tile 0: kernel entry; tile 1: roles start; tile 2: teardown
  kTraceMmaFullWait = 8,    // MMA issuer: cycles spent waiting for stages to land, this tile
  kTraceProducerWait = 9,   // producer: cycles spent waiting for free stages, this tile
  kTraceEpiStoreWait = 10,  // first epilogue warp: cycles spent waiting for staging boxes to be read out
  kTraceEpiTmemWait = 11,   // first epilogue warp: cycles spent waiting for tensor-memory loads
  kTraceEpiMath = 12,       // first epilogue warp: cycles in arithmetic and staging writes
  kTraceEpiFence = 13,      // first epilogue warp: cycles in the proxy fence and warp barrier
  kTraceEpiIssue = 14,      // first epilogue warp: cycles issuing the bulk store
  kTraceEpiWarpStart = 16,  // + epilogue warp index: that warp saw the accumulator complete
  kTraceEpiWarpEnd = 24,    // + epilogue warp index: that warp released the accumulator
};
__device__ __forceinline__ void trace_value(const long long* base, uint32_t tile_iter, int slot, long long v) {
  if (kTraceEnabled && base != nullptr && tile_iter < static_cast<uint32_t>(kTraceTiles))
    const_cast<long long*>(base)[(static_cast<size_t>(blockIdx.x) * kTraceTiles + tile_iter) * kTraceSlots + slot] = v;
}
__device__ __forceinline__ void trace_mark(const long long* base, uint32_t tile_iter, int slot) {
  if (kTraceEnabled && base != nullptr && tile_iter < static_cast<uint32_t>(kTraceTiles))
    const_cast<long long*>(base)[(static_cast<size_t>(blockIdx.x) * kTraceTiles + tile_iter) * kTraceSlots + slot] = clock64();
}

struct TileCoord {
  int32_t batch, m_blk, n_blk;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmKernelParams& p, int32_t tile) {
  const int32_t per_batch = p.m_blocks * p.n_blocks;
  TileCoord t;
  t.batch = tile / per_batch;
  const int32_t r = tile - t.batch * per_batch;
  const int32_t group_tiles = p.group_m * p.n_blocks;
  const int32_t g = r / group_tiles;
  const int32_t first_m = g * p.group_m;
  const int32_t gm = min(p.group_m, p.m_blocks - first_m);
  const int32_t rr = r - g * group_tiles;
  t.n_blk = rr / gm;
  t.m_blk = first_m + (rr - t.n_blk * gm);
  return t;
}

// ---------------------------------------------------------------- epilogue math

__device__ __forceinline__ float gelu_tanh_f32(float x) {
  // 0.5*x*(1+tanh(u)) == x / (1 + exp(-2u)),  u = 0.79788456*(x + 0.044715*x^3)
  const float u = 0.7978845608028654f * fmaf(0.044715f * x, x * x, x);
  return __fdividef(x, 1.0f + __expf(-2.0f * u));
}

// d/dx of the tanh-form GELU: with s = sigmoid(2u), tanh(u) = 2s - 1, so 0.5(1 + tanh u) = s and
// 1 - tanh^2 u = 4s(1 - s); u' = 0.79788456 * (1 + 0.134145 x^2)  (3 * 0.044715 = 0.134145).
__device__ __forceinline__ float gelu_tanh_grad_f32(float x) {
  const float x2 = x * x;
  const float u = 0.7978845608028654f * fmaf(0.044715f * x, x2, x);
  const float s = __fdividef(1.0f, 1.0f + __expf(-2.0f * u));
  const float du = 0.7978845608028654f * fmaf(0.134145f, x2, 1.0f);
  return fmaf(2.0f * x * du, s * (1.0f - s), s);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// 32 consecutive elements of one row of an epilogue operand (residual, live C, GELU pre-activation) as floats:
// 16-byte loads when the span is whole and aligned, guarded element loads at ragged edges.
template <typename OutT>
__device__ __forceinline__ void load_row32(const OutT* ptr, int32_t ncols, float (&out)[32]) {
  constexpr int kPerVec = 16 / static_cast<int>(sizeof(OutT));
  if (ncols == 32 && (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0u) {
#pragma unroll
    for (int j = 0; j < 32; j += kPerVec) {
      union { uint4 u; OutT e[kPerVec]; } pk;
      pk.u = *reinterpret_cast<const uint4*>(ptr + j);
#pragma unroll
      for (int e = 0; e < kPerVec; ++e) out[j + e] = to_f32<OutT>(pk.e[e]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) out[j] = j < ncols ? to_f32<OutT>(ptr[j]) : 0.0f;
  }
}

// One thread finishes 32 consecutive columns of one output row: accumulator + init, activation.
// `row_ok` guards the residual read of rows past M (their accumulators are zeros from the fill).
template <typename OutT>
__device__ __forceinline__ void epilogue_math(const GemmKernelParams& p, const uint32_t (&acc)[32], float (&v)[32],
                                              int32_t batch, int32_t row, int32_t col0, bool row_ok) {
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(acc[j]);
  const int32_t ncols = min(32, p.N - col0);
  if (p.init == NOVA_B200_INIT_LN_FOLD) {
    // layer norm folded into the contraction: v = rstd_i * (acc - mean_i * c_j) + d_j, all in fp32
    const float* c = reinterpret_cast<const float*>(p.bias) + col0;
    const float* d = c + p.N;
    const float2 st = row_ok ? __ldg(reinterpret_cast<const float2*>(p.residual) + row) : make_float2(0.0f, 0.0f);
    if (ncols == 32 && ((reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(d)) & 15u) == 0u) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 cq = __ldg(reinterpret_cast<const float4*>(c + j)), dq = __ldg(reinterpret_cast<const float4*>(d + j));
        v[j] = fmaf(st.y, fmaf(-st.x, cq.x, v[j]), dq.x);
        v[j + 1] = fmaf(st.y, fmaf(-st.x, cq.y, v[j + 1]), dq.y);
        v[j + 2] = fmaf(st.y, fmaf(-st.x, cq.z, v[j + 2]), dq.z);
        v[j + 3] = fmaf(st.y, fmaf(-st.x, cq.w, v[j + 3]), dq.w);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) v[j] = fmaf(st.y, fmaf(-st.x, __ldg(c + j), v[j]), __ldg(d + j));
    }
  }
  if (p.init == NOVA_B200_INIT_BIAS_ROW || p.init == NOVA_B200_INIT_BIAS_AND_RESIDUAL) {
    const OutT* b = reinterpret_cast<const OutT*>(p.bias) + col0;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) v[j] += to_f32<OutT>(__ldg(b + j));
  }
  if ((p.init == NOVA_B200_INIT_RESIDUAL_FULL || p.init == NOVA_B200_INIT_FROM_C ||
       p.init == NOVA_B200_INIT_BIAS_AND_RESIDUAL) && row_ok) {
    const OutT* r = p.init == NOVA_B200_INIT_FROM_C
                        ? reinterpret_cast<const OutT*>(p.C) + static_cast<int64_t>(batch) * p.stride_c +
                              static_cast<int64_t>(row) * p.ldc + col0
                        : reinterpret_cast<const OutT*>(p.residual) + static_cast<int64_t>(batch) * p.stride_r +
                              static_cast<int64_t>(row) * p.ldr + col0;
    float add[32];
    load_row32<OutT>(r, ncols, add);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += add[j];
  }
  if (p.act == NOVA_B200_ACT_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
  } else if (p.act == NOVA_B200_ACT_GELU_TANH) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_f32(v[j]);
  } else if (p.act == NOVA_B200_ACT_GELU_TANH_GRAD && row_ok) {
    // the forward pre-activation arrives through the residual pointer and is a multiplier, not an addend
    const OutT* z = reinterpret_cast<const OutT*>(p.residual) + static_cast<int64_t>(batch) * p.stride_r +
                    static_cast<int64_t>(row) * p.ldr + col0;
    float zf[32];
    load_row32<OutT>(z, ncols, zf);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= gelu_tanh_grad_f32(zf[j]);
  }
}

// Writes a staged box (32 rows x 128 B, swizzled) row by row with element stores, lane == column pair:
// the path for outputs whose base or pitch is not 16-byte aligned.  Each store instruction covers a
// contiguous span of one output row.
template <typename OutT>
__device__ __forceinline__ void epilogue_store_rows(const GemmKernelParams& p, const uint8_t* box, int lane,
                                                    int32_t batch, int32_t row0, int32_t col0) {
  constexpr int kPerLane = 4 / static_cast<int>(sizeof(OutT));  // elements in one 32-bit word
  OutT* cbase = reinterpret_cast<OutT*>(p.C) + static_cast<int64_t>(batch) * p.stride_c + col0 + lane * kPerLane;
  const int32_t col = col0 + lane * kPerLane;
#pragma unroll 4
  for (int r = 0; r < 32; ++r) {
    const int32_t row = row0 + r;
    if (row >= p.M) break;  // uniform across the warp
    union { uint32_t u; OutT e[kPerLane]; } w;
    w.u = *reinterpret_cast<const uint32_t*>(box + r * kSwizzleBytes + (((lane >> 2) ^ (r & 7)) << 4) + (lane & 3) * 4);
    OutT* dst = cbase + static_cast<int64_t>(row) * p.ldc;
#pragma unroll
    for (int e = 0; e < kPerLane; ++e)
      if (col + e < p.N) dst[e] = w.e[e];
  }
}

// 32 columns of one row into the warp's staging box (32 rows x 128 B, 16-byte chunks XOR-swizzled by
// row & 7, the layout a SWIZZLE_128B tensor map expects).  `first_chunk` is the index of the first
// 16-byte chunk these 32 columns occupy within the 128-byte row.
template <typename OutT>
__device__ __forceinline__ void epilogue_stage(uint8_t* box, const float (&v)[32], int lane, int first_chunk) {
  constexpr int kPerVec = 16 / static_cast<int>(sizeof(OutT));
#pragma unroll
  for (int j = 0; j < 32; j += kPerVec) {
    union { uint4 u; OutT e[kPerVec]; } pk;
#pragma unroll
    for (int e = 0; e < kPerVec; ++e) pk.e[e] = from_f32<OutT>(v[j + e]);
    const int chunk = first_chunk + j / kPerVec;
    *reinterpret_cast<uint4*>(box + lane * kSwizzleBytes + ((chunk ^ (lane & 7)) << 4)) = pk.u;
  }
}

// The staged box (32 rows x 128 B, swizzled) once more, into every peer GPU's copy of the output: lane l stores the
// 16-byte chunks l, l + 32, ... (chunk = row * 8 + position in the row), so a warp instruction covers four whole
// 128-byte row segments; plain st.global to peer-mapped addresses (no TMA, no multicast).  The host guarantees
// 16-byte-aligned pitches and N a multiple of the chunk width, so a chunk is either whole or absent.
template <typename OutT>
__device__ __forceinline__ void epilogue_push_box(const GemmKernelParams& p, const uint8_t* box, int lane, int32_t batch,
                                                  int32_t row0, int32_t col0) {
  constexpr int kPerChunk = 16 / static_cast<int>(sizeof(OutT));
  uint4 v[8];
  int64_t off[8];  // element offset of each chunk in the output, -1 when it lies outside
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = lane + 32 * i, r = idx >> 3, c = idx & 7;
    const int32_t row = row0 + r, col = col0 + c * kPerChunk;
    v[i] = *reinterpret_cast<const uint4*>(box + r * kSwizzleBytes + ((c ^ (r & 7)) << 4));
    off[i] = (row < p.M && col < p.N) ? static_cast<int64_t>(batch) * p.stride_c + static_cast<int64_t>(row) * p.ldc + col : -1;
  }
  for (int peer = 0; peer < p.n_peers; ++peer) {
    OutT* base = reinterpret_cast<OutT*>(p.peer_c[peer]);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (off[i] >= 0) *reinterpret_cast<uint4*>(base + off[i]) = v[i];
  }
}

// One epilogue warp drains kCols columns of its 32 accumulator rows, one 128-byte-wide box at a time.
// kBoxes staging boxes per warp: with two, the TMA store of one box overlaps the whole of the next; with
// one, it overlaps only the next box's first tensor-memory load and its arithmetic.
template <typename OutT, int kCols, int kBoxes = 2, int kSecondAcc = 0>
__device__ __forceinline__ void epilogue_tile(const GemmKernelParams& p, const CUtensorMap* tmap_c, uint32_t taddr,
                                              uint8_t* staging, uint32_t& box_iter, int lane, int32_t batch,
                                              int32_t row0, int32_t n0, long long* waits = nullptr) {
  constexpr int kColsPerBox = kSwizzleBytes / static_cast<int>(sizeof(OutT));  // 64 (16-bit) or 32 (f32)
  constexpr int kLoadsPerBox = kColsPerBox / 32;
  constexpr int kChunkStep = 32 * static_cast<int>(sizeof(OutT)) / 16;  // 16-byte chunks per 32 columns
  const int32_t row = row0 + lane;
  const bool row_ok = row < p.M;
#pragma unroll 1
  for (int c = 0; c < kCols / kColsPerBox; ++c) {
    const int32_t col0 = n0 + c * kColsPerBox;
    if (col0 >= p.N) break;  // uniform across the warp
    uint8_t* box = staging + (kBoxes == 2 ? (box_iter & 1u) : 0u) * (32 * kSwizzleBytes);
#pragma unroll
    for (int h = 0; h < kLoadsPerBox; ++h) {
      uint32_t r[32];
      long long t0 = 0;
      if (waits) t0 = clock64();
      tmem_ld_32x32(taddr + c * kColsPerBox + h * 32, r);
      if (kSecondAcc > 0) {
        // kSecondAcc columns further: the accumulator of the small 3xTF32 terms, added here with rounding
        uint32_t r2[32];
        tmem_ld_32x32(taddr + kSecondAcc + c * kColsPerBox + h * 32, r2);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
      }
      tmem_ld_wait();
      if (waits) waits[1] += clock64() - t0;
      float v[32];
      if (waits) t0 = clock64();
      epilogue_math<OutT>(p, r, v, batch, row, col0 + h * 32, row_ok);
      if (waits) waits[2] += clock64() - t0;
      if (h == 0 && p.vec_store) {
        // the TMA store that last used this box must have read it out
        if (waits) t0 = clock64();
        if (lane == 0) tma_store_wait_read<kBoxes - 1>();
        __syncwarp();
        if (waits) waits[0] += clock64() - t0;
      }
      if (waits) t0 = clock64();
      epilogue_stage<OutT>(box, v, lane, h * kChunkStep);
      if (waits) waits[2] += clock64() - t0;
    }
    if (p.vec_store) {
      long long t1 = 0;
      if (waits) t1 = clock64();
      fence_proxy_async_smem();
      __syncwarp();
      if (waits) { const long long t2 = clock64(); waits[3] += t2 - t1; t1 = t2; }
      if (lane == 0) {
        tma_store_3d(tmap_c, smem_u32(box), col0, row0, batch);  // rows >= M and columns >= N are clipped
        tma_store_commit();
      }
      if (p.n_peers > 0) epilogue_push_box<OutT>(p, box, lane, batch, row0, col0);
      if (waits) waits[4] += clock64() - t1;
    } else {
      __syncwarp();
      epilogue_store_rows<OutT>(p, box, lane, batch, row0, col0);
      __syncwarp();
    }
    ++box_iter;
  }
}

// Predicated 16-byte read-only load: zero when `pred` is false (no branch, so several can be in flight).
__device__ __forceinline__ uint4 ldg_v4_if(const uint4* ptr, bool pred) {
  uint4 v;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %5, 0;\n\t"
      "mov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t"
      "@p ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(ptr), "r"(static_cast<uint32_t>(pred)));
  return v;
}

// The 16 bytes that start `sh` bytes (0..15, a multiple of the element size) into the 32-byte window
// (lo, hi).  `sh` is warp-uniform where this is called, so the switch does not diverge.
__device__ __forceinline__ uint4 shift_window_16(const uint4& lo, const uint4& hi, int sh) {
  const uint32_t bs = static_cast<uint32_t>(sh & 3) * 8u;
  uint4 o;
  switch (sh >> 2) {
    case 0:
      o.x = __funnelshift_r(lo.x, lo.y, bs); o.y = __funnelshift_r(lo.y, lo.z, bs);
      o.z = __funnelshift_r(lo.z, lo.w, bs); o.w = __funnelshift_r(lo.w, hi.x, bs);
      break;
    case 1:
      o.x = __funnelshift_r(lo.y, lo.z, bs); o.y = __funnelshift_r(lo.z, lo.w, bs);
      o.z = __funnelshift_r(lo.w, hi.x, bs); o.w = __funnelshift_r(hi.x, hi.y, bs);
      break;
    case 2:
      o.x = __funnelshift_r(lo.z, lo.w, bs); o.y = __funnelshift_r(lo.w, hi.x, bs);
      o.z = __funnelshift_r(hi.x, hi.y, bs); o.w = __funnelshift_r(hi.y, hi.z, bs);
      break;
    default:
      o.x = __funnelshift_r(lo.w, hi.x, bs); o.y = __funnelshift_r(hi.x, hi.y, bs);
      o.z = __funnelshift_r(hi.y, hi.z, bs); o.w = __funnelshift_r(hi.z, hi.w, bs);
      break;
  }
  return o;
}

// zeroes the bytes at or beyond `nvalid` (0..16)
__device__ __forceinline__ uint4 mask_tail_16(uint4 v, int nvalid) {
  uint32_t o[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int vb = nvalid - 4 * i;  // valid bytes in this word
    o[i] = vb >= 4 ? o[i] : (vb <= 0 ? 0u : (o[i] & ((1u << (8 * vb)) - 1u)));
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

static constexpr int kLoaderUnroll = 8;  // warp tasks whose loads are issued before the first is consumed

// Fills one operand tile of a ring stage from a matrix whose rows are only element-aligned.
//
// A warp task is four shared-memory rows x eight 16-byte chunks, lane = (row, chunk).  The four rows are 8
// apart, so they share the misalignment `sh` of their global address (8 pitches are a multiple of 16 bytes).
// Each lane loads the 16-byte-ALIGNED chunk that holds the first byte it needs — a warp instruction covers
// four contiguous 128-byte spans — takes the following aligned chunk from the next lane by shuffle (the row's
// last chunk loads it itself) and funnel-shifts the pair into place.  kLoaderUnroll tasks are in flight at
// once.  kInterior: the stage has no row / column / K tail, so nothing is predicated or masked; otherwise an
// aligned chunk is read only if it holds at least one byte of its row (never a foreign page) and bytes past
// the matrix are zeroed.
//   shared-memory row r (128 B): K-major  -> r indexes M (or N), the 128 B span BLOCK_K elements of K
//                                MN-major -> r = chunk * BLOCK_K + k, the 128 B span one chunk of M (or N)
template <int kElemBytes, bool kMn, int kBlockK, bool kInterior>
__device__ __forceinline__ void loader_fill(uint8_t* __restrict__ dst, const uint8_t* __restrict__ gbase, int64_t ld,
                                            int mn0, int k0, int mn_limit, int k_limit, int total_rows, int wg,
                                            int lane) {
  constexpr int kElemsPerChunk = 16 / kElemBytes;
  constexpr int kElemsPerRow = kSwizzleBytes / kElemBytes;
  const int sub = lane >> 3, ch = lane & 7;
  const int ntasks = total_rows / 4;
  const int64_t pitch = ld * kElemBytes;
  for (int task0 = wg * kLoaderUnroll; task0 < ntasks; task0 += kLoaderWarpsPerGroup * kLoaderUnroll) {
    uint4 lo[kLoaderUnroll], hi[kLoaderUnroll];
    int meta[kLoaderUnroll];  // (nvalid << 20) | (sh << 16) | byte offset of the destination chunk
#pragma unroll
    for (int u = 0; u < kLoaderUnroll; ++u) {
      const int task = task0 + u;
      const bool live = task < ntasks;  // uniform across the warp
      const int r = (task & 7) + 8 * (4 * (task >> 3) + sub);
      int64_t outer;  // index along the pitched (outer) global dimension
      int inner0;     // first index of this lane's chunk along the contiguous global dimension
      if (!kMn) { outer = mn0 + r; inner0 = k0 + ch * kElemsPerChunk; }
      else { outer = k0 + (r % kBlockK); inner0 = mn0 + (r / kBlockK) * kElemsPerRow + ch * kElemsPerChunk; }
      const uint8_t* row_base = gbase + outer * pitch;
      const uintptr_t ga = reinterpret_cast<uintptr_t>(row_base) + static_cast<uintptr_t>(inner0 * kElemBytes);
      const int sh = static_cast<int>(ga & 15u);  // identical in all 32 lanes of the task
      const uint4* p0 = reinterpret_cast<const uint4*>(ga - sh);
      // 16-bit and K-major tiles: 16-byte chunks XOR (row & 7).  32-bit MN-major tiles use the 128-byte
      // swizzle with 32-byte atoms: the 32-byte pair index XOR (row & 3).
      const int sw = (kElemBytes == 4 && kMn) ? ((((ch >> 1) ^ (r & 3)) << 1) | (ch & 1)) : (ch ^ (r & 7));
      int nvalid = 16;
      if (kInterior) {
        lo[u] = ldg_v4_if(p0, live);
        hi[u] = ldg_v4_if(p0 + 1, live && ch == 7 && sh != 0);
      } else {
        const int outer_limit = kMn ? k_limit : mn_limit, inner_limit = kMn ? mn_limit : k_limit;
        const bool row_ok = live && outer < outer_limit;
        nvalid = row_ok ? max(0, min(kElemsPerChunk, inner_limit - inner0)) * kElemBytes : 0;
        const uintptr_t row_end = reinterpret_cast<uintptr_t>(row_base) + static_cast<uintptr_t>(inner_limit) * kElemBytes;
        lo[u] = ldg_v4_if(p0, row_ok && reinterpret_cast<uintptr_t>(p0) < row_end);
        hi[u] = ldg_v4_if(p0 + 1, row_ok && ch == 7 && sh != 0 && reinterpret_cast<uintptr_t>(p0 + 1) < row_end);
      }
      meta[u] = (nvalid << 20) | (sh << 16) | (r * kSwizzleBytes + (sw << 4));
    }
#pragma unroll
    for (int u = 0; u < kLoaderUnroll; ++u) {
      if (task0 + u >= ntasks) break;  // uniform
      uint4 nx;
      nx.x = __shfl_down_sync(0xffffffffu, lo[u].x, 1);
      nx.y = __shfl_down_sync(0xffffffffu, lo[u].y, 1);
      nx.z = __shfl_down_sync(0xffffffffu, lo[u].z, 1);
      nx.w = __shfl_down_sync(0xffffffffu, lo[u].w, 1);
      if (ch == 7) nx = hi[u];
      uint4 v = shift_window_16(lo[u], nx, (meta[u] >> 16) & 15);
      if (!kInterior) v = mask_tail_16(v, meta[u] >> 20);
      *reinterpret_cast<uint4*>(dst + (meta[u] & 0xffff)) = v;
    }
  }
}

// ---------------------------------------------------------------- the kernel
//
// kElemBytes : 2 (f16 / bf16, kind::f16) or 4 (f32 read as tf32, kind::tf32)
// kTerms     : 1, or 3 for the hi/lo split (operand term 0 = hi, 1 = lo; products lo*hi + hi*lo + hi*hi)
// kAMn/kBMn  : operand is MN-major in global memory (A stored [K,M]; B stored [K,N]) instead of K-major
// kLoader    : compiled with the ld.global loader warps (448 threads) or without them
// kEpiWarps  : 4, or 8 for contractions so short that draining the accumulators dominates: two warps share
//              each tensor-memory lane quarter and each drains half of the tile's columns
template <int kBlockN, int kElemBytes, int kTerms, bool kAMn, bool kBMn, int kStages, bool kLoader, int kEpiWarps>
__global__ void __launch_bounds__(kLoader ? kThreadsWithLoader : 32 * (kFirstEpilogueWarp + kEpiWarps), 1)
nova_gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a0, const __grid_constant__ CUtensorMap tmap_a1,
                       const __grid_constant__ CUtensorMap tmap_b0, const __grid_constant__ CUtensorMap tmap_b1,
                       const __grid_constant__ CUtensorMap tmap_c, const GemmKernelParams p) {
  constexpr int kOpTerms = kTerms == 3 ? 2 : 1;
  using L = GemmSmemLayout<kBlockN, kOpTerms, kStages, kEpiWarps>;
  static_assert(kEpiWarps == 4 || (kEpiWarps == 8 && !kLoader), "warp roles");
  constexpr int kElemsPerRow = kSwizzleBytes / kElemBytes;  // 64 (16-bit) or 32 (tf32): BLOCK_K and MN chunk
  constexpr int kBlockK = kElemsPerRow;
  constexpr int kUmmaK = 32 / kElemBytes;
  constexpr int kKSteps = kBlockK / kUmmaK;  // 4
  // 3xTF32: the two small products (lo x hi, hi x lo) go to accumulators of their own, so that the big one takes a third
  // of the additions: the tensor core adds with truncation and the drift of a sum grows with its number of additions.
  constexpr bool kTwoAcc = kTerms == 3;
  constexpr uint32_t kTmemCols = (kTwoAcc ? 4 : 2) * kBlockN < 32 ? 32 : (kTwoAcc ? 4 : 2) * kBlockN;
  static_assert(kBlockN % 32 == 0 && kBlockN >= 32 && kBlockN <= 256, "UMMA N / epilogue chunking");
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns must be a power of two <= 512");
  static_assert(L::kDynamicBytes <= 227 * 1024, "shared memory budget");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::kBarrierOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOffset);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kMiscOffset + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool use_loader = kLoader && (p.loader_a | p.loader_b) != 0;

  if (threadIdx.x == 0) {
    // arrivals per phase on a full barrier: the producer's expect_tx arrive, plus one per loader warp
    const uint32_t full_count = 1u + (use_loader ? kLoaderWarpsPerGroup : 0u);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), full_count);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), kEpiWarps * 32);
    }
    *abort_flag = 0u;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // everything above touched only this CTA's shared and tensor memory: it may overlap the previous kernel's tail
  griddep_launch_dependents();
  griddep_wait();

  if (warp == 0) {
    // ============================================================ TMA producer
    if (lane == 0) {
      if (!p.loader_a) { tma_prefetch_desc(&tmap_a0); if (kOpTerms == 2) tma_prefetch_desc(&tmap_a1); }
      if (!p.loader_b) { tma_prefetch_desc(&tmap_b0); if (kOpTerms == 2) tma_prefetch_desc(&tmap_b1); }
      uint32_t expect = 0;
      if (!p.loader_a) expect += kOpTerms * L::kATile;
      if (!p.loader_b) expect += kOpTerms * L::kBTile;
      uint32_t it = 0;
      bool ok = true;
      for (int32_t tile = blockIdx.x; ok && tile < p.tiles; tile += gridDim.x) {
        const TileCoord t = decode_tile(p, tile);
        const int m0 = t.m_blk * kBlockM, n0 = t.n_blk * kBlockN;
        // a split product: launch batch index = operand batch * ranges + range (see split_k_len)
        const int ob = p.split_k_ranges > 1 ? t.batch / p.split_k_ranges : t.batch;
        const int k_first = p.split_k_ranges > 1 ? (t.batch - ob * p.split_k_ranges) * p.split_k_len : 0;
        const int za = ob * p.a_batch_mul, zb = ob * p.b_batch_mul;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, kStatusProducerEmptyWait)) { ok = false; break; }
          const uint32_t stage = smem_base + s * L::kStageBytes;
          const uint32_t bar = full_bar(s);
          mbar_arrive_expect_tx(bar, expect);
          const int k0 = k_first + kb * kBlockK;
#pragma unroll
          for (int term = 0; term < kOpTerms; ++term) {
            if (!p.loader_a) {
              const CUtensorMap* ma = term == 0 ? &tmap_a0 : &tmap_a1;
              const uint32_t dst = stage + term * L::kATile;
              if (!kAMn) {
                tma_load_3d(dst, ma, bar, k0, m0, za);  // box {BLOCK_K, 128 rows}
              } else {
#pragma unroll
                for (int c = 0; c < kBlockM / kElemsPerRow; ++c)  // box {chunk of M, BLOCK_K rows}
                  tma_load_3d(dst + c * (kBlockK * kSwizzleBytes), ma, bar, m0 + c * kElemsPerRow, k0, za);
              }
            }
            if (!p.loader_b) {
              const CUtensorMap* mb = term == 0 ? &tmap_b0 : &tmap_b1;
              const uint32_t dst = stage + kOpTerms * L::kATile + term * L::kBTile;
              if (!kBMn) {
                tma_load_3d(dst, mb, bar, k0, n0, zb);  // box {BLOCK_K, kBlockN rows}
              } else {
#pragma unroll
                for (int c = 0; c < kBlockN / kElemsPerRow; ++c)  // box {chunk of N, BLOCK_K rows}
                  tma_load_3d(dst + c * (kBlockK * kSwizzleBytes), mb, bar, n0 + c * kElemsPerRow, k0, zb);
              }
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ============================================================ MMA issuer
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int32_t tile = blockIdx.x; ok && tile < p.tiles; tile += gridDim.x, ++tile_iter) {
        const uint32_t acc = tile_iter & 1u;
        const uint32_t acc_ph = (tile_iter >> 1) & 1u;
        if (!mbar_wait(tmem_empty_bar(acc), acc_ph ^ 1u, abort_flag, p.status, kStatusMmaTmemEmptyWait)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kBlockN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(full_bar(s), ph, abort_flag, p.status, kStatusMmaFullWait)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_stage = smem_base + s * L::kStageBytes;
          const uint32_t b_stage = a_stage + kOpTerms * L::kATile;
#pragma unroll
          for (int k = 0; k < kKSteps; ++k) {
            const uint32_t first = (kb | k) == 0 ? 0u : 1u;
            const uint64_t a_hi = make_smem_desc(a_stage + k * p.a_kstep, p.a_desc_lbo, p.a_desc_hi);
            const uint64_t b_hi = make_smem_desc(b_stage + k * p.b_kstep, p.b_desc_lbo, p.b_desc_hi);
            if (kElemBytes == 2) {
              umma_f16(d_tmem, a_hi, b_hi, p.idesc, first);
            } else if (kTerms == 1) {
              umma_tf32(d_tmem, a_hi, b_hi, p.idesc, first);
            } else {
              const uint64_t a_lo = make_smem_desc(a_stage + L::kATile + k * p.a_kstep, p.a_desc_lbo, p.a_desc_hi);
              const uint64_t b_lo = make_smem_desc(b_stage + L::kBTile + k * p.b_kstep, p.b_desc_lbo, p.b_desc_hi);
              umma_tf32(d_tmem + 2 * kBlockN, a_lo, b_hi, p.idesc, first);  // the small terms: their own accumulator
              umma_tf32(d_tmem + 2 * kBlockN, a_hi, b_lo, p.idesc, 1u);
              umma_tf32(d_tmem, a_hi, b_hi, p.idesc, first);
            }
          }
          umma_commit(empty_bar(s));  // stage reusable once these MMAs have read it
        }
        if (ok) umma_commit(tmem_full_bar(acc));  // accumulator complete
      }
    }
    __syncwarp();
  } else if (warp < kFirstEpilogueWarp + kEpiWarps) {
    // ============================================================ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* staging = smem_gen + L::kStagingOffset + (warp - kFirstEpilogueWarp) * (2 * L::kStageOutBox);
    if (p.vec_store && lane == 0) tma_prefetch_desc(&tmap_c);
    uint32_t tile_iter = 0;
    uint32_t box_iter = 0;
    for (int32_t tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++tile_iter) {
      const TileCoord t = decode_tile(p, tile);
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_ph = (tile_iter >> 1) & 1u;
      if (!mbar_wait(tmem_full_bar(acc), acc_ph, abort_flag, p.status, kStatusEpilogueTmemFullWait)) break;
      tc_fence_after_sync();
      constexpr int kColsPerWarp = kBlockN / (kEpiWarps / 4);
      const int cg = (warp - kFirstEpilogueWarp) >> 2;  // which column group of the tile this warp drains
      const int32_t row0 = t.m_blk * kBlockM + q * 32;
      const int32_t n0 = t.n_blk * kBlockN + cg * kColsPerWarp;
      const uint32_t taddr = tmem_base + acc * kBlockN + cg * kColsPerWarp + (static_cast<uint32_t>(q * 32) << 16);
      if (p.out_dtype == NOVA_B200_BF16)
        epilogue_tile<__nv_bfloat16, kColsPerWarp, 2, kTwoAcc ? 2 * kBlockN : 0>(p, &tmap_c, taddr, staging, box_iter, lane, t.batch, row0, n0);
      else if (p.out_dtype == NOVA_B200_F16)
        epilogue_tile<__half, kColsPerWarp, 2, kTwoAcc ? 2 * kBlockN : 0>(p, &tmap_c, taddr, staging, box_iter, lane, t.batch, row0, n0);
      else
        epilogue_tile<float, kColsPerWarp, 2, kTwoAcc ? 2 * kBlockN : 0>(p, &tmap_c, taddr, staging, box_iter, lane, t.batch, row0, n0);
      tc_fence_before_sync();
      mbar_arrive(tmem_empty_bar(acc));
    }
    if (p.vec_store && lane == 0) tma_store_wait_read<0>();  // staged boxes read out before shared memory goes away
    __syncwarp();
  } else if (kLoader) {
    // ============================================================ ld.global loader (operands TMA cannot address)
    // Each stage's operand tile is written exactly as TMA would write it: 128-byte rows whose
    // 16-byte chunks are XOR-swizzled with (row & 7); out-of-range elements are zero.
    // Group g fills the stages of k-block iterations it == g (mod kLoaderGroups): each group's global-memory
    // latency overlaps the other groups' work, so several stages are in flight at once.
    const int lw = warp - kFirstLoaderWarp;
    const int group = lw / kLoaderWarpsPerGroup;
    uint32_t it = 0;
    bool ok = true;
    for (int32_t tile = blockIdx.x; ok && tile < p.tiles; tile += gridDim.x) {
      const TileCoord t = decode_tile(p, tile);
      const int m0 = t.m_blk * kBlockM, n0 = t.n_blk * kBlockN;
      for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
        if (static_cast<int>(it % kLoaderGroups) != group) continue;
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status, kStatusLoaderEmptyWait)) { ok = false; break; }
        uint8_t* stage = smem_gen + s * L::kStageBytes;
        const int k0 = kb * kBlockK;
#pragma unroll
        for (int op = 0; op < 2; ++op) {
          if (op == 0 ? !p.loader_a : !p.loader_b) continue;
          const bool mn = op == 0 ? kAMn : kBMn;
          const int rows_mn = op == 0 ? kBlockM : kBlockN;  // extent of the tile along M (or N)
          const int mn0 = op == 0 ? m0 : n0;
          const int mn_limit = op == 0 ? p.M : p.N;
          const int64_t ld = op == 0 ? p.lda : p.ldb;
          const uint8_t* gbase = reinterpret_cast<const uint8_t*>(op == 0 ? p.A : p.B) +
                                 static_cast<int64_t>(t.batch) * (op == 0 ? p.a_batch_mul * p.stride_a
                                                                          : p.b_batch_mul * p.stride_b) * kElemBytes;
          uint8_t* dst = stage + (op == 0 ? 0 : kOpTerms * L::kATile);
          // smem row r (128 B): K-major -> r indexes M/N, 128 B span BLOCK_K elements of K
          //                     MN-major -> rows are grouped per chunk of kElemsPerRow M/N elements:
          //                                 row = chunk * BLOCK_K + k, 128 B span the chunk
          const int total_rows = mn ? (rows_mn / kElemsPerRow) * kBlockK : rows_mn;
          const int wg = lw % kLoaderWarpsPerGroup;
          // interior tiles (no row, column or K tail inside this stage) take the predicate-free path
          const bool interior = mn0 + rows_mn <= mn_limit && k0 + kBlockK <= p.K;
          if (mn) {
            if (interior) loader_fill<kElemBytes, true, kBlockK, true>(dst, gbase, ld, mn0, k0, mn_limit, p.K, total_rows, wg, lane);
            else loader_fill<kElemBytes, true, kBlockK, false>(dst, gbase, ld, mn0, k0, mn_limit, p.K, total_rows, wg, lane);
          } else {
            if (interior) loader_fill<kElemBytes, false, kBlockK, true>(dst, gbase, ld, mn0, k0, mn_limit, p.K, total_rows, wg, lane);
            else loader_fill<kElemBytes, false, kBlockK, false>(dst, gbase, ld, mn0, k0, mn_limit, p.K, total_rows, wg, lane);
          }
        }
        fence_proxy_async_smem();  // make the generic-proxy writes visible to the tensor core (async proxy)
        __syncwarp();
        if (lane == 0) mbar_arrive(full_bar(s));
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u && threadIdx.x == 0) {
    // a wait gave up: let this CTA's in-flight bulk copies land before its shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------- helper kernels

// hi = x rounded to tf32 (round-to-nearest), lo = x - hi (exact in fp32); written to compact
// [batch, rows, ld_out] buffers whose pitch is a multiple of 16 bytes whatever the input pitch was.
// One launch splits both operands: blockIdx.y == 0 handles A, 1 handles B.
struct SplitOperand {
  const float* x;
  float* hi;
  float* lo;
  int64_t rows_total, ld_in, stride_in;
  int32_t rows_per_batch, cols, ld_out;
};

__global__ void nova_split_tf32_kernel(const SplitOperand oa, const SplitOperand ob) {
  // the contraction that consumes this scratch is launched with programmatic serialization: let its prologue
  // (barriers, tensor-memory allocation) start now; it waits for this whole grid before its first global access
  griddep_launch_dependents();
  const SplitOperand& o = blockIdx.y == 0 ? oa : ob;
  // four output columns per thread (ld_out is a multiple of 4 and the scratch is 16-byte aligned); the input is
  // read as one float4 when its row start allows, else element-wise
  const int32_t quads = o.ld_out >> 2;
  const int64_t n = o.rows_total * quads;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / quads;
    const int32_t c = static_cast<int32_t>(i - r * quads) << 2;
    const int64_t b = r / o.rows_per_batch;
    const float* src = o.x + b * o.stride_in + (r - b * o.rows_per_batch) * o.ld_in + c;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (c + 4 <= o.cols && (reinterpret_cast<uintptr_t>(src) & 15u) == 0u) {
      const float4 q = *reinterpret_cast<const float4*>(src);
      v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (c + e < o.cols) v[e] = src[e];
    }
    float h[4], l[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      uint32_t hb;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(v[e]));
      h[e] = __uint_as_float(hb);
      l[e] = v[e] - h[e];
    }
    reinterpret_cast<float4*>(o.hi)[i] = make_float4(h[0], h[1], h[2], h[3]);
    reinterpret_cast<float4*>(o.lo)[i] = make_float4(l[0], l[1], l[2], l[3]);
  }
}

// Re-pitch: copies an operand whose base or row pitch is not a multiple of 16 bytes (so no tensor map can
// describe it) into [batch, rows, ld_out] scratch whose pitch is, one 16-byte chunk per thread.  Source reads
// are element-wise (consecutive threads read consecutive 16-byte spans of a row, so every sector is still
// fetched once); columns past `cols` are written as zeros.  blockIdx.y == 0 handles oa, 1 handles ob (rows_total
// == 0 skips an operand).
struct RepitchOperand {
  const void* src;
  void* dst;
  int64_t rows_total, ld_in, stride_in;  // elements
  int32_t rows_per_batch, cols, ld_out;
};

template <typename ElemT>
__global__ void nova_repitch_kernel(const RepitchOperand oa, const RepitchOperand ob) {
  constexpr int kPerChunk = 16 / static_cast<int>(sizeof(ElemT));
  griddep_launch_dependents();  // as in nova_split_tf32_kernel
  const RepitchOperand& o = blockIdx.y == 0 ? oa : ob;
  const int32_t chunks_per_row = o.ld_out / kPerChunk;
  const int64_t n = o.rows_total * chunks_per_row;
  const ElemT* src = static_cast<const ElemT*>(o.src);
  uint4* dst = static_cast<uint4*>(o.dst);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / chunks_per_row;
    const int32_t c0 = static_cast<int32_t>(i - r * chunks_per_row) * kPerChunk;
    const int64_t b = r / o.rows_per_batch;
    const ElemT* row = src + b * o.stride_in + (r - b * o.rows_per_batch) * o.ld_in + c0;
    union { uint4 u; ElemT e[kPerChunk]; } v;
#pragma unroll
    for (int e = 0; e < kPerChunk; ++e) v.e[e] = c0 + e < o.cols ? __ldg(row + e) : ElemT(0);
    dst[i] = v.u;
  }
}

// Second half of a K-split product: C[m, n] = round(act(init + sum over ranges of partial[s][m][n])), the ranges added in
// ascending order, init / activation exactly as the contraction's own epilogue applies them.
struct SplitKReduce {
  const float* partial;   // [batch][ranges][M][ldp]
  void* C;
  const void* bias;
  const void* residual;
  int64_t M, N, ldp, ldc, ldr, batch, stride_c, stride_r;
  int32_t ranges, init, act, out_dtype;
};

template <typename OutT>
__device__ __forceinline__ float splitk_finish(const SplitKReduce& r, float v, int64_t m, int64_t col, const OutT* bias,
                                               const OutT* res, const OutT* c) {
  if (r.init == NOVA_B200_INIT_LN_FOLD) {
    // v = rstd_m * (acc - mean_m * c_n) + d_n: bias = the fp32 arrays c then d, residual = {mean, rstd} per row
    const float* cd = static_cast<const float*>(r.bias);
    const float2 st = static_cast<const float2*>(r.residual)[m];
    v = fmaf(st.y, fmaf(-st.x, cd[col], v), cd[r.N + col]);
  }
  if (r.init == NOVA_B200_INIT_BIAS_ROW || r.init == NOVA_B200_INIT_BIAS_AND_RESIDUAL) v += to_f32<OutT>(bias[col]);
  if (r.init == NOVA_B200_INIT_RESIDUAL_FULL || r.init == NOVA_B200_INIT_BIAS_AND_RESIDUAL) v += to_f32<OutT>(res[m * r.ldr + col]);
  if (r.init == NOVA_B200_INIT_FROM_C) v += to_f32<OutT>(c[m * r.ldc + col]);
  if (r.act == NOVA_B200_ACT_RELU) v = fmaxf(v, 0.0f);
  else if (r.act == NOVA_B200_ACT_GELU_TANH) v = gelu_tanh_f32(v);
  else if (r.act == NOVA_B200_ACT_GELU_TANH_GRAD) v *= gelu_tanh_grad_f32(to_f32<OutT>(res[m * r.ldr + col]));
  return v;
}

// One thread finishes four consecutive columns: 16-byte loads of the partials (their pitch is a multiple of four
// floats), four loads in flight per range step; the ragged last columns of a row fall back to single elements.
template <typename OutT>
__global__ void __launch_bounds__(256) nova_splitk_reduce_kernel(const SplitKReduce r) {
  griddep_wait();  // launched with programmatic serialization behind the contraction that writes the partials
  const int64_t quads = r.ldp >> 2;
  const int64_t per_batch = r.M * quads;
  const int64_t n = r.batch * per_batch;
  const int64_t plane = r.M * r.ldp;
  const OutT* bias = static_cast<const OutT*>(r.bias);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = i / per_batch, ib = i - b * per_batch;
    const int64_t m = ib / quads, col = (ib - m * quads) << 2;
    if (col >= r.N) continue;
    OutT* c = static_cast<OutT*>(r.C) + b * r.stride_c;
    // (the LN fold keeps per-row statistics, not a matrix, behind `residual`; it is never batched)
    const OutT* res = r.init == NOVA_B200_INIT_LN_FOLD ? static_cast<const OutT*>(r.residual)
                                                        : static_cast<const OutT*>(r.residual) + b * r.stride_r;
    const float4* pp = reinterpret_cast<const float4*>(r.partial + b * r.ranges * plane + m * r.ldp + col);
    const int64_t plane4 = plane >> 2;
    float4 acc = pp[0];
    int32_t s = 1;
    for (; s + 3 < r.ranges; s += 4) {   // ascending range order, four loads in flight
      const float4 q0 = pp[s * plane4], q1 = pp[(s + 1) * plane4], q2 = pp[(s + 2) * plane4], q3 = pp[(s + 3) * plane4];
      acc.x = (((acc.x + q0.x) + q1.x) + q2.x) + q3.x;
      acc.y = (((acc.y + q0.y) + q1.y) + q2.y) + q3.y;
      acc.z = (((acc.z + q0.z) + q1.z) + q2.z) + q3.z;
      acc.w = (((acc.w + q0.w) + q1.w) + q2.w) + q3.w;
    }
    for (; s < r.ranges; ++s) {
      const float4 q = pp[s * plane4];
      acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
    }
    const float v[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (col + e < r.N) c[m * r.ldc + col + e] = from_f32<OutT>(splitk_finish<OutT>(r, v[e], m, col + e, bias, res, c));
  }
}

// C = act(init) for K == 0 (an empty contraction leaves the accumulator at its initial value).
template <typename OutT>
__global__ void nova_gemm_k0_kernel(GemmKernelParams p) {
  const int64_t per_batch = static_cast<int64_t>(p.M) * p.N;
  const int64_t n = per_batch * p.batch;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t b = i / per_batch;
    const int64_t r = (i - b * per_batch) / p.N;
    const int64_t c = i - b * per_batch - r * p.N;
    OutT* dst = reinterpret_cast<OutT*>(p.C) + b * p.stride_c + r * p.ldc + c;
    float v = 0.0f;
    if (p.init == NOVA_B200_INIT_LN_FOLD) v = reinterpret_cast<const float*>(p.bias)[p.N + c];  // K == 0: only d_j is left
    if (p.init == NOVA_B200_INIT_BIAS_ROW || p.init == NOVA_B200_INIT_BIAS_AND_RESIDUAL)
      v = to_f32<OutT>(reinterpret_cast<const OutT*>(p.bias)[c]);
    if (p.init == NOVA_B200_INIT_RESIDUAL_FULL || p.init == NOVA_B200_INIT_BIAS_AND_RESIDUAL)
      v += to_f32<OutT>(reinterpret_cast<const OutT*>(p.residual)[b * p.stride_r + r * p.ldr + c]);
    else if (p.init == NOVA_B200_INIT_FROM_C) v = to_f32<OutT>(*dst);
    if (p.act == NOVA_B200_ACT_RELU) v = fmaxf(v, 0.0f);
    else if (p.act == NOVA_B200_ACT_GELU_TANH) v = gelu_tanh_f32(v);
    else if (p.act == NOVA_B200_ACT_GELU_TANH_GRAD)
      v *= gelu_tanh_grad_f32(to_f32<OutT>(reinterpret_cast<const OutT*>(p.residual)[b * p.stride_r + r * p.ldr + c]));
    *dst = from_f32<OutT>(v);
  }
}

}  // namespace nova
