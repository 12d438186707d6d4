// Host side of the contraction: argument validation, kernel selection ("plan"),
// tensor-map encoding and launch.  See gemm_kernel.cuh for the device code.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cstring>

#include "gemm_kernel.cuh"
#include "gemm_kernel_pair.cuh"

namespace nova {
namespace {

struct Plan {
  nova_b200_gemm_plan_info info{};
  int elem_bytes = 2;
  int terms = 1;
  bool a_mn = false, b_mn = false;
  int out_bytes = 2;
  bool k_zero = false;
  bool empty = false;
  bool pair = false;  // CTA-pair kernel (cta_group::2, 256 x 256 tiles)
  bool short_k = false;  // contraction so short that the epilogue dominates: 8 epilogue warps, 3 stages
  int64_t repitch_a_ld = 0, repitch_b_ld = 0;  // > 0: the operand is first copied to scratch with this pitch
  int prefetch_dist = 0;  // pair kernel: ring stages the L2 prefetch cursor runs ahead of the loads
  // K split into this many equal ranges that run as the batches of one launch and are summed (in a fixed order) by a
  // second kernel that also applies the epilogue: for products with too few output tiles to fill the GPU
  int split_k = 1;
  int64_t split_len = 0;         // K elements per range (a multiple of the k-block)
  int64_t split_ldp = 0;         // pitch of one partial matrix (floats)
  int64_t split_offset = 0;      // byte offset of the partials in the stream's scratch
};

constexpr int64_t kMaxExtent = (1ll << 31) - 1;

int32_t validate_and_plan(const nova_b200_gemm_args* a, Plan* plan, int sm_count, bool allow_split_k = true) {
  if (!a) return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: args is null");
  if (a->struct_size != sizeof(nova_b200_gemm_args))
    return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: struct_size does not match this library's nova_b200_gemm_args");
  if (a->dtype_ab != NOVA_B200_F32 && a->dtype_ab != NOVA_B200_F16 && a->dtype_ab != NOVA_B200_BF16)
    return fail(NOVA_B200_ERR_UNSUPPORTED, "gemm: dtype_ab must be f32, f16 or bf16");
  if (!is_float_dtype(a->dtype_c)) return fail(NOVA_B200_ERR_UNSUPPORTED, "gemm: dtype_c must be f32, f16 or bf16");
  if (a->act < NOVA_B200_ACT_NONE || a->act > NOVA_B200_ACT_GELU_TANH_GRAD)
    return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: unknown activation");
  if (a->init < NOVA_B200_INIT_ZERO || a->init > NOVA_B200_INIT_LN_FOLD)
    return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: unknown accumulator init");
  if (a->init == NOVA_B200_INIT_LN_FOLD) {
    if (a->batch > 1) return fail(NOVA_B200_ERR_UNSUPPORTED, "gemm: INIT_LN_FOLD takes one matrix (flatten batch into rows)");
    if (a->act == NOVA_B200_ACT_GELU_TANH_GRAD) return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: INIT_LN_FOLD excludes ACT_GELU_TANH_GRAD");
    if (!a->bias || !a->residual)
      return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: INIT_LN_FOLD needs bias = fp32 {c, d} and residual = fp32 row statistics");
    if (reinterpret_cast<uintptr_t>(a->residual) % 8 != 0) return fail(NOVA_B200_ERR_LAYOUT, "gemm: row statistics must be 8-byte aligned");
  }
  if (a->f32_mode != NOVA_B200_TF32X3 && a->f32_mode != NOVA_B200_TF32X1)
    return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: unknown f32_mode");
  if (a->batch < 0 || a->M < 0 || a->N < 0 || a->K < 0)
    return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: negative extent");
  if (a->batch > kMaxExtent || a->M > kMaxExtent || a->N > kMaxExtent || a->K > kMaxExtent)
    return fail(NOVA_B200_ERR_TOO_LARGE, "gemm: extent exceeds 2^31-1");
  plan->empty = a->batch == 0 || a->M == 0 || a->N == 0;
  plan->k_zero = a->K == 0;
  plan->elem_bytes = dtype_bytes(a->dtype_ab);
  plan->out_bytes = dtype_bytes(a->dtype_c);
  plan->a_mn = a->trans_a != 0;  // A stored [K, M]: M is the contiguous (MN-major) dimension
  plan->b_mn = a->trans_b == 0;  // B stored [K, N]: N is the contiguous (MN-major) dimension
  if (plan->empty) return NOVA_B200_OK;

  if (!a->C) return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: C is null");
  if (!plan->k_zero && (!a->A || !a->B)) return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: A or B is null");
  if (init_has_bias(a->init) && !a->bias) return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: bias is null");
  if (a->act == NOVA_B200_ACT_GELU_TANH_GRAD && init_has_residual(a->init))
    return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: with ACT_GELU_TANH_GRAD the residual pointer holds the pre-activation; "
                                           "init must be ZERO, BIAS_ROW or FROM_C");
  if (reads_residual(a->init, a->act) && !a->residual)
    return fail(NOVA_B200_ERR_INVALID_ARG, "gemm: residual is null");
  const int64_t a_inner = a->trans_a ? a->M : a->K;
  const int64_t b_inner = a->trans_b ? a->K : a->N;
  if (!plan->k_zero && (a->lda < a_inner || a->ldb < b_inner))
    return fail(NOVA_B200_ERR_LAYOUT, "gemm: lda/ldb smaller than the contiguous extent");
  if (a->ldc < a->N) return fail(NOVA_B200_ERR_LAYOUT, "gemm: ldc smaller than N");
  if (reads_residual(a->init, a->act) && a->ldr < a->N)
    return fail(NOVA_B200_ERR_LAYOUT, "gemm: ldr smaller than N");
  if (a->batch_stride_a < 0 || a->batch_stride_b < 0 || a->batch_stride_c < 0 || a->batch_stride_r < 0)
    return fail(NOVA_B200_ERR_LAYOUT, "gemm: negative batch stride");
  if (a->batch > 1 && a->batch_stride_c < a->M * a->ldc && a->batch_stride_c != 0)
    return fail(NOVA_B200_ERR_LAYOUT, "gemm: batch_stride_c makes output batches overlap");
  if (a->batch > 1 && a->batch_stride_c == 0)
    return fail(NOVA_B200_ERR_LAYOUT, "gemm: output cannot be shared across batches");

  nova_b200_gemm_plan_info& pi = plan->info;
  const int es = plan->elem_bytes;
  auto tma_ok = [&](const void* base, int64_t ld, int64_t bstride) {
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return false;
    if ((ld * es) % 16 != 0) return false;
    if (a->batch > 1 && bstride != 0 && (bstride * es) % 16 != 0) return false;
    if (static_cast<unsigned long long>(ld) * es >= (1ull << 40)) return false;
    if (static_cast<unsigned long long>(bstride) * es >= (1ull << 40)) return false;
    return true;
  };
  plan->terms = (a->dtype_ab == NOVA_B200_F32 && a->f32_mode == NOVA_B200_TF32X3) ? 3 : 1;
  if (plan->terms == 3) {
    pi.loader_a = pi.loader_b = 0;  // operands are re-laid out by the hi/lo split into aligned scratch
    const int64_t a_rows = a->trans_a ? a->K : a->M, a_cols = a->trans_a ? a->M : a->K;
    const int64_t b_rows = a->trans_b ? a->N : a->K, b_cols = a->trans_b ? a->K : a->N;
    const int64_t a_b = a->batch_stride_a == 0 ? 1 : a->batch, b_b = a->batch_stride_b == 0 ? 1 : a->batch;
    pi.scratch_bytes = 2 * 4 * (a_b * a_rows * ((a_cols + 3) & ~3ll) + b_b * b_rows * ((b_cols + 3) & ~3ll));
  } else {
    pi.loader_a = tma_ok(a->A, a->lda, a->batch_stride_a) ? 0 : 1;
    pi.loader_b = tma_ok(a->B, a->ldb, a->batch_stride_b) ? 0 : 1;
    pi.scratch_bytes = 0;
    // An operand no tensor map can describe is first re-pitched into aligned scratch (one extra read and write
    // of the operand, then the full-rate TMA kernels).  Measured from 500^3 (11.9 us against 29.2) to
    // 4095 x 11007 x 4097 (0.32 ms against 1.70) that beats reading it in place with the loader warps, which
    // remain for callers that want no scratch traffic: NOVA_B200_REPITCH=0.
    const bool repitch = (pi.loader_a || pi.loader_b) && options().repitch.load() != 0;
    if (repitch) {
      const int per_chunk = 16 / es;
      const int64_t a_rows = a->trans_a ? a->K : a->M, a_cols = a->trans_a ? a->M : a->K;
      const int64_t b_rows = a->trans_b ? a->N : a->K, b_cols = a->trans_b ? a->K : a->N;
      const int64_t a_b = a->batch_stride_a == 0 ? 1 : a->batch, b_b = a->batch_stride_b == 0 ? 1 : a->batch;
      if (pi.loader_a) {
        plan->repitch_a_ld = (a_cols + per_chunk - 1) / per_chunk * per_chunk;
        pi.scratch_bytes += (a_b * a_rows * plan->repitch_a_ld * es + 255) / 256 * 256;
        pi.loader_a = 2;
      }
      if (pi.loader_b) {
        plan->repitch_b_ld = (b_cols + per_chunk - 1) / per_chunk * per_chunk;
        pi.scratch_bytes += (b_b * b_rows * plan->repitch_b_ld * es + 255) / 256 * 256;
        pi.loader_b = 2;
      }
    }
  }
  const int osz = plan->out_bytes;
  // The TMA-store epilogue writes whole 16-byte chunks: a row whose last chunk is partial (N * element size not a
  // multiple of 16) inside a wider buffer would have the bytes after column N overwritten, so it takes element stores.
  const bool c_vec = reinterpret_cast<uintptr_t>(a->C) % 16 == 0 && (a->ldc * osz) % 16 == 0 &&
                     (a->N * osz) % 16 == 0 && (a->batch <= 1 || (a->batch_stride_c * osz) % 16 == 0);
  pi.store_c = c_vec ? 0 : 1;

  pi.block_m = kBlockM;
  pi.block_k = kSwizzleBytes / es;
  const int64_t m_blocks = (a->M + kBlockM - 1) / kBlockM;
  // Tile shape.  Three candidates: 128 x 128 and 128 x 256 tiles on single CTAs (one per SM), 256 x 256 tiles on
  // CTA pairs (one per two SMs).  Each is priced as waves x (cycles of one tile's K loop) + the part of a launch
  // that does not overlap (launch, first loads, last epilogue), with constants fitted to B200 timings: every
  // shape streams at 8.5-9.3 cycles per K element per wave (a 128 x 128 tile is bound by shared-memory reads,
  // not by the tensor pipe, so it is no faster than a 128 x 256 one), never faster than its epilogue drains a
  // tile; pairs stream ~7 % faster and cost a cluster launch and cluster barriers up front.
  const int sms = sm_count > 0 ? sm_count : 148;
  const bool both_tma = pi.loader_a != 1 && pi.loader_b != 1;
  const int64_t n64 = (a->N + 63) / 64, n128 = (a->N + 127) / 128, n256 = (a->N + 255) / 256;
  const int64_t tiles64 = a->batch * m_blocks * n64;
  const int64_t tiles128 = a->batch * m_blocks * n128, tiles256 = a->batch * m_blocks * n256;
  const int64_t pair_tiles = a->batch * ((a->M + kPairBlockM - 1) / kPairBlockM) * ((a->N + kPairBlockN - 1) / kPairBlockN);
  auto waves = [](int64_t tiles, int64_t slots) { return static_cast<double>((tiles + slots - 1) / slots); };
  const double kd = static_cast<double>(a->K);
  // (128 x 64 tiles only pay when the problem is a fraction of a wave: twice the CTAs, each half the K-loop work)
  const double cost64 = waves(tiles64, sms) * std::max(7.0 * kd, 2000.0) + 10500.0;
  const double cost128 = waves(tiles128, sms) * std::max(9.3 * kd, 3000.0) + 11000.0;
  // (the short-K build below drains a 128 x 256 tile with eight warps)
  const double drain256 = (a->K <= 256 && pi.store_c == 0) ? 3900.0 : 6000.0;
  const double cost256 = waves(tiles256, sms) * std::max(9.1 * kd, drain256) + 11800.0;
  const double cost_pair = waves(pair_tiles, sms / 2) * std::max(8.5 * kd, 5000.0) + 13100.0;
  // (contractions shorter than two 128-element stages are bound by their epilogue, which pairs do not help)
  bool pair = plan->terms == 1 && both_tma && a->K >= 256 && cost_pair <= cost128 && cost_pair <= cost256 &&
              cost_pair <= cost64;
  int block_n = 256;
  if (plan->terms == 3) block_n = tiles128 <= sms / 4 ? 64 : 128;  // two operand copies per stage: 256 does not fit
  else if (both_tma && plan->terms == 1 && cost64 < cost128 && (a->N <= 128 || cost64 < cost256)) block_n = 64;
  else if (a->N <= 128) block_n = 128;
  else if (both_tma && plan->terms == 1) block_n = cost128 < cost256 ? 128 : 256;
  else if (tiles256 < sms) block_n = 128;  // loader warps: keep every SM's loaders busy
  {
    const int v = static_cast<int>(options().block_n.load());
    if ((v == 128 || v == 256) && plan->terms != 3) { block_n = v; pair = false; }
    if (v == 64 && (plan->terms == 3 || both_tma)) { block_n = v; pair = false; }
    const int pv = static_cast<int>(options().pair.load());
    if (pv == 0) pair = false;
    else if (pv > 0) pair = plan->terms == 1 && both_tma && a->K >= 256;
  }
  pi.block_n = block_n;
  const int64_t tiles = block_n == 256 ? tiles256 : (block_n == 128 ? tiles128 : tiles64);
  if (tiles > kMaxExtent) return fail(NOVA_B200_ERR_TOO_LARGE, "gemm: more than 2^31-1 output tiles");
  pi.tiles = tiles;
  pi.stages = plan->terms == 3 ? (block_n == 64 ? 4 : 3) : (block_n == 256 ? 4 : (block_n == 128 ? 6 : 8));
  pi.grid = static_cast<int32_t>(tiles < sms ? tiles : sms);
  plan->pair = pair;
  // K <= 256 with full-width tiles: the mainloop of a tile is at most four k-blocks, the time goes into
  // draining 128 x 256 accumulators, so trade one ring stage for a second set of epilogue warps.
  plan->short_k = !pair && plan->terms == 1 && both_tma && block_n == 256 && a->K <= 256 && pi.store_c == 0;
  if (options().short_k.load() == 0) plan->short_k = false;
  if (plan->short_k) pi.stages = 3;
  if (pair) {
    pi.block_m = kPairBlockM;
    pi.block_n = kPairBlockN;
    pi.stages = kPairStages;
    pi.tiles = pair_tiles;
    pi.grid = static_cast<int32_t>(2 * (pair_tiles < sms / 2 ? pair_tiles : sms / 2));
    const int64_t pf = options().prefetch.load();
    plan->prefetch_dist = pf >= 0 ? static_cast<int>(std::min<int64_t>(pf, 64)) : 0;
  }
  // Split K: one matrix product whose output tiles fill at most half of the SMs (weight gradients: small M and
  // N, K = the token count; the small f32 product), or whose last wave is mostly empty while K is very long.  The K
  // ranges run as the batches of the same kernel into fp32 partials in scratch; nova_splitk_reduce_kernel adds them in
  // range order and applies init / activation / rounding exactly once.  Results differ from the unsplit product in the
  // last bits (the fp32 additions associate differently); option "split_k": -1 = this rule, 0 = never, n >= 2 = n ranges.
  {
    const int64_t opt = options().split_k.load();
    const int64_t stage_k = pi.block_k;
    const int64_t kb = (a->K + stage_k - 1) / stage_k;
    const int64_t tiles = pi.tiles;
    int64_t want = 1;
    const bool batched_ok = a->batch == 1 || (a->init != NOVA_B200_INIT_LN_FOLD && a->batch_stride_c > 0);
    if (allow_split_k && opt != 0 && batched_ok && !pair && both_tma && tiles > 0) {
      if (opt >= 2) want = opt;
      else if (tiles * 2 <= sms && kb >= 16) want = std::min<int64_t>(8, sms / tiles);
      else if (kb >= 256 && tiles < 4 * sms) {
        const double eff1 = static_cast<double>(tiles) / (waves(tiles, sms) * sms);
        if (eff1 < 0.72) {
          double best = eff1 + 0.1;
          for (int64_t sp = 2; sp <= 4; ++sp) {
            const double e = static_cast<double>(tiles * sp) / (waves(tiles * sp, sms) * sms);
            if (e > best) { best = e; want = sp; }
          }
        }
      }
      // f32 through 3xTF32: the tensor core adds every product group into its fp32 accumulator with truncation, a bias
      // that grows with the length of the chain (measured against float64: ~2.3e-9 x K with the small terms in their
      // own accumulator, ~7e-9 x K before that; cuBLAS fp32 stays at 3-8e-7).  Ranges of at most 2048 keep one chain
      // under 5e-6; the partials are then added with rounding.
      if (opt < 0 && plan->terms == 3) want = std::max<int64_t>(want, (a->K + 2047) / 2048);
    }
    int64_t sp = std::min<int64_t>(want, 64);
    while (sp > 1 && (kb + sp - 1) / sp < 4) --sp;   // at least four k-blocks per range
    int64_t kb_per = sp > 1 ? (kb + sp - 1) / sp : kb;
    if (sp > 1) sp = (kb + kb_per - 1) / kb_per;      // ranges of kb_per k-blocks; the last may be shorter (zeros past K)
    if (sp > 1) {
      plan->split_k = static_cast<int>(sp);
      plan->split_len = kb_per * stage_k;
      plan->split_ldp = (a->N + 3) & ~3ll;
      plan->split_offset = (pi.scratch_bytes + 255) / 256 * 256;
      pi.scratch_bytes = plan->split_offset + a->batch * sp * a->M * plan->split_ldp * 4;
      pi.tiles = tiles * sp;
      pi.grid = static_cast<int32_t>(pi.tiles < sms ? pi.tiles : sms);
      pi.store_c = 0;  // the kernel writes the aligned partials; the reduce kernel writes C
    }
  }
  return NOVA_B200_OK;
}

// rows x cols matrix with `cols` contiguous, pitch ld, `nb` batches `bstride` elements apart.
int32_t encode_operand_map(DeviceContext* ctx, CUtensorMap* out, const void* base, int es, CUtensorMapDataType dt,
                           int64_t rows, int64_t cols, int64_t ld, int64_t nb, int64_t bstride, uint32_t box_inner,
                           uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(nb)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * es,
                           nb > 1 ? static_cast<cuuint64_t>(bstride) * es : static_cast<cuuint64_t>(rows) * ld * es};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = ctx->encode_tiled(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(NOVA_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(r));
  return NOVA_B200_OK;
}

// Launch with programmatic stream serialization when asked: the kernels call griddepcontrol.wait before their
// first global access, so letting their prologue (barrier setup, tensor-memory allocation) overlap the tail of
// the previous kernel in the stream is always safe.
template <typename Kernel, typename... Args>
int32_t launch_ex(Kernel kernel, int grid, int threads, size_t smem, cudaStream_t st, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl ? 1 : 0;
  NOVA_CUDA_OK(cudaLaunchKernelEx(&cfg, kernel, args...));
  return NOVA_B200_OK;
}

template <int kBlockN, int kElemBytes, int kTerms, bool kAMn, bool kBMn, int kStages, bool kLoader, int kEpiWarps>
int32_t launch_instance(const CUtensorMap* maps, const GemmKernelParams& p, int grid, cudaStream_t st, bool pdl) {
  using L = GemmSmemLayout<kBlockN, (kTerms == 3 ? 2 : 1), kStages, kEpiWarps>;
  auto kernel = nova_gemm_sm100_kernel<kBlockN, kElemBytes, kTerms, kAMn, kBMn, kStages, kLoader, kEpiWarps>;
  static thread_local int configured_device = -1;
  int dev = 0;
  NOVA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    NOVA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
    configured_device = dev;
  }
  constexpr int kThreads = kLoader ? kThreadsWithLoader : 32 * (kFirstEpilogueWarp + kEpiWarps);
  return launch_ex(kernel, grid, kThreads, L::kDynamicBytes, st, pdl, maps[0], maps[1], maps[2], maps[3], maps[4], p);
}

template <int kBlockN, int kElemBytes, int kTerms, int kStages, bool kLoader, int kEpiWarps>
int32_t launch_majors(bool a_mn, bool b_mn, const CUtensorMap* maps, const GemmKernelParams& p, int grid,
                      cudaStream_t st, bool pdl) {
  if (!a_mn && b_mn)
    return launch_instance<kBlockN, kElemBytes, kTerms, false, true, kStages, kLoader, kEpiWarps>(maps, p, grid, st, pdl);
  if (!a_mn && !b_mn)
    return launch_instance<kBlockN, kElemBytes, kTerms, false, false, kStages, kLoader, kEpiWarps>(maps, p, grid, st, pdl);
  if (a_mn && b_mn)
    return launch_instance<kBlockN, kElemBytes, kTerms, true, true, kStages, kLoader, kEpiWarps>(maps, p, grid, st, pdl);
  return launch_instance<kBlockN, kElemBytes, kTerms, true, false, kStages, kLoader, kEpiWarps>(maps, p, grid, st, pdl);
}

// the loader-warp build only exists for the single-term kernels (the 3xTF32 split re-lays its operands out)
template <int kBlockN, int kElemBytes, int kStages>
int32_t launch_single_term(bool loader, bool a_mn, bool b_mn, const CUtensorMap* maps, const GemmKernelParams& p,
                           int grid, cudaStream_t st, bool pdl) {
  if (loader) return launch_majors<kBlockN, kElemBytes, 1, kStages, true, 4>(a_mn, b_mn, maps, p, grid, st, pdl);
  return launch_majors<kBlockN, kElemBytes, 1, kStages, false, 4>(a_mn, b_mn, maps, p, grid, st, pdl);
}

template <int kElemBytes, bool kAMn, bool kBMn, int kEpiWarps>
int32_t launch_pair_instance(const CUtensorMap* maps, const GemmKernelParams& p, int sm_count, cudaStream_t st, bool pdl) {
  constexpr int kThreads = 32 * (kFirstEpilogueWarp + kEpiWarps);
  using PairSmem = PairSmemLayout<kEpiWarps>;
  auto kernel = nova_gemm_sm100_pair_kernel<kElemBytes, kAMn, kBMn, kEpiWarps>;
  static thread_local int configured_device = -1;
  static thread_local int max_pairs = 0;
  int dev = 0;
  NOVA_CUDA_OK(cudaGetDevice(&dev));
  if (configured_device != dev) {
    NOVA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kDynamicBytes));
    // how many 2-CTA clusters of this kernel can be resident at once (GPCs with an odd SM count strand one SM)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count & ~1), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = PairSmem::kDynamicBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count / 2;
    }
    max_pairs = n < sm_count / 2 ? n : sm_count / 2;
    if (options().debug.load()) fprintf(stderr, "[nova_b200] pair kernel: %d resident clusters reported, using %d\n", n, max_pairs);
    configured_device = dev;
  }
  const int pairs = p.tiles < max_pairs ? p.tiles : max_pairs;
  return launch_ex(kernel, 2 * pairs, kThreads, PairSmem::kDynamicBytes, st, pdl, maps[0], maps[1], maps[2], p);
}

template <int kElemBytes, int kEpiWarps>
int32_t launch_pair_majors(bool a_mn, bool b_mn, const CUtensorMap* maps, const GemmKernelParams& p, int sm_count,
                           cudaStream_t st, bool pdl) {
  if (!a_mn && b_mn) return launch_pair_instance<kElemBytes, false, true, kEpiWarps>(maps, p, sm_count, st, pdl);
  if (!a_mn && !b_mn) return launch_pair_instance<kElemBytes, false, false, kEpiWarps>(maps, p, sm_count, st, pdl);
  if (a_mn && b_mn) return launch_pair_instance<kElemBytes, true, true, kEpiWarps>(maps, p, sm_count, st, pdl);
  return launch_pair_instance<kElemBytes, true, false, kEpiWarps>(maps, p, sm_count, st, pdl);
}

// Everything a launch needs, derived from the argument struct.  Building it costs a plan, up to five
// cuTensorMapEncodeTiled calls and the descriptor arithmetic (several microseconds, more than the kernel of a small
// contraction), so the last few are kept per host thread and reused while the arguments (pointers included), the
// device, the tuning options and the scratch buffer are the same.
struct Prepared {
  nova_b200_gemm_args key{};
  const void* key_status = nullptr;  // identifies the device context
  const void* key_scratch = nullptr;
  uint32_t key_epoch = 0;
  bool key_allow_split = true;
  uint32_t key_presplit = 0;
  bool valid = false;
  Plan plan;
  GemmKernelParams p{};
  CUtensorMap maps[5];
  int pre_kernel = 0;  // 0 none, 1 hi/lo split, 2 re-pitch
  SplitOperand split_a{}, split_b{};
  RepitchOperand rep_a{}, rep_b{};
  int pre_blocks = 0;
  SplitKReduce splitk{};
};
constexpr int kPlanCacheEntries = 32;

int32_t prepare(DeviceContext* ctx, const nova_b200_gemm_args* a, void* scratch, Prepared* out) {
  Plan& plan = out->plan;
  const nova_b200_gemm_plan_info& pi = plan.info;
  GemmKernelParams& p = out->p;
  p = GemmKernelParams{};
  p.M = static_cast<int32_t>(a->M); p.N = static_cast<int32_t>(a->N); p.K = static_cast<int32_t>(a->K);
  p.batch = static_cast<int32_t>(a->batch);
  p.C = a->C; p.bias = a->bias; p.residual = a->residual;
  p.ldc = a->ldc; p.stride_c = a->batch_stride_c; p.ldr = a->ldr; p.stride_r = a->batch_stride_r;
  p.act = a->act; p.init = a->init; p.out_dtype = a->dtype_c;
  p.status = ctx->status_word;
  out->pre_kernel = 0;
  if (plan.k_zero) return NOVA_B200_OK;

  int32_t st = NOVA_B200_OK;
  const int es = plan.elem_bytes;
  const int block_n = pi.block_n;
  const int block_k = pi.block_k;
  const int block_m = pi.block_m;  // 128, or 256 for a CTA pair
  p.m_blocks = static_cast<int32_t>((a->M + block_m - 1) / block_m);
  p.n_blocks = static_cast<int32_t>((a->N + block_n - 1) / block_n);
  const int stage_k = plan.pair ? block_k * kPairSubK : block_k;  // K elements consumed per ring stage
  p.k_blocks = static_cast<int32_t>((a->K + stage_k - 1) / stage_k);
  p.group_m = static_cast<int32_t>(options().group_m.load());
  if (p.group_m < 1) p.group_m = 1;
  p.tiles = static_cast<int32_t>(pi.tiles);
  p.a_batch_mul = a->batch_stride_a == 0 ? 0 : 1;
  p.b_batch_mul = a->batch_stride_b == 0 ? 0 : 1;
  p.loader_a = pi.loader_a == 1 ? 1 : 0; p.loader_b = pi.loader_b == 1 ? 1 : 0;
  p.A = a->A; p.B = a->B; p.lda = a->lda; p.ldb = a->ldb;
  p.stride_a = a->batch_stride_a; p.stride_b = a->batch_stride_b;
  p.vec_store = pi.store_c == 0 ? 1 : 0;
  p.prefetch_dist = plan.prefetch_dist;

  // tcgen05 instruction descriptor: D=f32 (bits 4-5 = 1), A/B format (bits 7-9 / 10-12: f16=0, bf16=1, tf32=2),
  // A/B major (bits 15/16: 1 = MN-major), N>>3 in bits 17-22, M>>4 in bits 24-28.
  const uint32_t fmt = a->dtype_ab == NOVA_B200_F16 ? 0u : (a->dtype_ab == NOVA_B200_BF16 ? 1u : 2u);
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((plan.a_mn ? 1u : 0u) << 15) | ((plan.b_mn ? 1u : 0u) << 16) |
            (static_cast<uint32_t>(block_n >> 3) << 17) | (static_cast<uint32_t>(block_m >> 4) << 24);
  // Shared-memory matrix descriptors (128-byte swizzle, version 1):
  //   K-major : rows of 128 B, 8-row groups 1024 B apart (SBO); LBO unused; one UMMA K step = 32 B.
  //   MN-major: 128 B = one chunk of MN elements for one k; 8 k-rows = 1024 B (SBO); the next chunk of
  //             MN elements starts BLOCK_K*128 B further (LBO); one UMMA K step = UMMA_K*128 B.
  //   MN-major 32-bit (tf32) operands exist only in the 128-byte swizzle with 32-byte atoms (layout type 1,
  //             the tensor map's SWIZZLE_128B_ATOM_32B): its pattern repeats every 4 k-rows, so SBO = 512 B.
  const uint32_t umma_k = 32u / es;
  const uint32_t lbo_mn = static_cast<uint32_t>(block_k) * kSwizzleBytes;
  auto desc_hi = [&](bool mn) {
    const bool atom32 = mn && es == 4;
    const uint32_t sbo = atom32 ? 512u : 1024u;
    return ((sbo >> 4) & 0x3fffu) | (1u << 14) | ((atom32 ? 1u : 2u) << 29);  // SBO | version 1 | layout type
  };
  p.a_desc_hi = desc_hi(plan.a_mn);
  p.b_desc_hi = desc_hi(plan.b_mn);
  p.a_desc_lbo = (plan.a_mn ? ((lbo_mn >> 4) & 0x3fffu) : 1u) << 16;
  p.b_desc_lbo = (plan.b_mn ? ((lbo_mn >> 4) & 0x3fffu) : 1u) << 16;
  p.a_kstep = plan.a_mn ? umma_k * kSwizzleBytes : 32u;
  p.b_kstep = plan.b_mn ? umma_k * kSwizzleBytes : 32u;

  // operand views (possibly redirected to scratch: the hi/lo split of f32 operands, re-pitched copies)
  const int64_t a_rows = a->trans_a ? a->K : a->M, a_cols = a->trans_a ? a->M : a->K;
  const int64_t b_rows = a->trans_b ? a->N : a->K, b_cols = a->trans_b ? a->K : a->N;
  const int64_t a_nb = a->batch_stride_a == 0 ? 1 : a->batch, b_nb = a->batch_stride_b == 0 ? 1 : a->batch;
  const void* a_src[2] = {a->A, nullptr};
  const void* b_src[2] = {a->B, nullptr};
  int64_t a_ld = a->lda, b_ld = a->ldb, a_bs = a->batch_stride_a, b_bs = a->batch_stride_b;
  if (plan.terms == 3) {
    const int64_t a_ldo = (a_cols + 3) & ~3ll, b_ldo = (b_cols + 3) & ~3ll;
    float* s = static_cast<float*>(scratch);
    float* a_hi = s; float* a_lo = a_hi + a_nb * a_rows * a_ldo;
    float* b_hi = a_lo + a_nb * a_rows * a_ldo; float* b_lo = b_hi + b_nb * b_rows * b_ldo;
    out->split_a = SplitOperand{static_cast<const float*>(a->A), a_hi, a_lo, a_nb * a_rows, a->lda, a->batch_stride_a,
                                static_cast<int32_t>(a_rows), static_cast<int32_t>(a_cols), static_cast<int32_t>(a_ldo)};
    out->split_b = SplitOperand{static_cast<const float*>(a->B), b_hi, b_lo, b_nb * b_rows, a->ldb, a->batch_stride_b,
                                static_cast<int32_t>(b_rows), static_cast<int32_t>(b_cols), static_cast<int32_t>(b_ldo)};
    const int64_t biggest = std::max(a_nb * a_rows * a_ldo, b_nb * b_rows * b_ldo);
    const int64_t want = (biggest / 4 + 255) / 256;  // four elements per thread
    out->pre_blocks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, ctx->sm_count * 8)));
    out->pre_kernel = 1;
    a_src[0] = a_hi; a_src[1] = a_lo; b_src[0] = b_hi; b_src[1] = b_lo;
    a_ld = a_ldo; b_ld = b_ldo; a_bs = a_rows * a_ldo; b_bs = b_rows * b_ldo;
    // an operand the caller had split in advance: read those halves, skip its half of the split pass
    if (a->batch == 1) {
      std::lock_guard<std::mutex> lock(ctx->presplit_mu);
      for (const DeviceContext::PreSplit& e : ctx->presplit) {
        if (e.x == a->A && e.rows == a_rows && e.cols == a_cols && e.ld == a->lda) {
          a_src[0] = e.hi; a_src[1] = e.lo; a_ld = e.ld_out; a_bs = a_rows * a_ld;
          out->split_a.rows_total = 0;
        }
        if (e.x == a->B && e.rows == b_rows && e.cols == b_cols && e.ld == a->ldb) {
          b_src[0] = e.hi; b_src[1] = e.lo; b_ld = e.ld_out; b_bs = b_rows * b_ld;
          out->split_b.rows_total = 0;
        }
      }
      if (out->split_a.rows_total == 0 && out->split_b.rows_total == 0) out->pre_kernel = 0;
    }
  } else if (plan.repitch_a_ld > 0 || plan.repitch_b_ld > 0) {
    uint8_t* s = static_cast<uint8_t*>(scratch);
    out->rep_a = RepitchOperand{};
    out->rep_b = RepitchOperand{};
    int64_t biggest = 0;
    if (plan.repitch_a_ld > 0) {
      out->rep_a = RepitchOperand{a->A, s, a_nb * a_rows, a->lda, a->batch_stride_a, static_cast<int32_t>(a_rows),
                                  static_cast<int32_t>(a_cols), static_cast<int32_t>(plan.repitch_a_ld)};
      a_src[0] = s; a_ld = plan.repitch_a_ld; a_bs = a_rows * a_ld;
      s += (a_nb * a_rows * a_ld * es + 255) / 256 * 256;
      biggest = std::max(biggest, a_nb * a_rows * a_ld * es / 16);
    }
    if (plan.repitch_b_ld > 0) {
      out->rep_b = RepitchOperand{a->B, s, b_nb * b_rows, a->ldb, a->batch_stride_b, static_cast<int32_t>(b_rows),
                                  static_cast<int32_t>(b_cols), static_cast<int32_t>(plan.repitch_b_ld)};
      b_src[0] = s; b_ld = plan.repitch_b_ld; b_bs = b_rows * b_ld;
      biggest = std::max(biggest, b_nb * b_rows * b_ld * es / 16);
    }
    const int64_t want = (biggest + 255) / 256;
    out->pre_blocks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, ctx->sm_count * 16)));
    out->pre_kernel = 2;
  }

  // Split K: range s of K becomes "batch" s of the launch: the producer adds s * split_len to its K coordinate, the
  // tensor maps of A and B stay those of the whole matrices (so a last range that runs past K reads zeros); the
  // output is the fp32 partial [s, M, ldp] in scratch, written with no init and no activation.
  int64_t a_rows_v = a_rows, a_cols_v = a_cols, b_rows_v = b_rows, b_cols_v = b_cols, a_nb_v = a_nb, b_nb_v = b_nb;
  out->splitk = SplitKReduce{};
  if (plan.split_k > 1) {
    const int64_t sp = plan.split_k;
    p.split_k_len = static_cast<int32_t>(plan.split_len);
    p.split_k_ranges = static_cast<int32_t>(sp);
    p.k_blocks = static_cast<int32_t>(plan.split_len / stage_k);
    p.batch = static_cast<int32_t>(a->batch * sp);
    float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + plan.split_offset);
    out->splitk = SplitKReduce{partial, a->C, a->bias, a->residual, a->M, a->N, plan.split_ldp, a->ldc, a->ldr,
                               a->batch, a->batch_stride_c, a->batch_stride_r,
                               static_cast<int32_t>(sp), a->init, a->act, a->dtype_c};
    p.C = partial; p.ldc = plan.split_ldp; p.stride_c = a->M * plan.split_ldp;
    p.bias = nullptr; p.residual = nullptr; p.init = NOVA_B200_INIT_ZERO; p.act = NOVA_B200_ACT_NONE;
    p.out_dtype = NOVA_B200_F32;
    p.vec_store = 1;
  }

  CUtensorMap* maps = out->maps;  // A hi, A lo, B hi, B lo, C
  std::memset(maps, 0, sizeof(out->maps));
  const CUtensorMapDataType tdt = a->dtype_ab == NOVA_B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                : a->dtype_ab == NOVA_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const uint32_t chunk = static_cast<uint32_t>(block_k);  // 128 B of elements
  auto swizzle_for = [&](bool mn) {
    return mn && es == 4 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
  };
  for (int t = 0; t < (plan.terms == 3 ? 2 : 1); ++t) {
    if (pi.loader_a != 1) {
      st = encode_operand_map(ctx, &maps[t], a_src[t], es, tdt, a_rows_v, a_cols_v, a_ld, a_nb_v, a_bs, chunk,
                              plan.a_mn ? static_cast<uint32_t>(block_k) : static_cast<uint32_t>(kBlockM),
                              swizzle_for(plan.a_mn));
      if (st != NOVA_B200_OK) return st;
    }
    if (pi.loader_b != 1) {
      st = encode_operand_map(ctx, &maps[2 + t], b_src[t], es, tdt, b_rows_v, b_cols_v, b_ld, b_nb_v, b_bs, chunk,
                              plan.b_mn ? static_cast<uint32_t>(block_k)
                                        : static_cast<uint32_t>(plan.pair ? block_n / 2 : block_n),  // a pair CTA loads half of N
                              swizzle_for(plan.b_mn));
      if (st != NOVA_B200_OK) return st;
    }
  }
  if (p.vec_store && plan.split_k > 1) {
    // (columns N .. ldp of a partial row may be written by the last 16-byte chunk: they are padding)
    st = encode_operand_map(ctx, &maps[4], p.C, 4, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a->M, plan.split_ldp, plan.split_ldp,
                            a->batch * plan.split_k, a->M * plan.split_ldp, static_cast<uint32_t>(kSwizzleBytes / 4), 32u,
                            CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != NOVA_B200_OK) return st;
  } else if (p.vec_store) {
    // output boxes: 32 rows x 128 bytes, clipped by the tensor map at M and N
    const int osz = plan.out_bytes;
    const CUtensorMapDataType cdt = a->dtype_c == NOVA_B200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                  : a->dtype_c == NOVA_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    st = encode_operand_map(ctx, &maps[4], a->C, osz, cdt, a->M, a->N, a->ldc, a->batch, a->batch_stride_c,
                            static_cast<uint32_t>(kSwizzleBytes / osz), 32u, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st != NOVA_B200_OK) return st;
  }
  return NOVA_B200_OK;
}

}  // namespace

// One operand copied to a 16-byte-aligned pitch (the copy nova_b200_operand_prepare keeps for a constant weight).
int32_t repitch_launch(const void* src, void* dst, int es, int64_t batch, int64_t rows, int64_t cols, int64_t ld_in,
                       int64_t stride_in, int64_t ld_out, int sm_count, cudaStream_t stream) {
  RepitchOperand o{src, dst, batch * rows, ld_in, stride_in, static_cast<int32_t>(rows), static_cast<int32_t>(cols),
                   static_cast<int32_t>(ld_out)};
  RepitchOperand none{};
  const int64_t want = (batch * rows * ld_out * es / 16 + 255) / 256;
  const int blocks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, static_cast<int64_t>(sm_count) * 16)));
  if (es == 2) nova_repitch_kernel<uint16_t><<<dim3(blocks, 1), 256, 0, stream>>>(o, none);
  else nova_repitch_kernel<uint32_t><<<dim3(blocks, 1), 256, 0, stream>>>(o, none);
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

// hi = rna-tf32(x), lo = x - hi of one f32 matrix into [rows, ld_out] buffers (nova_b200_f32_presplit).
int32_t split_launch(const float* x, float* hi, float* lo, int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                     int sm_count, cudaStream_t stream) {
  SplitOperand o{x, hi, lo, rows, ld_in, 0, static_cast<int32_t>(rows), static_cast<int32_t>(cols), static_cast<int32_t>(ld_out)};
  SplitOperand none{};
  const int64_t want = (rows * ld_out / 4 + 255) / 256;
  const int blocks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(want, static_cast<int64_t>(sm_count) * 8)));
  nova_split_tf32_kernel<<<dim3(blocks, 1), 256, 0, stream>>>(o, none);
  NOVA_CUDA_OK(cudaGetLastError());
  return NOVA_B200_OK;
}

int32_t gemm_plan_only(const nova_b200_gemm_args* args, nova_b200_gemm_plan_info* out, bool allow_split_k) {
  Plan plan;
  int sm = 148;  // the plan a B200 will execute; needs no device
  int32_t st = validate_and_plan(args, &plan, sm, allow_split_k);
  if (st != NOVA_B200_OK) return st;
  if (out) *out = plan.info;
  return NOVA_B200_OK;
}

int32_t gemm_launch(DeviceContext* ctx, const nova_b200_gemm_args* a, cudaStream_t stream, void* const* peers,
                    int32_t n_peers) {
  static thread_local Prepared cache[kPlanCacheEntries];
  static thread_local int next_slot = 0;
  if (!a || a->struct_size != sizeof(nova_b200_gemm_args)) {
    Plan tmp;
    return validate_and_plan(a, &tmp, ctx->sm_count);  // reports the argument error
  }
  Options& opt = options();
  const uint32_t epoch = opt.epoch.load();
  const bool use_cache = opt.plan_cache.load() != 0;
  // (the push epilogue stores finished boxes of C; a K-split product finishes in the reduce kernel: never split those)
  // (nor with the fixed scratch of the no-allocation entry point, whose size is promised in terms of A and B alone)
  const bool allow_split = n_peers == 0 && ctx->fixed_scratch == nullptr;
  uint32_t presplit_version;
  {
    std::lock_guard<std::mutex> lock(ctx->presplit_mu);
    presplit_version = ctx->presplit_version;
  }
  Prepared* hit = nullptr;
  if (use_cache) {
    for (int i = 0; i < kPlanCacheEntries; ++i) {
      Prepared& c = cache[i];
      if (c.valid && c.key_status == ctx->status_word && c.key_epoch == epoch && c.key_allow_split == allow_split &&
          c.key_presplit == presplit_version &&
          std::memcmp(&c.key, a, sizeof(nova_b200_gemm_args)) == 0) {
        hit = &c;
        break;
      }
    }
  }
  Prepared local;
  Prepared* pr = hit;
  int32_t st = NOVA_B200_OK;
  if (!pr) {
    pr = use_cache ? &cache[next_slot] : &local;
    pr->valid = false;
    pr->plan = Plan{};
    st = validate_and_plan(a, &pr->plan, ctx->sm_count, allow_split);
    if (st != NOVA_B200_OK) return st;
  }
  const Plan& plan = pr->plan;
  if (plan.empty) return NOVA_B200_OK;
  const nova_b200_gemm_plan_info& pi = plan.info;
  if (!hit) {  // (a hit has the same pointers on the same device: already checked)
    for (const void* ptr : {a->A, a->B, static_cast<const void*>(a->C)}) {
      st = check_pointer_device(ctx, ptr, "gemm: an operand");
      if (st != NOVA_B200_OK) return st;
    }
  }
  void* scratch = nullptr;
  if (pi.scratch_bytes > 0 && !plan.k_zero) {
    st = acquire_scratch(ctx, stream, static_cast<size_t>(pi.scratch_bytes), &scratch);
    if (st != NOVA_B200_OK) return st;
  }
  if (!hit || pr->key_scratch != scratch) {
    pr->valid = false;
    st = prepare(ctx, a, scratch, pr);
    if (st != NOVA_B200_OK) return st;
    pr->key = *a;
    pr->key_status = ctx->status_word;
    pr->key_scratch = scratch;
    pr->key_epoch = epoch;
    pr->key_allow_split = allow_split;
    pr->key_presplit = presplit_version;
    pr->valid = true;
    if (!hit && use_cache) next_slot = (next_slot + 1) % kPlanCacheEntries;
  }
  GemmKernelParams pushed;
  if (n_peers > 0) {
    // every output box also goes to the peers: needs the TMA-store epilogue (aligned C) and whole 16-byte chunks
    if (plan.k_zero || pi.store_c != 0 || (a->N * plan.out_bytes) % 16 != 0)
      return fail(NOVA_B200_ERR_LAYOUT, "gemm_push: C must be 16-byte aligned (base, pitch, batch stride), N * element size a multiple of 16, K > 0");
    if (n_peers > kMaxPushPeers || !peers) return fail(NOVA_B200_ERR_INVALID_ARG, "gemm_push: at most 7 peers");
    pushed = pr->p;
    pushed.n_peers = n_peers;
    for (int i = 0; i < n_peers; ++i) {
      if (!peers[i] || reinterpret_cast<uintptr_t>(peers[i]) % 16 != 0)
        return fail(NOVA_B200_ERR_INVALID_ARG, "gemm_push: a peer pointer is null or not 16-byte aligned");
      pushed.peer_c[i] = peers[i];
    }
  }
  const GemmKernelParams& p = n_peers > 0 ? pushed : pr->p;
  const CUtensorMap* maps = pr->maps;
  const bool pdl = opt.pdl.load() != 0;

  if (plan.k_zero) {
    const int64_t n = a->batch * a->M * a->N;
    const int grid = static_cast<int>(n / 256 + 1 < 148 * 8 ? n / 256 + 1 : 148 * 8);
    if (a->dtype_c == NOVA_B200_BF16) nova_gemm_k0_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
    else if (a->dtype_c == NOVA_B200_F16) nova_gemm_k0_kernel<__half><<<grid, 256, 0, stream>>>(p);
    else nova_gemm_k0_kernel<float><<<grid, 256, 0, stream>>>(p);
    NOVA_CUDA_OK(cudaGetLastError());
    return NOVA_B200_OK;
  }
  const int es = plan.elem_bytes;
  if (pr->pre_kernel == 1) {
    nova_split_tf32_kernel<<<dim3(pr->pre_blocks, 2), 256, 0, stream>>>(pr->split_a, pr->split_b);
    NOVA_CUDA_OK(cudaGetLastError());
  } else if (pr->pre_kernel == 2) {
    if (es == 2) nova_repitch_kernel<uint16_t><<<dim3(pr->pre_blocks, 2), 256, 0, stream>>>(pr->rep_a, pr->rep_b);
    else nova_repitch_kernel<uint32_t><<<dim3(pr->pre_blocks, 2), 256, 0, stream>>>(pr->rep_a, pr->rep_b);
    NOVA_CUDA_OK(cudaGetLastError());
  }

  const int block_n = pi.block_n;
  if (plan.pair) {
    const CUtensorMap pm[3] = {maps[0], maps[2], maps[4]};
    // NOVA_B200_TRACE=<file> (diagnostic builds only): the launch is synchronous and every CTA's role timeline
    // (clock64 samples, see TraceSlot) is written to the file as int64[grid][kTraceTiles][kTraceSlots].
    const char* trace_path = kTraceEnabled ? std::getenv("NOVA_B200_TRACE") : nullptr;
    const size_t trace_bytes = sizeof(long long) * pi.grid * kTraceTiles * kTraceSlots;
    GemmKernelParams pt = p;
    if (trace_path != nullptr) {
      NOVA_CUDA_OK(cudaMalloc(&pt.trace, trace_bytes));
      NOVA_CUDA_OK(cudaMemsetAsync(pt.trace, 0, trace_bytes, stream));
    }
    st = es == 2 ? launch_pair_majors<2, kPairEpilogueWarps>(plan.a_mn, plan.b_mn, pm, pt, ctx->sm_count, stream, pdl)
                 : launch_pair_majors<4, kPairEpilogueWarps>(plan.a_mn, plan.b_mn, pm, pt, ctx->sm_count, stream, pdl);
    if (trace_path != nullptr) {
      std::vector<long long> host(trace_bytes / sizeof(long long));
      cudaStreamSynchronize(stream);
      cudaMemcpy(host.data(), pt.trace, trace_bytes, cudaMemcpyDeviceToHost);
      cudaFree(pt.trace);
      if (FILE* f = std::fopen(trace_path, "wb")) {
        std::fwrite(host.data(), 1, trace_bytes, f);
        std::fclose(f);
      }
    }
    return st;
  }
  const bool loader = pi.loader_a == 1 || pi.loader_b == 1;
  const int grid = pi.grid;
  auto launch_single_cta = [&]() -> int32_t {
    if (plan.terms == 3) {
      if (block_n == 64) return launch_majors<64, 4, 3, 4, false, 4>(plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
      return launch_majors<128, 4, 3, 3, false, 4>(plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
    }
    if (block_n == 64) {  // TMA-only build: narrow tiles are chosen only for operands tensor maps can describe
      if (es == 2) return launch_majors<64, 2, 1, 8, false, 4>(plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
      return launch_majors<64, 4, 1, 8, false, 4>(plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
    }
    if (plan.short_k) {  // 256-wide tiles, three stages, eight epilogue warps
      if (es == 2) return launch_majors<256, 2, 1, 3, false, 8>(plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
      return launch_majors<256, 4, 1, 3, false, 8>(plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
    }
    if (es == 2) {
      if (block_n == 256) return launch_single_term<256, 2, 4>(loader, plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
      return launch_single_term<128, 2, 6>(loader, plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
    }
    if (block_n == 256) return launch_single_term<256, 4, 4>(loader, plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
    return launch_single_term<128, 4, 6>(loader, plan.a_mn, plan.b_mn, maps, p, grid, stream, pdl);
  };
  st = launch_single_cta();
  if (st != NOVA_B200_OK || plan.split_k <= 1) return st;
  {
    const SplitKReduce& r = pr->splitk;
    cudaLaunchConfig_t cfg = {};
    const int64_t want = (r.batch * r.M * (r.ldp / 4) + 255) / 256;
    cfg.gridDim = dim3(static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>(want, ctx->sm_count * 8))), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl ? 1 : 0;
    if (r.out_dtype == NOVA_B200_BF16) NOVA_CUDA_OK(cudaLaunchKernelEx(&cfg, nova_splitk_reduce_kernel<__nv_bfloat16>, r));
    else if (r.out_dtype == NOVA_B200_F16) NOVA_CUDA_OK(cudaLaunchKernelEx(&cfg, nova_splitk_reduce_kernel<__half>, r));
    else NOVA_CUDA_OK(cudaLaunchKernelEx(&cfg, nova_splitk_reduce_kernel<float>, r));
  }
  return NOVA_B200_OK;
}

}  // namespace nova
