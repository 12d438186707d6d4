// Internal declarations shared by the translation units of libnova_b200.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/nova_b200.h"

namespace nova {

// Codes written to the device status word by bounded waits that gave up.
enum DeviceStatusCode : uint32_t {
  kStatusOk = 0,
  kStatusProducerEmptyWait = 0x101,   // TMA producer waiting for a free pipeline stage
  kStatusMmaFullWait = 0x102,         // MMA issuer waiting for operand bytes to land
  kStatusMmaTmemEmptyWait = 0x103,    // MMA issuer waiting for the epilogue to drain an accumulator
  kStatusEpilogueTmemFullWait = 0x104,// epilogue waiting for an accumulator to be complete
  kStatusLoaderEmptyWait = 0x105      // ld.global loader warps waiting for a free stage
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static constexpr int kHostChunks = 8;   // chunks per dimension of the *_host entry points
static constexpr int kHostEvents = kHostChunks * kHostChunks;  // one event pair per (row block, column slab) tile

// Per-device state.  One instance per CUDA device the process touched through this library.
struct DeviceContext {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  int device_count = 1;             // visible devices: pointer-ownership checks only run when > 1
  uint32_t* status_word = nullptr;  // device memory, 4 bytes (+ padding)
  // Scratch (hi/lo split of f32 operands, re-pitched operand copies, partial sums of the row kernels): one buffer
  // per STREAM, so calls on different streams never share scratch.  A buffer that has to grow is replaced, and
  // the old one is kept until nova_b200_shutdown because kernels already enqueued (or captured into a CUDA
  // graph) may still read it: growing never synchronises and never frees.
  struct ScratchBuf { void* ptr = nullptr; size_t bytes = 0; };
  std::map<cudaStream_t, ScratchBuf> scratch_by_stream;
  std::vector<void*> retired_scratch;
  // a caller-provided fixed scratch (the static-array entry point): used instead of the pool, never grown
  void* fixed_scratch = nullptr;
  size_t fixed_scratch_bytes = 0;
  void* staging = nullptr;          // device staging for the *_host entry points
  size_t staging_bytes = 0;
  EncodeTiledFn encode_tiled = nullptr;
  // the *_host entry points pipeline H2D / kernel / D2H over three streams
  cudaStream_t s_in = nullptr, s_comp = nullptr, s_out = nullptr;
  cudaEvent_t ev_in[kHostEvents] = {}, ev_comp[kHostEvents] = {};
  std::mutex mu;       // guards the scratch pool
  std::mutex host_mu;  // guards staging (the *_host entry points)
  // f32 matrices whose hi / lo halves (the 3xTF32 split) a caller asked to keep: a contraction that is given one of
  // them as an operand reads the halves instead of splitting it again (nova_b200_f32_presplit)
  struct PreSplit { const void* x; int64_t rows, cols, ld; float* hi; float* lo; int64_t ld_out; };
  std::vector<PreSplit> presplit;
  uint32_t presplit_version = 0;   // bumped by every change: cached launch descriptions are keyed on it
  std::mutex presplit_mu;
};

void set_error(const std::string& msg);
int32_t fail(nova_b200_status st, const std::string& msg);
// Returns the context of the current device, initialising it on first use; nullptr + error on failure.
DeviceContext* current_context(int32_t* status_out);
// Scratch of at least `bytes` for work enqueued on `stream` (see DeviceContext).  Allocates only when the stream's
// buffer is too small; refuses (NOVA_B200_ERR_CUDA) to allocate while `stream` is being captured.
int32_t acquire_scratch(DeviceContext* ctx, cudaStream_t stream, size_t bytes, void** out);
// NOVA_B200_ERR_INVALID_ARG when `p` is device memory of another device than the current one (only checked in
// processes that see more than one device).  `what` names the operand in the message.
int32_t check_pointer_device(const DeviceContext* ctx, const void* p, const char* what);

// Tuning switches.  Seeded once from the environment (NOVA_B200_<NAME>), changed with nova_b200_set_option.
struct Options {
  std::atomic<int64_t> repitch{1};    // unaligned operands: 1 = re-pitch copy + TMA, 0 = in-place loader warps
  std::atomic<int64_t> pair{-1};      // CTA-pair kernel: -1 = cost model, 0 = never, 1 = whenever legal
  std::atomic<int64_t> block_n{0};    // 0 = cost model, else 64 / 128 / 256
  std::atomic<int64_t> short_k{1};    // 8 epilogue warps for K <= 256
  std::atomic<int64_t> group_m{16};   // raster group height in row blocks
  std::atomic<int64_t> prefetch{-1};  // L2 prefetch distance of the pair kernel in ring stages: -1 = planner, 0 = off
  std::atomic<int64_t> ring_stages{0}; // ring depth of those kernels: 0 = chosen from the row size, else 2..8 (tuning)
  std::atomic<int64_t> ring_ctas{0};   // their CTAs per SM: 0 = as many as fit (tuning)
  std::atomic<int64_t> plan_cache{1}; // reuse plans and tensor maps of repeated calls
  std::atomic<int64_t> pdl{1};        // launch contractions with programmatic stream serialization
  std::atomic<int64_t> ring_rows{1};  // layer_norm (forward / backward) rows of a few KB through the shared-memory ring kernels
  std::atomic<int64_t> split_k{-1};   // K ranges of a product with few output tiles: -1 = planner, 0 = never, n >= 2 = n
  std::atomic<int64_t> host_tiles{0}; // host pipeline of one large product: 0 = built-in, -1 = row blocks only, else rows * 100 + cols
  std::atomic<int64_t> debug{0};
  std::atomic<uint32_t> epoch{0};     // bumped by every change: cached plans are keyed on it
};
Options& options();
int32_t ensure_staging(DeviceContext* ctx, size_t bytes);
int32_t ensure_host_streams(DeviceContext* ctx);

inline int dtype_bytes(int32_t dt) {
  switch (dt) {
    case NOVA_B200_F32: case NOVA_B200_I32: return 4;
    case NOVA_B200_F16: case NOVA_B200_BF16: case NOVA_B200_I16: return 2;
    case NOVA_B200_I64: return 8;
    case NOVA_B200_I1: return 1;
    default: return 0;
  }
}
inline bool init_has_bias(int32_t init) { return init == NOVA_B200_INIT_BIAS_ROW || init == NOVA_B200_INIT_BIAS_AND_RESIDUAL; }
inline bool init_has_residual(int32_t init) {
  return init == NOVA_B200_INIT_RESIDUAL_FULL || init == NOVA_B200_INIT_BIAS_AND_RESIDUAL;
}
// the residual pointer is read either as an addend or as the pre-activation of a fused nova.gelu_backward
inline bool reads_residual(int32_t init, int32_t act) { return init_has_residual(init) || act == NOVA_B200_ACT_GELU_TANH_GRAD; }
inline bool is_float_dtype(int32_t dt) { return dt == NOVA_B200_F32 || dt == NOVA_B200_F16 || dt == NOVA_B200_BF16; }

#define NOVA_CUDA_OK(expr)                                                                          \
  do {                                                                                              \
    cudaError_t e__ = (expr);                                                                       \
    if (e__ != cudaSuccess)                                                                         \
      return ::nova::fail(NOVA_B200_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__)); \
  } while (0)

}  // namespace nova
