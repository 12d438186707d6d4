// Internal declarations shared by the translation units of libnova_b200.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <string>

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

static constexpr int kHostChunks = 8;   // pipeline depth of the *_host entry points

// Per-device state.  One instance per CUDA device the process touched through this library.
struct DeviceContext {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  uint32_t* status_word = nullptr;  // device memory, 4 bytes (+ padding)
  void* scratch = nullptr;          // hi/lo split buffers for the 3xTF32 path
  size_t scratch_bytes = 0;
  void* staging = nullptr;          // device staging for the *_host entry points
  size_t staging_bytes = 0;
  EncodeTiledFn encode_tiled = nullptr;
  // the *_host entry points pipeline H2D / kernel / D2H over three streams
  cudaStream_t s_in = nullptr, s_comp = nullptr, s_out = nullptr;
  cudaEvent_t ev_in[kHostChunks] = {}, ev_comp[kHostChunks] = {};
  std::mutex mu;       // guards scratch
  std::mutex host_mu;  // guards staging (the *_host entry points)
};

void set_error(const std::string& msg);
int32_t fail(nova_b200_status st, const std::string& msg);
// Returns the context of the current device, initialising it on first use; nullptr + error on failure.
DeviceContext* current_context(int32_t* status_out);
// Grows ctx->scratch to at least `bytes` (device-synchronising only when it has to reallocate).
int32_t ensure_scratch(DeviceContext* ctx, size_t bytes);
int32_t ensure_staging(DeviceContext* ctx, size_t bytes);
int32_t ensure_host_streams(DeviceContext* ctx);

inline int dtype_bytes(int32_t dt) {
  switch (dt) {
    case NOVA_B200_F32: case NOVA_B200_I32: return 4;
    case NOVA_B200_F16: case NOVA_B200_BF16: case NOVA_B200_I16: return 2;
    case NOVA_B200_I64: return 8;
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
