// nova_b200_gemm_f32_static: the f32 (3xTF32) contraction for callers that cannot allocate device memory.
//
// Who this is for: code that runs where cudaMalloc is off limits — a compiled Nova graph invoked from
// inside a memory-planned region whose allocator has already handed out the whole device, a plug-in
// running under a host framework that forbids allocations on its streams, or a real-time loop that must
// not take the allocator's locks.  The regular f32 path (nova_b200_gemm) grows a per-device scratch
// buffer with cudaMalloc on first use and keeps its status word in allocated memory; this variant keeps
// both in one fixed array that is part of the library image, so nothing is ever allocated or freed.
//
// The price is a hard size limit and one shared buffer: see the notes on the entry point below.
#include <cstring>

#include "runtime.h"

namespace nova {
int32_t gemm_plan_only(const nova_b200_gemm_args* args, nova_b200_gemm_plan_info* out, bool allow_split_k = true);
int32_t gemm_launch(DeviceContext* ctx, const nova_b200_gemm_args* a, cudaStream_t stream, void* const* peers = nullptr,
                    int32_t n_peers = 0);
}  // namespace nova

namespace {

constexpr size_t kStatusBytes = 256;                     // status word + padding, keeps the scratch 256-byte aligned
constexpr size_t kScratchBytes = size_t(16) << 20;       // 16 MiB of hi/lo split buffers
constexpr int kMaxDevices = 64;

// Every GPU on which the library is loaded holds these 16 MiB + 256 B until the process exits.
// In host code this name is only a handle for cudaGetSymbolAddress — it is NOT a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStatusBytes + kScratchBytes];

struct StaticDevice {
  bool ready = false;
  unsigned char* base = nullptr;  // device address of g_static_scratch on this device
  int sm_count = 0;
  nova::EncodeTiledFn encode_tiled = nullptr;
};
StaticDevice g_devices[kMaxDevices];
std::mutex g_setup_mu;

// Once per device, with that device current: resolve the array's device address and the driver entry
// point, read the SM count.  Allocates nothing.
int32_t setup_device(int dev, StaticDevice** out) {
  if (dev < 0 || dev >= kMaxDevices) return nova::fail(NOVA_B200_ERR_INVALID_ARG, "gemm_f32_static: device index out of range");
  std::lock_guard<std::mutex> lock(g_setup_mu);
  StaticDevice& d = g_devices[dev];
  if (!d.ready) {
    cudaDeviceProp prop;
    NOVA_CUDA_OK(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      return nova::fail(NOVA_B200_ERR_NO_DEVICE, "gemm_f32_static: the current device is not compute capability 10.x");
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
      cudaGetLastError();
      return nova::fail(NOVA_B200_ERR_CUDA, "gemm_f32_static: cuTensorMapEncodeTiled is not available from this driver");
    }
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr) {
      cudaGetLastError();
      return nova::fail(NOVA_B200_ERR_CUDA, std::string("gemm_f32_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    }
    d.base = static_cast<unsigned char*>(ptr);
    d.sm_count = prop.multiProcessorCount;
    d.encode_tiled = reinterpret_cast<nova::EncodeTiledFn>(fn);
    d.ready = true;
  }
  *out = &d;
  return NOVA_B200_OK;
}

}  // namespace

namespace nova {
// For nova_b200_device_status: reads (and clears) the static array's status word on `dev` if this entry point has
// been used there, so a caller that only enqueues (wait_code_out == NULL) can still learn that a bounded wait gave
// up.  The caller has synchronised the device.  Allocates nothing.
int32_t static_scratch_status(int dev, uint32_t* code_out) {
  *code_out = 0;
  if (dev < 0 || dev >= kMaxDevices) return NOVA_B200_OK;
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mu);
    if (!g_devices[dev].ready) return NOVA_B200_OK;
    base = g_devices[dev].base;
  }
  uint32_t code = 0;
  NOVA_CUDA_OK(cudaMemcpy(&code, base, 4, cudaMemcpyDeviceToHost));
  if (code != 0) NOVA_CUDA_OK(cudaMemset(base, 0, 4));
  *code_out = code;
  return NOVA_B200_OK;
}
}  // namespace nova

extern "C" int32_t nova_b200_gemm_f32_static(const nova_b200_gemm_args* args, void* stream, uint32_t* wait_code_out) {
  using namespace nova;
  nova_b200_gemm_plan_info info;
  int32_t st = gemm_plan_only(args, &info, /*allow_split_k=*/false);
  if (st != NOVA_B200_OK) return st;
  if (args->dtype_ab != NOVA_B200_F32 || args->f32_mode != NOVA_B200_TF32X3)
    return fail(NOVA_B200_ERR_UNSUPPORTED, "gemm_f32_static: only the f32 contraction in NOVA_B200_TF32X3 mode is offered here; 16-bit and "
                                           "TF32X1 contractions with 16-byte-aligned operands use no scratch in nova_b200_gemm "
                                           "(unaligned ones are re-pitched into allocated scratch there)");
  if (static_cast<size_t>(info.scratch_bytes) > kScratchBytes)
    return fail(NOVA_B200_ERR_TOO_LARGE,
                "gemm_f32_static: the hi/lo split of A and B needs " + std::to_string(info.scratch_bytes) +
                    " bytes but the static scratch holds " + std::to_string(kScratchBytes) +
                    " (8 bytes per element of A and B, rows padded to 4 elements); use nova_b200_gemm for larger operands");
  int count = 0, dev = -1;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    cudaGetLastError();
    return fail(NOVA_B200_ERR_NO_DEVICE, "no CUDA device is visible; libnova_b200 has no CPU fallback");
  }
  NOVA_CUDA_OK(cudaGetDevice(&dev));
  StaticDevice* d = nullptr;
  st = setup_device(dev, &d);
  if (st != NOVA_B200_OK) return st;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left.  The split kernels overwrite every scratch byte the
  // contraction reads (padding columns included); only the status word has to start from zero, and it does unless
  // an earlier call's wait gave up and nobody has read the code yet: a call that reports the code itself
  // (wait_code_out) clears the word first, an enqueue-only call leaves it for nova_b200_device_status.
  if (wait_code_out) NOVA_CUDA_OK(cudaMemsetAsync(d->base, 0, 4, s));
  DeviceContext ctx;  // a view of the static array in the shape the launcher expects; owns nothing
  ctx.device = dev;
  ctx.sm_count = d->sm_count;
  ctx.device_count = count;
  ctx.cc_major = 10;
  ctx.status_word = reinterpret_cast<uint32_t*>(d->base);
  ctx.fixed_scratch = d->base + kStatusBytes;  // the launcher takes its scratch from here and never allocates
  ctx.fixed_scratch_bytes = kScratchBytes;
  ctx.encode_tiled = d->encode_tiled;
  st = gemm_launch(&ctx, args, s);
  if (st != NOVA_B200_OK) return st;
  if (wait_code_out) {
    uint32_t code = 0;
    NOVA_CUDA_OK(cudaMemcpyAsync(&code, d->base, 4, cudaMemcpyDeviceToHost, s));
    NOVA_CUDA_OK(cudaStreamSynchronize(s));
    *wait_code_out = code;
    if (code != 0) return fail(NOVA_B200_ERR_DEVICE_TIMEOUT, "gemm_f32_static: a bounded in-kernel wait gave up");
  }
  return NOVA_B200_OK;
}
