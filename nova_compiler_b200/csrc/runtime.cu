// libnova_b200 runtime: per-device contexts, error reporting, the C-ABI entry points for the
// contraction (device-pointer, host-pointer and memref-descriptor forms).
#include "runtime.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <vector>

namespace nova {

int32_t gemm_plan_only(const nova_b200_gemm_args* args, nova_b200_gemm_plan_info* out, bool allow_split_k = true);
int32_t gemm_launch(DeviceContext* ctx, const nova_b200_gemm_args* a, cudaStream_t stream, void* const* peers = nullptr,
                    int32_t n_peers = 0);
int32_t static_scratch_status(int dev, uint32_t* code_out);
int32_t repitch_launch(const void* src, void* dst, int es, int64_t batch, int64_t rows, int64_t cols, int64_t ld_in,
                       int64_t stride_in, int64_t ld_out, int sm_count, cudaStream_t stream);
int32_t split_launch(const float* x, float* hi, float* lo, int64_t rows, int64_t cols, int64_t ld_in, int64_t ld_out,
                     int sm_count, cudaStream_t stream);

namespace {
thread_local std::string g_last_error;
std::mutex g_ctx_mu;
std::map<int, std::unique_ptr<DeviceContext>> g_contexts;
}  // namespace

void set_error(const std::string& msg) { g_last_error = msg; }
int32_t fail(nova_b200_status st, const std::string& msg) {
  g_last_error = msg;
  return st;
}

DeviceContext* current_context(int32_t* status_out) {
  int dev = -1;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    *status_out = fail(NOVA_B200_ERR_NO_DEVICE, "no CUDA device is visible; libnova_b200 has no CPU fallback");
    return nullptr;
  }
  e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    *status_out = fail(NOVA_B200_ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_ctx_mu);
  auto it = g_contexts.find(dev);
  if (it != g_contexts.end()) {
    *status_out = NOVA_B200_OK;
    return it->second.get();
  }
  auto ctx = std::make_unique<DeviceContext>();
  ctx->device = dev;
  ctx->device_count = count;
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, dev);
  if (e != cudaSuccess) {
    *status_out = fail(NOVA_B200_ERR_CUDA, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
    return nullptr;
  }
  ctx->cc_major = prop.major;
  ctx->cc_minor = prop.minor;
  ctx->sm_count = prop.multiProcessorCount;
  if (prop.major != 10) {
    *status_out = fail(NOVA_B200_ERR_NO_DEVICE, "device " + std::to_string(dev) + " is compute capability " +
                                                    std::to_string(prop.major) + "." + std::to_string(prop.minor) +
                                                    "; libnova_b200 is built for sm_100a only");
    return nullptr;
  }
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    *status_out = fail(NOVA_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return nullptr;
  }
  ctx->encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  e = cudaMalloc(reinterpret_cast<void**>(&ctx->status_word), 256);
  if (e == cudaSuccess) e = cudaMemset(ctx->status_word, 0, 256);
  if (e != cudaSuccess) {
    *status_out = fail(NOVA_B200_ERR_CUDA, std::string("status word allocation: ") + cudaGetErrorString(e));
    return nullptr;
  }
  DeviceContext* raw = ctx.get();
  g_contexts[dev] = std::move(ctx);
  *status_out = NOVA_B200_OK;
  return raw;
}

// Staging of the *_host entry points: those calls synchronise before they return, so by the time a later call
// finds the buffer too small nothing can still be using it.
static int32_t grow_staging(void** buf, size_t* have, size_t want) {
  if (*have >= want) return NOVA_B200_OK;
  if (*buf) {
    NOVA_CUDA_OK(cudaFree(*buf));
    *buf = nullptr;
    *have = 0;
  }
  size_t bytes = (want + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
  cudaError_t e = cudaMalloc(buf, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(NOVA_B200_ERR_CUDA, "staging: cudaMalloc of " + std::to_string(bytes) + " bytes failed: " +
                                        cudaGetErrorString(e));
  }
  *have = bytes;
  return NOVA_B200_OK;
}

int32_t acquire_scratch(DeviceContext* ctx, cudaStream_t stream, size_t bytes, void** out) {
  if (ctx->fixed_scratch) {
    if (bytes > ctx->fixed_scratch_bytes)
      return fail(NOVA_B200_ERR_TOO_LARGE, "scratch request of " + std::to_string(bytes) + " bytes exceeds the fixed scratch");
    *out = ctx->fixed_scratch;
    return NOVA_B200_OK;
  }
  std::lock_guard<std::mutex> lock(ctx->mu);
  DeviceContext::ScratchBuf& buf = ctx->scratch_by_stream[stream];
  if (buf.bytes < bytes) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) cudaGetLastError();
    if (cap != cudaStreamCaptureStatusNone)
      return fail(NOVA_B200_ERR_CUDA, "this call needs " + std::to_string(bytes) + " bytes of library scratch on a stream that is "
                  "being captured; make one such call (or nova_b200_reserve_scratch) on the stream before the capture");
    // at least double, so the retired buffers of a growing stream sum to less than the live one
    size_t want = std::max(bytes, 2 * buf.bytes);
    want = (want + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    void* fresh = nullptr;
    cudaError_t e = cudaMalloc(&fresh, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(NOVA_B200_ERR_CUDA, "scratch: cudaMalloc of " + std::to_string(want) + " bytes failed: " + cudaGetErrorString(e));
    }
    if (buf.ptr) ctx->retired_scratch.push_back(buf.ptr);  // enqueued or captured kernels may still use it
    buf.ptr = fresh;
    buf.bytes = want;
  }
  *out = buf.ptr;
  return NOVA_B200_OK;
}

int32_t check_pointer_device(const DeviceContext* ctx, const void* p, const char* what) {
  if (!p || ctx->device_count <= 1) return NOVA_B200_OK;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return NOVA_B200_OK;  // not a pointer CUDA knows: the launch itself will report it
  }
  if (attr.type == cudaMemoryTypeDevice && attr.device != ctx->device)
    return fail(NOVA_B200_ERR_INVALID_ARG, std::string(what) + " lives on device " + std::to_string(attr.device) +
                                               " but the current device is " + std::to_string(ctx->device) +
                                               ": make the operands' device current before the call");
  return NOVA_B200_OK;
}

namespace {
struct OptionEntry { const char* name; const char* env; std::atomic<int64_t> Options::*field; };
const OptionEntry kOptionTable[] = {
    {"repitch", "NOVA_B200_REPITCH", &Options::repitch},     {"pair", "NOVA_B200_PAIR", &Options::pair},
    {"block_n", "NOVA_B200_BLOCK_N", &Options::block_n},     {"short_k", "NOVA_B200_SHORT_K", &Options::short_k},
    {"group_m", "NOVA_B200_GROUP_M", &Options::group_m},     {"prefetch", "NOVA_B200_PREFETCH", &Options::prefetch},
    {"plan_cache", "NOVA_B200_PLAN_CACHE", &Options::plan_cache}, {"debug", "NOVA_B200_DEBUG", &Options::debug},
    {"pdl", "NOVA_B200_PDL", &Options::pdl},
    {"ring_rows", "NOVA_B200_RING_ROWS", &Options::ring_rows},
    {"ring_stages", "NOVA_B200_RING_STAGES", &Options::ring_stages},
    {"ring_ctas", "NOVA_B200_RING_CTAS", &Options::ring_ctas},
    {"host_tiles", "NOVA_B200_HOST_TILES", &Options::host_tiles},
    {"split_k", "NOVA_B200_SPLIT_K", &Options::split_k},
};
}  // namespace

Options& options() {
  static Options* opts = [] {
    Options* o = new Options();
    for (const OptionEntry& e : kOptionTable)
      if (const char* v = std::getenv(e.env)) (o->*(e.field)).store(std::strtoll(v, nullptr, 0));
    return o;
  }();
  return *opts;
}

int32_t ensure_host_streams(DeviceContext* ctx) {
  if (ctx->s_in) return NOVA_B200_OK;
  NOVA_CUDA_OK(cudaStreamCreateWithFlags(&ctx->s_in, cudaStreamNonBlocking));
  NOVA_CUDA_OK(cudaStreamCreateWithFlags(&ctx->s_comp, cudaStreamNonBlocking));
  NOVA_CUDA_OK(cudaStreamCreateWithFlags(&ctx->s_out, cudaStreamNonBlocking));
  for (int i = 0; i < kHostEvents; ++i) {
    NOVA_CUDA_OK(cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming));
    NOVA_CUDA_OK(cudaEventCreateWithFlags(&ctx->ev_comp[i], cudaEventDisableTiming));
  }
  return NOVA_B200_OK;
}

int32_t ensure_staging(DeviceContext* ctx, size_t bytes) { return grow_staging(&ctx->staging, &ctx->staging_bytes, bytes); }

}  // namespace nova

using namespace nova;

extern "C" {

int32_t nova_b200_abi_version(void) { return NOVA_B200_ABI_VERSION; }

const char* nova_b200_last_error_string(void) { return g_last_error.c_str(); }

int32_t nova_b200_init(int32_t device) {
  if (device >= 0) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
      cudaGetLastError();
      return fail(NOVA_B200_ERR_NO_DEVICE, "no CUDA device is visible; libnova_b200 has no CPU fallback");
    }
    if (device >= count) return fail(NOVA_B200_ERR_INVALID_ARG, "nova_b200_init: device index out of range");
    NOVA_CUDA_OK(cudaSetDevice(device));
  }
  int32_t st = NOVA_B200_OK;
  current_context(&st);
  return st;
}

int32_t nova_b200_shutdown(void) {
  std::lock_guard<std::mutex> lock(g_ctx_mu);
  int prev = -1;
  cudaGetDevice(&prev);
  for (auto& kv : g_contexts) {
    DeviceContext* c = kv.second.get();
    if (cudaSetDevice(c->device) != cudaSuccess) continue;
    cudaDeviceSynchronize();
    if (c->status_word) cudaFree(c->status_word);
    for (auto& sb : c->scratch_by_stream)
      if (sb.second.ptr) cudaFree(sb.second.ptr);
    for (void* r : c->retired_scratch) cudaFree(r);
    if (c->staging) cudaFree(c->staging);
    for (const DeviceContext::PreSplit& e : c->presplit) cudaFree(e.hi);  // halves nobody released (hi is the allocation's base)
    c->presplit.clear();
    if (c->s_in) {
      cudaStreamDestroy(c->s_in); cudaStreamDestroy(c->s_comp); cudaStreamDestroy(c->s_out);
      for (int i = 0; i < kHostEvents; ++i) { cudaEventDestroy(c->ev_in[i]); cudaEventDestroy(c->ev_comp[i]); }
    }
  }
  g_contexts.clear();
  if (prev >= 0) cudaSetDevice(prev);
  cudaGetLastError();
  return NOVA_B200_OK;
}

int32_t nova_b200_device_status(uint32_t* code_out) {
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  uint32_t code = 0;
  NOVA_CUDA_OK(cudaDeviceSynchronize());
  NOVA_CUDA_OK(cudaMemcpy(&code, ctx->status_word, 4, cudaMemcpyDeviceToHost));
  if (code != 0) NOVA_CUDA_OK(cudaMemset(ctx->status_word, 0, 4));
  // the static-array entry point keeps its own status word (it may not use allocated memory)
  uint32_t static_code = 0;
  st = static_scratch_status(ctx->device, &static_code);
  if (st != NOVA_B200_OK) return st;
  if (code == 0) code = static_code;
  if (code_out) *code_out = code;
  if (code != 0)
    return fail(NOVA_B200_ERR_DEVICE_TIMEOUT, "a bounded in-kernel wait gave up, code 0x" + [&] {
      char b[16];
      snprintf(b, sizeof b, "%x", code);
      return std::string(b);
    }());
  return NOVA_B200_OK;
}

int32_t nova_b200_set_option(const char* name, int64_t value) {
  if (!name) return fail(NOVA_B200_ERR_INVALID_ARG, "set_option: name is null");
  Options& o = options();
  for (const OptionEntry& e : kOptionTable) {
    if (std::strcmp(e.name, name) == 0) {
      (o.*(e.field)).store(value);
      o.epoch.fetch_add(1);
      return NOVA_B200_OK;
    }
  }
  return fail(NOVA_B200_ERR_INVALID_ARG, std::string("set_option: unknown option '") + name + "'");
}

int32_t nova_b200_get_option(const char* name, int64_t* value_out) {
  if (!name || !value_out) return fail(NOVA_B200_ERR_INVALID_ARG, "get_option: null argument");
  Options& o = options();
  for (const OptionEntry& e : kOptionTable) {
    if (std::strcmp(e.name, name) == 0) {
      *value_out = (o.*(e.field)).load();
      return NOVA_B200_OK;
    }
  }
  return fail(NOVA_B200_ERR_INVALID_ARG, std::string("get_option: unknown option '") + name + "'");
}

int32_t nova_b200_reserve_scratch(int64_t bytes, void* stream) {
  if (bytes < 0) return fail(NOVA_B200_ERR_INVALID_ARG, "reserve_scratch: negative size");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  void* unused = nullptr;
  return bytes == 0 ? NOVA_B200_OK : acquire_scratch(ctx, static_cast<cudaStream_t>(stream), static_cast<size_t>(bytes), &unused);
}

// ---------------------------------------------------------------- prepared operands

struct nova_b200_operand {
  void* data = nullptr;
  int device = -1;
  int32_t dtype = 0;
  int64_t batch = 0, rows = 0, cols = 0, ld = 0, batch_stride = 0;
};

int32_t nova_b200_operand_prepare(const void* src_dev, int32_t dtype, int64_t batch, int64_t rows, int64_t cols, int64_t ld,
                                  int64_t batch_stride, void* stream, nova_b200_operand** out) {
  if (!out) return fail(NOVA_B200_ERR_INVALID_ARG, "operand_prepare: out is null");
  *out = nullptr;
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "operand_prepare: dtype must be f32, f16 or bf16");
  if (batch < 1 || rows < 1 || cols < 1 || ld < cols || batch_stride < 0 || !src_dev)
    return fail(NOVA_B200_ERR_INVALID_ARG, "operand_prepare: bad extent, pitch or pointer");
  if (batch > 1 && batch_stride != 0 && batch_stride < (rows - 1) * ld + cols)
    return fail(NOVA_B200_ERR_LAYOUT, "operand_prepare: batches overlap");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  st = check_pointer_device(ctx, src_dev, "operand_prepare: the operand");
  if (st != NOVA_B200_OK) return st;
  const int es = dtype_bytes(dtype);
  const int per_chunk = 16 / es;
  auto op = std::make_unique<nova_b200_operand>();
  op->device = ctx->device;
  op->dtype = dtype;
  op->batch = batch_stride == 0 ? 1 : batch;
  op->rows = rows;
  op->cols = cols;
  op->ld = (cols + per_chunk - 1) / per_chunk * per_chunk;
  op->batch_stride = op->batch > 1 ? rows * op->ld : 0;
  const size_t bytes = static_cast<size_t>(op->batch) * rows * op->ld * es;
  cudaError_t e = cudaMalloc(&op->data, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(NOVA_B200_ERR_CUDA, "operand_prepare: cudaMalloc of " + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e));
  }
  st = repitch_launch(src_dev, op->data, es, op->batch, rows, cols, ld, batch_stride, op->ld, ctx->sm_count,
                      static_cast<cudaStream_t>(stream));
  if (st != NOVA_B200_OK) {
    cudaFree(op->data);
    return st;
  }
  *out = op.release();
  return NOVA_B200_OK;
}

int32_t nova_b200_operand_view(const nova_b200_operand* op, const void** data_dev, int64_t* ld, int64_t* batch_stride) {
  if (!op) return fail(NOVA_B200_ERR_INVALID_ARG, "operand_view: operand is null");
  if (data_dev) *data_dev = op->data;
  if (ld) *ld = op->ld;
  if (batch_stride) *batch_stride = op->batch_stride;
  return NOVA_B200_OK;
}

struct nova_b200_presplit_handle {
  int device;
  const void* x;
  float* base;   // hi then lo, one stream-ordered allocation
};

int32_t nova_b200_f32_presplit(const void* x_dev, int64_t rows, int64_t cols, int64_t ld, void* stream, void** handle_out) {
  if (!handle_out) return fail(NOVA_B200_ERR_INVALID_ARG, "f32_presplit: handle_out is null");
  *handle_out = nullptr;
  if (!x_dev || rows < 1 || cols < 1 || ld < cols) return fail(NOVA_B200_ERR_INVALID_ARG, "f32_presplit: bad extent, pitch or pointer");
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  st = check_pointer_device(ctx, x_dev, "f32_presplit: the matrix");
  if (st != NOVA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t ldo = (cols + 3) & ~3ll;
  const size_t half = static_cast<size_t>(rows) * ldo * sizeof(float);
  void* base = nullptr;
  cudaError_t e = cudaMallocAsync(&base, 2 * half, s);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(NOVA_B200_ERR_CUDA, "f32_presplit: allocation of " + std::to_string(2 * half) + " bytes failed: " + cudaGetErrorString(e));
  }
  float* hi = static_cast<float*>(base);
  float* lo = hi + static_cast<size_t>(rows) * ldo;
  st = split_launch(static_cast<const float*>(x_dev), hi, lo, rows, cols, ld, ldo, ctx->sm_count, s);
  if (st != NOVA_B200_OK) { cudaFreeAsync(base, s); return st; }
  {
    std::lock_guard<std::mutex> lock(ctx->presplit_mu);
    ctx->presplit.push_back(DeviceContext::PreSplit{x_dev, rows, cols, ld, hi, lo, ldo});
    ++ctx->presplit_version;
  }
  *handle_out = new nova_b200_presplit_handle{ctx->device, x_dev, hi};
  return NOVA_B200_OK;
}

int32_t nova_b200_f32_presplit_release(void* handle, void* stream) {
  if (!handle) return NOVA_B200_OK;
  auto* h = static_cast<nova_b200_presplit_handle*>(handle);
  int32_t st = NOVA_B200_OK;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  if (ctx->device != h->device) return fail(NOVA_B200_ERR_INVALID_ARG, "f32_presplit_release: the handle belongs to another device");
  {
    std::lock_guard<std::mutex> lock(ctx->presplit_mu);
    for (size_t i = 0; i < ctx->presplit.size(); ++i) {
      if (ctx->presplit[i].hi == h->base) {
        ctx->presplit.erase(ctx->presplit.begin() + static_cast<std::ptrdiff_t>(i));
        break;
      }
    }
    ++ctx->presplit_version;
  }
  cudaError_t e = cudaFreeAsync(h->base, static_cast<cudaStream_t>(stream));
  delete h;
  if (e != cudaSuccess) { cudaGetLastError(); return fail(NOVA_B200_ERR_CUDA, std::string("f32_presplit_release: ") + cudaGetErrorString(e)); }
  return NOVA_B200_OK;
}

void nova_b200_operand_free(nova_b200_operand* op) {
  if (!op) return;
  int prev = -1;
  cudaGetDevice(&prev);
  if (cudaSetDevice(op->device) == cudaSuccess) {
    cudaDeviceSynchronize();  // kernels that still read the copy
    cudaFree(op->data);
  }
  if (prev >= 0) cudaSetDevice(prev);
  cudaGetLastError();
  delete op;
}

int32_t nova_b200_gemm_plan(const nova_b200_gemm_args* args, nova_b200_gemm_plan_info* out) {
  return gemm_plan_only(args, out);
}

int32_t nova_b200_gemm(const nova_b200_gemm_args* args, void* stream) {
  // validate first so that argument errors are reported even on a machine without a GPU
  nova_b200_gemm_plan_info info;
  int32_t st = gemm_plan_only(args, &info);
  if (st != NOVA_B200_OK) return st;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  return gemm_launch(ctx, args, static_cast<cudaStream_t>(stream));
}

int32_t nova_b200_gemm_push(const nova_b200_gemm_args* args, void* const* peer_c, int32_t n_peers, void* stream) {
  if (n_peers < 0 || (n_peers > 0 && !peer_c)) return fail(NOVA_B200_ERR_INVALID_ARG, "gemm_push: bad peer list");
  nova_b200_gemm_plan_info info;
  int32_t st = gemm_plan_only(args, &info);
  if (st != NOVA_B200_OK) return st;
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  return gemm_launch(ctx, args, static_cast<cudaStream_t>(stream), peer_c, n_peers);
}

int32_t nova_b200_peer_buffer_alloc(int64_t bytes, void** ptr_out, unsigned char handle_out[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (bytes <= 0 || !ptr_out || !handle_out) return fail(NOVA_B200_ERR_INVALID_ARG, "peer_buffer_alloc: bad argument");
  int32_t st = NOVA_B200_OK;
  if (!current_context(&st)) return st;
  void* p = nullptr;
  NOVA_CUDA_OK(cudaMalloc(&p, static_cast<size_t>(bytes)));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return fail(NOVA_B200_ERR_CUDA, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
  }
  std::memcpy(handle_out, &h, 64);
  *ptr_out = p;
  return NOVA_B200_OK;
}

int32_t nova_b200_peer_buffer_open(const unsigned char handle[64], void** ptr_out) {
  if (!handle || !ptr_out) return fail(NOVA_B200_ERR_INVALID_ARG, "peer_buffer_open: bad argument");
  int32_t st = NOVA_B200_OK;
  if (!current_context(&st)) return st;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(NOVA_B200_ERR_CUDA, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
  }
  *ptr_out = p;
  return NOVA_B200_OK;
}

int32_t nova_b200_peer_buffer_close(void* opened_ptr) {
  if (!opened_ptr) return NOVA_B200_OK;
  NOVA_CUDA_OK(cudaIpcCloseMemHandle(opened_ptr));
  return NOVA_B200_OK;
}

int32_t nova_b200_peer_buffer_free(void* owned_ptr) {
  if (!owned_ptr) return NOVA_B200_OK;
  NOVA_CUDA_OK(cudaFree(owned_ptr));
  return NOVA_B200_OK;
}

int32_t nova_b200_gemm_flat(int64_t A, int64_t B, int64_t C, int64_t bias, int64_t residual, int64_t batch, int64_t M,
                            int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldr,
                            int64_t batch_stride_a, int64_t batch_stride_b, int64_t batch_stride_c, int64_t batch_stride_r,
                            int32_t dtype_ab, int32_t dtype_c, int32_t trans_a, int32_t trans_b, int32_t act, int32_t init,
                            int32_t f32_mode, int64_t stream) {
  nova_b200_gemm_args g{};
  g.struct_size = sizeof(g);
  g.dtype_ab = dtype_ab; g.dtype_c = dtype_c; g.trans_a = trans_a; g.trans_b = trans_b;
  g.act = act; g.init = init; g.f32_mode = f32_mode;
  g.batch = batch; g.M = M; g.N = N; g.K = K;
  g.A = reinterpret_cast<const void*>(static_cast<intptr_t>(A));
  g.B = reinterpret_cast<const void*>(static_cast<intptr_t>(B));
  g.C = reinterpret_cast<void*>(static_cast<intptr_t>(C));
  g.bias = reinterpret_cast<const void*>(static_cast<intptr_t>(bias));
  g.residual = reinterpret_cast<const void*>(static_cast<intptr_t>(residual));
  g.lda = lda; g.ldb = ldb; g.ldc = ldc; g.ldr = ldr;
  g.batch_stride_a = batch_stride_a; g.batch_stride_b = batch_stride_b; g.batch_stride_c = batch_stride_c;
  g.batch_stride_r = batch_stride_r;
  return nova_b200_gemm(&g, reinterpret_cast<void*>(static_cast<intptr_t>(stream)));
}

int32_t nova_b200_gemm_host(const nova_b200_gemm_args* args) {
  nova_b200_gemm_plan_info info;
  int32_t st = gemm_plan_only(args, &info);
  if (st != NOVA_B200_OK) return st;
  if (args->batch == 0 || args->M == 0 || args->N == 0) return NOVA_B200_OK;
  if (args->init == NOVA_B200_INIT_LN_FOLD)
    return fail(NOVA_B200_ERR_UNSUPPORTED, "gemm_host: INIT_LN_FOLD takes device-resident statistics and folded weights; use nova_b200_gemm");
  DeviceContext* ctx = current_context(&st);
  if (!ctx) return st;
  const nova_b200_gemm_args& a = *args;
  const int es = dtype_bytes(a.dtype_ab), os = dtype_bytes(a.dtype_c);
  auto span = [](int64_t batch, int64_t bstride, int64_t rows, int64_t ld, int64_t cols) -> int64_t {
    // elements from the first to one past the last addressed element
    if (rows == 0 || cols == 0) return 0;
    return (bstride == 0 ? 0 : (batch - 1) * bstride) + (rows - 1) * ld + cols;
  };
  const int64_t a_rows = a.trans_a ? a.K : a.M, a_cols = a.trans_a ? a.M : a.K;
  const int64_t b_rows = a.trans_b ? a.N : a.K, b_cols = a.trans_b ? a.K : a.N;
  const size_t a_bytes = a.K ? span(a.batch, a.batch_stride_a, a_rows, a.lda, a_cols) * es : 0;
  const size_t b_bytes = a.K ? span(a.batch, a.batch_stride_b, b_rows, a.ldb, b_cols) * es : 0;
  const size_t c_bytes = span(a.batch, a.batch_stride_c, a.M, a.ldc, a.N) * os;
  const size_t bias_bytes = init_has_bias(a.init) ? a.N * os : 0;
  const size_t r_bytes = reads_residual(a.init, a.act) ? span(a.batch, a.batch_stride_r, a.M, a.ldr, a.N) * os : 0;
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  const size_t total = up(a_bytes) + up(b_bytes) + up(c_bytes) + up(bias_bytes) + up(r_bytes);
  std::lock_guard<std::mutex> lock(ctx->host_mu);
  st = ensure_staging(ctx, total);
  if (st != NOVA_B200_OK) return st;
  char* base = static_cast<char*>(ctx->staging);
  char* dA = base; char* dB = dA + up(a_bytes); char* dC = dB + up(b_bytes);
  char* dBias = dC + up(c_bytes); char* dR = dBias + up(bias_bytes);
  const bool c_preload = a.init == NOVA_B200_INIT_FROM_C || a.ldc != a.N || (a.batch > 1 && a.batch_stride_c != a.M * a.ldc);

  // Pipelined form: the problem is cut into up to 8 chunks (batches, or row blocks of a single matrix) and
  // chunk i+1's host-to-device copy, chunk i's kernel and chunk i-1's device-to-host copy run concurrently
  // on three streams, so the two PCIe directions overlap.  Needs chunkable layouts; else one shot below.
  const bool by_batch = a.batch > 1 && a.batch_stride_a != 0 && a.batch_stride_c != 0 &&
                        (!reads_residual(a.init, a.act) || a.batch_stride_r != 0);
  const bool by_rows = a.batch == 1 && !a.trans_a && a.M >= 512 && a.K > 0;
  // One large matrix product: tiles of (row block of A and C) x (column slab of B and C).  The device-to-host copy of
  // C is the longest leg (C3: 180 MB against 157 MB in), so the first result tile should leave as early as possible:
  // after ONE row block of A and ONE column slab of B have arrived, not after the whole of B.  From then on the
  // two PCIe directions run concurrently.  Slabs are strided on both sides: 2-D copies.
  const int64_t tiles_opt = options().host_tiles.load();
  const bool by_tiles = tiles_opt >= 0 && by_rows && !a.trans_b && a.N >= 2048 && a.init != NOVA_B200_INIT_FROM_C &&
                        reinterpret_cast<uintptr_t>(dB) % 16 == 0 && (a.ldb * es) % 16 == 0;
  if (by_tiles) {
    st = ensure_host_streams(ctx);
    if (st != NOVA_B200_OK) return st;
    cudaStream_t s_in = ctx->s_in, s_comp = ctx->s_comp, s_out = ctx->s_out;
    const int64_t row_units = (a.M + 255) / 256, col_units = (a.N + 63) / 64;
    // tiles of about 2048 x 2048: large enough that a strided copy runs at the link's rate and that the distinct tile
    // shapes stay within the plan cache, small enough that the first results leave early
    int rb = static_cast<int>(std::clamp<int64_t>((a.M + 1024) / 2048, 1, kHostChunks));
    int cb = static_cast<int>(std::clamp<int64_t>((a.N + 1024) / 2048, 1, kHostChunks));
    while (rb * cb > 30) (rb >= cb ? rb : cb) -= 1;
    if (tiles_opt % 10000 > 0) {
      rb = static_cast<int>(std::clamp<int64_t>(tiles_opt % 10000 / 100, 1, std::min<int64_t>(row_units, kHostChunks)));
      cb = static_cast<int>(std::clamp<int64_t>(tiles_opt % 100, 1, std::min<int64_t>(col_units, kHostChunks)));
    }
    if (bias_bytes) NOVA_CUDA_OK(cudaMemcpyAsync(dBias, a.bias, bias_bytes, cudaMemcpyHostToDevice, s_in));
    // Tile order: growing square.  Step s brings row block s and column slab s and releases the tiles whose larger
    // index is s, so the bytes of C that may leave grow quadratically with the bytes that have arrived and the
    // device-to-host direction is busy long before the last operand byte is in.  (Slab by slab the first rb tiles each
    // wait for a row block of A, and the outbound link idles.)  Option host_tiles >= 10000: slab by slab.
    std::vector<std::pair<int, int>> order;
    order.reserve(static_cast<size_t>(rb) * cb);
    if (tiles_opt >= 10000) {
      for (int j = 0; j < cb; ++j)
        for (int i = 0; i < rb; ++i) order.emplace_back(i, j);
    } else {
      for (int s2 = 0; s2 < std::max(rb, cb); ++s2) {
        if (s2 < cb)
          for (int i = 0; i <= std::min(s2, rb - 1); ++i) order.emplace_back(i, s2);
        if (s2 < rb)
          for (int j = 0; j < std::min(s2, cb); ++j) order.emplace_back(s2, j);
      }
    }
    bool a_in[kHostChunks] = {}, b_in[kHostChunks] = {};
    int e = 0;
    for (const auto& [i, j] : order) {
      const int64_t c0 = col_units * j / cb * 64, c1 = std::min<int64_t>(col_units * (j + 1) / cb * 64, a.N);
      const int64_t r0 = row_units * i / rb * 256, r1 = std::min<int64_t>(row_units * (i + 1) / rb * 256, a.M);
      const int64_t ncols = c1 - c0, nrows = r1 - r0;
      if (!b_in[j]) {
        NOVA_CUDA_OK(cudaMemcpy2DAsync(dB + c0 * es, a.ldb * es, static_cast<const char*>(a.B) + c0 * es, a.ldb * es,
                                       ncols * es, a.K, cudaMemcpyHostToDevice, s_in));
        b_in[j] = true;
      }
      if (!a_in[i]) {
        NOVA_CUDA_OK(cudaMemcpy2DAsync(dA + r0 * a.lda * es, a.lda * es, static_cast<const char*>(a.A) + r0 * a.lda * es,
                                       a.lda * es, a.K * es, nrows, cudaMemcpyHostToDevice, s_in));
        a_in[i] = true;
      }
      if (r_bytes)
        NOVA_CUDA_OK(cudaMemcpy2DAsync(dR + (r0 * a.ldr + c0) * os, a.ldr * os,
                                       static_cast<const char*>(a.residual) + (r0 * a.ldr + c0) * os, a.ldr * os, ncols * os,
                                       nrows, cudaMemcpyHostToDevice, s_in));
      NOVA_CUDA_OK(cudaEventRecord(ctx->ev_in[e], s_in));
      NOVA_CUDA_OK(cudaStreamWaitEvent(s_comp, ctx->ev_in[e], 0));
      nova_b200_gemm_args d = a;
      d.M = nrows;
      d.N = ncols;
      d.A = dA + r0 * a.lda * es;
      d.B = dB + c0 * es;
      d.C = dC + (r0 * a.ldc + c0) * os;
      d.bias = dBias + c0 * os;
      d.residual = dR + (r0 * a.ldr + c0) * os;
      st = gemm_launch(ctx, &d, s_comp);
      if (st != NOVA_B200_OK) { cudaDeviceSynchronize(); return st; }
      NOVA_CUDA_OK(cudaEventRecord(ctx->ev_comp[e], s_comp));
      NOVA_CUDA_OK(cudaStreamWaitEvent(s_out, ctx->ev_comp[e], 0));
      NOVA_CUDA_OK(cudaMemcpy2DAsync(static_cast<char*>(a.C) + (r0 * a.ldc + c0) * os, a.ldc * os, dC + (r0 * a.ldc + c0) * os,
                                     a.ldc * os, ncols * os, nrows, cudaMemcpyDeviceToHost, s_out));
      ++e;
    }
    NOVA_CUDA_OK(cudaStreamSynchronize(s_out));
    NOVA_CUDA_OK(cudaStreamSynchronize(s_in));
    return NOVA_B200_OK;
  }
  if ((by_batch || by_rows) && a.K > 0) {
    st = ensure_host_streams(ctx);
    if (st != NOVA_B200_OK) return st;
    cudaStream_t s_in = ctx->s_in, s_comp = ctx->s_comp, s_out = ctx->s_out;
    const int64_t units = by_batch ? a.batch : (a.M + 255) / 256;   // batches, or 256-row blocks
    const int n_chunks = static_cast<int>(units < kHostChunks ? units : kHostChunks);
    // operands every chunk needs
    if (bias_bytes) NOVA_CUDA_OK(cudaMemcpyAsync(dBias, a.bias, bias_bytes, cudaMemcpyHostToDevice, s_in));
    if (by_rows || a.batch_stride_b == 0) NOVA_CUDA_OK(cudaMemcpyAsync(dB, a.B, b_bytes, cudaMemcpyHostToDevice, s_in));
    for (int c = 0; c < n_chunks; ++c) {
      const int64_t u0 = units * c / n_chunks, u1 = units * (c + 1) / n_chunks;
      nova_b200_gemm_args d = a;
      int64_t a_off, c_off, r_off = 0, b_off = 0;  // element offsets of the chunk
      size_t a_len, c_len, r_len = 0, b_len = 0;   // bytes of the chunk
      if (by_batch) {
        const int64_t nb = u1 - u0;
        d.batch = nb;
        a_off = u0 * a.batch_stride_a; c_off = u0 * a.batch_stride_c;
        a_len = span(nb, a.batch_stride_a, a_rows, a.lda, a_cols) * es;
        c_len = span(nb, a.batch_stride_c, a.M, a.ldc, a.N) * os;
        if (a.batch_stride_b != 0) { b_off = u0 * a.batch_stride_b; b_len = span(nb, a.batch_stride_b, b_rows, a.ldb, b_cols) * es; }
        if (r_bytes) { r_off = u0 * a.batch_stride_r; r_len = span(nb, a.batch_stride_r, a.M, a.ldr, a.N) * os; }
      } else {
        const int64_t r0 = u0 * 256, r1 = u1 * 256 < a.M ? u1 * 256 : a.M;
        d.M = r1 - r0;
        a_off = r0 * a.lda; c_off = r0 * a.ldc;
        a_len = span(1, 0, d.M, a.lda, a_cols) * es;
        c_len = span(1, 0, d.M, a.ldc, a.N) * os;
        if (r_bytes) { r_off = r0 * a.ldr; r_len = span(1, 0, d.M, a.ldr, a.N) * os; }
      }
      NOVA_CUDA_OK(cudaMemcpyAsync(dA + a_off * es, static_cast<const char*>(a.A) + a_off * es, a_len, cudaMemcpyHostToDevice, s_in));
      if (b_len) NOVA_CUDA_OK(cudaMemcpyAsync(dB + b_off * es, static_cast<const char*>(a.B) + b_off * es, b_len, cudaMemcpyHostToDevice, s_in));
      if (r_len) NOVA_CUDA_OK(cudaMemcpyAsync(dR + r_off * os, static_cast<const char*>(a.residual) + r_off * os, r_len, cudaMemcpyHostToDevice, s_in));
      if (c_preload) NOVA_CUDA_OK(cudaMemcpyAsync(dC + c_off * os, static_cast<const char*>(a.C) + c_off * os, c_len, cudaMemcpyHostToDevice, s_in));
      NOVA_CUDA_OK(cudaEventRecord(ctx->ev_in[c], s_in));
      NOVA_CUDA_OK(cudaStreamWaitEvent(s_comp, ctx->ev_in[c], 0));
      d.A = dA + a_off * es;
      d.B = dB + b_off * es;
      d.C = dC + c_off * os;
      d.bias = dBias;
      d.residual = dR + r_off * os;
      st = gemm_launch(ctx, &d, s_comp);
      if (st != NOVA_B200_OK) { cudaDeviceSynchronize(); return st; }
      NOVA_CUDA_OK(cudaEventRecord(ctx->ev_comp[c], s_comp));
      NOVA_CUDA_OK(cudaStreamWaitEvent(s_out, ctx->ev_comp[c], 0));
      NOVA_CUDA_OK(cudaMemcpyAsync(static_cast<char*>(a.C) + c_off * os, dC + c_off * os, c_len, cudaMemcpyDeviceToHost, s_out));
    }
    NOVA_CUDA_OK(cudaStreamSynchronize(s_out));
    NOVA_CUDA_OK(cudaStreamSynchronize(s_in));
    return NOVA_B200_OK;
  }

  cudaStream_t s = nullptr;
  if (a_bytes) NOVA_CUDA_OK(cudaMemcpyAsync(dA, a.A, a_bytes, cudaMemcpyHostToDevice, s));
  if (b_bytes) NOVA_CUDA_OK(cudaMemcpyAsync(dB, a.B, b_bytes, cudaMemcpyHostToDevice, s));
  if (bias_bytes) NOVA_CUDA_OK(cudaMemcpyAsync(dBias, a.bias, bias_bytes, cudaMemcpyHostToDevice, s));
  if (r_bytes) NOVA_CUDA_OK(cudaMemcpyAsync(dR, a.residual, r_bytes, cudaMemcpyHostToDevice, s));
  if (c_preload) NOVA_CUDA_OK(cudaMemcpyAsync(dC, a.C, c_bytes, cudaMemcpyHostToDevice, s));  // keep bytes the kernel does not write
  nova_b200_gemm_args d = a;
  d.A = dA; d.B = dB; d.C = dC; d.bias = dBias; d.residual = dR;
  st = gemm_launch(ctx, &d, s);
  if (st != NOVA_B200_OK) return st;
  NOVA_CUDA_OK(cudaMemcpyAsync(a.C, dC, c_bytes, cudaMemcpyDeviceToHost, s));
  NOVA_CUDA_OK(cudaStreamSynchronize(s));
  return NOVA_B200_OK;
}

// ---------------------------------------------------------------- memref-descriptor entry points

namespace {

bool is_device_pointer(const void* p) {
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

// Maps a rank-2 (or the inner two dims of a rank-3) descriptor onto {pointer, pitch, transposed}.
int32_t inner2(const int64_t* sizes, const int64_t* strides, int64_t* ld, int32_t* trans, const char* name) {
  auto at_least = [](int64_t v, int64_t lo) { return v < lo ? lo : v; };
  if (sizes[1] == 1 || strides[1] == 1) {
    *trans = 0;
    *ld = sizes[0] > 1 ? strides[0] : at_least(strides[0], sizes[1]);
    return NOVA_B200_OK;
  }
  if (sizes[0] == 1 || strides[0] == 1) {
    *trans = 1;
    *ld = sizes[1] > 1 ? strides[1] : at_least(strides[1], sizes[0]);
    return NOVA_B200_OK;
  }
  return fail(NOVA_B200_ERR_LAYOUT, std::string(name) + ": neither of the two inner strides is 1");
}

int32_t run_descriptor_gemm(nova_b200_gemm_args& g) {
  const bool dev = is_device_pointer(g.C);
  if (dev != is_device_pointer(g.A) || dev != is_device_pointer(g.B))
    return fail(NOVA_B200_ERR_INVALID_ARG, "memref entry point: operands must be all host or all device memory");
  if (dev) {
    int32_t st = nova_b200_gemm(&g, nullptr);
    if (st != NOVA_B200_OK) return st;
    NOVA_CUDA_OK(cudaStreamSynchronize(nullptr));
    return NOVA_B200_OK;
  }
  return nova_b200_gemm_host(&g);
}

}  // namespace

int32_t _mlir_ciface_nova_b200_matmul(nova_b200_memref2d* C, nova_b200_memref2d* A, nova_b200_memref2d* B,
                                      int32_t dtype) {
  if (!C || !A || !B) return fail(NOVA_B200_ERR_INVALID_ARG, "matmul: null descriptor");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "matmul: dtype must be f32, f16 or bf16");
  if (A->sizes[1] != B->sizes[0] || C->sizes[0] != A->sizes[0] || C->sizes[1] != B->sizes[1])
    return fail(NOVA_B200_ERR_INVALID_ARG, "matmul: shapes do not compose");  // MatmulOp::verify, NovaOps.cpp:1247-1254
  const int es = dtype_bytes(dtype);
  nova_b200_gemm_args g{};
  g.struct_size = sizeof(g);
  g.dtype_ab = g.dtype_c = dtype;
  g.batch = 1; g.M = A->sizes[0]; g.K = A->sizes[1]; g.N = B->sizes[1];
  int32_t st, tc = 0;
  if ((st = inner2(A->sizes, A->strides, &g.lda, &g.trans_a, "matmul A")) != NOVA_B200_OK) return st;
  if ((st = inner2(B->sizes, B->strides, &g.ldb, &g.trans_b, "matmul B")) != NOVA_B200_OK) return st;
  if ((st = inner2(C->sizes, C->strides, &g.ldc, &tc, "matmul C")) != NOVA_B200_OK) return st;
  if (tc) return fail(NOVA_B200_ERR_LAYOUT, "matmul: C must have unit inner stride");
  g.A = static_cast<char*>(A->aligned) + A->offset * es;
  g.B = static_cast<char*>(B->aligned) + B->offset * es;
  g.C = static_cast<char*>(C->aligned) + C->offset * es;
  return run_descriptor_gemm(g);
}

int32_t _mlir_ciface_nova_b200_batch_matmul(nova_b200_memref3d* C, nova_b200_memref3d* A, nova_b200_memref3d* B,
                                            int32_t ab_dtype, int32_t c_dtype) {
  if (!C || !A || !B) return fail(NOVA_B200_ERR_INVALID_ARG, "batch_matmul: null descriptor");
  if (!is_float_dtype(ab_dtype) || !is_float_dtype(c_dtype))
    return fail(NOVA_B200_ERR_UNSUPPORTED, "batch_matmul: dtypes must be f32, f16 or bf16");
  if (A->sizes[0] != C->sizes[0] || (B->sizes[0] != C->sizes[0] && B->sizes[0] != 1) || A->sizes[2] != B->sizes[1] ||
      C->sizes[1] != A->sizes[1] || C->sizes[2] != B->sizes[2])
    return fail(NOVA_B200_ERR_INVALID_ARG, "batch_matmul: shapes do not compose");
  nova_b200_gemm_args g{};
  g.struct_size = sizeof(g);
  g.dtype_ab = ab_dtype; g.dtype_c = c_dtype;
  g.batch = C->sizes[0]; g.M = A->sizes[1]; g.K = A->sizes[2]; g.N = B->sizes[2];
  int32_t st, tc = 0;
  if ((st = inner2(A->sizes + 1, A->strides + 1, &g.lda, &g.trans_a, "batch_matmul A")) != NOVA_B200_OK) return st;
  if ((st = inner2(B->sizes + 1, B->strides + 1, &g.ldb, &g.trans_b, "batch_matmul B")) != NOVA_B200_OK) return st;
  if ((st = inner2(C->sizes + 1, C->strides + 1, &g.ldc, &tc, "batch_matmul C")) != NOVA_B200_OK) return st;
  if (tc) return fail(NOVA_B200_ERR_LAYOUT, "batch_matmul: C must have unit inner stride");
  g.batch_stride_a = A->strides[0];
  g.batch_stride_b = B->sizes[0] == 1 ? 0 : B->strides[0];
  g.batch_stride_c = C->strides[0];
  const int es = dtype_bytes(ab_dtype), os = dtype_bytes(c_dtype);
  g.A = static_cast<char*>(A->aligned) + A->offset * es;
  g.B = static_cast<char*>(B->aligned) + B->offset * es;
  g.C = static_cast<char*>(C->aligned) + C->offset * os;
  return run_descriptor_gemm(g);
}

int32_t _mlir_ciface_nova_b200_batch_matmul_4d(nova_b200_memref4d* C, nova_b200_memref4d* A, nova_b200_memref4d* B,
                                               int32_t ab_dtype, int32_t c_dtype) {
  if (!C || !A || !B) return fail(NOVA_B200_ERR_INVALID_ARG, "batch_matmul_4d: null descriptor");
  for (int d = 0; d < 2; ++d) {
    if (A->sizes[d] != C->sizes[d] || (B->sizes[d] != C->sizes[d] && B->sizes[d] != 1))
      return fail(NOVA_B200_ERR_INVALID_ARG, "batch_matmul_4d: batch dims do not compose");
  }
  // A size-1 batch dim broadcasts: give it stride 0 so the arithmetic below treats every operand alike.
  auto bstride = [](const nova_b200_memref4d* m, int d, int64_t full) { return (m->sizes[d] == 1 && full > 1) ? 0 : m->strides[d]; };
  const int64_t b0 = C->sizes[0], b1 = C->sizes[1];
  // collapsing [b0, b1] to one batch dim is metadata when stride[0] == b1 * stride[1] (or either dim is 1)
  auto collapses = [&](const nova_b200_memref4d* m) {
    const int64_t s0 = bstride(m, 0, b0), s1 = bstride(m, 1, b1);
    return b0 == 1 || b1 == 1 || s0 == b1 * s1;
  };
  auto slice3 = [&](const nova_b200_memref4d* m, int64_t i0, bool collapse, int esz) {
    nova_b200_memref3d r{};
    const int64_t s0 = bstride(m, 0, b0), s1 = bstride(m, 1, b1);
    r.allocated = m->allocated;
    r.aligned = static_cast<char*>(m->aligned) + (m->offset + (collapse ? 0 : i0 * s0)) * esz;
    r.offset = 0;
    const bool bcast = m->sizes[0] == 1 && m->sizes[1] == 1 && b0 * b1 > 1;
    r.sizes[0] = bcast ? 1 : (collapse ? b0 * b1 : b1);
    r.strides[0] = collapse ? (b1 == 1 ? s0 : s1) : s1;
    r.sizes[1] = m->sizes[2]; r.sizes[2] = m->sizes[3];
    r.strides[1] = m->strides[2]; r.strides[2] = m->strides[3];
    return r;
  };
  const int es = dtype_bytes(ab_dtype), os = dtype_bytes(c_dtype);
  if (es == 0 || os == 0) return fail(NOVA_B200_ERR_UNSUPPORTED, "batch_matmul_4d: dtypes must be f32, f16 or bf16");
  // an operand that broadcasts along only ONE of the two batch dims cannot be a single strided batch
  auto mixed = [&](const nova_b200_memref4d* m) { return (m->sizes[0] == 1) != (m->sizes[1] == 1) && b0 > 1 && b1 > 1; };
  const bool one_call = collapses(C) && collapses(A) && collapses(B) && !mixed(B);
  if (one_call) {
    nova_b200_memref3d c3 = slice3(C, 0, true, os), a3 = slice3(A, 0, true, es), bb3 = slice3(B, 0, true, es);
    return _mlir_ciface_nova_b200_batch_matmul(&c3, &a3, &bb3, ab_dtype, c_dtype);
  }
  for (int64_t i0 = 0; i0 < b0; ++i0) {
    nova_b200_memref3d c3 = slice3(C, i0, false, os), a3 = slice3(A, i0, false, es), bb3 = slice3(B, i0, false, es);
    if (B->sizes[1] == 1 && b1 > 1) bb3.sizes[0] = 1;
    int32_t st = _mlir_ciface_nova_b200_batch_matmul(&c3, &a3, &bb3, ab_dtype, c_dtype);
    if (st != NOVA_B200_OK) return st;
  }
  return NOVA_B200_OK;
}

int32_t _mlir_ciface_nova_b200_linear(nova_b200_memref2d* Y, nova_b200_memref2d* X, nova_b200_memref2d* W,
                                      nova_b200_memref1d* bias, int32_t dtype, int32_t act) {
  if (!Y || !X || !W || !bias) return fail(NOVA_B200_ERR_INVALID_ARG, "linear: null descriptor");
  if (!is_float_dtype(dtype)) return fail(NOVA_B200_ERR_UNSUPPORTED, "linear: dtype must be f32, f16 or bf16");
  if (X->sizes[1] != W->sizes[0] || Y->sizes[0] != X->sizes[0] || Y->sizes[1] != W->sizes[1] ||
      bias->sizes[0] != W->sizes[1])
    return fail(NOVA_B200_ERR_INVALID_ARG, "linear: shapes do not compose");
  if (bias->sizes[0] > 1 && bias->strides[0] != 1) return fail(NOVA_B200_ERR_LAYOUT, "linear: bias must be contiguous");
  const int es = dtype_bytes(dtype);
  nova_b200_gemm_args g{};
  g.struct_size = sizeof(g);
  g.dtype_ab = g.dtype_c = dtype;
  g.act = act;
  g.init = NOVA_B200_INIT_BIAS_ROW;
  g.batch = 1; g.M = X->sizes[0]; g.K = X->sizes[1]; g.N = W->sizes[1];
  int32_t st, tc = 0;
  if ((st = inner2(X->sizes, X->strides, &g.lda, &g.trans_a, "linear X")) != NOVA_B200_OK) return st;
  if ((st = inner2(W->sizes, W->strides, &g.ldb, &g.trans_b, "linear W")) != NOVA_B200_OK) return st;
  if ((st = inner2(Y->sizes, Y->strides, &g.ldc, &tc, "linear Y")) != NOVA_B200_OK) return st;
  if (tc) return fail(NOVA_B200_ERR_LAYOUT, "linear: Y must have unit inner stride");
  g.A = static_cast<char*>(X->aligned) + X->offset * es;
  g.B = static_cast<char*>(W->aligned) + W->offset * es;
  g.C = static_cast<char*>(Y->aligned) + Y->offset * es;
  g.bias = static_cast<char*>(bias->aligned) + bias->offset * es;
  const bool dev = is_device_pointer(g.C);
  if (dev != is_device_pointer(g.bias))
    return fail(NOVA_B200_ERR_INVALID_ARG, "linear: operands must be all host or all device memory");
  return run_descriptor_gemm(g);
}

}  // extern "C"
