// Executor of the textual front-end and its C-ABI entry points (nova_b200_module_*): runs a planned
// function by calling the same entry points a lowered module would call (nova_b200_gemm, _layer_norm,
// _softmax, _gather, _activation, _add_rowbcast).  Intermediates come from cudaMallocAsync on the caller's
// stream, the way the reference's generated host code allocates (lib/Transforms/FixGpuLaunch.cpp:49-50).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <memory>
#include <vector>

#include "frontend.h"
#include "runtime.h"

struct nova_b200_module {
  nova::fe::Module module;
};

namespace nova {
namespace fe {
namespace {

struct Value {
  void* ptr = nullptr;
  int32_t dtype = -1;
  std::vector<int64_t> shape, strides;  // strides in elements
  bool contiguous() const {
    int64_t expect = 1;
    for (int i = static_cast<int>(shape.size()) - 1; i >= 0; --i) {
      if (shape[i] != 1 && strides[i] != expect) return false;
      expect *= shape[i];
    }
    return true;
  }
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
  }
};

std::vector<int64_t> row_major(const std::vector<int64_t>& shape) {
  std::vector<int64_t> st(shape.size(), 1);
  for (int i = static_cast<int>(shape.size()) - 2; i >= 0; --i) st[i] = st[i + 1] * shape[i + 1];
  return st;
}

struct Strided6 {
  int64_t shape[6], strides[6];
};

template <int kBytes>
__global__ void strided_copy_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, Strided6 s, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t rem = i, off = 0;
#pragma unroll
    for (int d = 5; d >= 0; --d) {
      const int64_t q = rem / s.shape[d];
      off += (rem - q * s.shape[d]) * s.strides[d];
      rem = q;
    }
#pragma unroll
    for (int b = 0; b < kBytes; ++b) dst[i * kBytes + b] = src[off * kBytes + b];
  }
}

template <typename Tin, typename Tout>
__global__ void cast_kernel(const Tin* __restrict__ x, Tout* __restrict__ y, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    y[i] = static_cast<Tout>(static_cast<float>(x[i]));  // extf / truncf (round to nearest even)
}

// i1 (one byte, 0 / 1) -> float
template <typename Tout>
__global__ void cast_i1_kernel(const uint8_t* __restrict__ x, Tout* __restrict__ y, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    y[i] = static_cast<Tout>(x[i] ? 1.0f : 0.0f);
}

// out[i] = a (cmp) b with right-aligned broadcasting (strides 0 on stretched dims), kind: eq ne lt le gt ge
template <typename T>
__global__ void compare_kernel(const T* __restrict__ a, const T* __restrict__ b, uint8_t* __restrict__ out, Strided6 sa,
                               Strided6 sb, int64_t n, int kind) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int64_t rem = i, oa = 0, ob = 0;
#pragma unroll
    for (int d = 5; d >= 0; --d) {
      const int64_t q = rem / sa.shape[d], r = rem - q * sa.shape[d];
      oa += r * sa.strides[d];
      ob += r * sb.strides[d];
      rem = q;
    }
    const float x = static_cast<float>(a[oa]), y = static_cast<float>(b[ob]);
    const bool v = kind == 0 ? x == y : kind == 1 ? x != y : kind == 2 ? x < y : kind == 3 ? x <= y : kind == 4 ? x > y : x >= y;
    out[i] = v ? 1 : 0;
  }
}

// out[0] = mean over all n elements of (a - b)^2: one CTA, fp32 accumulation in a fixed order (the loss scalar of the
// training-step fixtures; a few thousand elements)
template <typename T>
__global__ void __launch_bounds__(1024) mse_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n) {
  __shared__ float part[1024];
  float acc = 0.0f;
  for (int64_t i = threadIdx.x; i < n; i += 1024) {
    const float d = static_cast<float>(a[i]) - static_cast<float>(b[i]);
    acc = fmaf(d, d, acc);
  }
  part[threadIdx.x] = acc;
  __syncthreads();
  for (int s = 512; s > 0; s >>= 1) {
    if (static_cast<int>(threadIdx.x) < s) part[threadIdx.x] += part[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = static_cast<T>(part[0] / static_cast<float>(n));
}

template <typename T>
__global__ void fill_kernel(T* __restrict__ y, float v, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    y[i] = static_cast<T>(v);
}

int grid_for(int64_t n) { return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, 148 * 16))); }

struct Exec {
  const Function& f;
  const Plan& p;
  cudaStream_t stream;
  std::map<std::string, Value> vals;
  std::vector<void*> owned;
  // f32 intermediates that more than one contraction reads (the logits gradient feeds both backward products of the
  // vocabulary layer): split into hi / lo once and shared (nova_b200_f32_presplit), released when the run ends
  std::map<std::string, std::string> view_root;
  std::map<std::string, int> gemm_reads;
  struct Shared { const void* ptr; int64_t rows, cols, ld; void* handle; };
  std::vector<Shared> shared;

  void count_gemm_reads() {
    auto root_of = [&](const std::string& n) {
      auto it = view_root.find(n);
      return it == view_root.end() ? n : it->second;
    };
    for (const Step& s : p.steps) {
      if ((s.kind == "alias" || s.kind == "reshape" || s.kind == "transpose") && !s.inputs.empty() && !s.outputs.empty())
        view_root[s.outputs[0]] = root_of(s.inputs[0]);
      else if (s.kind == "gemm" && s.inputs.size() >= 2) {
        ++gemm_reads[root_of(s.inputs[0])];
        ++gemm_reads[root_of(s.inputs[1])];
      }
    }
  }
  // Called with an operand of a contraction about to run: shares its split when the value has another reader.
  void maybe_share_split(const std::string& name, const Value& v, int64_t ld, int32_t trans) {
    auto rt = view_root.find(name);
    const std::string& root = rt == view_root.end() ? name : rt->second;
    auto it = gemm_reads.find(root);
    if (it == gemm_reads.end() || it->second < 2 || v.dtype != NOVA_B200_F32 || v.shape.size() < 2) return;
    if (std::find(owned.begin(), owned.end(), v.ptr) == owned.end()) return;  // arguments may be written during the run
    const size_t r = v.shape.size();
    const int64_t rows = trans ? v.shape[r - 1] : v.shape[r - 2], cols = trans ? v.shape[r - 2] : v.shape[r - 1];
    for (const Shared& e : shared)
      if (e.ptr == v.ptr && e.rows == rows && e.cols == cols && e.ld == ld) return;
    void* handle = nullptr;
    if (nova_b200_f32_presplit(v.ptr, rows, cols, ld, stream, &handle) == NOVA_B200_OK)
      shared.push_back(Shared{v.ptr, rows, cols, ld, handle});  // on failure the contraction splits it itself
  }

  ~Exec() {
    for (const Shared& e : shared) nova_b200_f32_presplit_release(e.handle, stream);
    for (void* q : owned) cudaFreeAsync(q, stream);
  }
  std::string canon(const std::string& n) const {
    if (vals.count(n)) return n;
    if (vals.count(n + "#0")) return n + "#0";
    const size_t h = n.find("#0");
    if (h != std::string::npos && vals.count(n.substr(0, h))) return n.substr(0, h);
    return n;
  }
  int32_t get(const std::string& n, Value* out) {
    auto it = vals.find(canon(n));
    if (it == vals.end()) return fail(NOVA_B200_ERR_INVALID_ARG, "front-end: value %" + n + " has no storage");
    *out = it->second;
    return NOVA_B200_OK;
  }
  int32_t alloc(const Type& t, Value* out) {
    out->dtype = t.dtype;
    out->shape = t.shape;
    out->strides = row_major(t.shape);
    const size_t bytes = static_cast<size_t>(std::max<int64_t>(t.numel(), 1)) * dtype_bytes(t.dtype);
    NOVA_CUDA_OK(cudaMallocAsync(&out->ptr, bytes, stream));
    owned.push_back(out->ptr);
    return NOVA_B200_OK;
  }
  const Type& type_of(const std::string& n) const {
    auto it = p.types.find(n);
    if (it != p.types.end()) return it->second;
    it = p.types.find(n + "#0");
    if (it != p.types.end()) return it->second;
    const size_t h = n.find("#0");
    return p.types.at(h == std::string::npos ? n : n.substr(0, h));
  }
  // a contiguous row-major version of v (a copy only when v is a strided view)
  int32_t make_contiguous(const Value& v_in, Value* out) {
    const Value v = v_in;  // callers pass the same object as input and output
    if (v.contiguous()) { *out = v; out->strides = row_major(v.shape); return NOVA_B200_OK; }
    if (v.shape.size() > 6) return fail(NOVA_B200_ERR_UNSUPPORTED, "front-end: strided copy of rank > 6");
    Type t; t.dtype = v.dtype; t.shape = v.shape;
    int32_t st = alloc(t, out);
    if (st != NOVA_B200_OK) return st;
    Strided6 s;
    const int pad = 6 - static_cast<int>(v.shape.size());
    for (int d = 0; d < 6; ++d) {
      s.shape[d] = d < pad ? 1 : v.shape[d - pad];
      s.strides[d] = d < pad ? 0 : v.strides[d - pad];
    }
    const int64_t n = v.numel();
    const uint8_t* src = static_cast<const uint8_t*>(v.ptr);
    uint8_t* dst = static_cast<uint8_t*>(out->ptr);
    switch (dtype_bytes(v.dtype)) {
      case 1: strided_copy_kernel<1><<<grid_for(n), 256, 0, stream>>>(src, dst, s, n); break;
      case 2: strided_copy_kernel<2><<<grid_for(n), 256, 0, stream>>>(src, dst, s, n); break;
      case 4: strided_copy_kernel<4><<<grid_for(n), 256, 0, stream>>>(src, dst, s, n); break;
      default: strided_copy_kernel<8><<<grid_for(n), 256, 0, stream>>>(src, dst, s, n); break;
    }
    NOVA_CUDA_OK(cudaGetLastError());
    return NOVA_B200_OK;
  }

  int32_t run_gemm(const Step& s) {
    Value a, b;
    int32_t st;
    if ((st = get(s.inputs[0], &a)) != NOVA_B200_OK || (st = get(s.inputs[1], &b)) != NOVA_B200_OK) return st;
    const bool va = a.shape.size() == 1, vb = b.shape.size() == 1;
    if (va) { a.shape.insert(a.shape.begin(), 1); a.strides.insert(a.strides.begin(), 0); }
    if (vb) { b.shape.push_back(1); b.strides.push_back(1); }
    const Type& out_t = type_of(s.outputs[0]);
    Value c;
    if ((st = alloc(out_t, &c)) != NOVA_B200_OK) return st;
    nova_b200_gemm_args g{};
    g.struct_size = sizeof(g);
    g.dtype_ab = a.dtype;
    g.dtype_c = out_t.dtype;
    const size_t ra = a.shape.size(), rb = b.shape.size();
    g.M = a.shape[ra - 2]; g.K = a.shape[ra - 1]; g.N = b.shape[rb - 1];
    int64_t batch = 1;
    // batch = product of the output's leading dims (all but the last two of the promoted shape)
    {
      std::vector<int64_t> os = out_t.shape;
      if (va) os.insert(os.end() - (vb ? 0 : 1), 1);
      if (vb) os.push_back(1);
      for (size_t i = 0; i + 2 < os.size(); ++i) batch *= os[i];
    }
    g.batch = batch;
    // each operand: inner two dims may be a transposed view; leading dims must collapse to one stride (or be absent)
    auto inner = [&](Value& v, int64_t* ld, int32_t* trans, int64_t* bstride) -> int32_t {
      for (int attempt = 0; attempt < 2; ++attempt) {
        const size_t r = v.shape.size();
        const int64_t rows = v.shape[r - 2], cols = v.shape[r - 1], sr = v.strides[r - 2], sc = v.strides[r - 1];
        bool ok = true;
        if (sc == 1 || cols == 1) { *trans = 0; *ld = rows > 1 ? sr : std::max(sr, cols); }
        else if (sr == 1 || rows == 1) { *trans = 1; *ld = cols > 1 ? sc : std::max(sc, rows); }
        else ok = false;
        int64_t lead = 1;
        for (size_t i = 0; i + 2 < r; ++i) lead *= v.shape[i];
        if (ok && lead > 1) {
          // leading dims must walk memory with one stride
          int64_t expect = v.strides[r - 3];
          for (int i = static_cast<int>(r) - 4; i >= 0 && ok; --i) {
            if (v.shape[i] != 1 && v.strides[i] != expect * v.shape[i + 1]) ok = false;
            expect = v.strides[i];
          }
          *bstride = v.strides[r - 3];
          if (lead != batch) ok = false;  // broadcast across SOME batch dims only: materialise below
        } else {
          *bstride = 0;
        }
        if (ok) return NOVA_B200_OK;
        if (attempt == 1) break;
        Value cc;
        const int32_t st2 = make_contiguous(v, &cc);
        if (st2 != NOVA_B200_OK) return st2;
        v = cc;
      }
      return fail(NOVA_B200_ERR_LAYOUT, "front-end: operand layout cannot be expressed (partial batch broadcast)");
    };
    if ((st = inner(a, &g.lda, &g.trans_a, &g.batch_stride_a)) != NOVA_B200_OK) return st;
    if ((st = inner(b, &g.ldb, &g.trans_b, &g.batch_stride_b)) != NOVA_B200_OK) return st;
    g.A = a.ptr; g.B = b.ptr; g.C = c.ptr;
    if (g.batch == 1) {
      maybe_share_split(s.inputs[0], a, g.lda, g.trans_a);
      maybe_share_split(s.inputs[1], b, g.ldb, g.trans_b);
    }
    g.ldc = g.N;
    g.batch_stride_c = g.M * g.N;
    g.act = s.act;
    Value aux;
    if (!s.bias.empty()) {
      if ((st = get(s.bias, &aux)) != NOVA_B200_OK || (st = make_contiguous(aux, &aux)) != NOVA_B200_OK) return st;
      g.init = NOVA_B200_INIT_BIAS_ROW;
      g.bias = aux.ptr;
    }
    if (!s.residual.empty()) {
      if ((st = get(s.residual, &aux)) != NOVA_B200_OK || (st = make_contiguous(aux, &aux)) != NOVA_B200_OK) return st;
      g.init = s.bias.empty() ? NOVA_B200_INIT_RESIDUAL_FULL : NOVA_B200_INIT_BIAS_AND_RESIDUAL;
      g.residual = aux.ptr;
      g.ldr = g.N;
      g.batch_stride_r = g.M * g.N;
    }
    if (s.act == NOVA_B200_ACT_GELU_TANH_GRAD) {
      if ((st = get(s.act_operand, &aux)) != NOVA_B200_OK || (st = make_contiguous(aux, &aux)) != NOVA_B200_OK) return st;
      g.residual = aux.ptr;
      g.ldr = g.N;
      g.batch_stride_r = g.M * g.N;
    }
    st = nova_b200_gemm(&g, stream);
    if (st != NOVA_B200_OK) return st;
    vals[s.outputs[0]] = c;
    return NOVA_B200_OK;
  }

  int32_t run_step(const Step& s) {
    int32_t st;
    const std::string& k = s.kind;
    if (k == "gemm") return run_gemm(s);
    if (k == "empty") { Value v; if ((st = alloc(type_of(s.outputs[0]), &v)) != NOVA_B200_OK) return st; vals[s.outputs[0]] = v; return NOVA_B200_OK; }
    if (k == "alias") { Value v; if ((st = get(s.inputs[0], &v)) != NOVA_B200_OK) return st; vals[s.outputs[0]] = v; return NOVA_B200_OK; }
    if (k == "reshape") {
      Value v;
      if ((st = get(s.inputs[0], &v)) != NOVA_B200_OK || (st = make_contiguous(v, &v)) != NOVA_B200_OK) return st;
      v.shape = type_of(s.outputs[0]).shape;  // row-major reinterpretation, no data movement
      v.strides = row_major(v.shape);
      vals[s.outputs[0]] = v;
      return NOVA_B200_OK;
    }
    if (k == "transpose") {
      Value v;
      if ((st = get(s.inputs[0], &v)) != NOVA_B200_OK) return st;
      const int64_t r = static_cast<int64_t>(v.shape.size());
      int64_t a1 = s.attrs.count("axes1") ? s.attrs.at("axes1") : -1, a2 = s.attrs.count("axes2") ? s.attrs.at("axes2") : -2;
      if (a1 < 0) a1 += r;
      if (a2 < 0) a2 += r;
      std::swap(v.shape[a1], v.shape[a2]);      // a view: a following contraction reads it through trans_a / trans_b
      std::swap(v.strides[a1], v.strides[a2]);
      vals[s.outputs[0]] = v;
      return NOVA_B200_OK;
    }
    if (k == "store_to_arg") {
      Value src, dst;
      if ((st = get(s.inputs[0], &src)) != NOVA_B200_OK || (st = get(s.inputs[1], &dst)) != NOVA_B200_OK) return st;
      if ((st = make_contiguous(src, &src)) != NOVA_B200_OK) return st;
      NOVA_CUDA_OK(cudaMemcpyAsync(dst.ptr, src.ptr, static_cast<size_t>(src.numel()) * dtype_bytes(src.dtype),
                                   cudaMemcpyDeviceToDevice, stream));
      return NOVA_B200_OK;
    }
    // everything below works on contiguous inputs and writes a fresh contiguous output
    std::vector<Value> in(s.inputs.size());
    for (size_t i = 0; i < s.inputs.size(); ++i)
      if ((st = get(s.inputs[i], &in[i])) != NOVA_B200_OK || (st = make_contiguous(in[i], &in[i])) != NOVA_B200_OK) return st;
    std::vector<Value> out(s.outputs.size());
    for (size_t i = 0; i < s.outputs.size(); ++i)
      if ((st = alloc(type_of(s.outputs[i]), &out[i])) != NOVA_B200_OK) return st;
    const int64_t n = in.empty() ? out[0].numel() : in[0].numel();
    if (k == "activation") st = nova_b200_activation(in[0].ptr, out[0].ptr, n, in[0].dtype, s.act, stream);
    else if (k == "sce" || k == "sce_backward") {
      const int64_t Cn = in[0].shape.back();
      const int64_t rows = in[0].numel() / std::max<int64_t>(Cn, 1);
      if (k == "sce") st = nova_b200_sce(in[0].ptr, in[1].ptr, out[0].ptr, out[1].ptr, rows, Cn, in[0].dtype, in[1].dtype, nullptr, stream);
      else st = nova_b200_sce_backward_scaled(in[0].ptr, in[1].ptr, out[0].ptr, rows, Cn, in[0].dtype, in[1].dtype,
                                              s.attrs.count("scaled") ? static_cast<float>(s.fvalue) : 1.0f, stream);
    } else if (k == "scatter_add") {
      const int64_t r = static_cast<int64_t>(in[0].shape.size());
      int64_t axis = s.attrs.count("axis") ? s.attrs.at("axis") : 0;
      if (axis < 0) axis += r;
      int64_t pre = 1, post = 1;
      for (int64_t i = 0; i < axis; ++i) pre *= in[0].shape[i];
      for (int64_t i = axis + 1; i < r; ++i) post *= in[0].shape[i];
      NOVA_CUDA_OK(cudaMemcpyAsync(out[0].ptr, in[0].ptr, static_cast<size_t>(in[0].numel()) * dtype_bytes(in[0].dtype),
                                   cudaMemcpyDeviceToDevice, stream));
      st = nova_b200_scatter_add(out[0].ptr, in[1].ptr, in[2].ptr, pre, in[0].shape[axis], post, in[2].shape[axis],
                                 in[1].dtype, in[0].dtype, nullptr, stream);
    } else if (k == "layer_norm_backward") {
      const int64_t D = in[1].shape.back();
      st = nova_b200_layer_norm_backward(in[0].ptr, in[1].ptr, in[2].ptr, in[3].ptr, in[4].ptr, out[0].ptr, out[1].ptr,
                                         out[2].ptr, in[1].numel() / std::max<int64_t>(D, 1), D, in[1].dtype, stream);
    } else if (k == "gelu_backward") st = nova_b200_gelu_backward(in[0].ptr, in[1].ptr, out[0].ptr, n, in[0].dtype, stream);
    else if (k == "binary") {
      // right-aligned broadcast: an operand dim of extent 1 (or a missing leading dim) gets stride 0
      const std::vector<int64_t>& os = out[0].shape;
      const int r = static_cast<int>(os.size());
      if (r > 6) return fail(NOVA_B200_ERR_UNSUPPORTED, "front-end: elementwise op of rank > 6");
      int64_t shp[6], sa[6], sb[6];
      auto strides_for = [&](const Value& v, int64_t* dst) {
        const int pad = r - static_cast<int>(v.shape.size());
        for (int d = 0; d < r; ++d) dst[d] = (d < pad || v.shape[d - pad] == 1) ? 0 : v.strides[d - pad];
      };
      for (int d = 0; d < r; ++d) shp[d] = os[d];
      strides_for(in[0], sa);
      strides_for(in[1], sb);
      st = nova_b200_binary(in[0].ptr, in[1].ptr, out[0].ptr, r, shp, sa, sb, static_cast<int32_t>(s.attrs.at("op")), in[0].dtype, stream);
    } else if (k == "reduce_sum") {
      const int64_t lead = s.attrs.at("lead");
      int64_t rows = 1;
      for (int64_t i = 0; i < lead; ++i) rows *= in[0].shape[i];
      const int64_t cols = n / std::max<int64_t>(rows, 1);
      st = nova_b200_column_sum(in[0].ptr, out[0].ptr, rows, cols, in[0].dtype, stream);
    } else if (k == "column_sum") {
      const int64_t cols = in[0].shape.back();
      st = nova_b200_column_sum(in[0].ptr, out[0].ptr, n / std::max<int64_t>(cols, 1), cols, in[0].dtype, stream);
    } else if (k == "softmax") {
      const int64_t r = static_cast<int64_t>(in[0].shape.size());
      int64_t dim = s.attrs.count("dimension") ? s.attrs.at("dimension") : -1;
      if (dim > r) dim = r - 1;  // as the reference normalises it (NovaToLinalgGeneric.cpp:1442-1443)
      if (dim < 0) dim += r;
      if (dim != r - 1) return fail(NOVA_B200_ERR_UNSUPPORTED, "front-end: softmax along a non-last dimension is outside the supported subset");
      const int64_t D = in[0].shape.back();
      st = nova_b200_softmax(in[0].ptr, out[0].ptr, n / std::max<int64_t>(D, 1), D, in[0].dtype, stream);
    } else if (k == "layer_norm") {
      const int64_t D = in[0].shape.back();
      st = nova_b200_layer_norm(in[0].ptr, in[1].ptr, in[2].ptr, out[0].ptr, out[1].ptr, out[2].ptr,
                                n / std::max<int64_t>(D, 1), D, in[0].dtype, stream);
    } else if (k == "gather") {
      const Value &x = in[0], &idx = in[1];
      int64_t axis = s.attrs.count("axis") ? s.attrs.at("axis") : 0;
      if (axis < 0) axis += static_cast<int64_t>(x.shape.size());
      size_t batch_dims = 0;
      for (size_t i = 0; i < std::min<size_t>(axis, idx.shape.size()); ++i) {
        if (x.shape[i] != idx.shape[i]) break;
        ++batch_dims;
      }
      const bool batched = axis > 0 && batch_dims == static_cast<size_t>(axis);
      if (axis > 0 && !batched && batch_dims != 0) return fail(NOVA_B200_ERR_UNSUPPORTED, "front-end: partially batched gather");
      int64_t pre = 1, post = 1, n_idx = 1;
      for (int64_t i = 0; i < axis; ++i) pre *= x.shape[i];
      for (size_t i = axis + 1; i < x.shape.size(); ++i) post *= x.shape[i];
      for (size_t i = batched ? batch_dims : 0; i < idx.shape.size(); ++i) n_idx *= idx.shape[i];
      st = nova_b200_gather(x.ptr, idx.ptr, out[0].ptr, pre, x.shape[axis], post, n_idx, idx.dtype, batched ? 1 : 0,
                            dtype_bytes(x.dtype), nullptr, stream);
    } else if (k == "compare") {
      const std::vector<int64_t>& os = out[0].shape;
      const int r = static_cast<int>(os.size());
      if (r > 6) return fail(NOVA_B200_ERR_UNSUPPORTED, "front-end: compare of rank > 6");
      Strided6 sa, sb;
      auto fill6 = [&](const Value& v, Strided6* dst) {
        const int pad_out = 6 - r, pad_v = r - static_cast<int>(v.shape.size());
        for (int d = 0; d < 6; ++d) {
          const int od = d - pad_out;  // index into the output shape
          dst->shape[d] = od < 0 ? 1 : os[od];
          const int vd = od - pad_v;
          dst->strides[d] = (od < 0 || vd < 0 || v.shape[vd] == 1) ? 0 : v.strides[vd];
        }
      };
      fill6(in[0], &sa);
      fill6(in[1], &sb);
      const int64_t m = out[0].numel();
      const int kind = static_cast<int>(s.attrs.at("op"));
      uint8_t* o = static_cast<uint8_t*>(out[0].ptr);
      if (in[0].dtype == NOVA_B200_F32) compare_kernel<float><<<grid_for(m), 256, 0, stream>>>(static_cast<const float*>(in[0].ptr), static_cast<const float*>(in[1].ptr), o, sa, sb, m, kind);
      else if (in[0].dtype == NOVA_B200_F16) compare_kernel<__half><<<grid_for(m), 256, 0, stream>>>(static_cast<const __half*>(in[0].ptr), static_cast<const __half*>(in[1].ptr), o, sa, sb, m, kind);
      else compare_kernel<__nv_bfloat16><<<grid_for(m), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(in[0].ptr), static_cast<const __nv_bfloat16*>(in[1].ptr), o, sa, sb, m, kind);
      NOVA_CUDA_OK(cudaGetLastError());
      st = NOVA_B200_OK;
    } else if (k == "mse") {
      if (in[0].dtype == NOVA_B200_F32) mse_kernel<float><<<1, 1024, 0, stream>>>(static_cast<const float*>(in[0].ptr), static_cast<const float*>(in[1].ptr), static_cast<float*>(out[0].ptr), n);
      else if (in[0].dtype == NOVA_B200_F16) mse_kernel<__half><<<1, 1024, 0, stream>>>(static_cast<const __half*>(in[0].ptr), static_cast<const __half*>(in[1].ptr), static_cast<__half*>(out[0].ptr), n);
      else mse_kernel<__nv_bfloat16><<<1, 1024, 0, stream>>>(static_cast<const __nv_bfloat16*>(in[0].ptr), static_cast<const __nv_bfloat16*>(in[1].ptr), static_cast<__nv_bfloat16*>(out[0].ptr), n);
      NOVA_CUDA_OK(cudaGetLastError());
      st = NOVA_B200_OK;
    } else if (k == "cast" && in[0].dtype == NOVA_B200_I1) {
      const uint8_t* x = static_cast<const uint8_t*>(in[0].ptr);
      if (out[0].dtype == NOVA_B200_F32) cast_i1_kernel<float><<<grid_for(n), 256, 0, stream>>>(x, static_cast<float*>(out[0].ptr), n);
      else if (out[0].dtype == NOVA_B200_F16) cast_i1_kernel<__half><<<grid_for(n), 256, 0, stream>>>(x, static_cast<__half*>(out[0].ptr), n);
      else cast_i1_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>(x, static_cast<__nv_bfloat16*>(out[0].ptr), n);
      NOVA_CUDA_OK(cudaGetLastError());
      st = NOVA_B200_OK;
    } else if (k == "cast") {
      const int32_t di = in[0].dtype, dout = out[0].dtype;
#define NOVA_CAST(TI, TO) cast_kernel<TI, TO><<<grid_for(n), 256, 0, stream>>>(static_cast<const TI*>(in[0].ptr), static_cast<TO*>(out[0].ptr), n)
      if (di == NOVA_B200_F32 && dout == NOVA_B200_F16) NOVA_CAST(float, __half);
      else if (di == NOVA_B200_F32 && dout == NOVA_B200_BF16) NOVA_CAST(float, __nv_bfloat16);
      else if (di == NOVA_B200_F16 && dout == NOVA_B200_F32) NOVA_CAST(__half, float);
      else if (di == NOVA_B200_BF16 && dout == NOVA_B200_F32) NOVA_CAST(__nv_bfloat16, float);
      else if (di == NOVA_B200_F16 && dout == NOVA_B200_BF16) NOVA_CAST(__half, __nv_bfloat16);
      else if (di == NOVA_B200_BF16 && dout == NOVA_B200_F16) NOVA_CAST(__nv_bfloat16, __half);
      else NOVA_CUDA_OK(cudaMemcpyAsync(out[0].ptr, in[0].ptr, static_cast<size_t>(n) * dtype_bytes(di), cudaMemcpyDeviceToDevice, stream));
#undef NOVA_CAST
      NOVA_CUDA_OK(cudaGetLastError());
      st = NOVA_B200_OK;
    } else if (k == "fill" || k == "constant") {
      const int64_t m = out[0].numel();
      if (out[0].dtype == NOVA_B200_F32) fill_kernel<float><<<grid_for(m), 256, 0, stream>>>(static_cast<float*>(out[0].ptr), static_cast<float>(s.fvalue), m);
      else if (out[0].dtype == NOVA_B200_F16) fill_kernel<__half><<<grid_for(m), 256, 0, stream>>>(static_cast<__half*>(out[0].ptr), static_cast<float>(s.fvalue), m);
      else fill_kernel<__nv_bfloat16><<<grid_for(m), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(out[0].ptr), static_cast<float>(s.fvalue), m);
      NOVA_CUDA_OK(cudaGetLastError());
      st = NOVA_B200_OK;
    } else {
      return fail(NOVA_B200_ERR_UNSUPPORTED, "front-end: no executor for step '" + k + "'");
    }
    if (st != NOVA_B200_OK) return st;
    for (size_t i = 0; i < s.outputs.size(); ++i) vals[s.outputs[i]] = out[i];
    return NOVA_B200_OK;
  }
};

bool same_shape(const Type& t, const nova_b200_tensor& x) {
  if (x.rank != static_cast<int32_t>(t.shape.size()) || x.dtype != t.dtype) return false;
  for (int i = 0; i < x.rank; ++i)
    if (x.shape[i] != t.shape[i]) return false;
  return true;
}

}  // namespace
}  // namespace fe
}  // namespace nova

using namespace nova;

extern "C" {

int32_t nova_b200_module_parse(const char* text, nova_b200_module** out) {
  if (!text || !out) return fail(NOVA_B200_ERR_INVALID_ARG, "module_parse: null argument");
  auto m = std::make_unique<nova_b200_module>();
  std::string err;
  if (!fe::parse_module(text, &m->module, &err)) return fail(NOVA_B200_ERR_INVALID_ARG, "module_parse: " + err);
  // plan every function once so that unsupported ops and shape errors surface at parse time
  for (const fe::Function& f : m->module.functions) {
    fe::Plan p;
    if (!fe::plan_function(f, &p, &err)) return fail(NOVA_B200_ERR_UNSUPPORTED, "module_parse: @" + f.name + ": " + err);
  }
  *out = m.release();
  return NOVA_B200_OK;
}

void nova_b200_module_free(nova_b200_module* m) { delete m; }

int32_t nova_b200_module_signature(const nova_b200_module* m, const char* func, int32_t index, int32_t is_result,
                                   nova_b200_tensor* out, int32_t* count) {
  if (!m || !func) return fail(NOVA_B200_ERR_INVALID_ARG, "module_signature: null argument");
  const fe::Function* f = m->module.find(func);
  if (!f) return fail(NOVA_B200_ERR_INVALID_ARG, std::string("module_signature: no function @") + func);
  fe::Plan p;
  std::string err;
  if (!fe::plan_function(*f, &p, &err)) return fail(NOVA_B200_ERR_UNSUPPORTED, err);
  const int32_t n = static_cast<int32_t>(is_result ? p.results.size() : f->arg_types.size());
  if (count) *count = n;
  if (!out) return NOVA_B200_OK;
  if (index < 0 || index >= n) return fail(NOVA_B200_ERR_INVALID_ARG, "module_signature: index out of range");
  fe::Type t;
  if (is_result) {
    auto it = p.types.find(p.results[index]);
    if (it == p.types.end()) it = p.types.find(p.results[index] + "#0");
    t = it->second;
  } else {
    t = f->arg_types[index];
  }
  if (t.shape.size() > 6) return fail(NOVA_B200_ERR_UNSUPPORTED, "module_signature: rank > 6");
  std::memset(out, 0, sizeof(*out));
  out->dtype = t.dtype;
  out->rank = static_cast<int32_t>(t.shape.size());
  for (size_t i = 0; i < t.shape.size(); ++i) out->shape[i] = t.shape[i];
  return NOVA_B200_OK;
}

int32_t nova_b200_module_plan(const nova_b200_module* m, const char* func, char* buf, int64_t buflen) {
  if (!m || !func || !buf || buflen <= 0) return fail(NOVA_B200_ERR_INVALID_ARG, "module_plan: bad argument");
  const fe::Function* f = m->module.find(func);
  if (!f) return fail(NOVA_B200_ERR_INVALID_ARG, std::string("module_plan: no function @") + func);
  fe::Plan p;
  std::string err;
  if (!fe::plan_function(*f, &p, &err)) return fail(NOVA_B200_ERR_UNSUPPORTED, err);
  const std::string s = fe::describe_plan(*f, p);
  std::strncpy(buf, s.c_str(), static_cast<size_t>(buflen) - 1);
  buf[buflen - 1] = 0;
  return NOVA_B200_OK;
}

int32_t nova_b200_module_run(const nova_b200_module* m, const char* func, const nova_b200_tensor* args, int32_t n_args,
                             nova_b200_tensor* results, int32_t n_results, void* stream) {
  if (!m || !func) return fail(NOVA_B200_ERR_INVALID_ARG, "module_run: null argument");
  const fe::Function* f = m->module.find(func);
  if (!f) return fail(NOVA_B200_ERR_INVALID_ARG, std::string("module_run: no function @") + func);
  fe::Plan p;
  std::string err;
  if (!fe::plan_function(*f, &p, &err)) return fail(NOVA_B200_ERR_UNSUPPORTED, err);
  if (n_args != static_cast<int32_t>(f->arg_types.size()) || n_results != static_cast<int32_t>(p.results.size()))
    return fail(NOVA_B200_ERR_INVALID_ARG, "module_run: wrong number of arguments or results");
  if ((n_args && !args) || (n_results && !results)) return fail(NOVA_B200_ERR_INVALID_ARG, "module_run: null tensor list");
  int32_t st = NOVA_B200_OK;
  if (!current_context(&st)) return st;
  {
    // Intermediates come from the device's default stream-ordered pool.  With the pool's release threshold at its
    // default of 0 every synchronisation hands the freed blocks back to the driver and the next run allocates them
    // again (measured on the GPT fixture: 10.4 ms per step against 8.1 ms): keep them, unless the application has
    // already chosen a threshold of its own.
    static std::mutex mu;
    static std::vector<int> done;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) {
      std::lock_guard<std::mutex> lock(mu);
      if (std::find(done.begin(), done.end(), dev) == done.end()) {
        done.push_back(dev);
        cudaMemPool_t pool = nullptr;
        uint64_t cur = 0;
        if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess &&
            cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &cur) == cudaSuccess && cur == 0) {
          uint64_t keep = ~0ull;
          cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
        }
        cudaGetLastError();
      }
    }
  }
  fe::Exec ex{*f, p, static_cast<cudaStream_t>(stream), {}, {}};
  ex.count_gemm_reads();
  for (int32_t i = 0; i < n_args; ++i) {
    if (!fe::same_shape(f->arg_types[i], args[i]))
      return fail(NOVA_B200_ERR_INVALID_ARG, "module_run: argument " + std::to_string(i) + " does not match the signature");
    if (!args[i].data && f->arg_types[i].numel() > 0) return fail(NOVA_B200_ERR_INVALID_ARG, "module_run: null argument data");
    fe::Value v;
    v.ptr = args[i].data; v.dtype = args[i].dtype; v.shape = f->arg_types[i].shape; v.strides = fe::row_major(v.shape);
    ex.vals[f->arg_names[i]] = v;
  }
  for (const fe::Step& s : p.steps) {
    st = ex.run_step(s);
    if (st != NOVA_B200_OK) return st;
  }
  for (int32_t i = 0; i < n_results; ++i) {
    fe::Value v;
    if ((st = ex.get(p.results[i], &v)) != NOVA_B200_OK) return st;
    fe::Type t; t.dtype = v.dtype; t.shape = v.shape;
    if (!fe::same_shape(t, results[i]))
      return fail(NOVA_B200_ERR_INVALID_ARG, "module_run: result " + std::to_string(i) + " buffer does not match the inferred type");
    if ((st = ex.make_contiguous(v, &v)) != NOVA_B200_OK) return st;
    if (v.numel() > 0)
      NOVA_CUDA_OK(cudaMemcpyAsync(results[i].data, v.ptr, static_cast<size_t>(v.numel()) * dtype_bytes(v.dtype),
                                   cudaMemcpyDeviceToDevice, ex.stream));
  }
  return NOVA_B200_OK;
}

int32_t nova_b200_module_call_ciface(const nova_b200_module* m, const char* func, void* result, void** args) {
  if (!m || !func) return fail(NOVA_B200_ERR_INVALID_ARG, "module_call_ciface: null argument");
  const fe::Function* f = m->module.find(func);
  if (!f) return fail(NOVA_B200_ERR_INVALID_ARG, std::string("module_call_ciface: no function @") + func);
  fe::Plan p;
  std::string err;
  if (!fe::plan_function(*f, &p, &err)) return fail(NOVA_B200_ERR_UNSUPPORTED, err);
  const int32_t n_args = static_cast<int32_t>(f->arg_types.size()), n_results = static_cast<int32_t>(p.results.size());
  if ((n_args && !args) || (n_results && !result)) return fail(NOVA_B200_ERR_INVALID_ARG, "module_call_ciface: null descriptor list");
  int32_t st = NOVA_B200_OK;
  if (!current_context(&st)) return st;

  struct Staged { void* dev = nullptr; void* host = nullptr; size_t bytes = 0; };
  std::vector<Staged> temps;       // device copies of host buffers (inputs and outputs)
  std::vector<Staged> copy_back;   // outputs that live in host memory
  auto cleanup = [&]() { for (Staged& t : temps) cudaFree(t.dev); };
  auto is_device = [](const void* ptr) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) { cudaGetLastError(); return false; }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
  };
  // descriptor {allocated, aligned, offset, sizes[R], strides[R]} -> a contiguous row-major tensor on the device
  auto bind = [&](const int64_t* d, const fe::Type& t, bool is_output, const std::string& what, nova_b200_tensor* out) -> int32_t {
    const int rank = static_cast<int>(t.shape.size());
    if (rank > 6) return fail(NOVA_B200_ERR_UNSUPPORTED, what + ": rank > 6");
    const int64_t* sizes = d + 3;
    const int64_t* strides = d + 3 + rank;
    int64_t expect = 1;
    for (int i = rank - 1; i >= 0; --i) {
      if (sizes[i] != t.shape[i]) return fail(NOVA_B200_ERR_INVALID_ARG, what + ": descriptor sizes do not match the signature");
      if (sizes[i] != 1 && strides[i] != expect) return fail(NOVA_B200_ERR_LAYOUT, what + ": descriptor is not row-major contiguous");
      expect *= sizes[i];
    }
    const int es = dtype_bytes(t.dtype);
    void* aligned = reinterpret_cast<void*>(static_cast<uintptr_t>(d[1]));
    if (!aligned && t.numel() > 0) return fail(NOVA_B200_ERR_INVALID_ARG, what + ": null buffer (results are caller-provided)");
    char* ptr = static_cast<char*>(aligned) + d[2] * es;
    const size_t bytes = static_cast<size_t>(t.numel()) * es;
    std::memset(out, 0, sizeof(*out));
    out->dtype = t.dtype;
    out->rank = rank;
    for (int i = 0; i < rank; ++i) out->shape[i] = t.shape[i];
    if (bytes == 0 || is_device(ptr)) {
      out->data = ptr;
      return NOVA_B200_OK;
    }
    Staged sgd;
    sgd.host = ptr;
    sgd.bytes = bytes;
    NOVA_CUDA_OK(cudaMalloc(&sgd.dev, bytes));
    temps.push_back(sgd);
    if (!is_output) NOVA_CUDA_OK(cudaMemcpyAsync(sgd.dev, ptr, bytes, cudaMemcpyHostToDevice, nullptr));
    else copy_back.push_back(sgd);
    out->data = sgd.dev;
    return NOVA_B200_OK;
  };
  std::vector<nova_b200_tensor> in(static_cast<size_t>(n_args)), outs(static_cast<size_t>(n_results));
  for (int32_t i = 0; i < n_args; ++i) {
    if (!args[i]) { cleanup(); return fail(NOVA_B200_ERR_INVALID_ARG, "module_call_ciface: null argument descriptor"); }
    st = bind(static_cast<const int64_t*>(args[i]), f->arg_types[i], false, "argument " + std::to_string(i), &in[i]);
    if (st != NOVA_B200_OK) { cleanup(); return st; }
  }
  const int64_t* rd = static_cast<const int64_t*>(result);
  for (int32_t i = 0; i < n_results; ++i) {
    auto it = p.types.find(p.results[i]);
    if (it == p.types.end()) it = p.types.find(p.results[i] + "#0");
    if (it == p.types.end()) { cleanup(); return fail(NOVA_B200_ERR_INVALID_ARG, "module_call_ciface: untyped result"); }
    st = bind(rd, it->second, true, "result " + std::to_string(i), &outs[i]);
    if (st != NOVA_B200_OK) { cleanup(); return st; }
    rd += 3 + 2 * it->second.shape.size();
  }
  st = nova_b200_module_run(m, func, in.data(), n_args, outs.data(), n_results, nullptr);
  if (st == NOVA_B200_OK) {
    for (Staged& c : copy_back)
      if (cudaMemcpyAsync(c.host, c.dev, c.bytes, cudaMemcpyDeviceToHost, nullptr) != cudaSuccess) st = fail(NOVA_B200_ERR_CUDA, "module_call_ciface: copy back failed");
  }
  if (cudaStreamSynchronize(nullptr) != cudaSuccess && st == NOVA_B200_OK) st = fail(NOVA_B200_ERR_CUDA, "module_call_ciface: synchronize failed");
  cleanup();
  return st;
}

}  // extern "C"
