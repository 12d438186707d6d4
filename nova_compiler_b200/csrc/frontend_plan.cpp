// Shape / dtype inference and fusion for the textual front-end (see frontend.h).  No GPU needed.
//
// Inference follows the reference's op definitions: MatmulOp::inferReturnTypes
// (lib/Dialect/nova/NovaOps.cpp:1116-1285: [...,M,K] x [...,K,N], numpy batch broadcast, K must match),
// LinearOp (:2075-2103: rank 2 or 3 input), GatherOp (:1898-1946: leading equal dims are batch dims),
// ReshapeOp verify (:1885-1895: equal element count), LayerNormOp (:2032-2054: stats drop the last dim).
// One deliberate difference: 16-bit contractions keep their input dtype (the reference infers f16 for
// all of them, :1198).
//
// Fusion mirrors FuseMatmulBias (lib/Transforms/FuseMatmulBias.cpp:95-193: a matmul whose only real
// consumer is an elementwise add takes the other addend as its accumulator init) and the epilogue
// classification (lib/Transforms/LLVMGPU/Config/NovaKernelConfig.cpp:1876-1895: a trailing ReLU / GELU
// within reach of the contraction runs in its epilogue).
#include <set>
#include <sstream>

#include "frontend.h"

namespace nova {
namespace fe {
namespace {

const char* dtype_name(int32_t d) {
  switch (d) {
    case NOVA_B200_F32: return "f32";
    case NOVA_B200_F16: return "f16";
    case NOVA_B200_BF16: return "bf16";
    case NOVA_B200_I16: return "i16";
    case NOVA_B200_I32: return "i32";
    case NOVA_B200_I64: return "i64";
    case NOVA_B200_I1: return "i1";
    default: return "?";
  }
}

std::string type_str(const Type& t) {
  std::ostringstream o;
  o << "tensor<";
  for (int64_t d : t.shape) o << d << "x";
  o << dtype_name(t.dtype) << ">";
  return o.str();
}

bool is_float(int32_t d) { return d == NOVA_B200_F32 || d == NOVA_B200_F16 || d == NOVA_B200_BF16; }

struct Ctx {
  const Function& f;
  Plan& p;
  std::string* err;
  std::map<std::string, int> uses;            // SSA name -> number of uses
  std::map<std::string, const Op*> producer;  // SSA name -> defining op
  std::set<const Op*> absorbed;
  bool fail(const Op& op, const std::string& msg) {
    *err = "line " + std::to_string(op.line) + " (" + op.name + "): " + msg;
    return false;
  }
  std::string canon(const std::string& n) const {  // %x and %x#0 name the same value
    if (p.types.count(n)) return n;
    if (p.types.count(n + "#0")) return n + "#0";
    const size_t h = n.find("#0");
    if (h != std::string::npos && p.types.count(n.substr(0, h))) return n.substr(0, h);
    return n;
  }
  const Type* type_of(const std::string& n) const {
    auto it = p.types.find(canon(n));
    return it == p.types.end() ? nullptr : &it->second;
  }
};

bool broadcast_batch(const std::vector<int64_t>& a, const std::vector<int64_t>& b, std::vector<int64_t>* out) {
  const size_t n = std::max(a.size(), b.size());
  out->assign(n, 1);
  for (size_t i = 0; i < n; ++i) {
    const int64_t da = i < n - a.size() ? 1 : a[i - (n - a.size())];
    const int64_t db = i < n - b.size() ? 1 : b[i - (n - b.size())];
    if (da != db && da != 1 && db != 1) return false;
    (*out)[i] = da == 1 ? db : da;
  }
  return true;
}

// b broadcasts along the rows of a: [N], [1,N], [1,1,N] ... against [..., N]
bool is_row_broadcast(const Type& a, const Type& b) {
  if (a.shape.empty() || b.shape.empty()) return false;
  if (b.shape.back() != a.shape.back()) return false;
  for (size_t i = 0; i + 1 < b.shape.size(); ++i)
    if (b.shape[i] != 1) return false;
  return b.numel() == a.shape.back();
}

bool infer_matmul(Ctx& c, const Op& op, const Type& a, const Type& b, Type* out) {
  if (!is_float(a.dtype) || a.dtype != b.dtype) return c.fail(op, "operands must share a float dtype (f32, f16, bf16)");
  std::vector<int64_t> as = a.shape, bs = b.shape;
  if (as.empty() || bs.empty()) return c.fail(op, "rank-0 operand");
  const bool va = as.size() == 1, vb = bs.size() == 1;
  if (va) as.insert(as.begin(), 1);
  if (vb) bs.push_back(1);
  if (as.back() != bs[bs.size() - 2])
    return c.fail(op, "contraction dims differ: " + std::to_string(as.back()) + " vs " + std::to_string(bs[bs.size() - 2]));
  std::vector<int64_t> batch;
  if (!broadcast_batch(std::vector<int64_t>(as.begin(), as.end() - 2), std::vector<int64_t>(bs.begin(), bs.end() - 2), &batch))
    return c.fail(op, "batch dims do not broadcast");
  out->dtype = a.dtype;
  out->shape = batch;
  if (!va) out->shape.push_back(as[as.size() - 2]);
  if (!vb) out->shape.push_back(bs.back());
  return true;
}

}  // namespace

bool plan_function(const Function& f, Plan* out, std::string* error) {
  Ctx c{f, *out, error, {}, {}, {}};
  Plan& p = *out;
  for (size_t i = 0; i < f.arg_names.size(); ++i) p.types[f.arg_names[i]] = f.arg_types[i];
  auto count_use = [&](const std::string& n) { c.uses[n]++; const size_t h = n.find('#'); if (h != std::string::npos && n.substr(h) == "#0") c.uses[n.substr(0, h)]++; };
  for (const Op& op : f.ops) {
    for (const std::string& o : op.operands) count_use(o);
    for (const std::string& o : op.index_operands) count_use(o);
    for (const std::string& r : op.results) c.producer[r] = &op;
  }
  for (const std::string& r : f.returned) count_use(r);

  // ---- pass 1: types
  for (const Op& op : f.ops) {
    std::vector<const Type*> in;
    for (const std::string& o : op.operands) {
      const Type* t = c.type_of(o);
      if (!t) return c.fail(op, "use of undefined value %" + o);
      in.push_back(t);
    }
    auto set = [&](size_t k, const Type& t) { if (k < op.results.size()) p.types[op.results[k]] = t; };
    const std::string& n = op.name;
    if (n == "nova.matmul") {
      if (in.size() != 2) return c.fail(op, "expects two operands");
      Type t;
      if (!infer_matmul(c, op, *in[0], *in[1], &t)) return false;
      set(0, t);
    } else if (n == "nova.linear") {
      if (in.size() != 3) return c.fail(op, "expects input, weight, bias");
      const Type &x = *in[0], &w = *in[1], &b = *in[2];
      if (x.shape.size() != 2 && x.shape.size() != 3) return c.fail(op, "input must be rank 2 or 3");
      if (w.shape.size() != 2) return c.fail(op, "weight must be rank 2");
      if (x.shape.back() != w.shape[0]) return c.fail(op, "input and weight do not compose");
      if (b.numel() != w.shape[1]) return c.fail(op, "bias must hold N elements");
      if (!is_float(x.dtype) || x.dtype != w.dtype || x.dtype != b.dtype) return c.fail(op, "operands must share a float dtype");
      Type t = x;
      t.shape.back() = w.shape[1];
      set(0, t);
    } else if (n == "linalg.matmul" || n == "linalg.batch_matmul") {
      if (in.size() != 3 || op.num_ins != 2) return c.fail(op, "expects ins(A, B) outs(C)");
      const size_t r = n == "linalg.matmul" ? 2 : 3;
      if (in[0]->shape.size() != r || in[1]->shape.size() != r || in[2]->shape.size() != r) return c.fail(op, "wrong operand rank");
      const Type &a = *in[0], &b = *in[1], &cc = *in[2];
      if (a.shape[r - 1] != b.shape[r - 2] || cc.shape[r - 2] != a.shape[r - 2] || cc.shape[r - 1] != b.shape[r - 1])
        return c.fail(op, "shapes do not compose");
      if (r == 3 && (a.shape[0] != cc.shape[0] || b.shape[0] != cc.shape[0])) return c.fail(op, "batch sizes differ");
      if (!is_float(a.dtype) || a.dtype != b.dtype || !is_float(cc.dtype)) return c.fail(op, "unsupported dtypes");
      set(0, cc);
    } else if (n == "nova.matmul_backward") {
      // grad_a has a's type, grad_b has b's type (MatmulBackwardOp::inferReturnTypes, NovaOps.cpp:1287-1303)
      if (in.size() != 3 || op.results.size() != 2) return c.fail(op, "expects grad_out, a, b and two results");
      const Type &go = *in[0], &a = *in[1], &b = *in[2];
      if (a.shape.size() < 2 || a.shape.size() != b.shape.size() || go.shape.size() != a.shape.size())
        return c.fail(op, "operands must share a rank >= 2");
      const size_t r = a.shape.size();
      if (go.shape[r - 2] != a.shape[r - 2] || go.shape[r - 1] != b.shape[r - 1] || a.shape[r - 1] != b.shape[r - 2])
        return c.fail(op, "shapes do not compose");
      if (!is_float(a.dtype) || a.dtype != b.dtype || a.dtype != go.dtype) return c.fail(op, "operands must share a float dtype");
      set(0, a); set(1, b);
    } else if (n == "nova.linear_backward") {
      // grad_input ~ input, grad_weight ~ weight, grad_bias = [N] (LinearBackwardOp::inferReturnTypes, NovaOps.cpp:2105-2128)
      if (in.size() != 3 || op.results.size() != 3) return c.fail(op, "expects grad_out, input, weight and three results");
      const Type &go = *in[0], &x = *in[1], &w = *in[2];
      if (w.shape.size() != 2 || x.shape.empty() || x.shape.back() != w.shape[0] || go.shape.size() != x.shape.size() ||
          go.shape.back() != w.shape[1])
        return c.fail(op, "shapes do not compose");
      if (!is_float(x.dtype) || x.dtype != w.dtype || x.dtype != go.dtype) return c.fail(op, "operands must share a float dtype");
      Type gb; gb.dtype = w.dtype; gb.shape = {w.shape[1]};
      set(0, x); set(1, w); set(2, gb);
    } else if (n == "linalg.fill") {
      if (in.size() != 2) return c.fail(op, "expects ins(scalar) outs(tensor)");
      set(0, *in[1]);
    } else if (n == "tensor.empty" || n == "arith.constant") {
      if (op.result_types.empty()) return c.fail(op, "missing result type");
      set(0, op.result_types[0]);
    } else if (n == "nova.gelu" || n == "nova.relu" || n == "nova.softmax") {
      if (in.size() != 1 || !is_float(in[0]->dtype)) return c.fail(op, "expects one float tensor");
      set(0, *in[0]);
    } else if (n == "nova.sce") {
      // (logits [..., C], targets [...]) -> (softmax ~ logits, loss [1])  (SceOp::inferReturnTypes, NovaOps.cpp:1648-1677)
      if (in.size() != 2 || !is_float(in[0]->dtype) || is_float(in[1]->dtype) || in[0]->shape.empty())
        return c.fail(op, "expects float logits and integer targets");
      if (in[1]->numel() != in[0]->numel() / std::max<int64_t>(in[0]->shape.back(), 1))
        return c.fail(op, "one target per row of logits");
      if (op.results.size() != 2) return c.fail(op, "produces softmax and loss");
      Type loss = *in[0];
      loss.shape = {1};
      set(0, *in[0]); set(1, loss);
    } else if (n == "nova.sce_backward") {
      // (softmax, targets) {dim} -> grad ~ softmax  (SceBackwardOp::inferReturnTypes, NovaOps.cpp:2148-2160)
      if (in.size() != 2 || !is_float(in[0]->dtype) || is_float(in[1]->dtype) || in[0]->shape.empty())
        return c.fail(op, "expects the forward's softmax and integer targets");
      const int64_t r = static_cast<int64_t>(in[0]->shape.size());
      const int64_t dim = op.attrs.count("dim") ? op.attrs.at("dim") : -1;
      if (dim != -1 && dim != r - 1) return c.fail(op, "only the last dimension as class dimension is supported");
      if (in[1]->numel() != in[0]->numel() / std::max<int64_t>(in[0]->shape.back(), 1))
        return c.fail(op, "one target per row");
      set(0, *in[0]);
    } else if (n == "nova.scatter_add") {
      // (input, indices, src) axis -> input's type; shapes match except at axis (ScatterAddOp::verify, NovaOps.cpp:1990-2026)
      if (in.size() != 3 || !is_float(in[0]->dtype) || is_float(in[1]->dtype) || in[2]->dtype != in[0]->dtype)
        return c.fail(op, "expects float input, integer indices, src of the input's type");
      const int64_t r = static_cast<int64_t>(in[0]->shape.size());
      int64_t axis = op.attrs.count("axis") ? op.attrs.at("axis") : 0;
      if (axis < 0) axis += r;
      if (static_cast<int64_t>(in[2]->shape.size()) != r) return c.fail(op, "input and src must have same rank");
      if (axis < 0 || axis >= r) return c.fail(op, "axis is out of bounds");
      for (int64_t i = 0; i < r; ++i) {
        if (i == axis) { if (in[2]->shape[i] != in[1]->numel()) return c.fail(op, "src dimension at axis must match index size"); }
        else if (in[0]->shape[i] != in[2]->shape[i]) return c.fail(op, "input and src shapes must match except at axis");
      }
      set(0, *in[0]);
    } else if (n == "nova.layer_norm_backward") {
      // (grad_y, x, gamma, mean_sum, rstd) -> (x's type, gamma's, gamma's)  (NovaOps.td:1038-1049, NovaOps.cpp:2055-2075)
      if (in.size() != 5) return c.fail(op, "expects grad_y, x, gamma, mean_sum, rstd");
      const Type& x = *in[1];
      if (!is_float(x.dtype) || x.shape.empty() || !(in[0]->shape == x.shape) || in[2]->numel() != x.shape.back() ||
          in[3]->numel() != x.numel() / std::max<int64_t>(x.shape.back(), 1) || in[4]->numel() != in[3]->numel())
        return c.fail(op, "operand shapes do not agree");
      for (int i = 0; i < 5; ++i)
        if (in[i]->dtype != x.dtype) return c.fail(op, "mixed dtypes are outside the supported subset");
      if (op.results.size() != 3) return c.fail(op, "produces grad_x, grad_gamma, grad_beta");
      set(0, x); set(1, *in[2]); set(2, *in[2]);
    } else if (n == "nova.gelu_backward") {
      // (grad_out, input) -> the input's type (GeluBackwardOp::inferReturnTypes, NovaOps.cpp:2130)
      if (in.size() != 2 || !is_float(in[1]->dtype) || in[0]->dtype != in[1]->dtype || !(in[0]->shape == in[1]->shape))
        return c.fail(op, "expects grad_out and input of one float type and shape");
      set(0, *in[1]);
    } else if (n == "nova.add" || n == "nova.sub" || n == "nova.mul") {
      // numpy broadcasting, right-aligned (inference: NovaOps.cpp:20-138 -> Broadcast.cpp:9-52)
      if (in.size() != 2) return c.fail(op, "expects two operands");
      if (in[0]->dtype != in[1]->dtype || !is_float(in[0]->dtype)) return c.fail(op, "mixed or non-float dtypes are outside the supported subset");
      Type t;
      t.dtype = in[0]->dtype;
      if (!broadcast_batch(in[0]->shape, in[1]->shape, &t.shape)) return c.fail(op, "operand shapes do not broadcast");
      set(0, t);
    } else if (n == "nova.compare") {
      // elementwise comparison with broadcasting -> i1 (CompareOp::inferReturnTypes, NovaOps.cpp:1006-1040)
      static const char* kinds[] = {"eq", "ne", "lt", "le", "gt", "ge"};
      bool known = false;
      for (const char* k : kinds) known = known || op.kind_attr == k;
      if (in.size() != 2 || !known) return c.fail(op, "expects compare<eq|ne|lt|le|gt|ge> of two operands");
      if (in[0]->dtype != in[1]->dtype || !is_float(in[0]->dtype)) return c.fail(op, "mixed or non-float dtypes are outside the supported subset");
      Type t;
      t.dtype = NOVA_B200_I1;
      if (!broadcast_batch(in[0]->shape, in[1]->shape, &t.shape)) return c.fail(op, "operand shapes do not broadcast");
      set(0, t);
    } else if (n == "nova.mse") {
      // mean over every element of (lhs - rhs)^2 -> tensor<1> (NovaMseForwardLowering, NovaToLinalgGeneric.cpp:367-428)
      if (in.size() != 2 || !is_float(in[0]->dtype) || in[0]->dtype != in[1]->dtype || !(in[0]->shape == in[1]->shape))
        return c.fail(op, "expects two float tensors of one type and shape");
      Type t;
      t.dtype = in[0]->dtype;
      t.shape = {1};
      set(0, t);
    } else if (n == "nova.constant") {
      // {value = dense<v> : T} : T  -- a splat; the written type is the result type
      if (!in.empty() || op.operand_types.empty()) return c.fail(op, "expects `{value = dense<v> : T} : T`");
      if (!is_float(op.operand_types[0].dtype)) return c.fail(op, "only float splat constants are supported");
      set(0, op.operand_types[0]);
    } else if (n == "nova.reduce") {
      // sum over the LEADING dims `dimension = [0, .., k-1]`, reduced dims dropped (ReduceOp, NovaOps.td:191-230): the
      // gradient accumulations of the backward graphs (ltest/test.mlir:45, ltest/testing.mlir:21-33)
      if (in.size() != 1 || !is_float(in[0]->dtype)) return c.fail(op, "expects one float tensor");
      if (op.kind_attr != "sum") return c.fail(op, "only reduce<sum> is inside the supported subset");
      if (op.attrs.count("keepdims") && op.attrs.at("keepdims") != 0) return c.fail(op, "keepdims is outside the supported subset");
      auto it = op.int_lists.find("dimension");
      if (it == op.int_lists.end() || it->second.empty()) return c.fail(op, "expects `dimension = [0, ..]`");
      const std::vector<int64_t>& dims = it->second;
      if (dims.size() >= in[0]->shape.size() + 0 && dims.size() > in[0]->shape.size()) return c.fail(op, "too many dimensions");
      for (size_t k = 0; k < dims.size(); ++k)
        if (dims[k] != static_cast<int64_t>(k)) return c.fail(op, "only the leading dimensions can be reduced");
      Type t;
      t.dtype = in[0]->dtype;
      t.shape.assign(in[0]->shape.begin() + dims.size(), in[0]->shape.end());
      set(0, t);
    } else if (n == "nova.layer_norm") {
      if (in.size() != 3) return c.fail(op, "expects input, gamma, beta");
      const Type& x = *in[0];
      if (x.shape.empty() || in[1]->numel() != x.shape.back() || in[2]->numel() != x.shape.back())
        return c.fail(op, "gamma / beta must hold D elements");
      Type stats = x;
      stats.shape.pop_back();
      if (op.results.size() == 1) {  // `%y = nova.layer_norm` binds the first result; the others stay addressable as #1, #2
        p.types[op.results[0]] = x;
        p.types[op.results[0] + "#1"] = stats;
        p.types[op.results[0] + "#2"] = stats;
      } else {
        set(0, x); set(1, stats); set(2, stats);
      }
    } else if (n == "nova.gather") {
      if (in.size() != 1 || op.index_operands.size() != 1) return c.fail(op, "expects input [indices]");
      const Type* idx = c.type_of(op.index_operands[0]);
      if (!idx) return c.fail(op, "use of undefined value %" + op.index_operands[0]);
      if (idx->dtype != NOVA_B200_I16 && idx->dtype != NOVA_B200_I32 && idx->dtype != NOVA_B200_I64)
        return c.fail(op, "indices must be i16, i32 or i64");
      const Type& x = *in[0];
      int64_t axis = op.attrs.count("axis") ? op.attrs.at("axis") : 0;
      if (axis < 0) axis += static_cast<int64_t>(x.shape.size());
      if (axis < 0 || axis >= static_cast<int64_t>(x.shape.size())) return c.fail(op, "axis out of range");
      size_t batch_dims = 0;
      for (size_t i = 0; i < std::min<size_t>(axis, idx->shape.size()); ++i) {
        if (x.shape[i] != idx->shape[i]) break;
        ++batch_dims;
      }
      Type t;
      t.dtype = x.dtype;
      for (int64_t i = 0; i < axis; ++i) t.shape.push_back(x.shape[i]);
      for (size_t i = batch_dims; i < idx->shape.size(); ++i) t.shape.push_back(idx->shape[i]);
      for (size_t i = axis + 1; i < x.shape.size(); ++i) t.shape.push_back(x.shape[i]);
      set(0, t);
    } else if (n == "nova.reshape") {
      if (in.size() != 1 || op.result_types.empty()) return c.fail(op, "expects `%x : Tin -> Tout`");
      if (op.result_types[0].numel() != in[0]->numel()) return c.fail(op, "element counts differ");
      Type t = op.result_types[0];
      t.dtype = in[0]->dtype;
      set(0, t);
    } else if (n == "nova.transpose") {
      if (in.size() != 1) return c.fail(op, "expects one operand");
      Type t = *in[0];
      const int64_t r = static_cast<int64_t>(t.shape.size());
      int64_t a1 = op.attrs.count("axes1") ? op.attrs.at("axes1") : -1;
      int64_t a2 = op.attrs.count("axes2") ? op.attrs.at("axes2") : -2;
      if (a1 < 0) a1 += r;
      if (a2 < 0) a2 += r;
      if (r < 2 || a1 < 0 || a2 < 0 || a1 >= r || a2 >= r) return c.fail(op, "axes out of range");
      std::swap(t.shape[a1], t.shape[a2]);
      set(0, t);
    } else if (n == "nova.cast") {
      if (in.size() != 1 || op.result_types.empty()) return c.fail(op, "expects `%x : Tin -> Tout`");
      if (!(is_float(in[0]->dtype) || in[0]->dtype == NOVA_B200_I1) || !is_float(op.result_types[0].dtype) ||
          op.result_types[0].shape != in[0]->shape)
        return c.fail(op, "only float-to-float and i1-to-float casts of equal shape are supported");
      set(0, op.result_types[0]);
    } else if (n == "nova.to_device" || n == "bufferization.to_tensor") {
      if (in.size() != 1) return c.fail(op, "expects one operand");
      set(0, *in[0]);
    } else if (n == "bufferization.materialize_in_destination") {
      if (in.size() != 2) return c.fail(op, "expects `%t in writable %dest`");
      if (in[0]->shape != in[1]->shape || in[0]->dtype != in[1]->dtype) return c.fail(op, "source and destination types differ");
    } else {
      return c.fail(op, "operation is outside the supported subset");
    }
    // written types, when present, must agree with what was inferred
    if (!op.result_types.empty() && !op.results.empty() && n != "nova.reshape" && n != "nova.cast") {
      const Type* got = c.type_of(op.results[0]);
      if (got && (got->shape != op.result_types[0].shape))
        return c.fail(op, "written result type " + type_str(op.result_types[0]) + " differs from the inferred " + type_str(*got));
    }
  }
  for (const std::string& r : f.returned)
    if (!c.type_of(r)) { *error = "return of undefined value %" + r; return false; }

  // ---- pass 2: steps with fusion
  auto single_user = [&](const std::string& v) -> const Op* {
    if (c.uses[v] != 1) return nullptr;
    for (const Op& u : f.ops) {
      if (c.absorbed.count(&u)) continue;
      for (const std::string& o : u.operands)
        if (o == v) return &u;
    }
    return nullptr;
  };
  // a value can be used by a step emitted at op `at` only if it is an argument or defined by an earlier op
  auto defined_before = [&](const std::string& v, const Op* at) {
    auto it = c.producer.find(v);
    if (it == c.producer.end()) {
      const size_t h = v.find('#');
      if (h != std::string::npos) it = c.producer.find(v.substr(0, h));
      if (it == c.producer.end()) return true;  // a function argument
    }
    return it->second < at;  // ops live in one vector: address order is program order
  };
  const Op* current = nullptr;
  // a contraction whose only user is nova.gelu_backward, as its grad_out operand: the multiplication by
  // gelu'(input) moves into the contraction's epilogue (the residual pointer then carries `input`)
  auto absorb_gelu_backward = [&](Step& s, std::string& v) {
    if (s.act != NOVA_B200_ACT_NONE || !s.residual.empty()) return;
    const Op* u = single_user(v);
    if (!(u && u->name == "nova.gelu_backward" && u->operands.size() == 2 && u->operands[0] == v && u->operands[1] != v)) return;
    if (!defined_before(u->operands[1], current)) return;
    s.act = NOVA_B200_ACT_GELU_TANH_GRAD;
    s.act_operand = u->operands[1];
    c.absorbed.insert(u);
    s.note += " + " + u->name;
    p.alias[v] = u->results[0];
    v = u->results[0];
  };
  auto absorb_tail = [&](Step& s, std::string v) {
    const Type out_t = *c.type_of(v);
    // accumulator init: the other addend of a following add (FuseMatmulBias) -- a row-broadcast bias, a
    // full-shape residual, or one of each ("out + x + b_down" after the FFN-down contraction)
    for (int round = 0; round < 2 && s.act == NOVA_B200_ACT_NONE; ++round) {
      const Op* u = single_user(v);
      if (!(u && u->name == "nova.add" && u->operands.size() == 2)) break;
      const std::string other = u->operands[0] == v ? u->operands[1] : u->operands[0];
      const Type* ot = c.type_of(other);
      if (!(ot && other != v && ot->dtype == out_t.dtype && defined_before(other, current))) break;
      bool fused = false;
      if (ot->shape == out_t.shape) {
        if (s.residual.empty()) { s.residual = other; fused = true; }
      } else if (is_row_broadcast(out_t, *ot)) {
        if (s.bias.empty()) { s.bias = other; fused = true; }
      }
      if (!fused) break;
      c.absorbed.insert(u);
      s.note += " + " + u->name;
      p.alias[v] = u->results[0];
      v = u->results[0];
    }
    absorb_gelu_backward(s, v);
    if (s.act == NOVA_B200_ACT_NONE) {
      const Op* u = single_user(v);
      if (u && (u->name == "nova.relu" || u->name == "nova.gelu")) {
        s.act = u->name == "nova.relu" ? NOVA_B200_ACT_RELU : NOVA_B200_ACT_GELU_TANH;
        c.absorbed.insert(u);
        s.note += " + " + u->name;
        p.alias[v] = u->results[0];
        v = u->results[0];
      }
    }
    s.outputs = {v};
  };

  for (const Op& op : f.ops) {
    if (c.absorbed.count(&op)) continue;
    current = &op;
    const std::string& n = op.name;
    Step s;
    s.attrs = op.attrs;
    s.note = n;
    if (n == "nova.matmul") {
      s.kind = "gemm";
      s.inputs = {op.operands[0], op.operands[1]};
      absorb_tail(s, op.results[0]);
    } else if (n == "nova.linear") {
      s.kind = "gemm";
      s.inputs = {op.operands[0], op.operands[1]};
      s.bias = op.operands[2];
      absorb_tail(s, op.results[0]);
    } else if (n == "linalg.matmul" || n == "linalg.batch_matmul") {
      s.kind = "gemm";
      s.inputs = {op.operands[0], op.operands[1]};
      // outs: a zero fill is INIT_ZERO; anything else is a live accumulator (bias / residual already moved there)
      const std::string outs = op.operands[2];
      const Op* prod = c.producer.count(outs) ? c.producer[outs] : nullptr;
      bool zero = false;
      if (prod && prod->name == "linalg.fill") {
        const Op* cst = c.producer.count(prod->operands[0]) ? c.producer[prod->operands[0]] : nullptr;
        zero = cst && cst->name == "arith.constant" && cst->fvalue == 0.0;
      }
      if (!zero) s.residual = outs;
      absorb_tail(s, op.results[0]);
    } else if (n == "nova.matmul_backward" || n == "nova.linear_backward") {
      // Expanded into views + contractions (+ a column sum): the transposes are strided views that the
      // contraction reads through trans_a / trans_b, the flattening of batch*M rows is a reshape view.
      const std::string tag = "__bw" + std::to_string(op.line) + "_";
      auto view = [&](const char* kind, const std::string& src, const std::string& dst, const Type& t,
                      std::map<std::string, int64_t> attrs = {}) {
        Step v; v.kind = kind; v.inputs = {src}; v.outputs = {dst}; v.attrs = attrs; v.note = n;
        p.types[dst] = t;
        p.steps.push_back(v);
      };
      auto swapped = [](Type t) { std::swap(t.shape[t.shape.size() - 1], t.shape[t.shape.size() - 2]); return t; };
      auto gemm = [&](const std::string& a, const std::string& b, std::string out, const char* what) {
        Step g; g.kind = "gemm"; g.inputs = {a, b}; g.note = n + std::string(" ") + what;
        absorb_gelu_backward(g, out);  // e.g. grad_input of the FFN-down layer feeding nova.gelu_backward
        g.outputs = {out};
        p.steps.push_back(g);
      };
      const std::string &go = op.operands[0], &x = op.operands[1], &w = op.operands[2];
      const Type &tgo = *c.type_of(go), &tx = *c.type_of(x), &tw = *c.type_of(w);
      if (n == "nova.matmul_backward") {
        view("transpose", w, tag + "bt", swapped(tw));
        gemm(go, tag + "bt", op.results[0], "grad_a = grad_out x b^T");
        view("transpose", x, tag + "at", swapped(tx));
        gemm(tag + "at", go, op.results[1], "grad_b = a^T x grad_out");
      } else {
        view("transpose", w, tag + "wt", swapped(tw));
        gemm(go, tag + "wt", op.results[0], "grad_input = grad_out x W^T");
        Type xf = tx, gf = tgo;
        xf.shape = {tx.numel() / tx.shape.back(), tx.shape.back()};
        gf.shape = {tgo.numel() / tgo.shape.back(), tgo.shape.back()};
        view("reshape", x, tag + "xf", xf);
        view("reshape", go, tag + "gf", gf);
        view("transpose", tag + "xf", tag + "xft", swapped(xf));
        gemm(tag + "xft", tag + "gf", op.results[1], "grad_weight = flatX^T x flatGo");
        Step cs; cs.kind = "column_sum"; cs.inputs = {tag + "gf"}; cs.outputs = {op.results[2]}; cs.note = n + " grad_bias";
        p.steps.push_back(cs);
      }
      continue;
    } else if (n == "nova.gelu" || n == "nova.relu") {
      s.kind = "activation";
      s.act = n == "nova.relu" ? NOVA_B200_ACT_RELU : NOVA_B200_ACT_GELU_TANH;
      s.inputs = op.operands; s.outputs = op.results;
    } else if (n == "nova.sce" || n == "nova.sce_backward" || n == "nova.scatter_add") {
      s.kind = n.substr(5);
      s.inputs = op.operands; s.outputs = op.results;
      if (n == "nova.sce_backward") {
        // grad * (one-element constant), its only use: the multiplication joins the pass that writes grad (an
        // all-parallel consumer of a root, which the reference's tile-and-fuse pipeline fuses as well: isEpilogue,
        // NovaKernelConfig.cpp:1876-1895)
        const Op* u = single_user(op.results[0]);
        if (u && u->name == "nova.mul" && u->operands.size() == 2 && u->operands[0] != u->operands[1]) {
          const std::string& other = u->operands[0] == op.results[0] ? u->operands[1] : u->operands[0];
          const Op* cst = c.producer.count(other) ? c.producer[other] : nullptr;
          const Type* ct = c.type_of(other);
          if (cst && (cst->name == "nova.constant" || cst->name == "arith.constant") && ct && ct->numel() == 1) {
            s.attrs["scaled"] = 1;
            s.fvalue = cst->fvalue;
            s.outputs = u->results;
            s.note = "nova.sce_backward + nova.mul by %" + other;
            c.absorbed.insert(u);
          }
        }
      }
    } else if (n == "nova.layer_norm_backward") {
      s.kind = "layer_norm_backward";
      s.inputs = op.operands; s.outputs = op.results;
    } else if (n == "nova.gelu_backward") {
      s.kind = "gelu_backward";
      s.inputs = op.operands; s.outputs = op.results;
    } else if (n == "nova.add" || n == "nova.sub" || n == "nova.mul") {
      s.kind = "binary";
      s.attrs["op"] = n == "nova.add" ? NOVA_B200_BIN_ADD : (n == "nova.sub" ? NOVA_B200_BIN_SUB : NOVA_B200_BIN_MUL);
      s.inputs = op.operands; s.outputs = op.results;
    } else if (n == "nova.compare") {
      static const char* kinds[] = {"eq", "ne", "lt", "le", "gt", "ge"};
      s.kind = "compare";
      for (int k = 0; k < 6; ++k)
        if (op.kind_attr == kinds[k]) s.attrs["op"] = k;
      s.inputs = op.operands; s.outputs = op.results;
    } else if (n == "nova.mse") {
      s.kind = "mse"; s.inputs = op.operands; s.outputs = op.results;
    } else if (n == "nova.constant") {
      s.kind = "constant"; s.fvalue = op.fvalue; s.outputs = op.results;
    } else if (n == "nova.reduce") {
      s.kind = "reduce_sum"; s.attrs["lead"] = static_cast<int64_t>(op.int_lists.at("dimension").size());
      s.inputs = op.operands; s.outputs = op.results;
    } else if (n == "nova.softmax") { s.kind = "softmax"; s.inputs = op.operands; s.outputs = op.results; }
    else if (n == "nova.layer_norm") {
      s.kind = "layer_norm"; s.inputs = op.operands;
      if (op.results.size() == 1) s.outputs = {op.results[0], op.results[0] + "#1", op.results[0] + "#2"};
      else s.outputs = op.results;
    } else if (n == "nova.gather") { s.kind = "gather"; s.inputs = {op.operands[0], op.index_operands[0]}; s.outputs = op.results; }
    else if (n == "nova.reshape") { s.kind = "reshape"; s.inputs = op.operands; s.outputs = op.results; }
    else if (n == "nova.transpose") { s.kind = "transpose"; s.inputs = op.operands; s.outputs = op.results; }
    else if (n == "nova.cast") { s.kind = "cast"; s.inputs = op.operands; s.outputs = op.results; }
    else if (n == "nova.to_device" || n == "bufferization.to_tensor") { s.kind = "alias"; s.inputs = op.operands; s.outputs = op.results; }
    else if (n == "bufferization.materialize_in_destination") { s.kind = "store_to_arg"; s.inputs = op.operands; }
    else if (n == "linalg.fill") {
      // a zero fill that only initialises a contraction is folded into it (INIT_ZERO)
      const Op* cst = c.producer.count(op.operands[0]) ? c.producer[op.operands[0]] : nullptr;
      bool only_gemm_outs = c.uses[op.results[0]] > 0;
      for (const Op& u : f.ops)
        for (size_t k = 0; k < u.operands.size(); ++k)
          if (u.operands[k] == op.results[0] && !((u.name == "linalg.matmul" || u.name == "linalg.batch_matmul") && k == 2))
            only_gemm_outs = false;
      if (cst && cst->fvalue == 0.0 && only_gemm_outs) continue;
      s.kind = "fill"; s.fvalue = cst ? cst->fvalue : 0.0; s.inputs = {op.operands[1]}; s.outputs = op.results;
    } else if (n == "tensor.empty") { s.kind = "empty"; s.outputs = op.results; }
    else if (n == "arith.constant") { continue; }
    p.steps.push_back(s);
  }
  p.results = f.returned;
  return true;
}

std::string describe_plan(const Function& f, const Plan& p) {
  std::ostringstream o;
  o << "func @" << f.name << "(";
  for (size_t i = 0; i < f.arg_names.size(); ++i) o << (i ? ", " : "") << "%" << f.arg_names[i] << ": " << type_str(f.arg_types[i]);
  o << ")\n";
  for (const Step& s : p.steps) {
    o << "  " << s.kind;
    if (s.kind == "gemm") {
      o << " init=" << (!s.bias.empty() && !s.residual.empty() ? "bias_row(%" + s.bias + ")+residual(%" + s.residual + ")"
                        : !s.bias.empty()                      ? "bias_row(%" + s.bias + ")"
                        : !s.residual.empty()                  ? "residual(%" + s.residual + ")"
                                                               : std::string("zero"));
      o << " act=" << (s.act == NOVA_B200_ACT_RELU ? "relu" : s.act == NOVA_B200_ACT_GELU_TANH ? "gelu_tanh"
                       : s.act == NOVA_B200_ACT_GELU_TANH_GRAD ? "gelu_tanh_grad(%" + s.act_operand + ")" : std::string("none"));
    }
    o << " (";
    for (size_t i = 0; i < s.inputs.size(); ++i) o << (i ? ", " : "") << "%" << s.inputs[i];
    o << ") -> (";
    for (size_t i = 0; i < s.outputs.size(); ++i) {
      o << (i ? ", " : "") << "%" << s.outputs[i];
      auto it = p.types.find(s.outputs[i]);
      if (it != p.types.end()) o << ": " << type_str(it->second);
    }
    o << ")  [" << s.note << "]\n";
  }
  o << "  return";
  for (const std::string& r : p.results) o << " %" << r;
  o << "\n";
  return o.str();
}

}  // namespace fe
}  // namespace nova
