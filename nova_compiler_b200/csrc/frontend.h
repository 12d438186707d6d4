// Textual front-end: parses the restricted nova / linalg subset that reaches the contraction path and
// turns a function into a list of C-ABI calls (with the bias / activation fusion FuseMatmulBias and the
// epilogue classification would perform).  Stand-in for the MLIR lowering pass, which needs MLIR 21 to
// build; it lets the reference's .mlir graphs run on libnova_b200 unchanged.
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "../../include/nova_b200.h"

namespace nova {
namespace fe {

struct Type {
  int32_t dtype = -1;          // nova_b200_dtype; -1 = not a tensor
  std::vector<int64_t> shape;  // static shapes only
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t d : shape) n *= d;
    return n;
  }
};

struct Op {
  std::string name;                   // e.g. "nova.matmul", "linalg.batch_matmul", "return"
  std::vector<std::string> results;   // SSA names without '%'
  std::vector<std::string> operands;  // ins first, then outs for linalg ops
  std::vector<std::string> index_operands;  // nova.gather [%idx]
  int num_ins = 0;                    // linalg ops: operands[0..num_ins) are ins
  std::map<std::string, int64_t> attrs;  // axis, dimension, axes1, axes2
  std::map<std::string, std::vector<int64_t>> int_lists;  // dimension = [0, 1]
  std::string kind_attr;              // nova.reduce<sum>, nova.compare<gt>: the text between the angle brackets
  bool from_generic = false;          // a linalg.generic bias / ReLU consumer rewritten into the nova op it came from
  double fvalue = 0.0;                // arith.constant, nova.constant (splat)
  std::vector<Type> operand_types;    // as written after ':'
  std::vector<Type> result_types;     // as written after '->' (may be empty: inferred)
  int line = 0;
};

struct Function {
  std::string name;
  std::vector<std::string> arg_names;
  std::vector<Type> arg_types;
  std::vector<Type> result_types;
  std::vector<Op> ops;
  std::vector<std::string> returned;  // operands of the return
};

struct Module {
  std::vector<Function> functions;
  const Function* find(const std::string& name) const {
    for (const Function& f : functions)
      if (f.name == name) return &f;
    return nullptr;
  }
};

// Parses `text`; on failure returns false and describes the problem (with a line number) in *error.
bool parse_module(const std::string& text, Module* out, std::string* error);

// One executable step after shape inference and fusion.
struct Step {
  std::string kind;  // "gemm", "layer_norm", "softmax", "gather", "activation", "add", "cast", "view", "fill", "copy"
  std::vector<std::string> inputs;   // SSA names
  std::vector<std::string> outputs;  // SSA names
  // gemm
  std::string bias, residual;
  int32_t act = NOVA_B200_ACT_NONE;
  std::string act_operand;  // ACT_GELU_TANH_GRAD: the forward pre-activation the result is multiplied by
  bool accumulate_into_out = false;
  // misc
  std::map<std::string, int64_t> attrs;
  double fvalue = 0.0;
  std::string note;  // which source ops were folded into this step
};

struct Plan {
  std::map<std::string, Type> types;  // every SSA value (after inference)
  std::map<std::string, std::string> alias;  // value -> value it is a pure view / fused result of
  std::vector<Step> steps;
  std::vector<std::string> results;   // SSA names returned
};

// Shape / dtype inference following the reference's op definitions, plus fusion.  No GPU needed.
bool plan_function(const Function& f, Plan* out, std::string* error);
std::string describe_plan(const Function& f, const Plan& p);

}  // namespace fe
}  // namespace nova
