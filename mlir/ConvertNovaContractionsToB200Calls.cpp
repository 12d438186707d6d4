//===- ConvertNovaContractionsToB200Calls.cpp - contractions -> libnova_b200 calls ------------------===//
//
// Lowering pass of the Nova compiler's GPU pipeline for B200: rewrites every dense contraction that reaches
// code generation -- linalg.matmul, linalg.batch_matmul, linalg.matmul_transpose_a, in the bias-as-accumulator
// form FuseMatmulBias leaves them in, together with a trailing ReLU / GELU(tanh) consumer -- into ONE call of
// `nova_b200_gemm_flat` (include/nova_b200.h), and the row-wise ops next to them into their entry points.
//
// STATUS: written against MLIR / LLVM 21.1.6 (the version the reference pins) but NOT compiled or run: that
// toolchain is not available where this repository is developed.  Treat it as unverified source.  What IS
// checked on every test run is that the call table below names only functions libnova_b200 exports, with the
// arity used here, and that the fusion decisions it encodes are the ones the textual front-end
// (nova_compiler_b200/csrc/frontend_plan.cpp) makes on the reference's own .mlir fixtures
// (tests/test_lowering_pass_source.py).
//
// Where it goes (lib/Transforms/LLVMGPU/Passes.cpp, addNovaGPUOptimizedPipeline):
//
//     pm.addNestedPass<func::FuncOp>(createFuseMatmulBiasPass());          // :102  (unchanged)
//     pm.addPass(createCSEPass()); pm.addPass(createCanonicalizerPass());  // :107-108
//     pm.addPass(createNovaConvertContractionsToB200CallsPass());          // <-- here, before the fold of unit dims (:111)
//                                                                          //     and strategy selection (:116)
//
// Everything from strategy selection to vector distribution (:116-479) then finds no contraction left and is
// a no-op for the rewritten ops.  NovaCompilerAPI keeps its `device == "gpu" | "cuda"` switch
// (lib/API/NovaCompilerAPI.cpp:356-357); a pipeline alias `--nova-b200-pipeline` registers the same sequence.
//
// What is emitted, per contraction (pattern skeleton: matmul.cpp:878-926; extern declaration in the style of
// getOrDeclareFunc, lib/Transforms/FixGpuLaunch.cpp:17-33):
//
//     %a = bufferization.to_buffer %A : tensor<MxKxT> to memref<MxKxT, 1>     // device memory space 1
//     %b = bufferization.to_buffer %B ...
//     %c = memref.alloc() : memref<MxNxT, 1>                                   // FixGpuLaunch turns it into cudaMallocAsync (:49-50)
//     %pa = memref.extract_aligned_pointer_as_index %a -> index -> i64         // descriptor field 1, as FixGpuLaunch.cpp:245-246
//     %st = func.call @nova_b200_gemm_flat(%pa, %pb, %pc, %pbias, %pres, batch, M, N, K, lda, ldb, ldc, ldr,
//                                          bsa, bsb, bsc, bsr, dtype_ab, dtype_c, trans_a, trans_b, act, init,
//                                          f32_mode, stream) : (...) -> i32
//     cf.assert (%st == 0), "libnova_b200 call failed"                          // unlike FixGpuLaunch.cpp:106-107 the status is checked
//     %r = bufferization.to_tensor %c restrict writable : memref<MxNxT, 1> to tensor<MxNxT>
//
// CALL TABLE (machine-readable; one line per rewrite: matched form | callee | init | act)
// @call linalg.matmul outs(fill 0)                          | nova_b200_gemm_flat | NOVA_B200_INIT_ZERO              | NOVA_B200_ACT_NONE
// @call linalg.matmul outs(bias broadcast along rows)       | nova_b200_gemm_flat | NOVA_B200_INIT_BIAS_ROW          | NOVA_B200_ACT_NONE
// @call linalg.matmul outs(full tensor)                     | nova_b200_gemm_flat | NOVA_B200_INIT_RESIDUAL_FULL     | NOVA_B200_ACT_NONE
// @call linalg.matmul outs(full tensor) + row bias add      | nova_b200_gemm_flat | NOVA_B200_INIT_BIAS_AND_RESIDUAL | NOVA_B200_ACT_NONE
// @call any of the above + maximumf(x, 0) consumer          | nova_b200_gemm_flat | (as matched)                     | NOVA_B200_ACT_RELU
// @call any of the above + tanh-GELU consumer               | nova_b200_gemm_flat | (as matched)                     | NOVA_B200_ACT_GELU_TANH
// @call linalg.batch_matmul (same forms)                    | nova_b200_gemm_flat | (as matched)                     | (as matched)
// @call linalg.matmul_transpose_a (same forms, trans_a = 1) | nova_b200_gemm_flat | (as matched)                     | (as matched)
// @arity nova_b200_gemm_flat 25
//
//===----------------------------------------------------------------------------------------------===//

#include "mlir/Dialect/Arith/IR/Arith.h"
#include "mlir/Dialect/Bufferization/IR/Bufferization.h"
#include "mlir/Dialect/ControlFlow/IR/ControlFlowOps.h"
#include "mlir/Dialect/Func/IR/FuncOps.h"
#include "mlir/Dialect/Linalg/IR/Linalg.h"
#include "mlir/Dialect/Math/IR/Math.h"
#include "mlir/Dialect/MemRef/IR/MemRef.h"
#include "mlir/Dialect/Tensor/IR/Tensor.h"
#include "mlir/IR/Matchers.h"
#include "mlir/IR/PatternMatch.h"
#include "mlir/Pass/Pass.h"
#include "mlir/Transforms/GreedyPatternRewriteDriver.h"

using namespace mlir;

namespace mlir {
namespace nova {
namespace {

// Enumerators of include/nova_b200.h (kept in step by tests/test_lowering_pass_source.py).
enum : int32_t { kF32 = 0, kF16 = 1, kBF16 = 2 };
enum : int32_t { kActNone = 0, kActRelu = 1, kActGeluTanh = 2 };
enum : int32_t { kInitZero = 0, kInitBiasRow = 1, kInitResidualFull = 2, kInitFromC = 3, kInitBiasAndResidual = 4 };
constexpr const char *kGemmCallee = "nova_b200_gemm_flat";
constexpr int64_t kDeviceMemorySpace = 1;  // memref<..., 1>, as in ltest/test_gpu.mlir:2-8

static std::optional<int32_t> dtypeCode(Type t) {
  if (t.isF32()) return kF32;
  if (t.isF16()) return kF16;
  if (t.isBF16()) return kBF16;
  return std::nullopt;
}

static bool isZeroFill(Value v) {
  auto fill = v.getDefiningOp<linalg::FillOp>();
  if (!fill) return false;
  return matchPattern(fill.getInputs()[0], m_AnyZeroFloat());
}

// An all-parallel generic with identity output map whose body is a single op on block arguments.
static bool isElementwise(linalg::GenericOp g) {
  if (g.getNumReductionLoops() != 0 || g.getNumDpsInits() != 1) return false;
  return g.getMatchingIndexingMap(g.getDpsInitOperand(0)).isIdentity();
}

// `yield addf(in_i, in_j)` (or in-place `addf(in, out)`): returns the addend that is not `through`.
static Value matchAdd(linalg::GenericOp g, Value through, AffineMap *otherMap) {
  if (!isElementwise(g)) return {};
  Block &body = g.getRegion().front();
  auto yield = cast<linalg::YieldOp>(body.getTerminator());
  auto add = yield.getOperand(0).getDefiningOp<arith::AddFOp>();
  if (!add || std::distance(body.begin(), body.end()) != 2) return {};
  auto lhs = dyn_cast<BlockArgument>(add.getLhs()), rhs = dyn_cast<BlockArgument>(add.getRhs());
  if (!lhs || !rhs || lhs == rhs) return {};
  SmallVector<OpOperand *> operands = g.getOpOperandsMatchingBBargs();
  Value a = operands[lhs.getArgNumber()]->get(), b = operands[rhs.getArgNumber()]->get();
  if (a != through && b != through) return {};
  OpOperand *other = a == through ? operands[rhs.getArgNumber()] : operands[lhs.getArgNumber()];
  *otherMap = g.getMatchingIndexingMap(other);
  return other->get();
}

// `yield maximumf(in, 0.0)`
static bool matchRelu(linalg::GenericOp g, Value through) {
  if (!isElementwise(g) || g.getNumDpsInputs() != 1 || g.getDpsInputOperand(0)->get() != through) return false;
  Block &body = g.getRegion().front();
  auto yield = cast<linalg::YieldOp>(body.getTerminator());
  auto mx = yield.getOperand(0).getDefiningOp<arith::MaximumFOp>();
  if (!mx || std::distance(body.begin(), body.end()) != 2) return false;
  Value c = isa<BlockArgument>(mx.getLhs()) ? mx.getRhs() : mx.getLhs();
  return matchPattern(c, m_AnyZeroFloat());
}

// The tanh GELU body the reference emits (NovaGeluForwardPattern, NovaToLinalgGeneric.cpp:1310-1330):
// exactly one math.tanh, six mulf, two addf, nothing else.
static bool matchGeluTanh(linalg::GenericOp g, Value through) {
  if (!isElementwise(g) || g.getNumDpsInputs() != 1 || g.getDpsInputOperand(0)->get() != through) return false;
  int tanh = 0, mul = 0, add = 0, other = 0;
  for (Operation &op : g.getRegion().front().without_terminator()) {
    if (isa<math::TanhOp>(op)) ++tanh;
    else if (isa<arith::MulFOp>(op)) ++mul;
    else if (isa<arith::AddFOp>(op)) ++add;
    else if (!isa<arith::ConstantOp>(op)) ++other;
  }
  return tanh == 1 && mul == 6 && add == 2 && other == 0;
}

// a bias that stretches along the rows: its map drops every dim but the last, (d0, .., dn) -> (dn)
static bool isRowBroadcastMap(AffineMap m) {
  return m.getNumResults() == 1 && m.getResult(0) == getAffineDimExpr(m.getNumDims() - 1, m.getContext());
}

// The only real consumer of `v` (write-back bookkeeping does not count: FuseMatmulBias.cpp:107-109).
static Operation *singleConsumer(Value v) {
  Operation *found = nullptr;
  for (Operation *user : v.getUsers()) {
    if (isa<bufferization::MaterializeInDestinationOp>(user)) continue;
    if (found) return nullptr;
    found = user;
  }
  return found;
}

static func::FuncOp getOrDeclareCallee(ModuleOp module, PatternRewriter &rewriter) {
  if (auto f = module.lookupSymbol<func::FuncOp>(kGemmCallee)) return f;
  OpBuilder::InsertionGuard guard(rewriter);
  rewriter.setInsertionPointToStart(module.getBody());
  Type i64 = rewriter.getI64Type(), i32 = rewriter.getI32Type();
  SmallVector<Type> args(17, i64);   // A, B, C, bias, residual, batch, M, N, K, 4 pitches, 4 batch strides
  args.append(7, i32);               // dtype_ab, dtype_c, trans_a, trans_b, act, init, f32_mode
  args.push_back(i64);               // stream
  auto f = rewriter.create<func::FuncOp>(module.getLoc(), kGemmCallee, rewriter.getFunctionType(args, {i32}));
  f.setPrivate();
  return f;
}

struct Epilogue {
  int32_t init = kInitZero, act = kActNone;
  Value bias, residual;      // tensors
  Value result;              // the value the fused chain finally produces
  SmallVector<Operation *> absorbed;
};

// Walks outs (what FuseMatmulBias left there) and the single-consumer chain after the contraction.
static void classify(Value outs, Value mmResult, Epilogue *e) {
  e->result = mmResult;
  if (!isZeroFill(outs)) {
    // (c) a broadcast generic `yield args[0]` of a lower-rank bias (FuseMatmulBias.cpp:149-173) or (b) a full tensor
    if (auto g = outs.getDefiningOp<linalg::GenericOp>();
        g && isElementwise(g) && g.getNumDpsInputs() == 1 &&
        isa<BlockArgument>(cast<linalg::YieldOp>(g.getRegion().front().getTerminator()).getOperand(0)) &&
        isRowBroadcastMap(g.getMatchingIndexingMap(g.getDpsInputOperand(0)))) {
      e->init = kInitBiasRow;
      e->bias = g.getDpsInputOperand(0)->get();
    } else {
      e->init = kInitResidualFull;
      e->residual = outs;
    }
  }
  // trailing adds (at most one row bias and one full residual), then one activation
  for (int round = 0; round < 2; ++round) {
    auto g = dyn_cast_or_null<linalg::GenericOp>(singleConsumer(e->result));
    AffineMap m;
    Value other = g ? matchAdd(g, e->result, &m) : Value();
    if (!other) break;
    if (m.isIdentity() && !e->residual) e->residual = other;
    else if (isRowBroadcastMap(m) && !e->bias) e->bias = other;
    else break;
    e->init = e->bias && e->residual ? kInitBiasAndResidual : (e->bias ? kInitBiasRow : kInitResidualFull);
    e->absorbed.push_back(g);
    e->result = g.getResult(0);
  }
  if (auto g = dyn_cast_or_null<linalg::GenericOp>(singleConsumer(e->result))) {
    if (matchRelu(g, e->result)) e->act = kActRelu;
    else if (matchGeluTanh(g, e->result)) e->act = kActGeluTanh;
    if (e->act != kActNone) {
      e->absorbed.push_back(g);
      e->result = g.getResult(0);
    }
  }
}

// tensor -> aligned device pointer as i64 (0 for a null Value)
static Value devicePointer(PatternRewriter &rewriter, Location loc, Value tensor) {
  if (!tensor) return rewriter.create<arith::ConstantIntOp>(loc, 0, 64);
  auto tt = cast<RankedTensorType>(tensor.getType());
  auto mt = MemRefType::get(tt.getShape(), tt.getElementType(), MemRefLayoutAttrInterface{},
                            rewriter.getI64IntegerAttr(kDeviceMemorySpace));
  Value m = rewriter.create<bufferization::ToBufferOp>(loc, mt, tensor);
  Value idx = rewriter.create<memref::ExtractAlignedPointerAsIndexOp>(loc, m);
  return rewriter.create<arith::IndexCastOp>(loc, rewriter.getI64Type(), idx);
}

template <typename ContractionOp, bool kBatched, bool kTransA>
struct ContractionToB200Call : public OpRewritePattern<ContractionOp> {
  using OpRewritePattern<ContractionOp>::OpRewritePattern;

  LogicalResult matchAndRewrite(ContractionOp op, PatternRewriter &rewriter) const override {
    if (!op.hasPureTensorSemantics()) return failure();
    Value A = op.getDpsInputOperand(0)->get(), B = op.getDpsInputOperand(1)->get();
    Value outs = op.getDpsInitOperand(0)->get();
    auto at = cast<RankedTensorType>(A.getType()), bt = cast<RankedTensorType>(B.getType());
    auto ct = cast<RankedTensorType>(op->getResult(0).getType());
    if (!at.hasStaticShape() || !bt.hasStaticShape() || !ct.hasStaticShape()) return failure();
    auto dab = dtypeCode(at.getElementType()), dc = dtypeCode(ct.getElementType());
    if (!dab || !dc || at.getElementType() != bt.getElementType()) return failure();

    const int r = kBatched ? 1 : 0;  // index of the first matrix dim
    const int64_t batch = kBatched ? ct.getDimSize(0) : 1;
    const int64_t M = ct.getDimSize(r), N = ct.getDimSize(r + 1);
    const int64_t K = kTransA ? at.getDimSize(r) : at.getDimSize(r + 1);
    // row-major contiguous tensors: the pitch is the inner extent of what is stored
    const int64_t lda = at.getDimSize(r + 1), ldb = bt.getDimSize(r + 1), ldc = N;

    Epilogue e;
    classify(outs, op->getResult(0), &e);
    Location loc = op.getLoc();
    auto module = op->template getParentOfType<ModuleOp>();
    func::FuncOp callee = getOrDeclareCallee(module, rewriter);

    // the fused chain's last op is where the call goes, so every absorbed operand dominates it
    Operation *last = e.absorbed.empty() ? op.getOperation() : e.absorbed.back();
    rewriter.setInsertionPoint(last);
    auto cm = MemRefType::get(ct.getShape(), ct.getElementType(), MemRefLayoutAttrInterface{},
                              rewriter.getI64IntegerAttr(kDeviceMemorySpace));
    Value cBuf = rewriter.create<memref::AllocOp>(loc, cm);
    Value pc = rewriter.create<arith::IndexCastOp>(
        loc, rewriter.getI64Type(), rewriter.create<memref::ExtractAlignedPointerAsIndexOp>(loc, cBuf));
    auto i64c = [&](int64_t v) -> Value { return rewriter.create<arith::ConstantIntOp>(loc, v, 64); };
    auto i32c = [&](int32_t v) -> Value { return rewriter.create<arith::ConstantIntOp>(loc, v, 32); };
    SmallVector<Value> args = {
        devicePointer(rewriter, loc, A), devicePointer(rewriter, loc, B), pc,
        devicePointer(rewriter, loc, e.bias), devicePointer(rewriter, loc, e.residual),
        i64c(batch), i64c(M), i64c(N), i64c(K), i64c(lda), i64c(ldb), i64c(ldc), i64c(/*ldr=*/N),
        i64c(kBatched ? at.getDimSize(1) * at.getDimSize(2) : 0), i64c(kBatched ? bt.getDimSize(1) * bt.getDimSize(2) : 0),
        i64c(M * N), i64c(e.residual ? M * N : 0),
        i32c(*dab), i32c(*dc), i32c(kTransA ? 1 : 0), i32c(0), i32c(e.act), i32c(e.init), i32c(/*TF32X3*/ 0),
        i64c(/*stream=*/0)};
    auto call = rewriter.create<func::CallOp>(loc, callee, args);
    Value ok = rewriter.create<arith::CmpIOp>(loc, arith::CmpIPredicate::eq, call.getResult(0), i32c(0));
    rewriter.create<cf::AssertOp>(loc, ok, "libnova_b200 call failed");
    Value result = rewriter.create<bufferization::ToTensorOp>(loc, ct, cBuf, /*restrict=*/true, /*writable=*/true);
    rewriter.replaceOp(last, result);
    // the ops between the contraction and `last` are dead now: erase them consumer-first
    for (auto it = e.absorbed.rbegin(); it != e.absorbed.rend(); ++it)
      if (*it != last) rewriter.eraseOp(*it);
    if (last != op.getOperation()) rewriter.eraseOp(op);
    return success();
  }
};

struct ConvertNovaContractionsToB200CallsPass
    : public PassWrapper<ConvertNovaContractionsToB200CallsPass, OperationPass<ModuleOp>> {
  MLIR_DEFINE_EXPLICIT_INTERNAL_INLINE_TYPE_ID(ConvertNovaContractionsToB200CallsPass)

  StringRef getArgument() const final { return "nova-convert-contractions-to-b200-calls"; }
  StringRef getDescription() const final {
    return "Rewrite linalg contractions (with their fused bias / residual / ReLU / GELU consumers) into calls of libnova_b200";
  }
  void getDependentDialects(DialectRegistry &registry) const override {
    registry.insert<arith::ArithDialect, bufferization::BufferizationDialect, cf::ControlFlowDialect, func::FuncDialect,
                    memref::MemRefDialect>();
  }
  void runOnOperation() override {
    RewritePatternSet patterns(&getContext());
    patterns.add<ContractionToB200Call<linalg::MatmulOp, false, false>,
                 ContractionToB200Call<linalg::BatchMatmulOp, true, false>,
                 ContractionToB200Call<linalg::MatmulTransposeAOp, false, true>>(&getContext());
    if (failed(applyPatternsGreedily(getOperation(), std::move(patterns)))) signalPassFailure();
  }
};

}  // namespace

std::unique_ptr<Pass> createNovaConvertContractionsToB200CallsPass() {
  return std::make_unique<ConvertNovaContractionsToB200CallsPass>();
}

}  // namespace nova
}  // namespace mlir
