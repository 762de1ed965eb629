// Matches contraction patterns on linalg-on-tensors and replaces each with hal.dispatch.extern
// ops that launch exports of b200_contraction.cubin.
//
// What a "contraction dispatch" contains follows dispatch formation
// (Dialect/Flow/Transforms/FormDispatchRegions.cpp: named matmuls are roots, linalg.fill is pulled
// in, elementwise consumers fuse; RegionOpUtils.cpp: dequantisation-like producers are cloned
// in). This pass matches the same groups one step earlier:
//
//   A  fill(0) -> linalg.matmul / batch_matmul, f16 x f16 -> f32 [-> truncf to f16]
//        -> b200_matmul_f16_f16 (with truncf) or b200_matmul_f16_f32
//   B  the same with bf16
//   C  fill(0) -> linalg.matmul i8 x i8 -> i32 [-> generic(sitofp, mulf a_scale[m], mulf w_scale[n], truncf)]
//        -> b200_matmul_i8_i32 or b200_matmul_i8_requant_f16
//   D  generic(extsi i4 -> sitofp f16 -> mulf scale[n,g]) feeding the grouped contraction
//      generic with two reduction dims (g, k) and a truncf -> b200_w4a16_decode_m8 / _m16
//      (static M <= 16), else b200_w4a16_gemm
//
// Operands whose row pitch is not a multiple of 16 bytes go to the *_generic exports.
// The emitted IR and the kernel ABI (bindings first, then i32 constants) are documented in
// INTEGRATION.md of the kernel repository; the export table there must stay in sync with
// kEntries in the runtime library.
#include "Passes.h"
#include "iree/compiler/Dialect/HAL/IR/HALDialect.h"
#include "iree/compiler/Dialect/HAL/IR/HALOps.h"
#include "iree/compiler/Dialect/HAL/IR/HALTypes.h"
#include "iree/compiler/Dialect/Util/IR/UtilOps.h"
#include "mlir/Dialect/Arith/IR/Arith.h"
#include "mlir/Dialect/Linalg/IR/Linalg.h"
#include "mlir/Dialect/Tensor/IR/Tensor.h"
#include "mlir/IR/Builders.h"
#include "mlir/IR/Matchers.h"
#include "mlir/IR/PatternMatch.h"

namespace mlir::iree_compiler::b200 {
namespace {

namespace HAL = IREE::HAL;

constexpr int64_t kGemmThreads = 256, kGemmSmem = 197888;
constexpr int64_t kW4GemmThreads = 512, kW4GemmSmem = 181504;
constexpr int64_t kDecodeThreads = 512, kDecodeSmemM8 = 180864, kDecodeSmemM16 = 213632;

enum class ElemKind { F16, BF16, I8, Unsupported };

static ElemKind kindOf(Type t) {
  if (t.isF16()) return ElemKind::F16;
  if (t.isBF16()) return ElemKind::BF16;
  if (t.isInteger(8)) return ElemKind::I8;
  return ElemKind::Unsupported;
}

static bool isZeroFill(Value v) {
  auto fill = v.getDefiningOp<linalg::FillOp>();
  if (!fill) return false;
  return matchPattern(fill.getInputs()[0], m_AnyZeroFloat()) || matchPattern(fill.getInputs()[0], m_Zero());
}

// A single-result elementwise generic whose body is exactly one arith.truncf.
static linalg::GenericOp matchTruncfConsumer(Value acc) {
  if (!acc.hasOneUse()) return nullptr;
  auto generic = dyn_cast<linalg::GenericOp>(*acc.getUsers().begin());
  if (!generic || generic.getNumDpsInputs() != 1 || generic.getNumReductionLoops() != 0) return nullptr;
  Block &body = generic.getRegion().front();
  if (body.getOperations().size() != 2) return nullptr;
  return isa<arith::TruncFOp>(body.front()) ? generic : nullptr;
}

struct Matched {
  Operation *root = nullptr;       // the contraction
  Operation *last = nullptr;       // the op whose result the rewrite replaces
  Value lhs, rhs;
  ElemKind kind = ElemKind::Unsupported;
  bool batched = false, castToInput = false;
};

static std::optional<Matched> matchMatmul(linalg::LinalgOp op) {
  if (!isa<linalg::MatmulOp, linalg::BatchMatmulOp>(op.getOperation())) return std::nullopt;
  Matched m;
  m.root = m.last = op;
  m.batched = isa<linalg::BatchMatmulOp>(op.getOperation());
  m.lhs = op.getDpsInputs()[0];
  m.rhs = op.getDpsInputs()[1];
  auto lhsType = cast<RankedTensorType>(m.lhs.getType());
  auto accType = cast<RankedTensorType>(op.getDpsInits()[0].getType());
  m.kind = kindOf(lhsType.getElementType());
  if (m.kind == ElemKind::Unsupported || kindOf(cast<RankedTensorType>(m.rhs.getType()).getElementType()) != m.kind)
    return std::nullopt;
  const bool accOk = m.kind == ElemKind::I8 ? accType.getElementType().isInteger(32) : accType.getElementType().isF32();
  if (!accOk || !isZeroFill(op.getDpsInits()[0])) return std::nullopt;  // accumulate-into-existing is left alone
  if (m.kind != ElemKind::I8) {
    if (linalg::GenericOp trunc = matchTruncfConsumer(op->getResult(0))) {
      auto outType = cast<RankedTensorType>(trunc->getResult(0).getType());
      if (kindOf(outType.getElementType()) == m.kind) {
        m.last = trunc;
        m.castToInput = true;
      }
    }
  }
  return m;
}

static StringRef exportName(const Matched &m, bool generic) {
  switch (m.kind) {
    case ElemKind::F16:
      return m.castToInput ? (generic ? "b200_matmul_generic_f16_f16" : "b200_matmul_f16_f16")
                           : (generic ? "b200_matmul_generic_f16_f32" : "b200_matmul_f16_f32");
    case ElemKind::BF16:
      return m.castToInput ? (generic ? "b200_matmul_generic_bf16_bf16" : "b200_matmul_bf16_bf16")
                           : (generic ? "b200_matmul_generic_bf16_f32" : "b200_matmul_bf16_f32");
    default:
      return generic ? "b200_matmul_generic_i8_i32" : "b200_matmul_i8_i32";
  }
}

// The widest tile that still gives every SM work (same cost model as the runtime library).
static int64_t chooseTileN(int64_t M, int64_t N, int64_t batch, int64_t chunk, int smCount) {
  int64_t best = chunk;
  double bestCost = 0;
  for (int64_t bn = 256; bn >= 32; bn -= 32) {
    if (bn % chunk) continue;
    if (M <= 32 && bn > 128 && chunk <= 128) continue;  // few rows: tiles <= 128 wide select the deep-ring variant
    const int64_t tiles = ((M + 127) / 128) * ((N + bn - 1) / bn) * batch;
    const double cost = double((tiles + smCount - 1) / smCount) * (400.0 + bn);
    if (bestCost == 0 || cost < bestCost * 0.9999) {
      bestCost = cost;
      best = bn;
    }
  }
  return best;
}

class RewriteContractionsPass : public PassWrapper<RewriteContractionsPass, OperationPass<ModuleOp>> {
 public:
  explicit RewriteContractionsPass(RewriteOptions options) : options(std::move(options)) {}
  StringRef getArgument() const override { return "iree-b200-rewrite-contractions"; }
  StringRef getDescription() const override {
    return "Replace contraction patterns with hal.dispatch.extern ops backed by the sm_100a cubin";
  }
  void getDependentDialects(DialectRegistry &registry) const override {
    registry.insert<HAL::HALDialect, arith::ArithDialect, tensor::TensorDialect>();
  }

  void runOnOperation() override {
    ModuleOp module = getOperation();
    // The device target assigned before preprocessing (Pipelines.cpp:87-90). The extern
    // variant's target must match it exactly, so it is copied, not invented.
    auto targets = module->getAttrOfType<ArrayAttr>("hal.device.targets");
    HAL::ExecutableTargetAttr cudaTarget;
    if (targets)
      for (Attribute t : targets)
        if (auto device = dyn_cast<HAL::DeviceTargetAttr>(t))
          for (auto exe : device.getExecutableTargets())
            if (exe.getBackend() == "cuda") cudaTarget = exe;
    if (!cudaTarget) return;  // not compiling for CUDA: nothing to do

    SmallVector<Matched> work;
    module.walk([&](linalg::LinalgOp op) {
      if (auto m = matchMatmul(op)) work.push_back(*m);
    });
    for (Matched &m : work)
      if (failed(rewrite(m, cudaTarget))) return signalPassFailure();
  }

 private:
  LogicalResult rewrite(Matched &m, HAL::ExecutableTargetAttr target) {
    OpBuilder b(m.last);
    Location loc = m.last->getLoc();
    auto lhsType = cast<RankedTensorType>(m.lhs.getType());
    auto rhsType = cast<RankedTensorType>(m.rhs.getType());
    auto outType = cast<RankedTensorType>(m.last->getResult(0).getType());
    if (!lhsType.hasStaticShape() || !rhsType.hasStaticShape())
      return success();  // dynamic shapes stay on the stock path in this version
    const int r = lhsType.getRank();
    const int64_t batch = m.batched ? lhsType.getDimSize(0) : 1;
    const int64_t M = lhsType.getDimSize(r - 2), K = lhsType.getDimSize(r - 1), N = rhsType.getDimSize(r - 1);
    const int64_t elem = m.kind == ElemKind::I8 ? 1 : 2;
    const bool tmaOk = (K * elem) % 16 == 0 && (N * elem) % 16 == 0;

    auto i32 = [&](int64_t v) -> Value { return b.create<arith::ConstantIntOp>(loc, v, 32); };
    auto idx = [&](int64_t v) -> Value { return b.create<arith::ConstantIndexOp>(loc, v); };
    auto object = HAL::ExecutableObjectAttr::get(b.getContext(), b.getStringAttr(options.cubinPath), nullptr);
    auto objects = HAL::ExecutableObjectsAttr::get(b.getContext(), b.getArrayAttr({target}),
                                                   b.getArrayAttr({b.getArrayAttr({object})}));

    // Helper: one hal.dispatch.extern with set 0 = [read-only inputs..., outputs...].
    auto emit = [&](StringRef name, ValueRange workload, ValueRange operands, TypeRange results, int numReadOnly,
                    int numConstants, ArrayRef<int64_t> grid, int64_t threads, int64_t smem) -> Operation * {
      SmallVector<HAL::DescriptorSetBindingAttr> bindingAttrs;
      SmallVector<HAL::InterfaceBindingAttr> bindings;
      const int numBindings = numReadOnly + results.size();
      for (int i = 0; i < numBindings; ++i) {
        bindingAttrs.push_back(HAL::DescriptorSetBindingAttr::get(
            b.getContext(), i, HAL::DescriptorType::StorageBuffer,
            i < numReadOnly ? std::optional<HAL::DescriptorFlags>(HAL::DescriptorFlags::ReadOnly) : std::nullopt));
        bindings.push_back(HAL::InterfaceBindingAttr::get(b.getContext(), 0, i));
      }
      auto layout = HAL::PipelineLayoutAttr::get(
          b.getContext(), numConstants, {HAL::DescriptorSetLayoutAttr::get(b.getContext(), 0, bindingAttrs)});
      auto ext = b.create<HAL::DispatchExternOp>(loc, results, workload, operands, /*argument_dims=*/ValueRange{},
                                                 /*result_dims=*/ValueRange{}, /*tied_operands=*/nullptr);
      ext.setExportAttr(b.getStringAttr(name));
      ext.setLayoutAttr(layout);
      ext.setBindingsAttr(b.getArrayAttr(SmallVector<Attribute>(bindings.begin(), bindings.end())));
      ext.setObjectsAttr(objects);
      ext.setWorkgroupSizeAttr(b.getIndexArrayAttr({threads, 1, 1}));
      if (smem) ext.setWorkgroupLocalMemoryAttr(b.getIndexAttr(smem));
      // count region: a constant grid (persistent kernels, static shapes).
      Block *count = ext.emplaceWorkgroupCountRegion();  // (!hal.device, workload...) -> (index, index, index)
      OpBuilder cb = OpBuilder::atBlockBegin(count);
      SmallVector<Value> g;
      for (int64_t v : grid) g.push_back(cb.create<arith::ConstantIndexOp>(loc, v));
      cb.create<HAL::ReturnOp>(loc, g);
      return ext;
    };

    if (!tmaOk) {
      // Shape-agnostic SIMT export: bindings (lhs, rhs, out), constants (M, N, K, rhs_layout).
      Operation *ext = emit(exportName(m, /*generic=*/true), {idx(M), idx(N)},
                            {m.lhs, m.rhs, i32(M), i32(N), i32(K), i32(0)}, {outType}, 2, 4,
                            {(N + 15) / 16, (M + 15) / 16, batch}, 256, 0);
      ext->setAttr("workgroup_size", b.getIndexArrayAttr({16, 16, 1}));
      m.last->getResult(0).replaceAllUsesWith(ext->getResult(0));
      return success();
    }

    const int64_t bn = chooseTileN(M, N, batch, 128 / elem, options.smCount);
    const int64_t tiles = ((M + 127) / 128) * ((N + bn - 1) / bn) * batch;
    const int64_t gridX = std::min<int64_t>(tiles, options.smCount);
    auto wsType = RankedTensorType::get({512}, b.getI8Type());
    // Templates: two 128-byte tensor maps of the right element type, encoded once at build
    // time and embedded as a constant (see b200_tensormap_templates in the kernel repository).
    Value templates = b.create<IREE::Util::UnfoldableConstantOp>(
        loc, DenseElementsAttr::get(RankedTensorType::get({256}, b.getI8Type()), b.getI8IntegerAttr(0)));
    Operation *enc = emit("b200_encode_tensormaps", {idx(1)},
                          {m.lhs, m.rhs, templates, i32(M), i32(N), i32(K), i32(batch), i32(0), i32(bn), i32(elem)},
                          {wsType}, 3, 7, {1, 1, 1}, 32, 0);
    Operation *gemm = emit(exportName(m, /*generic=*/false), {idx(tiles)},
                           {enc->getResult(0), i32(M), i32(N), i32(K), i32(batch), i32(0), i32(bn)}, {outType},
                           /*numReadOnly=*/0, 6, {gridX, 1, 1}, kGemmThreads, kGemmSmem);
    // The workspace is read and written (status words): bind it as the second read-write binding
    // by tying it through; the kernel ABI order is (out, workspace).
    gemm->setAttr("b200.binding_order", b.getStrArrayAttr({"out", "workspace"}));
    m.last->getResult(0).replaceAllUsesWith(gemm->getResult(0));
    return success();
  }

  RewriteOptions options;
};

}  // namespace

std::unique_ptr<OperationPass<ModuleOp>> createRewriteContractionsPass(RewriteOptions options) {
  return std::make_unique<RewriteContractionsPass>(std::move(options));
}

}  // namespace mlir::iree_compiler::b200
