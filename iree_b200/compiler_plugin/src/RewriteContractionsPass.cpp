// Matches contraction patterns on linalg-on-tensors and replaces each with hal.dispatch.extern
// ops that launch exports of b200_contraction.cubin.
//
// What a "contraction dispatch" contains follows dispatch formation
// (Dialect/Flow/Transforms/FormDispatchRegions.cpp: named matmuls are roots, linalg.fill is pulled
// in, elementwise consumers fuse; RegionOpUtils.cpp: dequantisation-like producers are cloned
// in). This pass matches the same groups one step earlier:
//
//   A  fill(0) -> linalg.matmul / batch_matmul, f16 x f16 -> f32 [-> truncf to f16]
//        -> b200_matmul[_pair]_f16_f16 (with truncf) or b200_matmul[_pair]_f16_f32
//   B  the same with bf16
//   C  fill(0) -> linalg.matmul i8 x i8 -> i32 [-> generic(sitofp, mulf a_scale[m], mulf w_scale[n], truncf)]
//        -> b200_matmul[_pair]_i8_i32 or b200_matmul[_pair]_i8_requant_f16
//   D  generic(extsi i4 -> sitofp f16 -> mulf scale[n,g]) feeding the grouped contraction
//      generic with two reduction dims (g, k) and a truncf (the IR of
//      Dialect/Flow/Transforms/test/pipeline_tests.mlir:53-99, signed weights, no zero point)
//        -> b200_w4a16_decode_m8 / _m16 (static M <= 16), b200_w4a16_gemm_wt (M > 16, aligned result),
//           else b200_w4a16_gemm
//
// Operands whose row pitch is not a multiple of 16 bytes go to the *_generic exports.
// Kernel ABI: every binding as a pointer, then every i32 constant, in the order given here; thread
// counts and dynamic shared-memory sizes must equal the runtime library's export table (a test of
// the kernel repository compares the constants below with it). Tensor maps cannot travel as kernel
// parameters and the stock CUDA HAL driver never encodes any, so each map is built on the device
// by a b200_encode_tensormap(s) dispatch from a template embedded as a constant.
#include <algorithm>
#include <optional>

#include "Passes.h"
#include "iree/compiler/Dialect/Flow/IR/FlowOps.h"
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

// kTensorMapTemplates[6][128]: one encoded tensor map per kind (element type, rank, swizzle),
// written by compiler_plugin/gen_templates.py on a machine with the CUDA driver.
#include "TensorMapTemplates.inc"

constexpr int64_t kGemmThreads = 256, kGemmSmem = 230656;
constexpr int64_t kW4GemmThreads = 512, kW4GemmSmem = 230656, kW4WtThreads = 512, kW4WtSmem = 214528;
constexpr int64_t kDecodeThreads = 512, kDecodeSmemM8 = 217984, kDecodeSmemM16 = 213760;
constexpr int64_t kDecodeSliceK = 4096;
// indices into the template table (IREE_B200_TEMPLATE_* of the runtime library's header)
enum Template { kF16Sw128R3 = 0, kBF16Sw128R3 = 1, kU8Sw128R3 = 2, kU8Sw64R3 = 3, kF16PlainR2 = 4, kU64PlainR2 = 5 };

enum class ElemKind { F16, BF16, I8, Unsupported };
enum class Epilogue { Accumulator, Cast, RequantF16 };

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

// The body of `generic`, without its terminator, as a list of operation names.
static bool bodyIs(linalg::GenericOp generic, ArrayRef<StringRef> names) {
  Block &body = generic.getRegion().front();
  if (body.getOperations().size() != names.size() + 1) return false;
  auto it = body.begin();
  for (StringRef n : names)
    if ((it++)->getName().getStringRef() != n) return false;
  return true;
}

// The only user of `v`, if it is an all-parallel generic with exactly this body.
static linalg::GenericOp matchConsumer(Value v, ArrayRef<StringRef> body) {
  if (!v.hasOneUse()) return nullptr;
  auto generic = dyn_cast<linalg::GenericOp>(*v.getUsers().begin());
  if (!generic || generic.getNumReductionLoops() != 0 || generic.getNumDpsInits() != 1) return nullptr;
  return bodyIs(generic, body) ? generic : nullptr;
}

// Result positions of an indexing map as a list of dimension indices; empty if not a projection.
static SmallVector<int64_t> dimsOf(AffineMap map) {
  SmallVector<int64_t> dims;
  for (AffineExpr e : map.getResults()) {
    auto d = dyn_cast<AffineDimExpr>(e);
    if (!d) return {};
    dims.push_back(d.getPosition());
  }
  return dims;
}

struct Matched {
  Operation *last = nullptr;  // the op whose result the rewrite replaces
  // patterns A-C
  Value lhs, rhs, rowScale, colScale;
  ElemKind kind = ElemKind::Unsupported;
  Epilogue epilogue = Epilogue::Accumulator;
  bool batched = false;
  // pattern D
  bool grouped = false;
  Value activations, weights, scales;  // weights: i4 [N, G, group] or the i8 [N, K/2] they were bitcast from
  int64_t M = 0, N = 0, K = 0, group = 0;
};

static std::optional<Matched> matchMatmul(linalg::LinalgOp op) {
  if (!isa<linalg::MatmulOp, linalg::BatchMatmulOp>(op.getOperation())) return std::nullopt;
  Matched m;
  m.last = op;
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
    // A, B: truncf consumer back to the operand type
    if (linalg::GenericOp trunc = matchConsumer(op->getResult(0), {"arith.truncf"})) {
      auto outType = cast<RankedTensorType>(trunc->getResult(0).getType());
      if (trunc.getNumDpsInputs() == 1 && kindOf(outType.getElementType()) == m.kind) {
        m.last = trunc;
        m.epilogue = Epilogue::Cast;
      }
    }
    return m;
  }
  // C: the requantisation consumer f16(f32(acc) * a_scale[m] * w_scale[n]), operation order as written
  if (m.batched) return m;
  linalg::GenericOp q = matchConsumer(op->getResult(0), {"arith.sitofp", "arith.mulf", "arith.mulf", "arith.truncf"});
  if (!q || q.getNumDpsInputs() != 3 || q.getDpsInputs()[0] != op->getResult(0)) return m;
  auto maps = q.getIndexingMapsArray();
  auto rowType = dyn_cast<RankedTensorType>(q.getDpsInputs()[1].getType());
  auto colType = dyn_cast<RankedTensorType>(q.getDpsInputs()[2].getType());
  auto outType = cast<RankedTensorType>(q->getResult(0).getType());
  if (!rowType || !colType || !rowType.getElementType().isF32() || !colType.getElementType().isF32() ||
      !outType.getElementType().isF16())
    return m;
  if (dimsOf(maps[0]) != SmallVector<int64_t>{0, 1} || dimsOf(maps[1]) != SmallVector<int64_t>{0} ||
      dimsOf(maps[2]) != SmallVector<int64_t>{1})
    return m;
  // the body must multiply the converted accumulator by the row scale first, then by the column scale
  Block &body = q.getRegion().front();
  auto it = body.begin();
  Operation *conv = &*it++, *mul0 = &*it++, *mul1 = &*it++, *trunc = &*it++;
  auto usesBoth = [](Operation *mul, Value a, Value b) {
    return (mul->getOperand(0) == a && mul->getOperand(1) == b) || (mul->getOperand(0) == b && mul->getOperand(1) == a);
  };
  if (conv->getOperand(0) != body.getArgument(0) || !usesBoth(mul0, conv->getResult(0), body.getArgument(1)) ||
      !usesBoth(mul1, mul0->getResult(0), body.getArgument(2)) || trunc->getOperand(0) != mul1->getResult(0))
    return m;
  m.rowScale = q.getDpsInputs()[1];
  m.colScale = q.getDpsInputs()[2];
  m.last = q;
  m.epilogue = Epilogue::RequantF16;
  return m;
}

// D: contraction generic (m, n, g, k) over activations [M, G, group] and dequantised weights
// [N, G, group], whose producer is the dequantisation generic; consumer truncf to f16.
static std::optional<Matched> matchGroupedDequant(linalg::GenericOp op) {
  if (op.getNumLoops() != 4 || op.getNumReductionLoops() != 2 || op.getNumDpsInputs() != 2) return std::nullopt;
  SmallVector<utils::IteratorType> iters = op.getIteratorTypesArray();
  if (iters[0] != utils::IteratorType::parallel || iters[1] != utils::IteratorType::parallel) return std::nullopt;
  if (!bodyIs(op, {"arith.extf", "arith.extf", "arith.mulf", "arith.addf"}) || !isZeroFill(op.getDpsInits()[0]))
    return std::nullopt;
  auto maps = op.getIndexingMapsArray();
  if (dimsOf(maps[0]) != SmallVector<int64_t>{0, 2, 3} || dimsOf(maps[1]) != SmallVector<int64_t>{1, 2, 3} ||
      dimsOf(maps[2]) != SmallVector<int64_t>{0, 1})
    return std::nullopt;
  auto deq = op.getDpsInputs()[1].getDefiningOp<linalg::GenericOp>();
  if (!deq || deq.getNumReductionLoops() != 0 || deq.getNumDpsInputs() != 2 ||
      !bodyIs(deq, {"arith.extsi", "arith.sitofp", "arith.mulf"}))
    return std::nullopt;
  auto dmaps = deq.getIndexingMapsArray();
  if (dimsOf(dmaps[0]) != SmallVector<int64_t>{0, 1, 2} || dimsOf(dmaps[1]) != SmallVector<int64_t>{0, 1})
    return std::nullopt;
  auto actType = cast<RankedTensorType>(op.getDpsInputs()[0].getType());
  auto wType = cast<RankedTensorType>(deq.getDpsInputs()[0].getType());
  auto sType = cast<RankedTensorType>(deq.getDpsInputs()[1].getType());
  if (!actType.hasStaticShape() || !wType.hasStaticShape() || !actType.getElementType().isF16() ||
      !wType.getElementType().isInteger(4) || !sType.getElementType().isF16())
    return std::nullopt;
  linalg::GenericOp trunc = matchConsumer(op->getResult(0), {"arith.truncf"});
  if (!trunc || !cast<RankedTensorType>(trunc->getResult(0).getType()).getElementType().isF16()) return std::nullopt;
  Matched m;
  m.grouped = true;
  m.last = trunc;
  m.activations = op.getDpsInputs()[0];
  m.weights = deq.getDpsInputs()[0];
  // int4 tensors reach programs as bytes and are bitcast (the Torch frontend's bitcast_quant_tensor): bind the bytes
  if (auto cast = m.weights.getDefiningOp<IREE::Flow::TensorBitCastOp>()) m.weights = cast.getSource();
  m.scales = deq.getDpsInputs()[1];
  m.M = actType.getDimSize(0);
  m.N = wType.getDimSize(0);
  m.group = wType.getDimSize(2);
  m.K = wType.getDimSize(1) * m.group;
  if (actType.getDimSize(1) != wType.getDimSize(1) || actType.getDimSize(2) != m.group) return std::nullopt;
  return m;
}

static StringRef exportName(const Matched &m, bool generic, bool pairs) {
  const char *stem = nullptr;
  switch (m.kind) {
    case ElemKind::F16: stem = m.epilogue == Epilogue::Cast ? "f16_f16" : "f16_f32"; break;
    case ElemKind::BF16: stem = m.epilogue == Epilogue::Cast ? "bf16_bf16" : "bf16_f32"; break;
    default: stem = m.epilogue == Epilogue::RequantF16 ? "i8_requant_f16" : "i8_i32"; break;
  }
  static thread_local std::string name;
  name = std::string(generic ? "b200_matmul_generic_" : pairs ? "b200_matmul_pair_" : "b200_matmul_") + stem;
  return name;
}

// CTA pairs (256-row tiles, tcgen05 cta_group::2) pay off when there are enough 256 x 256 tiles to
// fill the SM pairs (the runtime library's rule).
static bool usePairs(int64_t M, int64_t N, int64_t K, int64_t batch, int smCount) {
  const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256) * batch;
  return M >= 256 && tiles >= (smCount & ~1) / 2 && K >= 512;
}

// The widest tile that still gives every SM (pair) work (same cost model as the runtime library).
static int64_t chooseTileN(int64_t M, int64_t N, int64_t batch, int64_t chunk, int smCount, bool pairs) {
  int64_t best = chunk;
  double bestCost = 0;
  const int64_t units = (smCount & ~1) / (pairs ? 2 : 1), rows = pairs ? 256 : 128;
  for (int64_t bn = 256; bn >= 32; bn -= 32) {
    if (bn % chunk) continue;
    if (M <= 32 && bn > 128 && chunk <= 128) continue;  // few rows: tiles <= 128 wide select the deep-ring variant
    const int64_t tiles = ((M + rows - 1) / rows) * ((N + bn - 1) / bn) * batch;
    const double cost = double((tiles + units - 1) / units) * (400.0 + bn);
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
    if (targets)
      for (Attribute t : targets)
        if (auto device = dyn_cast<HAL::DeviceTargetAttr>(t))
          for (auto exe : device.getExecutableTargets())
            if (exe.getBackend() == "cuda") cudaTarget = exe;
    if (!cudaTarget) return;  // not compiling for CUDA: nothing to do

    SmallVector<Matched> work;
    module.walk([&](linalg::LinalgOp op) {
      if (auto m = matchMatmul(op)) {
        work.push_back(*m);
      } else if (auto generic = dyn_cast<linalg::GenericOp>(op.getOperation())) {
        if (auto g = matchGroupedDequant(generic)) work.push_back(*g);
      }
    });
    for (Matched &m : work)
      if (failed(m.grouped ? rewriteGrouped(m) : rewriteMatmul(m))) return signalPassFailure();
  }

 private:
  // One hal.dispatch.extern: set 0 = [read-only inputs..., results...], then the i32 constants.
  Operation *emit(OpBuilder &b, Location loc, StringRef name, ValueRange workload, ValueRange operands, TypeRange results,
                  int numReadOnly, int numConstants, ArrayRef<int64_t> grid, ArrayRef<int64_t> block, int64_t smem) {
    SmallVector<HAL::DescriptorSetBindingAttr> bindingAttrs;
    SmallVector<Attribute> bindings;
    const int numBindings = numReadOnly + results.size();
    for (int i = 0; i < numBindings; ++i) {
      bindingAttrs.push_back(HAL::DescriptorSetBindingAttr::get(
          b.getContext(), i, HAL::DescriptorType::StorageBuffer,
          i < numReadOnly ? std::optional<HAL::DescriptorFlags>(HAL::DescriptorFlags::ReadOnly) : std::nullopt));
      bindings.push_back(HAL::InterfaceBindingAttr::get(b.getContext(), 0, i));
    }
    auto layout = HAL::PipelineLayoutAttr::get(b.getContext(), numConstants,
                                               {HAL::DescriptorSetLayoutAttr::get(b.getContext(), 0, bindingAttrs)});
    auto object = HAL::ExecutableObjectAttr::get(b.getContext(), b.getStringAttr(options.cubinPath), nullptr);
    auto objects = HAL::ExecutableObjectsAttr::get(b.getContext(), b.getArrayAttr({cudaTarget}),
                                                   b.getArrayAttr({b.getArrayAttr({object})}));
    auto ext = b.create<HAL::DispatchExternOp>(loc, results, workload, operands, /*argument_dims=*/ValueRange{},
                                               /*result_dims=*/ValueRange{}, /*tied_operands=*/nullptr);
    ext.setExportAttr(b.getStringAttr(name));
    ext.setLayoutAttr(layout);
    ext.setBindingsAttr(b.getArrayAttr(bindings));
    ext.setObjectsAttr(objects);
    ext.setWorkgroupSizeAttr(b.getIndexArrayAttr(block));
    if (smem) ext.setWorkgroupLocalMemoryAttr(b.getIndexAttr(smem));
    // count region: a constant grid (persistent kernels, static shapes).
    Block *count = ext.emplaceWorkgroupCountRegion();  // (!hal.device, workload...) -> (index, index, index)
    OpBuilder cb = OpBuilder::atBlockBegin(count);
    SmallVector<Value> g;
    for (int64_t v : grid) g.push_back(cb.create<arith::ConstantIndexOp>(loc, v));
    cb.create<HAL::ReturnOp>(loc, g);
    return ext;
  }

  Value i32(OpBuilder &b, Location loc, int64_t v) { return b.create<arith::ConstantIntOp>(loc, v, 32); }
  Value idx(OpBuilder &b, Location loc, int64_t v) { return b.create<arith::ConstantIndexOp>(loc, v); }

  // The template table as an embedded constant (768 bytes).
  Value templates(OpBuilder &b, Location loc) {
    SmallVector<int8_t> bytes(reinterpret_cast<const int8_t *>(kTensorMapTemplates),
                              reinterpret_cast<const int8_t *>(kTensorMapTemplates) + sizeof kTensorMapTemplates);
    auto type = RankedTensorType::get({static_cast<int64_t>(bytes.size())}, b.getI8Type());
    return b.create<IREE::Util::UnfoldableConstantOp>(loc, DenseElementsAttr::get(type, ArrayRef<int8_t>(bytes)));
  }

  // b200_encode_tensormap: one map at byte `slot` of the workspace (tied through as result).
  // dims / box innermost first; strides = byte pitches of dims 1 and 2.
  Value encodeMap(OpBuilder &b, Location loc, Value tensor, Value table, Value workspace, int64_t slot, Template tmpl, int rank,
                  ArrayRef<int64_t> dims, ArrayRef<int64_t> strides, ArrayRef<int64_t> box, int64_t elemBytes, int64_t flags) {
    int64_t d[3] = {1, 1, 1}, bx[3] = {1, 1, 1}, st[2] = {0, 0};
    std::copy(dims.begin(), dims.end(), d);
    std::copy(box.begin(), box.end(), bx);
    std::copy(strides.begin(), strides.end(), st);
    SmallVector<Value> operands = {tensor, table, workspace};
    for (int64_t v : {slot, int64_t(tmpl), int64_t(rank), d[0], d[1], d[2], int64_t(int32_t(uint32_t(st[0]))), st[0] >> 32,
                      int64_t(int32_t(uint32_t(st[1]))), st[1] >> 32, bx[0], bx[1], bx[2], bx[0] * bx[1] * bx[2] * elemBytes, flags})
      operands.push_back(i32(b, loc, v));
    Operation *ext = emit(b, loc, "b200_encode_tensormap", {idx(b, loc, 1)}, operands, {workspace.getType()},
                          /*numReadOnly=*/2, 15, {1, 1, 1}, {32, 1, 1}, 0);
    ext->setAttr("tied_operands", b.getIndexArrayAttr({2}));  // the workspace is updated in place
    return ext->getResult(0);
  }

  // A zero-filled workspace of `bytes` bytes.
  Value workspace(OpBuilder &b, Location loc, int64_t bytes) {
    auto type = RankedTensorType::get({bytes}, b.getI8Type());
    Value zero = b.create<arith::ConstantIntOp>(loc, 0, 8);
    Value empty = b.create<tensor::EmptyOp>(loc, type.getShape(), b.getI8Type());
    return b.create<linalg::FillOp>(loc, zero, empty).getResult(0);
  }

  LogicalResult rewriteMatmul(Matched &m) {
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
    const bool tmaOk = (K * elem) % 16 == 0 && (N * elem) % 16 == 0 && K > 0;
    const bool requant = m.epilogue == Epilogue::RequantF16;
    SmallVector<Value> scales;
    if (requant) scales = {m.rowScale, m.colScale};

    if (!tmaOk) {
      // Shape-agnostic SIMT export: bindings (lhs, rhs, out[, a_scale, w_scale]), constants (M, N, K, rhs_layout).
      SmallVector<Value> operands = {m.lhs, m.rhs};
      operands.append(scales);
      for (int64_t v : {M, N, K, int64_t(0)}) operands.push_back(i32(b, loc, v));
      Operation *ext = emit(b, loc, exportName(m, /*generic=*/true, false), {idx(b, loc, M), idx(b, loc, N)}, operands,
                            {outType}, 2 + scales.size(), 4, {(N + 15) / 16, (M + 15) / 16, batch}, {16, 16, 1}, 0);
      // kernel parameter order differs from (read-only..., result): out is the third pointer
      ext->setAttr("b200.binding_order", b.getStrArrayAttr(requant ? ArrayRef<StringRef>{"lhs", "rhs", "out", "a_scale", "w_scale"}
                                                                   : ArrayRef<StringRef>{"lhs", "rhs", "out"}));
      m.last->getResult(0).replaceAllUsesWith(ext->getResult(0));
      return success();
    }

    const bool pairs = usePairs(M, N, K, batch, options.smCount);
    const int64_t bn = chooseTileN(M, N, batch, (pairs ? 2 : 1) * 128 / elem, options.smCount, pairs);
    const int64_t rows = pairs ? 256 : 128;
    const int64_t tiles = ((M + rows - 1) / rows) * ((N + bn - 1) / bn) * batch;
    const int64_t gridX = pairs ? 2 * std::min<int64_t>(tiles, (options.smCount & ~1) / 2) : std::min<int64_t>(tiles, options.smCount);
    auto wsType = RankedTensorType::get({512}, b.getI8Type());
    // The A / B templates of the operand type: rows (2 kind) and (2 kind + 1) of the pair table this export reads.
    const Template tmpl = m.kind == ElemKind::I8 ? kU8Sw128R3 : m.kind == ElemKind::BF16 ? kBF16Sw128R3 : kF16Sw128R3;
    SmallVector<int8_t> pair(256);
    std::copy_n(reinterpret_cast<const int8_t *>(kTensorMapTemplates[tmpl]), 128, pair.begin());
    std::copy_n(reinterpret_cast<const int8_t *>(kTensorMapTemplates[tmpl]), 128, pair.begin() + 128);
    Value pairTable = b.create<IREE::Util::UnfoldableConstantOp>(
        loc, DenseElementsAttr::get(RankedTensorType::get({256}, b.getI8Type()), ArrayRef<int8_t>(pair)));
    // in pair mode each CTA loads half of the right-hand tile: the map's box is half as wide
    SmallVector<Value> encOperands = {m.lhs, m.rhs, pairTable};
    for (int64_t v : {M, N, K, batch, int64_t(0), pairs ? bn / 2 : bn, elem}) encOperands.push_back(i32(b, loc, v));
    Operation *enc = emit(b, loc, "b200_encode_tensormaps", {idx(b, loc, 1)}, encOperands, {wsType}, 3, 7, {1, 1, 1}, {32, 1, 1}, 0);
    // GEMM: bindings (out[, a_scale, w_scale], workspace), constants (M, N, K, batch, rhs_layout, tile_n)
    SmallVector<Value> operands(scales.begin(), scales.end());
    operands.push_back(enc->getResult(0));
    for (int64_t v : {M, N, K, batch, int64_t(0), bn}) operands.push_back(i32(b, loc, v));
    Operation *gemm = emit(b, loc, exportName(m, /*generic=*/false, pairs), {idx(b, loc, tiles)}, operands, {outType},
                           /*numReadOnly=*/scales.size(), 6, {gridX, 1, 1}, {kGemmThreads, 1, 1}, kGemmSmem);
    // The workspace is read and written (status words): it is the last read-write binding.
    gemm->setAttr("b200.binding_order", b.getStrArrayAttr(requant ? ArrayRef<StringRef>{"out", "a_scale", "w_scale", "workspace"}
                                                                  : ArrayRef<StringRef>{"out", "workspace"}));
    m.last->getResult(0).replaceAllUsesWith(gemm->getResult(0));
    return success();
  }

  LogicalResult rewriteGrouped(Matched &m) {
    OpBuilder b(m.last);
    Location loc = m.last->getLoc();
    auto outType = cast<RankedTensorType>(m.last->getResult(0).getType());
    const int64_t M = m.M, N = m.N, K = m.K, ldo = N, nOff = 0;
    const int sms = options.smCount;
    if (m.group != 128 || K % 128) {
      // any group size: one thread per output. bindings (a, wq, scales, out), constants (M, N, K, group, ldo, n_off)
      SmallVector<Value> operands = {m.activations, m.weights, m.scales};
      for (int64_t v : {M, N, K, m.group, ldo, nOff}) operands.push_back(i32(b, loc, v));
      Operation *ext = emit(b, loc, "b200_w4a16_generic", {idx(b, loc, M), idx(b, loc, N)}, operands, {outType}, 3, 6,
                            {(N + 255) / 256, M, 1}, {256, 1, 1}, 0);
      m.last->getResult(0).replaceAllUsesWith(ext->getResult(0));
      return success();
    }
    Value table = templates(b, loc);
    if (M <= 16 && N % 16 == 0 && K % 256 == 0 && K <= 4 * kDecodeSliceK) {
      // decode: HBM-bound weight streaming. Workspace: header, a counter per 16-row tile (padded to 256 bytes),
      // one 1 KiB partial tile per tile and K slice. K beyond one slice: the weight map is built first.
      const int64_t slices = (K + kDecodeSliceK - 1) / kDecodeSliceK;
      const int64_t counters = ((N / 16) * 4 + 255) / 256 * 256;
      Value ws = workspace(b, loc, 512 + counters + (N / 16) * slices * 1024);
      if (slices > 1)
        ws = encodeMap(b, loc, m.weights, table, ws, 0, kU64PlainR2, 2, {K / 16, N}, {K / 2}, {256, 8}, 8, /*flags=*/3);
      const int64_t walkers = std::max<int64_t>(1, std::min<int64_t>(N / 16, sms / slices));
      SmallVector<Value> operands = {m.activations, m.weights, m.scales, ws};
      for (int64_t v : {M, N, K, ldo, nOff}) operands.push_back(i32(b, loc, v));
      Operation *ext = emit(b, loc, M <= 8 ? "b200_w4a16_decode_m8" : "b200_w4a16_decode_m16", {idx(b, loc, N / 16)}, operands,
                            {outType}, 3, 5, {walkers * slices, 1, 1}, {kDecodeThreads, 1, 1}, M <= 8 ? kDecodeSmemM8 : kDecodeSmemM16);
      ext->setAttr("b200.binding_order", b.getStrArrayAttr({"a", "wq", "scales", "out", "workspace"}));
      m.last->getResult(0).replaceAllUsesWith(ext->getResult(0));
      return success();
    }
    if ((ldo * 2) % 16 == 0 && nOff % 8 == 0) {
      // more than sixteen rows: weights as the tensor-memory operand; 128 weight rows x 128 (M <= 128) or 256
      // activation rows per tile; results leave by TMA stores through the output map at byte 512 of the
      // workspace (one destination), which needs the result's pitch and offset on 16-byte boundaries
      Value ws = workspace(b, loc, 512 + 8 * 128 + 8 * 8);
      ws = encodeMap(b, loc, m.activations, table, ws, 0, kF16Sw128R3, 3, {K, M, 1}, {K * 2, M * K * 2}, {64, 128, 1}, 2, 1);
      ws = encodeMap(b, loc, m.weights, table, ws, 128, kU8Sw64R3, 3, {K / 2, N, 1}, {K / 2, N * (K / 2)}, {64, 128, 1}, 1, 0);
      // the result tensor the kernel stores into is the extern op's own result: the map is built over it by tying
      // an empty tensor through the builder dispatch
      Value result = b.create<tensor::EmptyOp>(loc, outType.getShape(), outType.getElementType());
      ws = encodeMap(b, loc, result, table, ws, 512, kF16PlainR2, 2, {nOff + N, M}, {ldo * 2}, {128, 64}, 2, 0);
      const int64_t tiles = ((M + 255) / 256) * ((N + 127) / 128);
      SmallVector<Value> operands = {m.scales, result, ws};
      for (int64_t v : {M, N, K, ldo, nOff, int64_t((1 << 8) | 0), int64_t(0)}) operands.push_back(i32(b, loc, v));
      Operation *ext = emit(b, loc, "b200_w4a16_gemm_wt", {idx(b, loc, tiles)}, operands, {outType}, 1, 7,
                            {std::min<int64_t>(tiles, sms), 1, 1}, {kW4WtThreads, 1, 1}, kW4WtSmem);
      ext->setAttr("tied_operands", b.getIndexArrayAttr({1}));  // writes the tensor the output map was built over
      ext->setAttr("b200.binding_order", b.getStrArrayAttr({"scales", "out", "workspace"}));
      m.last->getResult(0).replaceAllUsesWith(ext->getResult(0));
      return success();
    }
    // 128-row tiles, expanded weights as the shared-memory operand; tile width: a multiple of 16, at most 128
    int64_t bn = 0;
    double best = 0;
    for (int64_t cand = 128; cand >= 16; cand -= 16) {
      const int64_t t = ((M + 127) / 128) * ((N + cand - 1) / cand);
      const double cost = double((t + sms - 1) / sms) * (400.0 + cand);
      if (!bn || cost < best * 0.9999) bn = cand, best = cost;
    }
    Value ws = workspace(b, loc, 512);
    ws = encodeMap(b, loc, m.activations, table, ws, 0, kF16Sw128R3, 3, {K, M, 1}, {K * 2, M * K * 2}, {64, 128, 1}, 2, 1);
    ws = encodeMap(b, loc, m.weights, table, ws, 128, kU8Sw64R3, 3, {K / 2, N, 1}, {K / 2, N * (K / 2)}, {64, bn, 1}, 1, 0);
    const int64_t tiles = ((M + 127) / 128) * ((N + bn - 1) / bn);
    SmallVector<Value> operands = {m.scales, ws};
    for (int64_t v : {M, N, K, ldo, nOff, bn}) operands.push_back(i32(b, loc, v));
    Operation *ext = emit(b, loc, "b200_w4a16_gemm", {idx(b, loc, tiles)}, operands, {outType}, 1, 6,
                          {std::min<int64_t>(tiles, sms), 1, 1}, {kW4GemmThreads, 1, 1}, kW4GemmSmem);
    ext->setAttr("b200.binding_order", b.getStrArrayAttr({"scales", "out", "workspace"}));
    m.last->getResult(0).replaceAllUsesWith(ext->getResult(0));
    return success();
  }

  RewriteOptions options;
  HAL::ExecutableTargetAttr cudaTarget;
};

}  // namespace

std::unique_ptr<OperationPass<ModuleOp>> createRewriteContractionsPass(RewriteOptions options) {
  return std::make_unique<RewriteContractionsPass>(std::move(options));
}

}  // namespace mlir::iree_compiler::b200
