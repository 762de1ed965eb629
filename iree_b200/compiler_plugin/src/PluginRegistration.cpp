// b200_contraction: routes contraction dispatches to hand-written sm_100a kernels.
//
// The session adds one pass at the preprocessing hook
// (PluginAPI/Client.h: extendPreprocessingPassPipeline, called from
// Preprocessing/Passes.cpp before the transform-spec and PDL steps). There is no hook inside
// dispatch formation itself, so "during dispatch formation" is realised as "immediately before
// it", exactly as the custom_dispatch samples do.
#include "Passes.h"
#include "iree/compiler/PluginAPI/Client.h"
#include "mlir/Pass/PassManager.h"

using namespace mlir;
using namespace mlir::iree_compiler;

namespace {

struct B200Options {
  std::string cubinPath = "b200_contraction.cubin";
  int smCount = 148;
  bool deviceTensorMaps = true;

  void bindOptions(OptionsBinder &binder) {
    static llvm::cl::OptionCategory category("B200 contraction plugin");
    binder.opt<std::string>("iree-b200-cubin", cubinPath, llvm::cl::cat(category),
                            llvm::cl::desc("File name of the sm_100a cubin recorded in the "
                                           "#hal.executable.object of every rewritten dispatch."));
    binder.opt<int>("iree-b200-sm-count", smCount, llvm::cl::cat(category),
                    llvm::cl::desc("SM count the persistent kernels' grids are capped at."));
    binder.opt<bool>("iree-b200-device-tensor-maps", deviceTensorMaps, llvm::cl::cat(category),
                     llvm::cl::desc("Emit the b200_encode_tensormaps dispatch ahead of each "
                                    "tensor-core contraction (required with the stock CUDA driver)."));
  }
};

// Explicit activation: the plugin only acts when named with --iree-plugin=b200_contraction.
struct B200Session : public PluginSession<B200Session, B200Options, PluginActivationPolicy::Explicit> {
  void extendPreprocessingPassPipeline(OpPassManager &pm) override {
    b200::RewriteOptions opts;
    opts.cubinPath = options.cubinPath;
    opts.smCount = options.smCount;
    opts.deviceTensorMaps = options.deviceTensorMaps;
    pm.addPass(b200::createRewriteContractionsPass(opts));
  }
};

}  // namespace

IREE_DEFINE_COMPILER_OPTION_FLAGS(B200Options);

extern "C" bool iree_register_compiler_plugin_b200_contraction(mlir::iree_compiler::PluginRegistrar *registrar) {
  registrar->registerPlugin<B200Session>("b200_contraction");
  return true;
}
