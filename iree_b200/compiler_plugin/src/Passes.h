// Pass entry points of the b200_contraction plugin.
#ifndef IREE_B200_CONTRACTION_PASSES_H_
#define IREE_B200_CONTRACTION_PASSES_H_

#include <memory>
#include <string>

#include "mlir/Pass/Pass.h"

namespace mlir::iree_compiler::b200 {

struct RewriteOptions {
  // File name recorded in #hal.executable.object; resolved on
  // --iree-hal-executable-object-search-path like any external object.
  std::string cubinPath = "b200_contraction.cubin";
  // Number of SMs the persistent kernels are sized for (B200: 148).
  int smCount = 148;
  // Build tensor maps with the b200_encode_tensormaps dispatch (needed with the stock CUDA HAL
  // driver, which never calls cuTensorMapEncodeTiled).
  bool deviceTensorMaps = true;
};

// Replaces matched contraction patterns with hal.dispatch.extern ops. Runs on the module at
// the plugin's extendPreprocessingPassPipeline hook, i.e. before dispatch formation.
std::unique_ptr<OperationPass<ModuleOp>> createRewriteContractionsPass(RewriteOptions options);

}  // namespace mlir::iree_compiler::b200

#endif  // IREE_B200_CONTRACTION_PASSES_H_
