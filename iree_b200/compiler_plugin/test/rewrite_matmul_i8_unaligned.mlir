// RUN: iree-opt --iree-plugin=b200_contraction --pass-pipeline="builtin.module(iree-b200-rewrite-contractions)" %s | FileCheck %s
// A row pitch that is not a multiple of 16 bytes (K = 789 i8) cannot go through TMA: the
// shape-agnostic export is chosen, with no tensor-map dispatch.

#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>
module attributes {hal.device.targets = [#cuda]} {
  util.func public @matmul_i8(%lhs: tensor<123x789xi8>, %rhs: tensor<789x456xi8>) -> tensor<123x456xi32> {
    %zero = arith.constant 0 : i32
    %e = tensor.empty() : tensor<123x456xi32>
    %fill = linalg.fill ins(%zero : i32) outs(%e : tensor<123x456xi32>) -> tensor<123x456xi32>
    %mm = linalg.matmul ins(%lhs, %rhs : tensor<123x789xi8>, tensor<789x456xi8>)
                        outs(%fill : tensor<123x456xi32>) -> tensor<123x456xi32>
    util.return %mm : tensor<123x456xi32>
  }
}

// CHECK-LABEL: util.func public @matmul_i8
//   CHECK-NOT:   b200_encode_tensormaps
//       CHECK:   hal.dispatch.extern "b200_matmul_generic_i8_i32"
//       CHECK:     push_constants = 4
//       CHECK:     workgroup_size = [16 : index, 16 : index, 1 : index]
