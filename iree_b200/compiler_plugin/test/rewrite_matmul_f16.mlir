// RUN: iree-opt --iree-plugin=b200_contraction --pass-pipeline="builtin.module(iree-b200-rewrite-contractions)" %s | FileCheck %s
// (lit-style expectation; not executed in the kernel repository, which has no iree-opt)

#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>
module attributes {hal.device.targets = [#cuda]} {
  util.func public @matmul_f16(%lhs: tensor<4096x4096xf16>, %rhs: tensor<4096x4096xf16>) -> tensor<4096x4096xf16> {
    %zero = arith.constant 0.0 : f32
    %e = tensor.empty() : tensor<4096x4096xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<4096x4096xf32>) -> tensor<4096x4096xf32>
    %mm = linalg.matmul ins(%lhs, %rhs : tensor<4096x4096xf16>, tensor<4096x4096xf16>)
                        outs(%fill : tensor<4096x4096xf32>) -> tensor<4096x4096xf32>
    %o = tensor.empty() : tensor<4096x4096xf16>
    %t = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%mm : tensor<4096x4096xf32>) outs(%o : tensor<4096x4096xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<4096x4096xf16>
    util.return %t : tensor<4096x4096xf16>
  }
}

// 4096^3 fills the SM pairs: the CTA-pair export; each CTA loads half of the 256-wide right-hand tile, so the
// encode dispatch gets 128.
// CHECK-LABEL: util.func public @matmul_f16
//   CHECK-NOT:   linalg.matmul
//       CHECK:   %[[WS:.+]] = hal.dispatch.extern "b200_encode_tensormaps"
//  CHECK-SAME:       %c4096_i32, %c4096_i32, %c4096_i32, %c1_i32, %c0_i32, %c128_i32, %c2_i32
//  CHECK-SAME:       -> tensor<512xi8>
//       CHECK:     push_constants = 7
//       CHECK:     #hal.executable.object<{path = "b200_contraction.cubin"}>
//       CHECK:     workgroup_size = [32 : index, 1 : index, 1 : index]
//       CHECK:   %[[OUT:.+]] = hal.dispatch.extern "b200_matmul_pair_f16_f16"
//  CHECK-SAME:       (%[[WS]], %c4096_i32, %c4096_i32, %c4096_i32, %c1_i32, %c0_i32, %c256_i32)
//       CHECK:     hal.return %c148, %c1, %c1
//       CHECK:     push_constants = 6
//       CHECK:     workgroup_local_memory = 230656 : index
//       CHECK:   util.return %[[OUT]]
