// RUN: iree-opt --iree-plugin=b200_contraction --pass-pipeline="builtin.module(iree-b200-rewrite-contractions)" %s | FileCheck %s
// (lit-style expectation; not executed in the kernel repository, which has no iree-opt)

#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>
module attributes {hal.device.targets = [#cuda]} {
  util.func public @w8a8_m16(%lhs: tensor<16x4096xi8>, %rhs: tensor<4096x11008xi8>, %a_scale: tensor<16xf32>, %w_scale: tensor<11008xf32>) -> tensor<16x11008xf16> {
    %zero = arith.constant 0 : i32
    %e = tensor.empty() : tensor<16x11008xi32>
    %fill = linalg.fill ins(%zero : i32) outs(%e : tensor<16x11008xi32>) -> tensor<16x11008xi32>
    %acc = linalg.matmul ins(%lhs, %rhs : tensor<16x4096xi8>, tensor<4096x11008xi8>)
        outs(%fill : tensor<16x11008xi32>) -> tensor<16x11008xi32>
    %o = tensor.empty() : tensor<16x11008xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>,
                                          affine_map<(d0, d1) -> (d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc, %a_scale, %w_scale : tensor<16x11008xi32>, tensor<16xf32>, tensor<11008xf32>) outs(%o : tensor<16x11008xf16>) {
      ^bb0(%in: i32, %sa: f32, %sw: f32, %out: f16):
        %f = arith.sitofp %in : i32 to f32
        %x = arith.mulf %f, %sa : f32
        %y = arith.mulf %x, %sw : f32
        %t = arith.truncf %y : f32 to f16
        linalg.yield %t : f16
    } -> tensor<16x11008xf16>
    util.return %r : tensor<16x11008xf16>
  }
}

// Pattern C: i8 matmul + (sitofp, mulf a_scale[m], mulf w_scale[n], truncf) consumer. Sixteen rows: the
// few-rows variant of the 1-CTA export (tiles 128 wide, deep ring), 86 tiles.
// CHECK-LABEL: util.func public @w8a8_m16
//   CHECK-NOT:   linalg.matmul
//   CHECK-NOT:   arith.sitofp
//       CHECK:   %[[WS:.+]] = hal.dispatch.extern "b200_encode_tensormaps"
//  CHECK-SAME:       %c16_i32, %c11008_i32, %c4096_i32, %c1_i32, %c0_i32, %c128_i32, %c1_i32
//  CHECK-SAME:       -> tensor<512xi8>
//       CHECK:   %[[OUT:.+]] = hal.dispatch.extern "b200_matmul_i8_requant_f16"
//  CHECK-SAME:       (%a_scale, %w_scale, %[[WS]], %c16_i32, %c11008_i32, %c4096_i32, %c1_i32, %c0_i32, %c128_i32)
//       CHECK:     hal.return %c86, %c1, %c1
//       CHECK:     push_constants = 6
//       CHECK:     workgroup_size = [256 : index, 1 : index, 1 : index], workgroup_local_memory = 230656 : index
//       CHECK:   util.return %[[OUT]]
