// RUN: iree-opt --iree-plugin=b200_contraction --pass-pipeline="builtin.module(iree-b200-rewrite-contractions)" %s | FileCheck %s
// (lit-style expectation; not executed in the kernel repository, which has no iree-opt)

#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>
module attributes {hal.device.targets = [#cuda]} {
  util.func public @w4a16_m2048(%a: tensor<2048x32x128xf16>, %wq: tensor<11008x2048xi8>, %scales: tensor<11008x32xf16>) -> tensor<2048x11008xf16> {
    %w4 = flow.tensor.bitcast %wq : tensor<11008x2048xi8> -> tensor<11008x32x128xi4>
    %we = tensor.empty() : tensor<11008x32x128xf16>
    %deq = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2) -> (d0, d1, d2)>, affine_map<(d0, d1, d2) -> (d0, d1)>,
                                            affine_map<(d0, d1, d2) -> (d0, d1, d2)>],
                           iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%w4, %scales : tensor<11008x32x128xi4>, tensor<11008x32xf16>) outs(%we : tensor<11008x32x128xf16>) {
      ^bb0(%in: i4, %s: f16, %out: f16):
        %i = arith.extsi %in : i4 to i32
        %f = arith.sitofp %i : i32 to f16
        %d = arith.mulf %f, %s : f16
        linalg.yield %d : f16
    } -> tensor<11008x32x128xf16>
    %zero = arith.constant 0.000000e+00 : f32
    %e = tensor.empty() : tensor<2048x11008xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<2048x11008xf32>) -> tensor<2048x11008xf32>
    %acc = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2, d3) -> (d0, d2, d3)>, affine_map<(d0, d1, d2, d3) -> (d1, d2, d3)>,
                                            affine_map<(d0, d1, d2, d3) -> (d0, d1)>],
                           iterator_types = ["parallel", "parallel", "reduction", "reduction"]}
        ins(%a, %deq : tensor<2048x32x128xf16>, tensor<11008x32x128xf16>) outs(%fill : tensor<2048x11008xf32>) {
      ^bb0(%x: f16, %w: f16, %out: f32):
        %xe = arith.extf %x : f16 to f32
        %we2 = arith.extf %w : f16 to f32
        %p = arith.mulf %xe, %we2 : f32
        %sum = arith.addf %p, %out : f32
        linalg.yield %sum : f32
    } -> tensor<2048x11008xf32>
    %o = tensor.empty() : tensor<2048x11008xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc : tensor<2048x11008xf32>) outs(%o : tensor<2048x11008xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<2048x11008xf16>
    util.return %r : tensor<2048x11008xf16>
  }
}

// Pattern D: dequantisation producer (extsi i4, sitofp, mulf by the group's scale) + contraction over
// (group, k) + truncf consumer. 2048 rows: the kernel that keeps the expanded weights in tensor memory;
// its three tensor maps (activations, raw weights, result) are built on the device from the template table.
// CHECK-LABEL: util.func public @w4a16_m2048
//   CHECK-NOT:   linalg.generic
//       CHECK:   %[[T:.+]] = util.unfoldable_constant dense<{{.*}}> : tensor<768xi8>
//       CHECK:   %[[W0:.+]] = hal.dispatch.extern "b200_encode_tensormap"
//  CHECK-SAME:       (%a, %[[T]],
//       CHECK:   %[[W1:.+]] = hal.dispatch.extern "b200_encode_tensormap"
//  CHECK-SAME:       %[[W0]]
//       CHECK:   %[[W2:.+]] = hal.dispatch.extern "b200_encode_tensormap"
//  CHECK-SAME:       %[[W1]]
//       CHECK:   %[[OUT:.+]] = hal.dispatch.extern "b200_w4a16_gemm_wt"
//  CHECK-SAME:       %[[W2]], %c2048_i32, %c11008_i32, %c4096_i32, %c11008_i32, %c0_i32, %c256_i32, %c0_i32
//       CHECK:     hal.return %c148, %c1, %c1
//       CHECK:     push_constants = 7
//       CHECK:     workgroup_size = [512 : index, 1 : index, 1 : index], workgroup_local_memory = 214528 : index
//       CHECK:   util.return %[[OUT]]
