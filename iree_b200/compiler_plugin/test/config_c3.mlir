// The benchmark configuration c3 as linalg-on-tensors, in the op shapes the rewrite pass matches.
// Written by `python -m iree_b200.mlir_frontend c3`; lowered to a host plan by
// iree_b200.mlir_frontend.plans_from_mlir (tests/test_dispatch_plan.py).
#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>
module attributes {hal.device.targets = [#cuda]} {
  util.func public @c3_m1(%lhs: tensor<1x4096xi8>, %rhs: tensor<4096x11008xi8>, %a_scale: tensor<1xf32>, %w_scale: tensor<11008xf32>) -> tensor<1x11008xf16> {
    %zero = arith.constant 0 : i32
    %e = tensor.empty() : tensor<1x11008xi32>
    %fill = linalg.fill ins(%zero : i32) outs(%e : tensor<1x11008xi32>) -> tensor<1x11008xi32>
    %acc = linalg.matmul ins(%lhs, %rhs : tensor<1x4096xi8>, tensor<4096x11008xi8>)
        outs(%fill : tensor<1x11008xi32>) -> tensor<1x11008xi32>
    %o = tensor.empty() : tensor<1x11008xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>,
                                          affine_map<(d0, d1) -> (d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc, %a_scale, %w_scale : tensor<1x11008xi32>, tensor<1xf32>, tensor<11008xf32>) outs(%o : tensor<1x11008xf16>) {
      ^bb0(%in: i32, %sa: f32, %sw: f32, %out: f16):
        %f = arith.sitofp %in : i32 to f32
        %x = arith.mulf %f, %sa : f32
        %y = arith.mulf %x, %sw : f32
        %t = arith.truncf %y : f32 to f16
        linalg.yield %t : f16
    } -> tensor<1x11008xf16>
    util.return %r : tensor<1x11008xf16>
  }
  util.func public @c3_m16(%lhs: tensor<16x4096xi8>, %rhs: tensor<4096x11008xi8>, %a_scale: tensor<16xf32>, %w_scale: tensor<11008xf32>) -> tensor<16x11008xf16> {
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
  util.func public @c3_m512(%lhs: tensor<512x4096xi8>, %rhs: tensor<4096x11008xi8>, %a_scale: tensor<512xf32>, %w_scale: tensor<11008xf32>) -> tensor<512x11008xf16> {
    %zero = arith.constant 0 : i32
    %e = tensor.empty() : tensor<512x11008xi32>
    %fill = linalg.fill ins(%zero : i32) outs(%e : tensor<512x11008xi32>) -> tensor<512x11008xi32>
    %acc = linalg.matmul ins(%lhs, %rhs : tensor<512x4096xi8>, tensor<4096x11008xi8>)
        outs(%fill : tensor<512x11008xi32>) -> tensor<512x11008xi32>
    %o = tensor.empty() : tensor<512x11008xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>,
                                          affine_map<(d0, d1) -> (d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc, %a_scale, %w_scale : tensor<512x11008xi32>, tensor<512xf32>, tensor<11008xf32>) outs(%o : tensor<512x11008xf16>) {
      ^bb0(%in: i32, %sa: f32, %sw: f32, %out: f16):
        %f = arith.sitofp %in : i32 to f32
        %x = arith.mulf %f, %sa : f32
        %y = arith.mulf %x, %sw : f32
        %t = arith.truncf %y : f32 to f16
        linalg.yield %t : f16
    } -> tensor<512x11008xf16>
    util.return %r : tensor<512x11008xf16>
  }
  util.func public @c3_m4096(%lhs: tensor<4096x4096xi8>, %rhs: tensor<4096x11008xi8>, %a_scale: tensor<4096xf32>, %w_scale: tensor<11008xf32>) -> tensor<4096x11008xf16> {
    %zero = arith.constant 0 : i32
    %e = tensor.empty() : tensor<4096x11008xi32>
    %fill = linalg.fill ins(%zero : i32) outs(%e : tensor<4096x11008xi32>) -> tensor<4096x11008xi32>
    %acc = linalg.matmul ins(%lhs, %rhs : tensor<4096x4096xi8>, tensor<4096x11008xi8>)
        outs(%fill : tensor<4096x11008xi32>) -> tensor<4096x11008xi32>
    %o = tensor.empty() : tensor<4096x11008xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0)>,
                                          affine_map<(d0, d1) -> (d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc, %a_scale, %w_scale : tensor<4096x11008xi32>, tensor<4096xf32>, tensor<11008xf32>) outs(%o : tensor<4096x11008xf16>) {
      ^bb0(%in: i32, %sa: f32, %sw: f32, %out: f16):
        %f = arith.sitofp %in : i32 to f32
        %x = arith.mulf %f, %sa : f32
        %y = arith.mulf %x, %sw : f32
        %t = arith.truncf %y : f32 to f16
        linalg.yield %t : f16
    } -> tensor<4096x11008xf16>
    util.return %r : tensor<4096x11008xf16>
  }
}
