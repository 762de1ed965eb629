// The benchmark configuration c2 as linalg-on-tensors, in the op shapes the rewrite pass matches.
// Written by `python -m iree_b200.mlir_frontend c2`; lowered to a host plan by
// iree_b200.mlir_frontend.plans_from_mlir (tests/test_dispatch_plan.py).
#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>
module attributes {hal.device.targets = [#cuda]} {
  util.func public @c2(%lhs: tensor<4096x4096xf16>, %rhs: tensor<4096x4096xf16>) -> tensor<4096x4096xf16> {
    %zero = arith.constant 0.000000e+00 : f32
    %e = tensor.empty() : tensor<4096x4096xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<4096x4096xf32>) -> tensor<4096x4096xf32>
    %acc = linalg.matmul ins(%lhs, %rhs : tensor<4096x4096xf16>, tensor<4096x4096xf16>)
        outs(%fill : tensor<4096x4096xf32>) -> tensor<4096x4096xf32>
    %o = tensor.empty() : tensor<4096x4096xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc : tensor<4096x4096xf32>) outs(%o : tensor<4096x4096xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<4096x4096xf16>
    util.return %r : tensor<4096x4096xf16>
  }
  util.func public @c2_bmm(%lhs: tensor<32x512x128xf16>, %rhs: tensor<32x128x512xf16>) -> tensor<32x512x512xf16> {
    %zero = arith.constant 0.000000e+00 : f32
    %e = tensor.empty() : tensor<32x512x512xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<32x512x512xf32>) -> tensor<32x512x512xf32>
    %acc = linalg.batch_matmul ins(%lhs, %rhs : tensor<32x512x128xf16>, tensor<32x128x512xf16>)
        outs(%fill : tensor<32x512x512xf32>) -> tensor<32x512x512xf32>
    %o = tensor.empty() : tensor<32x512x512xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2) -> (d0, d1, d2)>, affine_map<(d0, d1, d2) -> (d0, d1, d2)>],
                         iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%acc : tensor<32x512x512xf32>) outs(%o : tensor<32x512x512xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<32x512x512xf16>
    util.return %r : tensor<32x512x512xf16>
  }
}
