// The benchmark configuration c1 as linalg-on-tensors, in the op shapes the rewrite pass matches.
// Written by `python -m iree_b200.mlir_frontend c1`; lowered to a host plan by
// iree_b200.mlir_frontend.plans_from_mlir (tests/test_dispatch_plan.py).
#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>
module attributes {hal.device.targets = [#cuda]} {
  util.func public @c1(%lhs: tensor<1024x1024xi8>, %rhs: tensor<1024x1024xi8>) -> tensor<1024x1024xi32> {
    %zero = arith.constant 0 : i32
    %e = tensor.empty() : tensor<1024x1024xi32>
    %fill = linalg.fill ins(%zero : i32) outs(%e : tensor<1024x1024xi32>) -> tensor<1024x1024xi32>
    %acc = linalg.matmul ins(%lhs, %rhs : tensor<1024x1024xi8>, tensor<1024x1024xi8>)
        outs(%fill : tensor<1024x1024xi32>) -> tensor<1024x1024xi32>
    util.return %acc : tensor<1024x1024xi32>
  }
}
