// The benchmark configuration c5 as linalg-on-tensors, in the op shapes the rewrite pass matches.
// Written by `python -m iree_b200.mlir_frontend c5`; lowered to a host plan by
// iree_b200.mlir_frontend.plans_from_mlir (tests/test_dispatch_plan.py).
#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>
module attributes {hal.device.targets = [#cuda]} {
  util.func public @c5_m16(%a: tensor<16x64x128xf16>, %wq: tensor<28672x4096xi8>, %scales: tensor<28672x64xf16>) -> tensor<16x28672xf16> {
    %w4 = flow.tensor.bitcast %wq : tensor<28672x4096xi8> -> tensor<28672x64x128xi4>
    %we = tensor.empty() : tensor<28672x64x128xf16>
    %deq = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2) -> (d0, d1, d2)>, affine_map<(d0, d1, d2) -> (d0, d1)>,
                                            affine_map<(d0, d1, d2) -> (d0, d1, d2)>],
                           iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%w4, %scales : tensor<28672x64x128xi4>, tensor<28672x64xf16>) outs(%we : tensor<28672x64x128xf16>) {
      ^bb0(%in: i4, %s: f16, %out: f16):
        %i = arith.extsi %in : i4 to i32
        %f = arith.sitofp %i : i32 to f16
        %d = arith.mulf %f, %s : f16
        linalg.yield %d : f16
    } -> tensor<28672x64x128xf16>
    %zero = arith.constant 0.000000e+00 : f32
    %e = tensor.empty() : tensor<16x28672xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<16x28672xf32>) -> tensor<16x28672xf32>
    %acc = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2, d3) -> (d0, d2, d3)>, affine_map<(d0, d1, d2, d3) -> (d1, d2, d3)>,
                                            affine_map<(d0, d1, d2, d3) -> (d0, d1)>],
                           iterator_types = ["parallel", "parallel", "reduction", "reduction"]}
        ins(%a, %deq : tensor<16x64x128xf16>, tensor<28672x64x128xf16>) outs(%fill : tensor<16x28672xf32>) {
      ^bb0(%x: f16, %w: f16, %out: f32):
        %xe = arith.extf %x : f16 to f32
        %we2 = arith.extf %w : f16 to f32
        %p = arith.mulf %xe, %we2 : f32
        %sum = arith.addf %p, %out : f32
        linalg.yield %sum : f32
    } -> tensor<16x28672xf32>
    %o = tensor.empty() : tensor<16x28672xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc : tensor<16x28672xf32>) outs(%o : tensor<16x28672xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<16x28672xf16>
    util.return %r : tensor<16x28672xf16>
  }
  util.func public @c5_m4096(%a: tensor<4096x64x128xf16>, %wq: tensor<28672x4096xi8>, %scales: tensor<28672x64xf16>) -> tensor<4096x28672xf16> {
    %w4 = flow.tensor.bitcast %wq : tensor<28672x4096xi8> -> tensor<28672x64x128xi4>
    %we = tensor.empty() : tensor<28672x64x128xf16>
    %deq = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2) -> (d0, d1, d2)>, affine_map<(d0, d1, d2) -> (d0, d1)>,
                                            affine_map<(d0, d1, d2) -> (d0, d1, d2)>],
                           iterator_types = ["parallel", "parallel", "parallel"]}
        ins(%w4, %scales : tensor<28672x64x128xi4>, tensor<28672x64xf16>) outs(%we : tensor<28672x64x128xf16>) {
      ^bb0(%in: i4, %s: f16, %out: f16):
        %i = arith.extsi %in : i4 to i32
        %f = arith.sitofp %i : i32 to f16
        %d = arith.mulf %f, %s : f16
        linalg.yield %d : f16
    } -> tensor<28672x64x128xf16>
    %zero = arith.constant 0.000000e+00 : f32
    %e = tensor.empty() : tensor<4096x28672xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<4096x28672xf32>) -> tensor<4096x28672xf32>
    %acc = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2, d3) -> (d0, d2, d3)>, affine_map<(d0, d1, d2, d3) -> (d1, d2, d3)>,
                                            affine_map<(d0, d1, d2, d3) -> (d0, d1)>],
                           iterator_types = ["parallel", "parallel", "reduction", "reduction"]}
        ins(%a, %deq : tensor<4096x64x128xf16>, tensor<28672x64x128xf16>) outs(%fill : tensor<4096x28672xf32>) {
      ^bb0(%x: f16, %w: f16, %out: f32):
        %xe = arith.extf %x : f16 to f32
        %we2 = arith.extf %w : f16 to f32
        %p = arith.mulf %xe, %we2 : f32
        %sum = arith.addf %p, %out : f32
        linalg.yield %sum : f32
    } -> tensor<4096x28672xf32>
    %o = tensor.empty() : tensor<4096x28672xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc : tensor<4096x28672xf32>) outs(%o : tensor<4096x28672xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<4096x28672xf16>
    util.return %r : tensor<4096x28672xf16>
  }
}
