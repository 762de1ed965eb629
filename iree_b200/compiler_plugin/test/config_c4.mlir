// The benchmark configuration c4 as linalg-on-tensors, in the op shapes the rewrite pass matches.
// Written by `python -m iree_b200.mlir_frontend c4`; lowered to a host plan by
// iree_b200.mlir_frontend.plans_from_mlir (tests/test_dispatch_plan.py).
#cuda = #hal.device.target<"cuda", [#hal.executable.target<"cuda", "cuda-nvptx-fb", {}>]>
module attributes {hal.device.targets = [#cuda]} {
  util.func public @c4_m1(%a: tensor<1x32x128xf16>, %wq: tensor<11008x2048xi8>, %scales: tensor<11008x32xf16>) -> tensor<1x11008xf16> {
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
    %e = tensor.empty() : tensor<1x11008xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<1x11008xf32>) -> tensor<1x11008xf32>
    %acc = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2, d3) -> (d0, d2, d3)>, affine_map<(d0, d1, d2, d3) -> (d1, d2, d3)>,
                                            affine_map<(d0, d1, d2, d3) -> (d0, d1)>],
                           iterator_types = ["parallel", "parallel", "reduction", "reduction"]}
        ins(%a, %deq : tensor<1x32x128xf16>, tensor<11008x32x128xf16>) outs(%fill : tensor<1x11008xf32>) {
      ^bb0(%x: f16, %w: f16, %out: f32):
        %xe = arith.extf %x : f16 to f32
        %we2 = arith.extf %w : f16 to f32
        %p = arith.mulf %xe, %we2 : f32
        %sum = arith.addf %p, %out : f32
        linalg.yield %sum : f32
    } -> tensor<1x11008xf32>
    %o = tensor.empty() : tensor<1x11008xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc : tensor<1x11008xf32>) outs(%o : tensor<1x11008xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<1x11008xf16>
    util.return %r : tensor<1x11008xf16>
  }
  util.func public @c4_m8(%a: tensor<8x32x128xf16>, %wq: tensor<11008x2048xi8>, %scales: tensor<11008x32xf16>) -> tensor<8x11008xf16> {
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
    %e = tensor.empty() : tensor<8x11008xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<8x11008xf32>) -> tensor<8x11008xf32>
    %acc = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2, d3) -> (d0, d2, d3)>, affine_map<(d0, d1, d2, d3) -> (d1, d2, d3)>,
                                            affine_map<(d0, d1, d2, d3) -> (d0, d1)>],
                           iterator_types = ["parallel", "parallel", "reduction", "reduction"]}
        ins(%a, %deq : tensor<8x32x128xf16>, tensor<11008x32x128xf16>) outs(%fill : tensor<8x11008xf32>) {
      ^bb0(%x: f16, %w: f16, %out: f32):
        %xe = arith.extf %x : f16 to f32
        %we2 = arith.extf %w : f16 to f32
        %p = arith.mulf %xe, %we2 : f32
        %sum = arith.addf %p, %out : f32
        linalg.yield %sum : f32
    } -> tensor<8x11008xf32>
    %o = tensor.empty() : tensor<8x11008xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc : tensor<8x11008xf32>) outs(%o : tensor<8x11008xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<8x11008xf16>
    util.return %r : tensor<8x11008xf16>
  }
  util.func public @c4_m16(%a: tensor<16x32x128xf16>, %wq: tensor<11008x2048xi8>, %scales: tensor<11008x32xf16>) -> tensor<16x11008xf16> {
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
    %e = tensor.empty() : tensor<16x11008xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<16x11008xf32>) -> tensor<16x11008xf32>
    %acc = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2, d3) -> (d0, d2, d3)>, affine_map<(d0, d1, d2, d3) -> (d1, d2, d3)>,
                                            affine_map<(d0, d1, d2, d3) -> (d0, d1)>],
                           iterator_types = ["parallel", "parallel", "reduction", "reduction"]}
        ins(%a, %deq : tensor<16x32x128xf16>, tensor<11008x32x128xf16>) outs(%fill : tensor<16x11008xf32>) {
      ^bb0(%x: f16, %w: f16, %out: f32):
        %xe = arith.extf %x : f16 to f32
        %we2 = arith.extf %w : f16 to f32
        %p = arith.mulf %xe, %we2 : f32
        %sum = arith.addf %p, %out : f32
        linalg.yield %sum : f32
    } -> tensor<16x11008xf32>
    %o = tensor.empty() : tensor<16x11008xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc : tensor<16x11008xf32>) outs(%o : tensor<16x11008xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<16x11008xf16>
    util.return %r : tensor<16x11008xf16>
  }
  util.func public @c4_m128(%a: tensor<128x32x128xf16>, %wq: tensor<11008x2048xi8>, %scales: tensor<11008x32xf16>) -> tensor<128x11008xf16> {
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
    %e = tensor.empty() : tensor<128x11008xf32>
    %fill = linalg.fill ins(%zero : f32) outs(%e : tensor<128x11008xf32>) -> tensor<128x11008xf32>
    %acc = linalg.generic {indexing_maps = [affine_map<(d0, d1, d2, d3) -> (d0, d2, d3)>, affine_map<(d0, d1, d2, d3) -> (d1, d2, d3)>,
                                            affine_map<(d0, d1, d2, d3) -> (d0, d1)>],
                           iterator_types = ["parallel", "parallel", "reduction", "reduction"]}
        ins(%a, %deq : tensor<128x32x128xf16>, tensor<11008x32x128xf16>) outs(%fill : tensor<128x11008xf32>) {
      ^bb0(%x: f16, %w: f16, %out: f32):
        %xe = arith.extf %x : f16 to f32
        %we2 = arith.extf %w : f16 to f32
        %p = arith.mulf %xe, %we2 : f32
        %sum = arith.addf %p, %out : f32
        linalg.yield %sum : f32
    } -> tensor<128x11008xf32>
    %o = tensor.empty() : tensor<128x11008xf16>
    %r = linalg.generic {indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
                         iterator_types = ["parallel", "parallel"]}
        ins(%acc : tensor<128x11008xf32>) outs(%o : tensor<128x11008xf16>) {
      ^bb0(%in: f32, %out: f16):
        %v = arith.truncf %in : f32 to f16
        linalg.yield %v : f16
    } -> tensor<128x11008xf16>
    util.return %r : tensor<128x11008xf16>
  }
  util.func public @c4_m2048(%a: tensor<2048x32x128xf16>, %wq: tensor<11008x2048xi8>, %scales: tensor<11008x32xf16>) -> tensor<2048x11008xf16> {
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
