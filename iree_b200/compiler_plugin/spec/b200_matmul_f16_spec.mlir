// Transform-dialect script that routes static 4096x4096x4096 f16 matmuls (fill + linalg.matmul +
// truncf) to the b200_matmul_f16_f16 export of b200_contraction.cubin with an UNMODIFIED
// iree-compile:
//
//   iree-compile model.mlir --iree-hal-target-backends=cuda --iree-hal-cuda-llvm-target-arch=sm_100a \
//       --iree-preprocessing-transform-spec-filename=b200_matmul_f16_spec.mlir \
//       --iree-hal-executable-object-search-path=<dir of b200_contraction.cubin> -o model.vmfb
//
// Structure follows samples/custom_dispatch/vulkan/shaders/example_transform_spec.mlir and
// samples/custom_dispatch/cpu/mlp_plugin/mlp_spec_matmul.mlir of the IREE tree: a hand-written
// util.func holds the hal.dispatch.extern ops (so push constants and binding order line up with
// the kernel ABI), a matcher finds the DAG, and cast_and_call rewires it.
// Not run in the repository this file ships in (no iree-compile there).

#cuda_target = #hal.executable.target<"cuda", "cuda-nvptx-fb", {}>

module attributes {transform.with_named_sequence} {

  util.func private @b200_matmul_f16_4096(%lhs: tensor<4096x4096xf16>, %rhs: tensor<4096x4096xf16>) -> tensor<4096x4096xf16> {
    %c1 = arith.constant 1 : index
    %tiles = arith.constant 512 : index                 // 32 x 16 tiles of 128 x 256
    %m = arith.constant 4096 : i32
    %one = arith.constant 1 : i32
    %kn = arith.constant 0 : i32                        // rhs is [K, N]
    %bn = arith.constant 256 : i32
    %elem = arith.constant 2 : i32
    // Two 128-byte tensor-map templates (f16, rank 3, 128-byte swizzle): row 0 of the table that
    // compiler_plugin/gen_templates.py writes from the runtime library, once for lhs and once for rhs.
    // The device-side builder replaces address, extents, strides and box; the address bytes in here
    // are those of the buffer the template was encoded over and mean nothing.
    %templates = util.unfoldable_constant dense<"0x000020B9CF7F0000206326002000000000200000000000000000000000000000FF000000FF0000000000000000000000000000000000003F070000000000000000040000000000000004000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000020B9CF7F0000206326002000000000200000000000000000000000000000FF000000FF0000000000000000000000000000000000003F070000000000000000040000000000000004000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000000"> : tensor<256xi8>

    // 1. tensor maps built on the device (bindings: lhs, rhs, templates, workspace)
    %ws = hal.dispatch.extern "b200_encode_tensormaps"[%c1](%lhs, %rhs, %templates, %m, %m, %m, %one, %kn, %bn, %elem)
        : (tensor<4096x4096xf16>, tensor<4096x4096xf16>, tensor<256xi8>, i32, i32, i32, i32, i32, i32, i32) -> tensor<512xi8>
      count(%device: !hal.device, %w: index) -> (index, index, index) {
        %c1_0 = arith.constant 1 : index
        hal.return %c1_0, %c1_0, %c1_0 : index, index, index
      }
      layout(#hal.pipeline.layout<push_constants = 7, sets = [
        <0, bindings = [
            <0, storage_buffer, ReadOnly>,
            <1, storage_buffer, ReadOnly>,
            <2, storage_buffer, ReadOnly>,
            <3, storage_buffer>
        ]>
      ]>)
      bindings([
        #hal.interface.binding<0, 0>,
        #hal.interface.binding<0, 1>,
        #hal.interface.binding<0, 2>,
        #hal.interface.binding<0, 3>
      ])
      objects({
        #cuda_target ordinal(0) = [#hal.executable.object<{path = "b200_contraction.cubin"}>]
      })
      attributes {workgroup_size = [32 : index, 1 : index, 1 : index]}

    // 2. the contraction (bindings: out, workspace; constants: M, N, K, batch, rhs_layout, tile_n).
    //    The workspace is tied through so that it is bound read-write after the result.
    %out:2 = hal.dispatch.extern "b200_matmul_f16_f16"[%tiles](%ws, %m, %m, %m, %one, %kn, %bn)
        : (tensor<512xi8>, i32, i32, i32, i32, i32, i32) -> (tensor<4096x4096xf16>, %ws)
      count(%device: !hal.device, %t: index) -> (index, index, index) {
        %c148 = arith.constant 148 : index              // one persistent CTA per SM
        %c1_0 = arith.constant 1 : index
        hal.return %c148, %c1_0, %c1_0 : index, index, index
      }
      layout(#hal.pipeline.layout<push_constants = 6, sets = [
        <0, bindings = [
            <0, storage_buffer>,
            <1, storage_buffer>
        ]>
      ]>)
      bindings([
        #hal.interface.binding<0, 0>,
        #hal.interface.binding<0, 1>
      ])
      objects({
        #cuda_target ordinal(0) = [#hal.executable.object<{path = "b200_contraction.cubin"}>]
      })
      attributes {workgroup_size = [256 : index, 1 : index, 1 : index], workgroup_local_memory = 230656 : index}
    util.return %out#0 : tensor<4096x4096xf16>
  }

  transform.named_sequence @match_f16_matmul_truncf(%root: !transform.any_op {transform.readonly})
      -> (!transform.any_value, !transform.any_value) {
    %ins, %outs = transform.iree.match.cast_compatible_dag_from_root %root {
      ^bb0(%lhs: tensor<4096x4096xf16>, %rhs: tensor<4096x4096xf16>, %acc_init: tensor<4096x4096xf32>, %out_init: tensor<4096x4096xf16>):
        %zero = arith.constant 0.0 : f32
        %fill = linalg.fill ins(%zero : f32) outs(%acc_init : tensor<4096x4096xf32>) -> tensor<4096x4096xf32>
        %mm = linalg.matmul ins(%lhs, %rhs : tensor<4096x4096xf16>, tensor<4096x4096xf16>)
                            outs(%fill : tensor<4096x4096xf32>) -> tensor<4096x4096xf32>
        %trunc = linalg.generic {
            indexing_maps = [affine_map<(d0, d1) -> (d0, d1)>, affine_map<(d0, d1) -> (d0, d1)>],
            iterator_types = ["parallel", "parallel"]}
            ins(%mm : tensor<4096x4096xf32>) outs(%out_init : tensor<4096x4096xf16>) {
          ^bb0(%in: f32, %o: f16):
            %t = arith.truncf %in : f32 to f16
            linalg.yield %t : f16
        } -> tensor<4096x4096xf16>
      } : (!transform.any_op) -> (!transform.any_value, !transform.any_value)
    transform.yield %ins, %outs : !transform.any_value, !transform.any_value
  }

  transform.named_sequence @call_b200(%ins: !transform.any_value {transform.readonly},
                                      %out: !transform.any_value {transform.readonly}) {
    %root = transform.get_defining_op %out : (!transform.any_value) -> !transform.any_op
    %module = transform.util.get_nearest_symbol_table %root : (!transform.any_op) -> !transform.any_op
    %func = transform.util.import_symbol @b200_matmul_f16_4096 into %module if undefined : (!transform.any_op) -> !transform.any_op
    // Only the two tensor operands are forwarded; the init tensors of the matched DAG are dropped.
    %lhs_rhs = transform.get_result %root[0] : (!transform.any_op) -> !transform.any_value
    transform.util.cast_and_call %func(%ins) -> %out after %root {
      transform.type_conversion.tensor.cast_shape_dynamic_dims
    } : (!transform.any_op, !transform.any_value, !transform.any_value, !transform.any_op) -> !transform.any_op
    transform.yield
  }

  transform.named_sequence @__transform_main(%module: !transform.any_op) {
    %funcs = transform.structured.match ops{["util.func"]} in %module : (!transform.any_op) -> !transform.any_op
    transform.foreach %funcs : !transform.any_op {
      ^bb1(%func: !transform.any_op):
        transform.foreach_match in %func
          @match_f16_matmul_truncf -> @call_b200
        : (!transform.any_op) -> (!transform.any_op)
    }
    transform.apply_dce to %module : !transform.any_op
    transform.apply_registered_pass "inline" to %module : (!transform.any_op) -> !transform.any_op
    transform.yield
  }
}
