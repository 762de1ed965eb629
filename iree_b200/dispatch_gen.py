"""Host plans for contraction dispatches: which exports of ``b200_contraction.cubin`` run, with
which bindings, push constants and grid.

This restates, in Python, the matching and lowering rules of the compiler plugin
(``iree_b200/compiler_plugin/src/RewriteContractionsPass.cpp``): the plugin emits the same
sequence as ``hal.dispatch.extern`` ops. A plan is plain data (JSON-serialisable); it is what
``iree_b200.run_module`` executes through the HAL-shaped layer of the C ABI (executable create,
push constants, descriptor set, dispatch), i.e. through the kernel ABI itself and not through the
operator-level C entry points. The export table must stay identical to ``kEntries`` in
``csrc/hal_b200.cc``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from typing import Dict, List, Optional, Tuple

GEMM_THREADS, GEMM_SMEM = 256, 230656
W4_THREADS, W4_SMEM = 512, 230656  # 1024 + 224 KiB + 256
W4_WT_THREADS = 512
W4_WT_SMEM = 214528               # b200_w4a16_gemm_wt: 1024 + 4 x 32 KiB + 6 x 8 KiB + 2 x 16 KiB + 512
DECODE_THREADS, DECODE_SMEM = 512, {8: 217984, 16: 213760}
DECODE_SLICE_K = 4096           # K per CTA of the decode kernels; K beyond it is split over CTAs
SM_COUNT = 148

ELEM_BYTES = {"f16": 2, "bf16": 2, "i8": 1, "i32": 4, "f32": 4}


@dataclass
class Dispatch:
    export: str
    bindings: List[str]            # names of tensors / scratch buffers, in kernel-parameter order
    constants: List[int]           # i32 push constants, in order
    grid: Tuple[int, int, int]
    block: Tuple[int, int, int]
    shared_memory: int


@dataclass
class Plan:
    function: str
    inputs: List[Dict]             # {"name", "shape", "dtype", optional "parameter": "scope::key"}
    outputs: List[Dict]
    transients: List[Dict]         # {"name", "bytes", "zero": bool, "templates": optional kind}
    dispatches: List[Dispatch] = field(default_factory=list)

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    def bind_parameters(self, bindings: Dict[str, str]) -> "Plan":
        """Marks inputs as program parameters: {"wq": "model::blk.0.wq"} (scope::key). They are then
        loaded from a parameter archive instead of arriving as function arguments, the way a
        compiled program's `#stream.parameter.named<"model"::"blk.0.wq">` globals are."""
        for decl in self.inputs:
            if decl["name"] in bindings:
                decl["parameter"] = bindings[decl["name"]]
        return self

    @staticmethod
    def from_json(text: str) -> "Plan":
        d = json.loads(text)
        d["dispatches"] = [Dispatch(**{**x, "grid": tuple(x["grid"]), "block": tuple(x["block"])})
                           for x in d["dispatches"]]
        return Plan(**d)


def use_pairs(M: int, N: int, K: int, batch: int, sm_count: int = SM_COUNT) -> bool:
    """CTA pairs (256-row tiles, tcgen05 cta_group::2) pay off when there are enough 256 x 256 tiles to
    fill the SM pairs (the runtime library's rule)."""
    tiles = ((M + 255) // 256) * ((N + 255) // 256) * batch
    return M >= 256 and tiles >= (sm_count & ~1) // 2 and K >= 512


def choose_tile_n(M: int, N: int, batch: int, chunk: int, sm_count: int = SM_COUNT, pairs: bool = False) -> int:
    """Widest tile that still gives every SM (or SM pair) work (same cost model as the runtime and the plugin).
    `chunk`: columns a tile width must be a multiple of (in pair mode each CTA holds half a tile)."""
    best, best_cost = 0, 0.0
    units = (sm_count & ~1) // (2 if pairs else 1)
    rows = 256 if pairs else 128
    for bn in range(256, 31, -32):
        if bn % chunk or (M <= 32 and bn > 128 and chunk <= 128):   # few rows: the deep-ring variant
            continue
        tiles = ((M + rows - 1) // rows) * ((N + bn - 1) // bn) * batch
        cost = ((tiles + units - 1) // units) * (400.0 + bn)
        if not best or cost < best_cost * 0.9999:
            best, best_cost = bn, cost
    return best


def matmul_export(kind: str, epilogue: str, generic: bool, pairs: bool = False) -> str:
    table = {("f16", "cast"): "f16_f16", ("f16", "acc"): "f16_f32", ("bf16", "cast"): "bf16_bf16",
             ("bf16", "acc"): "bf16_f32", ("i8", "acc"): "i8_i32", ("i8", "requant"): "i8_requant_f16"}
    if (kind, epilogue) not in table:
        raise ValueError("no kernel for %s with epilogue %s" % (kind, epilogue))
    prefix = "b200_matmul_generic_" if generic else ("b200_matmul_pair_" if pairs else "b200_matmul_")
    return prefix + table[(kind, epilogue)]


def plan_matmul(function: str, kind: str, epilogue: str, M: int, N: int, K: int, batch: int = 1,
                rhs_layout: str = "KN", device_tensor_maps: bool = True, sm_count: int = SM_COUNT) -> Plan:
    """fill + linalg.matmul / batch_matmul (+ truncf or requant consumer)."""
    es = ELEM_BYTES[kind]
    out_dtype = {"cast": kind, "acc": "i32" if kind == "i8" else "f32", "requant": "f16"}[epilogue]
    lead = [batch] if batch > 1 else []
    rhs_shape = lead + ([K, N] if rhs_layout == "KN" else [N, K])
    inputs = [{"name": "lhs", "shape": lead + [M, K], "dtype": kind}, {"name": "rhs", "shape": rhs_shape, "dtype": kind}]
    if epilogue == "requant":
        inputs += [{"name": "a_scale", "shape": [M], "dtype": "f32"}, {"name": "w_scale", "shape": [N], "dtype": "f32"}]
    outputs = [{"name": "out", "shape": lead + [M, N], "dtype": out_dtype}]
    layout = 0 if rhs_layout == "KN" else 1
    plan = Plan(function, inputs, outputs, [])
    tma_ok = (K * es) % 16 == 0 and (layout == 1 or (N * es) % 16 == 0) and K > 0
    scales = ["a_scale", "w_scale"] if epilogue == "requant" else []
    if not tma_ok:
        plan.dispatches.append(Dispatch(matmul_export(kind, epilogue, True), ["lhs", "rhs", "out"] + scales,
                                        [M, N, K, layout], ((N + 15) // 16, (M + 15) // 16, batch), (16, 16, 1), 0))
        return plan
    pairs = use_pairs(M, N, K, batch, sm_count)
    chunk = ((2 if pairs else 1) * 128 // es) if layout == 0 else (64 if pairs else 32)
    bn = choose_tile_n(M, N, batch, chunk, sm_count, pairs)
    rows = 256 if pairs else 128
    tiles = ((M + rows - 1) // rows) * ((N + bn - 1) // bn) * batch
    grid = 2 * min(tiles, (sm_count & ~1) // 2) if pairs else min(tiles, sm_count)   # whole pairs only
    plan.transients.append({"name": "workspace", "bytes": 512, "zero": True})
    if device_tensor_maps:
        plan.transients.append({"name": "templates", "bytes": 256, "zero": False, "templates": kind})
        # in pair mode each CTA loads half of the right-hand tile: the map's box is half as wide
        plan.dispatches.append(Dispatch("b200_encode_tensormaps", ["lhs", "rhs", "templates", "workspace"],
                                        [M, N, K, batch, layout, bn // 2 if pairs else bn, es], (1, 1, 1), (32, 1, 1), 0))
    else:
        plan.transients[0]["host_tensor_maps"] = {"kind": kind, "epilogue": epilogue, "M": M, "N": N, "K": K,
                                                  "batch": batch, "layout": layout, "tile_n": bn}
    plan.dispatches.append(Dispatch(matmul_export(kind, epilogue, False, pairs), ["out"] + scales + ["workspace"],
                                    [M, N, K, batch, layout, bn], (grid, 1, 1), (GEMM_THREADS, 1, 1), GEMM_SMEM))
    return plan


# Indices into the tensor-map template table (IREE_B200_TEMPLATE_* in include/iree_b200.h).
TEMPLATE_F16_SW128_R3, TEMPLATE_BF16_SW128_R3, TEMPLATE_U8_SW128_R3 = 0, 1, 2
TEMPLATE_U8_SW64_R3, TEMPLATE_F16_PLAIN_R2, TEMPLATE_U64_PLAIN_R2 = 3, 4, 5


def encode_map_dispatch(tensor: str, slot: int, template: int, rank: int, dims, strides, box, elem_bytes: int,
                        flags: int = 0) -> Dispatch:
    """One b200_encode_tensormap dispatch: builds, on the device, the tensor map of `tensor` at byte
    `slot` of the workspace. dims / box are innermost first; strides are the byte pitches of dims 1, 2."""
    dims, box, strides = list(dims) + [1] * (3 - len(dims)), list(box) + [1] * (3 - len(box)), list(strides) + [0] * (2 - len(strides))
    box_bytes = box[0] * box[1] * box[2] * elem_bytes
    lo_hi = [x for st in strides for x in (st & 0x7FFFFFFF | (-(st & 0x80000000)), st >> 32)]
    return Dispatch("b200_encode_tensormap", [tensor, "templates", "workspace"],
                    [slot, template, rank] + dims + lo_hi + box + [box_bytes, flags], (1, 1, 1), (32, 1, 1), 0)


def plan_w4a16(function: str, M: int, N: int, K: int, group: int = 128, ldo: Optional[int] = None,
               n_offset: int = 0, sm_count: int = SM_COUNT, device_tensor_maps: bool = False) -> Plan:
    """dequant-like generic (i4 -> f16 * scale) cloned into the grouped contraction + truncf.

    With device_tensor_maps the tensor maps the kernels need are built by b200_encode_tensormap
    dispatches ahead of them (what the compiler plugin emits: a stock runtime cannot encode maps on
    the host); otherwise the workspace carries a note for the host to encode them."""
    ldo = N if ldo is None else ldo
    inputs = [{"name": "a", "shape": [M, K], "dtype": "f16"}, {"name": "wq", "shape": [N, K // 2], "dtype": "i8"},
              {"name": "scales", "shape": [N, K // group], "dtype": "f16"}]
    outputs = [{"name": "out", "shape": [M, ldo], "dtype": "f16"}]
    plan = Plan(function, inputs, outputs, [])
    if group == 128 and M <= 16 and N % 16 == 0 and K % 256 == 0 and K <= 16384:
        # workspace: 512-byte header (status words at byte 384), a counter per 16-row tile padded to 256
        # bytes, one 1 KiB f32 partial tile per tile and K slice (only touched when K spans several slices)
        slices = (K + DECODE_SLICE_K - 1) // DECODE_SLICE_K
        counters = ((N // 16) * 4 + 255) // 256 * 256
        ws = {"name": "workspace", "bytes": 512 + counters + (N // 16) * slices * 1024, "zero": True}
        plan.transients.append(ws)
        if slices > 1:   # the kernel reads its weight tiles through a tensor map at the start of the workspace
            if device_tensor_maps:
                plan.transients.append({"name": "templates", "bytes": 768, "zero": False, "templates": "table"})
                plan.dispatches.append(encode_map_dispatch("wq", 0, TEMPLATE_U64_PLAIN_R2, 2, [K // 16, N], [K // 2],
                                                           [256, 8], 8, flags=3))
            else:
                ws["host_tensor_maps"] = {"kind": "w4a16_decode", "M": M, "N": N, "K": K}
        mh = 8 if M <= 8 else 16
        walkers = max(1, min(N // 16, sm_count // slices))
        plan.dispatches.append(Dispatch("b200_w4a16_decode_m%d" % mh, ["a", "wq", "scales", "out", "workspace"],
                                        [M, N, K, ldo, n_offset], (walkers * slices, 1, 1),
                                        (DECODE_THREADS, 1, 1), DECODE_SMEM[mh]))
    elif group == 128 and K % 128 == 0 and (ldo * 2) % 16 == 0 and n_offset % 8 == 0:
        # more than sixteen rows: the weights are the tensor-memory operand, tiles are 128 weight rows x 128
        # (M <= 128) or 256 activation rows, results leave by TMA stores through an output map in the
        # workspace (one destination here), which needs pitch and offset on 16-byte boundaries
        tiles = ((M + 255) // 256) * ((N + 127) // 128)
        ws = {"name": "workspace", "bytes": 512 + 8 * 128 + 8 * 8, "zero": True}
        plan.transients.append(ws)
        if device_tensor_maps:
            plan.transients.append({"name": "templates", "bytes": 768, "zero": False, "templates": "table"})
            plan.dispatches += [
                encode_map_dispatch("a", 0, TEMPLATE_F16_SW128_R3, 3, [K, M, 1], [K * 2, M * K * 2], [64, 128, 1], 2, flags=1),
                encode_map_dispatch("wq", 128, TEMPLATE_U8_SW64_R3, 3, [K // 2, N, 1], [K // 2, N * (K // 2)], [64, 128, 1], 1),
                encode_map_dispatch("out", 512, TEMPLATE_F16_PLAIN_R2, 2, [n_offset + N, M], [ldo * 2], [128, 64], 2)]
        else:
            ws["host_tensor_maps"] = {"kind": "w4a16_wt", "M": M, "N": N, "K": K, "ldo": ldo, "n_offset": n_offset}
        plan.dispatches.append(Dispatch("b200_w4a16_gemm_wt", ["scales", "out", "workspace"],
                                        [M, N, K, ldo, n_offset, (1 << 8) | 0, 0], (min(tiles, sm_count), 1, 1),
                                        (W4_WT_THREADS, 1, 1), W4_WT_SMEM))
    elif group == 128 and K % 128 == 0:
        # tiles: a multiple of 16, at most 128 columns; M >= 256 runs the kernel's 256-row variant
        tall = M >= 256
        rows = 256 if tall else 128
        bn, best = 0, 0.0
        for cand in range(128, 15, -16):
            t = ((M + rows - 1) // rows) * ((N + cand - 1) // cand)
            cost = ((t + sm_count - 1) // sm_count) * (400.0 + (2 * cand if tall else cand))
            if not bn or cost < best * 0.9999:
                bn, best = cand, cost
        tiles = ((M + rows - 1) // rows) * ((N + bn - 1) // bn)
        ws = {"name": "workspace", "bytes": 512, "zero": True}
        plan.transients.append(ws)
        if device_tensor_maps:
            plan.transients.append({"name": "templates", "bytes": 768, "zero": False, "templates": "table"})
            plan.dispatches += [
                encode_map_dispatch("a", 0, TEMPLATE_F16_SW128_R3, 3, [K, M, 1], [K * 2, M * K * 2], [64, 128, 1], 2, flags=1),
                encode_map_dispatch("wq", 128, TEMPLATE_U8_SW64_R3, 3, [K // 2, N, 1], [K // 2, N * (K // 2)], [64, bn, 1], 1)]
        else:
            ws["host_tensor_maps"] = {"kind": "w4a16", "M": M, "N": N, "K": K, "tile_n": bn}
        plan.dispatches.append(Dispatch("b200_w4a16_gemm", ["scales", "out", "workspace"],
                                        [M, N, K, ldo, n_offset, bn], (min(tiles, sm_count), 1, 1), (W4_THREADS, 1, 1),
                                        W4_SMEM))
    else:
        plan.dispatches.append(Dispatch("b200_w4a16_generic", ["a", "wq", "scales", "out"],
                                        [M, N, K, group, ldo, n_offset], ((N + 255) // 256, M, 1), (256, 1, 1), 0))
    return plan


def extern_mlir(plan: Plan, cubin: str = "b200_contraction.cubin") -> str:
    """The hal.dispatch.extern ops the plugin emits for this plan (textual sketch for review)."""
    lines = []
    written = {o["name"] for o in plan.outputs} | {t["name"] for t in plan.transients}
    for d in plan.dispatches:
        ro = [b for b in d.bindings if b not in written or b == "templates"]
        rw = [b for b in d.bindings if b not in ro]
        layout = ", ".join("<%d, storage_buffer%s>" % (i, ", ReadOnly" if b in ro else "") for i, b in enumerate(d.bindings))
        lines.append('hal.dispatch.extern "%s"[...](%s | %s)' % (d.export, ", ".join("%" + b for b in d.bindings),
                                                                   ", ".join("%d : i32" % c for c in d.constants)))
        lines.append("  count(...) { hal.return %d, %d, %d }" % d.grid)
        lines.append("  layout(#hal.pipeline.layout<push_constants = %d, sets = [<0, bindings = [%s]>]>)" % (
            len(d.constants), layout))
        lines.append('  objects({#cuda_target ordinal(0) = [#hal.executable.object<{path = "%s"}>]})' % cubin)
        lines.append("  attributes {workgroup_size = [%d, %d, %d], workgroup_local_memory = %d}  // writes: %s" % (
            d.block + (d.shared_memory, ", ".join(rw))))
    return "\n".join(lines)


# The five benchmark configurations (BASELINE.json order) as plans.
def baseline_plans(device_tensor_maps: bool = True) -> Dict[str, Plan]:
    p = {"c1_i8_1024": plan_matmul("c1", "i8", "acc", 1024, 1024, 1024, device_tensor_maps=device_tensor_maps),
         "c2_f16_4096": plan_matmul("c2", "f16", "cast", 4096, 4096, 4096, device_tensor_maps=device_tensor_maps),
         "c2_f16_bmm": plan_matmul("c2_bmm", "f16", "cast", 512, 512, 128, batch=32, device_tensor_maps=device_tensor_maps)}
    for m in (1, 16, 512, 4096):
        p["c3_w8a8_m%d" % m] = plan_matmul("c3_m%d" % m, "i8", "requant", m, 11008, 4096, device_tensor_maps=device_tensor_maps)
    for m in (1, 8, 16, 128, 2048):
        p["c4_w4a16_m%d" % m] = plan_w4a16("c4_m%d" % m, m, 11008, 4096)
    for m in (16, 4096):
        p["c5_w4a16_m%d" % m] = plan_w4a16("c5_m%d" % m, m, 28672, 8192)
    return p


if __name__ == "__main__":
    import sys
    for name, plan in baseline_plans().items():
        if len(sys.argv) < 2 or sys.argv[1] == name:
            print("// ---- %s" % name)
            print(extern_mlir(plan))
