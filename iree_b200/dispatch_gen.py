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

GEMM_THREADS, GEMM_SMEM = 256, 197888
W4_THREADS, W4_SMEM = 512, 230656  # 1024 + 224 KiB + 256
W4_WT_SMEM = 214528               # b200_w4a16_gemm_wt: 1024 + 4 x 32 KiB + 6 x 8 KiB + 2 x 16 KiB + 512
DECODE_THREADS, DECODE_SMEM = 512, {8: 180864, 16: 213632}
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


def choose_tile_n(M: int, N: int, batch: int, chunk: int, sm_count: int = SM_COUNT) -> int:
    """Widest tile that still gives every SM work (same cost model as the runtime and the plugin)."""
    best, best_cost = 0, 0.0
    for bn in range(256, 31, -32):
        if bn % chunk or (M <= 32 and bn > 128 and chunk <= 128):   # few rows: the deep-ring variant
            continue
        tiles = ((M + 127) // 128) * ((N + bn - 1) // bn) * batch
        cost = ((tiles + sm_count - 1) // sm_count) * (400.0 + bn)
        if not best or cost < best_cost * 0.9999:
            best, best_cost = bn, cost
    return best


def matmul_export(kind: str, epilogue: str, generic: bool) -> str:
    table = {("f16", "cast"): "f16_f16", ("f16", "acc"): "f16_f32", ("bf16", "cast"): "bf16_bf16",
             ("bf16", "acc"): "bf16_f32", ("i8", "acc"): "i8_i32", ("i8", "requant"): "i8_requant_f16"}
    if (kind, epilogue) not in table:
        raise ValueError("no kernel for %s with epilogue %s" % (kind, epilogue))
    return ("b200_matmul_generic_" if generic else "b200_matmul_") + table[(kind, epilogue)]


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
    bn = choose_tile_n(M, N, batch, 128 // es if layout == 0 else 32, sm_count)
    tiles = ((M + 127) // 128) * ((N + bn - 1) // bn) * batch
    plan.transients.append({"name": "workspace", "bytes": 512, "zero": True})
    if device_tensor_maps:
        plan.transients.append({"name": "templates", "bytes": 256, "zero": False, "templates": kind})
        plan.dispatches.append(Dispatch("b200_encode_tensormaps", ["lhs", "rhs", "templates", "workspace"],
                                        [M, N, K, batch, layout, bn, es], (1, 1, 1), (32, 1, 1), 0))
    else:
        plan.transients[0]["host_tensor_maps"] = {"kind": kind, "M": M, "N": N, "K": K, "batch": batch,
                                                  "layout": layout, "tile_n": bn}
    plan.dispatches.append(Dispatch(matmul_export(kind, epilogue, False), ["out"] + scales + ["workspace"],
                                    [M, N, K, batch, layout, bn], (min(tiles, sm_count), 1, 1), (GEMM_THREADS, 1, 1),
                                    GEMM_SMEM))
    return plan


def plan_w4a16(function: str, M: int, N: int, K: int, group: int = 128, ldo: Optional[int] = None,
               n_offset: int = 0, sm_count: int = SM_COUNT) -> Plan:
    """dequant-like generic (i4 -> f16 * scale) cloned into the grouped contraction + truncf."""
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
        if slices > 1:   # the kernel reads its weight tiles through a tensor map at the start of the workspace
            ws["host_tensor_maps"] = {"kind": "w4a16_decode", "M": M, "N": N, "K": K}
        plan.transients.append(ws)
        mh = 8 if M <= 8 else 16
        walkers = max(1, min(N // 16, sm_count // slices))
        plan.dispatches.append(Dispatch("b200_w4a16_decode_m%d" % mh, ["a", "wq", "scales", "out", "workspace"],
                                        [M, N, K, ldo, n_offset], (walkers * slices, 1, 1),
                                        (DECODE_THREADS, 1, 1), DECODE_SMEM[mh]))
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
        plan.transients.append({"name": "workspace", "bytes": 512, "zero": True,
                                "host_tensor_maps": {"kind": "w4a16", "M": M, "N": N, "K": K, "tile_n": bn}})
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
