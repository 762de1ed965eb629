"""``iree-run-module``-shaped command line over a host plan (``iree_b200.dispatch_gen.Plan``).

    python -m iree_b200.run_module --device=cuda --module=plan.json --function=c2 \
        --input=4096x4096xf16=@lhs.npy --input=4096x4096xf16=@rhs.npy \
        [--output=@out.npy] [--expected_output=4096x4096xf16=@want.npy] [--print_statistics]

Flag names, the ``EXEC @function`` line, the ``SHAPExTYPE=@file.npy`` input grammar and the
non-zero exit code on a mismatch follow runtime/src/iree/tooling/run_module.c:23-91,199-322. A real
.vmfb needs IREE's bytecode VM, which is outside this repository; the module here is the plan
(exports, bindings, push constants, grids) plus the cubin, executed through the same HAL calls a
compiled program makes: executable create from an ExecutableDef, push constants, push descriptor
set, dispatch. Only ``--device=cuda`` exists: there is no CPU path.
"""
from __future__ import annotations

import argparse
import sys

import numpy as np

from . import runtime as rt
from .dispatch_gen import Plan

_DTYPES = {"f16": np.float16, "bf16": np.uint16, "i8": np.int8, "si8": np.int8, "ui8": np.uint8, "u8": np.uint8,
           "i32": np.int32, "f32": np.float32}


def parse_tensor_flag(text: str):
    """``4096x4096xf16=@file.npy`` or ``2x2xi8=1 2 3 4`` -> ndarray (hal/string_util.c grammar)."""
    spec, _, value = text.partition("=")
    parts = spec.split("x")
    dtype = _DTYPES[parts[-1]]
    shape = tuple(int(p) for p in parts[:-1])
    if value.startswith("@"):
        arr = np.load(value[1:]) if value.endswith(".npy") else np.fromfile(value[1:], dtype=dtype)
        arr = np.ascontiguousarray(arr).view(dtype).reshape(shape)
    else:
        vals = value.replace(",", " ").split()
        arr = (np.full(shape, dtype(float(vals[0]))) if len(vals) == 1 else np.array([float(v) for v in vals])).astype(
            dtype).reshape(shape)
    return arr


def execute_plan(ctx: rt.Context, plan: Plan, inputs, parameters=None):
    """Runs every dispatch of the plan through the raw HAL-level calls; returns the outputs.

    Inputs the plan binds to a parameter (``"parameter": "scope::key"``, what a compiled program
    declares as ``#stream.parameter.named<"scope"::"key">``) are loaded from the archives in
    ``parameters`` (scope -> ParameterIndex) instead of being taken from ``inputs``.
    """
    free_inputs = [d for d in plan.inputs if "parameter" not in d]
    if len(inputs) != len(free_inputs):
        raise rt.IreeB200Error(3, "function expects %d inputs, %d given" % (len(free_inputs), len(inputs)))
    buffers, owned = {}, []
    for decl, arr in zip(free_inputs, inputs):
        if list(arr.shape) != list(decl["shape"]) and int(np.prod(arr.shape)) == int(np.prod(decl["shape"])) and \
                arr.shape[0] == decl["shape"][0]:
            arr = arr.reshape(decl["shape"])       # a reshape of the trailing dimensions: [M, G, 128] for [M, K]
        if list(arr.shape) != list(decl["shape"]):
            raise rt.IreeB200Error(3, "input %s: expected shape %s, got %s" % (decl["name"], decl["shape"], list(arr.shape)))
        buffers[decl["name"]] = ctx.to_device(arr)
    for decl in plan.inputs:
        if "parameter" not in decl:
            continue
        scope, _, key = decl["parameter"].rpartition("::")
        index = (parameters or {}).get(scope)
        if index is None:
            raise rt.IreeB200Error(5, "no parameter provider registered for scope '%s'" % scope)
        nbytes = int(np.prod(decl["shape"])) * np.dtype(_DTYPES[decl["dtype"]]).itemsize
        if index.lookup(key).length != nbytes:
            raise rt.IreeB200Error(3, "parameter %s holds %d bytes, the program expects %d" % (
                decl["parameter"], index.lookup(key).length, nbytes))
        buf = ctx.alloc(max(nbytes, 1))
        index.load(ctx, key, buf, nbytes)
        buffers[decl["name"]] = buf
    for decl in plan.outputs:
        n = int(np.prod(decl["shape"])) * np.dtype(_DTYPES[decl["dtype"]]).itemsize
        buffers[decl["name"]] = ctx.alloc(max(n, 1))
    for t in plan.transients:
        buf = ctx.alloc(t["bytes"])
        if t.get("zero"):
            buf.fill(0)
        if t.get("templates") == "table":      # every template kind, as the compiler plugin embeds them
            import ctypes as C
            host = C.create_string_buffer(768)
            rt.check(rt.library().iree_b200_tensormap_templates(ctx.handle, host))
            buf.upload(np.frombuffer(host.raw, np.uint8))
        elif t.get("templates"):
            kind = t["templates"]
            es = 1 if kind == "i8" else 2
            host = b"".join(ctx.encode_tensor_map(es, kind == "bf16", buf, 128 // es * 4, 256, 1, 128 // es, 64)
                            for _ in range(2))
            buf.upload(np.frombuffer(host, np.uint8))
        buffers[t["name"]] = buf
        if "host_tensor_maps" in t:
            _host_tensor_maps(ctx, t["host_tensor_maps"], buffers, buf)
    for d in plan.dispatches:
        ctx.dispatch(d.export, [buffers[b] for b in d.bindings], d.constants, d.grid)
    if "workspace" in buffers:
        ctx.workspace_status(buffers["workspace"])
    ctx.synchronize()
    outs = [buffers[o["name"]].download(_DTYPES[o["dtype"]], tuple(o["shape"])) for o in plan.outputs]
    for b in buffers.values():
        b.free()
    return outs


def _host_tensor_maps(ctx, spec, buffers, ws):
    if spec["kind"] == "w4a16_decode":
        p = rt.W4A16Params(spec["M"], spec["N"], spec["K"], 128, spec["N"], 0, rt.W4A16_DECODE, 0)
        ctx.w4a16_prepare(p, buffers["a"], buffers["wq"], buffers["scales"], buffers["out"], ws)
    elif spec["kind"] == "w4a16_wt":
        p = rt.W4A16Params(spec["M"], spec["N"], spec["K"], 128, spec["ldo"], spec["n_offset"], rt.W4A16_GEMM_WT, 0)
        ctx.w4a16_prepare(p, buffers["a"], buffers["wq"], buffers["scales"], buffers["out"], ws)
    elif spec["kind"] == "w4a16":
        p = rt.W4A16Params(spec["M"], spec["N"], spec["K"], 128, spec["N"], 0, rt.W4A16_GEMM, spec["tile_n"])
        ctx.w4a16_prepare(p, buffers["a"], buffers["wq"], buffers["scales"], buffers["out"], ws)
    else:
        kind = {"f16": rt.KIND_F16, "bf16": rt.KIND_BF16, "i8": rt.KIND_I8}[spec["kind"]]
        epilogue = {"cast": rt.EPILOGUE_CAST, "acc": rt.EPILOGUE_ACCUMULATOR, "requant": rt.EPILOGUE_REQUANT_F16}[
            spec.get("epilogue", "acc" if kind == rt.KIND_I8 else "cast")]
        p = rt.MatmulParams(kind, epilogue, spec["M"], spec["N"], spec["K"], spec["batch"], spec["layout"], spec["tile_n"], 0)
        ctx.matmul_prepare(p, buffers["lhs"], buffers["rhs"], ws)


def _run_bytecode_module(args, contents: bytes) -> int:
    """--module=x.vmfb: the bytecode-module subset (iree_b200/vm.py) instead of a JSON plan."""
    from . import vm, vmfb
    try:
        module = vmfb.read_module(contents)
    except vmfb.VmfbError as e:
        print(str(e), file=sys.stderr)
        return 1
    exported = [f.name for f in module.functions if f.name]
    function = args.function or (exported[0] if exported else "")
    if function not in exported:
        print("NOT_FOUND: no function @%s in the module (it exports %s)" % (function, ", ".join("@" + n for n in exported)),
              file=sys.stderr)
        return 1
    inputs = [parse_tensor_flag(t) for t in args.input]
    ordinal = int(args.device.split(":")[1]) if ":" in args.device else 0
    ctx = rt.Context(ordinal)
    try:
        print("EXEC @%s" % function)
        outs, _ = vm.run_vmfb(ctx, contents, function, inputs)
        for i, o in enumerate(outs):
            if i < len(args.output) and args.output[i].startswith("@"):
                np.save(args.output[i][1:], o)
            else:
                print("result[%d]: hal.buffer_view\n%sx%s=%s ..." % (i, "x".join(map(str, o.shape)), o.dtype,
                                                                   " ".join(str(v) for v in o.reshape(-1)[:8])))
        return 0
    finally:
        ctx.close()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="iree_b200.run_module", allow_abbrev=False)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--module", required=True)
    ap.add_argument("--function", default="")
    ap.add_argument("--input", action="append", default=[])
    ap.add_argument("--parameters", action="append", default=[],
                    help="[scope=]file.irpa: parameters of that scope come from the archive (tooling/parameter_util.c)")
    ap.add_argument("--output", action="append", default=[])
    ap.add_argument("--expected_output", action="append", default=[])
    ap.add_argument("--print_statistics", action="store_true")
    args = ap.parse_args(argv)
    if not args.device.startswith("cuda"):
        print("only --device=cuda is available (no CPU path)", file=sys.stderr)
        return 2
    raw = open(args.module, "rb").read()
    if not raw.lstrip()[:1] == b"{":
        return _run_bytecode_module(args, raw)
    plan = Plan.from_json(raw.decode())
    if args.function and args.function != plan.function:
        print("NOT_FOUND: no function @%s in the module (it holds @%s)" % (args.function, plan.function), file=sys.stderr)
        return 1
    inputs = [parse_tensor_flag(t) for t in args.input]
    from .parameters import ParameterIndex
    parameters = {}
    for spec in args.parameters:
        scope, sep, path = spec.partition("=")
        if not sep:
            scope, path = "", spec
        parameters[scope] = ParameterIndex(path)
    ordinal = int(args.device.split(":")[1]) if ":" in args.device else 0
    ctx = rt.Context(ordinal)
    try:
        print("EXEC @%s" % plan.function)
        outs = execute_plan(ctx, plan, inputs, parameters)
        for i, o in enumerate(outs):
            if i < len(args.output) and args.output[i].startswith("@"):
                np.save(args.output[i][1:], o)
            else:
                print("result[%d]: hal.buffer_view\n%sx%s=%s ..." % (i, "x".join(map(str, o.shape)), plan.outputs[i]["dtype"],
                                                                   " ".join(str(v) for v in o.reshape(-1)[:8])))
        rc = 0
        for i, text in enumerate(args.expected_output):
            want = parse_tensor_flag(text)
            ok = (outs[i] == want).all() if outs[i].dtype.kind in "iu" else np.allclose(
                outs[i].astype(np.float32), want.astype(np.float32), rtol=1e-2, atol=1e-2)
            print("[SUCCESS] all function outputs matched their expected values." if ok
                  else "[FAILED] result[%d]: element mismatch" % i)
            rc |= 0 if ok else 1
        if args.print_statistics:
            print("[[ statistics ]] kernel launches: %d" % ctx.launch_count)
        return rc
    finally:
        ctx.close()


if __name__ == "__main__":
    sys.exit(main())
