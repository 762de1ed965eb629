"""The bytecode-module subset: writer -> reader round trip, the loader's rejection rules, the
interpreter on a fake HAL module (CPU), and the same module executed on the GPU against the plan
executor. The reference holds no `.vmfb` fixture and its compiler cannot be built here, so the
reader has only met modules written by this repository's writer (parity unpinned)."""
import struct

import numpy as np
import pytest

from iree_b200 import dispatch_gen as dg
from iree_b200 import vm, vmfb


def tiny_module():
    """@add_one_and_two(): calls test.add(i32, i32) -> i32 twice and test.sum(variadic) once."""
    a = vmfb.Assembler()
    x, y = a.const_i32(40), a.const_i32(2)
    z = a.i32()
    a.call(0, [x, y], [z])
    big = a.const_i64(1 << 40)
    blob = a.const_ref_rodata(0)
    total = a.i64()
    a.call_variadic(1, [1, 3], [big, x, y, z], [total])
    a.ret([z, total, blob])
    m = vmfb.Module("tiny", version=3, types=["i32", "!vm.buffer"], dependencies=[("test", 1)],
                    imports=[vmfb.Import("test.add", "0ii_i"), vmfb.Import("test.sum", "0ICiD_I"),
                             vmfb.Import("test.optional", "0v_v", optional=True)],
                    rodata=[b"hello rodata", bytes(range(200))])
    m.functions.append(a.function("add_one_and_two", "0v_iIr"))
    return m


@pytest.mark.parametrize("external", [False, True])
def test_writer_reader_round_trip(external):
    m = tiny_module()
    data = vmfb.write_module(m, external_rodata=external)
    size = struct.unpack_from("<I", data, 0)[0]
    assert data[8:12] == b"IREE" and size <= len(data) - 4            # size prefix, file identifier
    back = vmfb.read_module(data)
    assert back == m
    # a polyglot zip prefix (local file header in front of the module) is skipped
    name = b"module.fb"
    pad = (64 - (30 + len(name)) % 64) % 64 if external else 0       # external segments are addressed from 64-byte boundaries
    zipped = struct.pack("<IHHHHHIIIHH", vmfb.ZIP_SIGNATURE, 20, 0, 0, 0, 0, 0, 0, 0, len(name), pad) + name + bytes(pad) + data
    assert vmfb.read_module(zipped) == m


def test_loader_rejection_rules():
    data = bytearray(vmfb.write_module(tiny_module()))
    with pytest.raises(vmfb.VmfbError) as e:
        vmfb.read_module(bytes(data[:12]))
    assert e.value.code == "INVALID_ARGUMENT"                         # less than 16 bytes
    bad = bytearray(data)
    struct.pack_into("<I", bad, 0, len(data))                          # length prefix beyond the file
    with pytest.raises(vmfb.VmfbError):
        vmfb.read_module(bytes(bad))
    bad = bytearray(data)
    bad[8:12] = b"NOPE"
    with pytest.raises(vmfb.VmfbError):
        vmfb.read_module(bytes(bad))
    m = tiny_module()
    m.bytecode_version = (14 << 16)                                    # other major version
    with pytest.raises(vmfb.VmfbError) as e:
        vmfb.read_module(vmfb.write_module(m))
    assert "version" in str(e.value)
    m.bytecode_version = vmfb.BYTECODE_VERSION + 1                     # newer minor version
    with pytest.raises(vmfb.VmfbError):
        vmfb.read_module(vmfb.write_module(m))


def test_interpreter_marshals_by_calling_convention():
    calls = []

    def add(a, b):
        calls.append(("add", a, b))
        return a + b

    def total(big, items):
        calls.append(("sum", big, items))
        return big + sum(v for (v,) in items)

    m = vmfb.read_module(vmfb.write_module(tiny_module()))
    interp = vm.Interpreter(m, {"test.add": add, "test.sum": total})
    z, t, blob = interp.invoke("add_one_and_two", [])
    assert (z, t, blob) == (42, (1 << 40) + 40 + 2 + 42, b"hello rodata")
    assert calls == [("add", 40, 2), ("sum", 1 << 40, [(40,), (2,), (42,)])]
    with pytest.raises(vm.VmError) as e:
        interp.invoke("missing", [])
    assert e.value.code == "NOT_FOUND"
    with pytest.raises(vm.VmError) as e:
        vm.Interpreter(m, {"test.add": add})                           # required import not registered
    assert e.value.code == "NOT_FOUND"


def test_interpreter_branches_and_refuses_unknown_opcodes():
    a = vmfb.Assembler()
    x = a.const_i32(5)
    nz = a.i32()
    a.code += bytes([vmfb.OP["CmpNZI32"]]) + struct.pack("<HH", x, nz)
    # cond_br nz, ^then(x -> r3), ^else(): two blocks follow
    r3 = a.i32()
    here = len(a.code)
    a.code += bytes([vmfb.OP["CondBranch"]]) + struct.pack("<H", nz)
    then_at = len(a.code)
    a.code += struct.pack("<i", 0)
    if len(a.code) % 2:
        a.code.append(0)
    a.code += struct.pack("<HHH", 1, x, r3)
    else_at = len(a.code)
    a.code += struct.pack("<i", 0)
    if len(a.code) % 2:
        a.code.append(0)
    a.code += struct.pack("<H", 0)
    else_block = len(a.code)
    a.code += bytes([vmfb.OP["Block"]])
    zero = a.const_i32(0)
    a.ret([zero])
    then_block = len(a.code)
    a.code += bytes([vmfb.OP["Block"]])
    a.ret([r3])
    struct.pack_into("<i", a.code, then_at, then_block)
    struct.pack_into("<i", a.code, else_at, else_block)
    a.blocks = 3
    m = vmfb.Module("br")
    m.functions.append(a.function("f", "0v_i"))
    assert vm.Interpreter(vmfb.read_module(vmfb.write_module(m)), {}).invoke("f", []) == [5]
    bad = vmfb.Module("bad")
    bad.functions.append(vmfb.Function("f", "0v_v", bytes([vmfb.OP["Block"], 0x22]), 1, 1))
    with pytest.raises(vm.VmError) as e:
        vm.Interpreter(bad, {}).invoke("f", [])
    assert e.value.code == "UNIMPLEMENTED"
    assert here > 0


class FakeHal:
    """Records the HAL calls of a program; buffers are numpy arrays."""

    def __init__(self):
        self.log = []

    def imports(self):
        def make(name):
            def fn(*args):
                self.log.append(name)
                if name.endswith("buffer_view.buffer"):
                    return args[0].buffer
                if name.endswith("buffer_view.create"):
                    return vm.BufferView(args[0], [d[0] for d in args[5]], args[3])
                if name.endswith("fence.await"):
                    return 0
                if name.endswith("dispatch"):
                    self.log.append(("grid", args[3], args[4], args[5], "entry", args[2]))
                if name.endswith("push_constants"):
                    self.log.append(("constants", [v for (v,) in args[3]]))
                if name.endswith("push_descriptor_set"):
                    self.log.append(("bindings", [b[0] for b in args[3]]))
                if name.endswith(("_v",)):
                    return None
                return object()
            return fn
        return {n: make(n) for n, _ in vm._HAL_IMPORTS}


def test_plan_becomes_a_module_whose_hal_calls_are_the_plans_dispatches():
    plan = dg.plan_matmul("mm", "f16", "cast", 256, 384, 512)
    ordinals = {d.export: 10 + i for i, d in enumerate(plan.dispatches)}
    module = vm.plan_to_module(plan, b"\x10\0\0\0CUDAnot-a-real-executable", ordinals, templates=bytes(256))
    data = vmfb.write_module(module)
    back = vmfb.read_module(data)
    assert back.functions[0].name == "mm" and back.functions[0].calling_convention == "0rr_r"
    assert [i.full_name for i in back.imports] == [n for n, _ in vm._HAL_IMPORTS]
    hal = FakeHal()
    lhs = vm.BufferView(np.zeros(1), [256, 512], vm.ELEMENT_TYPES["f16"])
    rhs = vm.BufferView(np.zeros(1), [512, 384], vm.ELEMENT_TYPES["f16"])
    (out,) = vm.Interpreter(back, hal.imports()).invoke("mm", [lhs, rhs])
    assert out.shape == [256, 384] and out.element_type == vm.ELEMENT_TYPES["f16"]
    grids = [x for x in hal.log if isinstance(x, tuple) and x[0] == "grid"]
    assert grids == [("grid",) + d.grid + ("entry", ordinals[d.export]) for d in plan.dispatches]
    consts = [x[1] for x in hal.log if isinstance(x, tuple) and x[0] == "constants"]
    assert consts == [d.constants for d in plan.dispatches]
    names = [x for x in hal.log if isinstance(x, str)]
    assert names[0] == "hal.devices.get" and names[-1] == "hal.buffer_view.create"
    assert names.index("hal.executable.create") < names.index("hal.command_buffer.create") < names.index(
        "hal.command_buffer.finalize") < names.index("hal.device.queue.execute") < names.index("hal.fence.await")


@pytest.mark.gpu
def test_module_runs_on_the_gpu_like_the_plan(ctx):
    from iree_b200 import run_module, workloads
    import ctypes as C
    import iree_b200 as ib
    plan = dg.plan_matmul("c1", "i8", "acc", 1024, 1024, 1024)
    a, b = workloads.c1_i8_matmul()
    want = run_module.execute_plan(ctx, plan, [a, b])[0]
    exe = vm.contraction_executable_def()
    table = C.create_string_buffer(768)
    ib.runtime.check(ib.library().iree_b200_tensormap_templates(ctx.handle, table))
    kind_row = {"f16": 0, "bf16": 1, "i8": 2}["i8"]
    pair = table.raw[128 * kind_row:128 * kind_row + 128] * 2
    module = vm.plan_to_module(plan, exe, vm.export_ordinals(exe), templates=pair)
    outs, trace = vm.run_vmfb(ctx, vmfb.write_module(module, external_rodata=True), "c1", [a, b])
    assert (outs[0] == want).all()
    assert trace.count("hal.command_buffer.dispatch") == len(plan.dispatches)


def test_writer_command_line_embeds_the_contraction_executable(built, tmp_path):
    out = tmp_path / "c3.vmfb"
    assert vm.main(["--plan", "c3_w8a8_m16", "-o", str(out)]) == 0
    m = vmfb.read_module(out.read_bytes())
    assert [f.name for f in m.functions] == ["c3_m16"] and m.functions[0].calling_convention == "0rrrr_r"
    exe = m.rodata[0]
    assert exe[4:8] == b"CUDA" and m.rodata[1] == b"PTXE"               # the ExecutableDef and its format string
    names = vm.export_ordinals(exe)
    assert "b200_matmul_i8_requant_f16" in names and "b200_encode_tensormaps" in names
    assert len(m.rodata[2]) == 256                                      # the operand pair's tensor-map templates
