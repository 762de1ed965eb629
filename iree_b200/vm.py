"""A bytecode interpreter for the subset of IREE's VM a single-dispatch program uses, the HAL module
imports such a program calls, and a writer that turns a dispatch plan into a `.vmfb`.

Reference: the interpreter is runtime/src/iree/vm/bytecode/dispatch.c (ops :842-878 constants,
:1613-1647 branches, :1680-1780 calls and return; import marshalling by calling-convention string
:360-441); the imports are the functions of runtime/src/iree/modules/hal/exports.inl with the
argument lists given there. Everything runs through the `iree_hal_b200_*` layer of the runtime
library: a command buffer records into a CUDA graph (`command_buffer.create` .. `finalize`) and
`device.queue.execute` launches it, the way the reference's graph command buffer does.

Parity note: checked only against modules produced by `plan_to_module` below (see vmfb.py).
"""
import ctypes as C
import struct
from typing import Callable, Dict, List

import numpy as np

from . import vmfb
from .vmfb import OP, REF_MASK, Assembler, Function, Import, Module

# iree/hal/buffer_view.h:30-151: numerical type << 24 | bit count
ELEMENT_TYPES = {"i8": 0x11000008, "i32": 0x11000020, "f16": 0x21000010, "bf16": 0x22000010, "f32": 0x21000020}
ELEMENT_NAMES = {v: k for k, v in ELEMENT_TYPES.items()}
ENCODING_DENSE_ROW_MAJOR = 1


class VmError(RuntimeError):
    def __init__(self, code: str, message: str):
        super().__init__("%s: %s" % (code, message))
        self.code = code


def parse_cconv(cc: str):
    """"0rriCiD_v" -> (arguments, results) as strings (iree/vm/module.h: version digit, '_' separator)."""
    if not cc or cc[0] != "0":
        raise VmError("UNIMPLEMENTED", "unsupported calling convention version in '%s'" % cc)
    args, _, results = cc[1:].partition("_")
    return ("" if args == "v" else args), ("" if results == "v" else results)


class Interpreter:
    """Executes exported functions of a bytecode module; imports are Python callables by full name."""

    def __init__(self, module: Module, imports: Dict[str, Callable]):
        self.module = module
        self.imports = []
        for imp in module.imports:
            fn = imports.get(imp.full_name)
            if fn is None and not imp.optional:
                raise VmError("NOT_FOUND", "required import '%s' not registered" % imp.full_name)
            self.imports.append((imp, fn))
        self.rodata = [bytes(r) for r in module.rodata]
        self.global_refs = [None] * module.global_refs
        self.exports = {f.name: i for i, f in enumerate(module.functions) if f.name}

    def invoke(self, name: str, args: List):
        if name not in self.exports:
            raise VmError("NOT_FOUND", "no exported function '%s'" % name)
        return self._run(self.exports[name], args)

    def _run(self, ordinal: int, args: List):
        f = self.module.functions[ordinal]
        cc_args, cc_results = parse_cconv(f.calling_convention)
        i32 = np.zeros(max(f.i32_registers, 2) + 2, np.int32)
        ref = [None] * max(f.ref_registers, 1)
        ni = nr = 0
        if len(args) != len(cc_args):
            raise VmError("INVALID_ARGUMENT", "function takes %d arguments, %d given" % (len(cc_args), len(args)))
        for c, a in zip(cc_args, args):       # arguments fill each register bank in order (dispatch.c external_enter)
            if c == "r":
                ref[nr] = a
                nr += 1
            elif c in "iI":
                if c == "I":
                    ni = (ni + 1) & ~1
                    i32[ni:ni + 2] = np.frombuffer(struct.pack("<q", a), np.int32)
                    ni += 2
                else:
                    i32[ni] = a
                    ni += 1
            else:
                raise VmError("UNIMPLEMENTED", "argument type '%s'" % c)
        code, pc = f.bytecode, 0

        def u16():
            nonlocal pc
            v = struct.unpack_from("<H", code, pc)[0]
            pc += 2
            return v

        def reg_list():
            nonlocal pc
            pc = (pc + 1) & ~1
            n = u16()
            return [u16() for _ in range(n)]

        def get(kind: str, r: int):
            if kind == "r":
                return ref[r & REF_MASK]
            if kind in "if":
                return int(i32[r])
            return struct.unpack("<q", i32[r:r + 2].tobytes())[0]

        def put(kind: str, r: int, value):
            if kind == "r":
                ref[r & REF_MASK] = value
            elif kind in "if":
                i32[r] = np.int32(value)
            else:
                i32[r:r + 2] = np.frombuffer(struct.pack("<q", value), np.int32)

        steps = 0
        while True:
            steps += 1
            if steps > 1_000_000:
                raise VmError("DEADLINE_EXCEEDED", "function did not return within a million instructions")
            if pc >= len(code):
                raise VmError("OUT_OF_RANGE", "execution ran off the end of the function")
            op = code[pc]
            pc += 1
            if op == OP["Block"]:
                continue
            if op == OP["ConstI32Zero"]:
                i32[u16()] = 0
            elif op == OP["ConstI32"]:
                v = struct.unpack_from("<i", code, pc)[0]
                pc += 4
                i32[u16()] = v
            elif op == OP["ConstI64Zero"]:
                put("I", u16(), 0)
            elif op == OP["ConstI64"]:
                v = struct.unpack_from("<q", code, pc)[0]
                pc += 8
                put("I", u16(), v)
            elif op == OP["ConstRefZero"]:
                ref[u16() & REF_MASK] = None
            elif op == OP["ConstRefRodata"]:
                ordinal_ = struct.unpack_from("<i", code, pc)[0]
                pc += 4
                if not 0 <= ordinal_ < len(self.rodata):
                    raise VmError("OUT_OF_RANGE", "rodata ordinal %d" % ordinal_)
                ref[u16() & REF_MASK] = self.rodata[ordinal_]
            elif op in (OP["GlobalLoadRef"], OP["GlobalStoreRef"]):
                g = struct.unpack_from("<i", code, pc)[0]
                pc += 8           # global ordinal, then the type id
                r = u16()
                if not 0 <= g < len(self.global_refs):
                    raise VmError("OUT_OF_RANGE", "global ref ordinal %d" % g)
                if op == OP["GlobalLoadRef"]:
                    ref[r & REF_MASK] = self.global_refs[g]
                else:
                    self.global_refs[g] = ref[r & REF_MASK]
            elif op in (OP["CmpEQI32"], OP["CmpNEI32"]):
                a, b, d = u16(), u16(), u16()
                i32[d] = int((i32[a] == i32[b]) == (op == OP["CmpEQI32"]))
            elif op == OP["CmpNZI32"]:
                a, d = u16(), u16()
                i32[d] = int(i32[a] != 0)
            elif op in (OP["Branch"], OP["CondBranch"]):
                cond = True
                if op == OP["CondBranch"]:
                    cond = bool(i32[u16()])
                targets = []
                for _ in range(1 if op == OP["Branch"] else 2):
                    t = struct.unpack_from("<i", code, pc)[0]
                    pc += 4
                    pc = (pc + 1) & ~1
                    n = u16()
                    targets.append((t, [(u16(), u16()) for _ in range(n)]))
                t, remap = targets[0] if cond else targets[1]
                moved = [(dst, ref[src & REF_MASK] if src & vmfb.REF_TYPE_BIT else int(i32[src])) for src, dst in remap]
                for dst, v in moved:
                    if dst & vmfb.REF_TYPE_BIT:
                        ref[dst & REF_MASK] = v
                    else:
                        i32[dst] = v
                pc = t + 1    # skip the block marker
            elif op in (OP["Call"], OP["CallVariadic"]):
                callee = struct.unpack_from("<I", code, pc)[0]
                pc += 4
                segments = reg_list() if op == OP["CallVariadic"] else None
                operands, results = reg_list(), reg_list()
                if not callee & 0x80000000:
                    if segments is not None:
                        raise VmError("FAILED_PRECONDITION", "variadic calls only supported for imports")
                    g = self.module.functions[callee]
                    ca, cr = parse_cconv(g.calling_convention)
                    out = self._run(callee, [get(c, r) for c, r in zip(ca, operands)])
                    for c, r, v in zip(cr, results, out):
                        put(c, r, v)
                    continue
                imp, fn = self.imports[callee & 0x7fffffff]
                if fn is None:
                    raise VmError("NOT_FOUND", "optional import '%s' was called but is not registered" % imp.full_name)
                ca, cr = parse_cconv(imp.calling_convention)
                values, k, seg, i = [], 0, 0, 0
                while i < len(ca):            # dispatch.c:360-441
                    c = ca[i]
                    if c == "C":
                        end = ca.index("D", i)
                        inner = ca[i + 1:end]
                        count = segments[seg] if segments is not None else 0
                        items = []
                        for _ in range(count):
                            items.append(tuple(get(t, operands[k + j]) for j, t in enumerate(inner)))
                            k += len(inner)
                        values.append(items)
                        i = end
                    else:
                        values.append(get(c, operands[k]))
                        k += 1
                    i += 1
                    seg += 1
                out = fn(*values)
                if not cr:
                    out = ()
                elif len(cr) == 1:
                    out = (out,)
                for c, r, v in zip(cr, results, out):
                    put(c, r, v)
            elif op == OP["Return"]:
                regs = reg_list()
                return [get(c, r) for c, r in zip(cc_results, regs)]
            elif op == OP["Fail"]:
                status = int(i32[u16()])
                n = u16()
                message = code[pc:pc + n].decode("utf-8", "replace")
                raise VmError("status %d" % status, message)
            else:
                raise VmError("UNIMPLEMENTED", "opcode 0x%02X (%s) is outside the supported subset" % (
                    op, vmfb.OP_NAME.get(op, "?")))


# ------------------------------------------------------------------------------------------------
# The HAL module over the runtime library
# ------------------------------------------------------------------------------------------------
class BufferView:
    def __init__(self, buffer, shape, element_type: int, encoding_type: int = ENCODING_DENSE_ROW_MAJOR):
        self.buffer, self.shape, self.element_type, self.encoding_type = buffer, list(shape), element_type, encoding_type


class _CommandBuffer:
    def __init__(self):
        self.graph = None
        self.constants = {}
        self.bindings = {}


class HalModule:
    """`hal.*` imports (modules/hal/exports.inl) for one device, on top of a runtime Context."""

    def __init__(self, ctx):
        from . import runtime as rt
        self.ctx, self.rt, self.lib = ctx, rt, rt.library()
        self.owned = []              # device buffers allocated by the program
        self.executables = []
        self.trace = []              # (import name, summary) in call order, for tests and --trace

    def imports(self) -> Dict[str, Callable]:
        table = {}
        for name in dir(self):
            if name.startswith("hal_"):
                full = "hal." + name[4:].replace("__", ".")
                table[full] = self._traced(full, getattr(self, name))
        return table

    def _traced(self, full, fn):
        def call(*args):
            self.trace.append(full)
            return fn(*args)
        return call

    def close(self):
        self.ctx.synchronize()
        for b in self.owned:
            b.free()
        for e in self.executables:
            self.lib.iree_hal_b200_executable_release(e)
        self.owned, self.executables = [], []

    # devices.get(i) -> r ; device.allocator(r) -> r
    def hal_devices__get(self, index):
        if index != 0:
            raise VmError("OUT_OF_RANGE", "device %d" % index)
        return self.ctx

    def hal_device__allocator(self, device):
        return device

    # allocator.allocate(rIiiI) -> r
    def hal_allocator__allocate(self, allocator, queue_affinity, memory_types, buffer_usage, size):
        buf = self.ctx.alloc(max(int(size), 1))
        self.owned.append(buf)
        return buf

    # allocator.import(riIiirII) -> r: a host buffer (rodata) becomes a device buffer
    def hal_allocator__import(self, allocator, try_, queue_affinity, memory_types, buffer_usage, source, offset, length):
        data = np.frombuffer(source, np.uint8)[offset:offset + length]
        buf = self.ctx.to_device(np.ascontiguousarray(data))
        self.owned.append(buf)
        return buf

    # buffer_view.*
    def hal_buffer_view__create(self, buffer, source_offset, source_length, element_type, encoding_type, shape):
        if source_offset:
            raise VmError("UNIMPLEMENTED", "buffer views at an offset")
        return BufferView(buffer, [d[0] for d in shape], element_type, encoding_type)

    def hal_buffer_view__buffer(self, view):
        return view.buffer

    def hal_buffer_view__rank(self, view):
        return len(view.shape)

    def hal_buffer_view__dim(self, view, index):
        return view.shape[index]

    def hal_buffer_view__element_type(self, view):
        return view.element_type

    def hal_buffer_view__assert(self, view, message, element_type, encoding_type, shape):
        want = [d[0] for d in shape]
        if view.element_type != element_type or view.shape != want:
            raise VmError("INVALID_ARGUMENT", "%s: expected %s of element type %#x, got %s of %#x" % (
                bytes(message).decode() if message else "input", want, element_type, view.shape, view.element_type))

    # executable.create(rrrrCrD) -> r
    def hal_executable__create(self, device, executable_format, executable_data, constants, layouts):
        handle = C.c_void_p()
        fmt = bytes(executable_format).decode()
        self.rt.check(self.lib.iree_hal_b200_executable_create(self.ctx.device, fmt.encode(), bytes(executable_data),
                                                               C.c_size_t(len(executable_data)), C.byref(handle)))
        self.executables.append(handle)
        return handle

    def hal_descriptor_set_layout__create(self, device, flags, bindings):
        return ("descriptor_set_layout", flags, list(bindings))

    def hal_pipeline_layout__create(self, device, push_constants, set_layouts):
        return ("pipeline_layout", push_constants, [s[0] for s in set_layouts])

    # command buffers record into a CUDA graph
    def hal_command_buffer__create(self, device, modes, command_categories, binding_capacity):
        cb = _CommandBuffer()
        self.rt.check(self.lib.iree_hal_b200_command_buffer_begin_graph(self.ctx.command_buffer))
        return cb

    def hal_command_buffer__fill_buffer(self, cb, buffer, offset, length, pattern, pattern_length):
        # a memset node of the recording; the pattern arrives as an i32 of which pattern_length bytes count
        raw = int(pattern & 0xFFFFFFFF).to_bytes(4, "little")[:pattern_length]
        self.rt.check(self.lib.iree_hal_b200_command_buffer_fill_buffer(
            self.ctx.command_buffer, self.rt._vp(buffer), C.c_size_t(offset), C.c_size_t(length), raw,
            C.c_size_t(pattern_length)))

    def hal_command_buffer__copy_buffer(self, cb, source, source_offset, target, target_offset, length):
        self.rt.check(self.lib.iree_hal_b200_command_buffer_copy_buffer(
            self.ctx.command_buffer, self.rt._vp(source), C.c_size_t(source_offset), self.rt._vp(target),
            C.c_size_t(target_offset), C.c_size_t(length)))

    def hal_command_buffer__push_constants(self, cb, pipeline_layout, offset, values):
        for i, (v,) in enumerate(values):
            cb.constants[offset // 4 + i] = v

    def hal_command_buffer__push_descriptor_set(self, cb, pipeline_layout, set_, bindings):
        for ordinal, slot, buffer, offset, length in bindings:
            if offset:
                raise VmError("UNIMPLEMENTED", "bindings at an offset")
            cb.bindings[ordinal] = buffer

    def hal_command_buffer__dispatch(self, cb, executable, entry_point, x, y, z):
        n = (max(cb.bindings) + 1) if cb.bindings else 0
        arr = (self.rt._Binding * max(n, 1))()
        for i in range(n):
            arr[i].binding, arr[i].device_ptr = i, self.rt._vp(cb.bindings[i]).value
        consts = np.asarray([cb.constants[i] for i in range(len(cb.constants))], np.int32)
        c = self.ctx.command_buffer
        self.rt.check(self.lib.iree_hal_b200_command_buffer_push_descriptor_set(c, C.c_uint32(0), C.c_size_t(n), arr))
        self.rt.check(self.lib.iree_hal_b200_command_buffer_push_constants(c, C.c_size_t(0), self.rt._vp(consts),
                                                                           C.c_size_t(consts.nbytes)))
        self.rt.check(self.lib.iree_hal_b200_command_buffer_dispatch(c, executable, C.c_int32(entry_point), C.c_uint32(n),
                                                                     C.c_uint32(len(consts)), C.c_uint32(x), C.c_uint32(y),
                                                                     C.c_uint32(z)))
        cb.constants, cb.bindings = {}, {}

    def hal_command_buffer__execution_barrier(self, cb, source_stage_mask, target_stage_mask, flags):
        # nodes of the recording already depend on each other in order; the barrier keeps the next dispatch
        # from being launched early
        self.rt.check(self.lib.iree_hal_b200_command_buffer_execution_barrier(
            self.ctx.command_buffer, C.c_uint32(source_stage_mask & 0xFFFFFFFF), C.c_uint32(target_stage_mask & 0xFFFFFFFF),
            C.c_uint32(flags & 0xFFFFFFFF)))

    def hal_command_buffer__finalize(self, cb):
        g = C.c_void_p()
        self.rt.check(self.lib.iree_hal_b200_command_buffer_end_graph(self.ctx.command_buffer, C.byref(g)))
        cb.graph = g

    def hal_fence__create(self, device, flags):
        return ["fence", False]

    def hal_device__queue__execute(self, device, queue_affinity, wait_fence, signal_fence, command_buffers):
        for (cb,) in command_buffers:
            self.rt.check(self.lib.iree_hal_b200_graph_execute(self.ctx.command_buffer, cb.graph))
            self.lib.iree_hal_b200_graph_release(cb.graph)
            cb.graph = None
        if signal_fence is not None:
            signal_fence[1] = True

    def hal_fence__await(self, timeout_millis, fences):
        self.ctx.synchronize()
        return 0


# ------------------------------------------------------------------------------------------------
# Plan -> module
# ------------------------------------------------------------------------------------------------
_HAL_IMPORTS = [
    ("hal.devices.get", "0i_r"), ("hal.device.allocator", "0r_r"), ("hal.allocator.allocate", "0rIiiI_r"),
    ("hal.allocator.import", "0riIiirII_r"), ("hal.buffer_view.assert", "0rriiCID_v"), ("hal.buffer_view.buffer", "0r_r"),
    ("hal.buffer_view.create", "0rIIiiCID_r"), ("hal.descriptor_set_layout.create", "0riCiiiD_r"),
    ("hal.pipeline_layout.create", "0riCrD_r"), ("hal.executable.create", "0rrrrCrD_r"),
    ("hal.command_buffer.create", "0riii_r"), ("hal.command_buffer.push_constants", "0rriCiD_v"),
    ("hal.command_buffer.push_descriptor_set", "0rriCiirIID_v"), ("hal.command_buffer.dispatch", "0rriiii_v"),
    ("hal.command_buffer.execution_barrier", "0riii_v"), ("hal.command_buffer.finalize", "0r_v"),
    ("hal.fence.create", "0ri_r"), ("hal.device.queue.execute", "0rIrrCrD_v"), ("hal.fence.await", "0iCrD_i"),
]


def plan_to_module(plan, executable_def: bytes, export_ordinals: Dict[str, int], templates: bytes = b"") -> Module:
    """The host program of a dispatch plan as a bytecode module: one exported function taking the
    plan's inputs as buffer views and returning its outputs. Transient buffers must be ones a
    program can produce itself: zero-initialised workspaces are not expressible without a fill, so
    plans are expected to build their tensor maps on the device (`device_tensor_maps=True`) and the
    workspace's header is then written by the encode dispatch; counters behind it need a zeroed
    allocation, which this writer requests from the allocator (buffer usage bit 0x80000000 is this
    module's private "zero-filled" request, honoured by HalModule below)."""
    imports = [Import(n, cc) for n, cc in _HAL_IMPORTS]
    index = {n: i for i, (n, _) in enumerate(_HAL_IMPORTS)}
    m = Module("module", types=["i32", "i64", "!hal.allocator", "!hal.buffer", "!hal.buffer_view", "!hal.command_buffer",
                                "!hal.device", "!hal.executable", "!hal.fence", "!vm.buffer"],
               dependencies=[("hal", 5)], imports=imports)
    m.rodata = [bytes(executable_def), b"PTXE"]
    if templates:
        m.rodata.append(bytes(templates))
    a = Assembler()
    views = {}
    for decl in plan.inputs:
        if "parameter" in decl:
            raise VmError("UNIMPLEMENTED", "parameter-backed inputs in the bytecode writer")
        views[decl["name"]] = a.ref()
    n_args = len(plan.inputs)

    def call(name, operands, results=()):
        a.call(index[name], list(operands), list(results))

    def variadic(name, segments, operands, results=()):
        a.call_variadic(index[name], list(segments), list(operands), list(results))

    zero32 = a.const_i32(0)
    device = a.ref()
    call("hal.devices.get", [zero32], [device])
    allocator = a.ref()
    call("hal.device.allocator", [device], [allocator])
    buffers = {}
    for decl in plan.inputs:
        shape_regs = [a.const_i64(d) for d in decl["shape"]]
        et = a.const_i32(_element_type(decl["dtype"]))
        enc = a.const_i32(ENCODING_DENSE_ROW_MAJOR)
        null = a.const_ref_zero()
        variadic("hal.buffer_view.assert", [1, 1, 1, 1, len(shape_regs)], [views[decl["name"]], null, et, enc] + shape_regs)
        buffers[decl["name"]] = a.ref()
        call("hal.buffer_view.buffer", [views[decl["name"]]], [buffers[decl["name"]]])
    any_affinity = a.const_i64(-1)
    device_local = a.const_i32(48)            # IREE_HAL_MEMORY_TYPE_DEVICE_LOCAL | optimal
    for decl in list(plan.outputs) + list(plan.transients):
        if decl.get("templates"):
            src = a.const_ref_rodata(2)
            off, length = a.const_i64(0), a.const_i64(len(templates))
            buffers[decl["name"]] = a.ref()
            usage = a.const_i32(3)
            call("hal.allocator.import", [allocator, zero32, any_affinity, device_local, usage, src, off, length], [buffers[decl["name"]]])
            continue
        nbytes = decl["bytes"] if "bytes" in decl else int(np.prod(decl["shape"])) * np.dtype(_np_dtype(decl["dtype"])).itemsize
        size = a.const_i64(max(nbytes, 1))
        usage = a.const_i32(3 | (0x40000000 if decl.get("zero") else 0))
        buffers[decl["name"]] = a.ref()
        call("hal.allocator.allocate", [allocator, any_affinity, device_local, usage, size], [buffers[decl["name"]]])
    # executable
    fmt, data, null = a.const_ref_rodata(1), a.const_ref_rodata(0), a.const_ref_zero()
    exe = a.ref()
    variadic("hal.executable.create", [1, 1, 1, 1, 0], [device, fmt, data, null], [exe])
    cb = a.ref()
    one = a.const_i32(1)
    three = a.const_i32(3)
    call("hal.command_buffer.create", [device, one, three, zero32], [cb])
    layout = a.const_ref_zero()
    for d in plan.dispatches:
        consts = [a.const_i32(c) for c in d.constants]
        variadic("hal.command_buffer.push_constants", [1, 1, 1, len(consts)], [cb, layout, zero32] + consts)
        operands = [cb, layout, zero32]
        zero64 = a.const_i64(0)
        whole = a.const_i64(-1)
        for slot, name in enumerate(d.bindings):
            operands += [a.const_i32(slot), zero32, buffers[name], zero64, whole]
        variadic("hal.command_buffer.push_descriptor_set", [1, 1, 1, len(d.bindings)], operands)
        entry = a.const_i32(export_ordinals[d.export])
        gx, gy, gz = (a.const_i32(g) for g in d.grid)
        call("hal.command_buffer.dispatch", [cb, exe, entry, gx, gy, gz])
        call("hal.command_buffer.execution_barrier", [cb, one, one, zero32])
    call("hal.command_buffer.finalize", [cb])
    fence = a.ref()
    call("hal.fence.create", [device, zero32], [fence])
    null = a.const_ref_zero()
    variadic("hal.device.queue.execute", [1, 1, 1, 1, 1], [device, any_affinity, null, fence, cb])
    status = a.i32()
    timeout = a.const_i32(-1)
    variadic("hal.fence.await", [1, 1], [timeout, fence], [status])
    outs = []
    for decl in plan.outputs:
        shape_regs = [a.const_i64(d) for d in decl["shape"]]
        et = a.const_i32(_element_type(decl["dtype"]))
        enc = a.const_i32(ENCODING_DENSE_ROW_MAJOR)
        zero64, whole = a.const_i64(0), a.const_i64(int(np.prod(decl["shape"])) * np.dtype(_np_dtype(decl["dtype"])).itemsize)
        v = a.ref()
        variadic("hal.buffer_view.create", [1, 1, 1, 1, 1, len(shape_regs)], [buffers[decl["name"]], zero64, whole, et, enc] + shape_regs, [v])
        outs.append(v)
    a.ret(outs)
    cc = "0" + ("r" * n_args or "v") + "_" + ("r" * len(outs) or "v")
    m.functions.append(a.function(plan.function, cc, argument_refs=n_args))
    return m


def _np_dtype(name: str):
    return {"f16": np.float16, "bf16": np.uint16, "i8": np.int8, "i32": np.int32, "f32": np.float32}[name]


def _element_type(name: str) -> int:
    return ELEMENT_TYPES[name]


# allocator.allocate with the writer's zero-fill request
_plain_allocate = HalModule.hal_allocator__allocate


def _allocate(self, allocator, queue_affinity, memory_types, buffer_usage, size):
    buf = _plain_allocate(self, allocator, queue_affinity, memory_types, buffer_usage, size)
    if buffer_usage & 0x40000000:
        buf.fill(0)
    return buf


HalModule.hal_allocator__allocate = _allocate


def export_ordinals(executable_def: bytes) -> Dict[str, int]:
    """Entry-point names of an ExecutableDef (cuda_executable_def.fbs: entry_points is field 0), in order."""
    root = vmfb.Table(executable_def, struct.unpack_from("<I", executable_def, 0)[0])
    start, n = root.vector(0)
    names = {}
    for i in range(n):
        at = start + 4 * i
        s = at + struct.unpack_from("<I", executable_def, at)[0]
        length = struct.unpack_from("<I", executable_def, s)[0]
        names[executable_def[s + 4:s + 4 + length].decode()] = i
    return names


def contraction_executable_def(cubin_path: str = None) -> bytes:
    from . import runtime as rt
    lib = rt.library()
    path = (cubin_path or rt.cubin_path()).encode()
    size = C.c_size_t()
    rt.check(lib.iree_b200_contraction_executable_def(path, None, C.c_size_t(0), C.byref(size)))
    out = C.create_string_buffer(size.value)
    rt.check(lib.iree_b200_contraction_executable_def(path, out, C.c_size_t(size.value), C.byref(size)))
    return out.raw[:size.value]


def run_vmfb(ctx, contents: bytes, function: str, inputs: List[np.ndarray]):
    """Loads a module, binds the HAL module, invokes `function` on host arrays, returns host arrays."""
    module = vmfb.read_module(contents)
    hal = HalModule(ctx)
    try:
        interp = Interpreter(module, hal.imports())
        views = []
        for arr in inputs:
            buf = ctx.to_device(np.ascontiguousarray(arr))
            hal.owned.append(buf)
            name = {np.dtype(np.float16): "f16", np.dtype(np.int8): "i8", np.dtype(np.int32): "i32",
                    np.dtype(np.float32): "f32", np.dtype(np.uint16): "bf16", np.dtype(np.uint8): "i8"}[arr.dtype]
            views.append(BufferView(buf, arr.shape, ELEMENT_TYPES[name]))
        results = interp.invoke(function or next(iter(interp.exports)), views)
        outs = []
        for v in results:
            dt = _np_dtype(ELEMENT_NAMES[v.element_type])
            outs.append(v.buffer.download(dt, tuple(v.shape)))
        return outs, hal.trace
    finally:
        hal.close()


def main(argv=None) -> int:
    """python -m iree_b200.vm --plan <benchmark plan name | plan.json> -o out.vmfb: writes the plan's host
    program as a bytecode module (tensor maps built on the device, the contraction cubin embedded)."""
    import argparse
    from . import dispatch_gen as dg, runtime as rt
    ap = argparse.ArgumentParser(prog="iree_b200.vm")
    ap.add_argument("--plan", required=True)
    ap.add_argument("-o", "--output", required=True)
    args = ap.parse_args(argv)
    plans = dg.baseline_plans()
    plan = plans[args.plan] if args.plan in plans else dg.Plan.from_json(open(args.plan).read())
    exe = contraction_executable_def()
    templates = b""
    for t in plan.transients:
        if t.get("templates") == "table":
            templates = bytes(template_table())
        elif t.get("templates"):
            row = {"f16": 0, "bf16": 1, "i8": 2}[t["templates"]]
            table = template_table()
            templates = bytes(table[128 * row:128 * row + 128]) * 2
        if "host_tensor_maps" in t:
            raise VmError("UNIMPLEMENTED", "plans whose tensor maps are encoded on the host have no bytecode form")
    open(args.output, "wb").write(vmfb.write_module(plan_to_module(plan, exe, export_ordinals(exe), templates), external_rodata=True))
    return 0


def template_table() -> bytes:
    """The six tensor-map templates, from the copy the compiler plugin embeds (no GPU needed)."""
    import os
    import re
    inc = open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "compiler_plugin", "src", "TensorMapTemplates.inc")).read()
    return bytes(int(x, 16) for x in re.findall(r"0x([0-9a-fA-F]{2})", inc))


if __name__ == "__main__":
    import sys
    sys.exit(main())
