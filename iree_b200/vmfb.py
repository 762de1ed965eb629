"""Reader and writer for IREE bytecode modules (`.vmfb`), and an assembler for the bytecode subset a
single-dispatch program needs.

File layout (runtime/src/iree/vm/bytecode/archive.c:60-140): an optional ZIP local-file header, a
32-bit size prefix, then a FlatBuffer with file identifier "IREE" whose root is `BytecodeModuleDef`
(runtime/src/iree/schemas/bytecode_module_def.fbs:232-298); read-only data may follow the
FlatBuffer, aligned to 64 bytes (`external_data_offset` is relative to that point).

Bytecode encoding (runtime/src/iree/vm/bytecode/dispatch_util.h:125-225, utils/isa.h:20-70):
one opcode byte (utils/generated/op_table.h), attributes little-endian inline, registers as 16-bit
ordinals (refs carry the type bit 0x8000 and the move bit 0x4000), register lists as a 16-bit count
followed by the ordinals, aligned to two bytes. Version 15.0.

Parity note: the reference holds no `.vmfb` fixture and its compiler cannot be built here, so this
reader has only met modules written by the writer below.
"""
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

BYTECODE_VERSION = (15 << 16) | 0      # isa.h:33-40, major in the upper half
SEGMENT_ALIGNMENT = 64                 # IREE_VM_ARCHIVE_SEGMENT_ALIGNMENT
ZIP_SIGNATURE = 0x04034B50

# utils/generated/op_table.h
OP = {"GlobalLoadRef": 0x08, "GlobalStoreRef": 0x09, "ConstI32Zero": 0x0C, "ConstI32": 0x0D, "ConstI64Zero": 0x0E,
      "ConstI64": 0x0F, "ConstRefZero": 0x10, "ConstRefRodata": 0x11, "CmpEQI32": 0x49, "CmpNEI32": 0x4A, "CmpNZI32": 0x4D,
      "Branch": 0x56, "CondBranch": 0x57, "Call": 0x58, "CallVariadic": 0x59, "Return": 0x5A, "Fail": 0x5B, "Block": 0x79}
OP_NAME = {v: k for k, v in OP.items()}
REF_TYPE_BIT, REF_MOVE_BIT, REF_MASK, I32_MASK = 0x8000, 0x4000, 0x3FFF, 0x7FFF


class VmfbError(ValueError):
    """Malformed module; `code` is the reference status it would be reported with."""

    def __init__(self, code: str, message: str):
        super().__init__("%s: %s" % (code, message))
        self.code = code


# ------------------------------------------------------------------------------------------------
# FlatBuffer reading (generic: tables through their vtables)
# ------------------------------------------------------------------------------------------------
class Table:
    def __init__(self, buf: bytes, pos: int):
        if pos < 0 or pos + 4 > len(buf):
            raise VmfbError("INVALID_ARGUMENT", "table offset out of bounds")
        self.buf, self.pos = buf, pos
        self.vt = pos - struct.unpack_from("<i", buf, pos)[0]
        if self.vt < 0 or self.vt + 4 > len(buf):
            raise VmfbError("INVALID_ARGUMENT", "vtable offset out of bounds")
        self.vt_size = struct.unpack_from("<H", buf, self.vt)[0]

    def _slot(self, field_id: int) -> int:
        o = 4 + 2 * field_id
        if o + 2 > self.vt_size:
            return 0
        return struct.unpack_from("<H", self.buf, self.vt + o)[0]

    def scalar(self, field_id: int, fmt: str, default=0):
        s = self._slot(field_id)
        return struct.unpack_from("<" + fmt, self.buf, self.pos + s)[0] if s else default

    def _indirect(self, field_id: int) -> Optional[int]:
        s = self._slot(field_id)
        if not s:
            return None
        at = self.pos + s
        target = at + struct.unpack_from("<I", self.buf, at)[0]
        if target + 4 > len(self.buf):
            raise VmfbError("INVALID_ARGUMENT", "offset out of bounds")
        return target

    def table(self, field_id: int) -> Optional["Table"]:
        t = self._indirect(field_id)
        return Table(self.buf, t) if t is not None else None

    def string(self, field_id: int) -> Optional[str]:
        t = self._indirect(field_id)
        if t is None:
            return None
        n = struct.unpack_from("<I", self.buf, t)[0]
        return self.buf[t + 4:t + 4 + n].decode("utf-8")

    def vector(self, field_id: int) -> Tuple[int, int]:
        """(position of element 0, element count); (0, 0) when absent."""
        t = self._indirect(field_id)
        if t is None:
            return 0, 0
        return t + 4, struct.unpack_from("<I", self.buf, t)[0]

    def tables(self, field_id: int) -> List["Table"]:
        start, n = self.vector(field_id)
        out = []
        for i in range(n):
            at = start + 4 * i
            out.append(Table(self.buf, at + struct.unpack_from("<I", self.buf, at)[0]))
        return out

    def bytes_(self, field_id: int) -> Optional[bytes]:
        start, n = self.vector(field_id)
        if not start:
            return None
        if start + n > len(self.buf):
            raise VmfbError("INVALID_ARGUMENT", "byte vector out of bounds")
        return bytes(self.buf[start:start + n])


# ------------------------------------------------------------------------------------------------
# FlatBuffer writing: a table is written first and its children after it (offsets point forward)
# ------------------------------------------------------------------------------------------------
_SCALAR = {"u8": ("B", 1), "i16": ("h", 2), "u16": ("H", 2), "i32": ("i", 4), "u32": ("I", 4), "u64": ("Q", 8)}


class Builder:
    def __init__(self):
        self.b = bytearray()

    def _align(self, n: int):
        while len(self.b) % n:
            self.b.append(0)

    def table(self, fields: Dict[int, Tuple[str, object]]) -> int:
        """fields: id -> (kind, value); kinds: scalars of _SCALAR, "str", "bytes" (value: (data, alignment)),
        "structs" (value: (data, count, alignment)), "table" (value: fields), "tables" (value: [fields])."""
        fields = {k: v for k, v in fields.items() if v[1] is not None}
        count = (max(fields) + 1) if fields else 0
        off, slots, big = 4, {}, 4
        for fid in sorted(fields):
            size = _SCALAR[fields[fid][0]][1] if fields[fid][0] in _SCALAR else 4
            off = (off + size - 1) // size * size
            slots[fid] = off
            off += size
            big = max(big, size)
        vt_size = 4 + 2 * count
        self._align(2)
        while (len(self.b) + vt_size) % big:
            self.b += b"\0\0"
        vt = len(self.b)
        self.b += struct.pack("<HH", vt_size, off)
        for fid in range(count):
            self.b += struct.pack("<H", slots.get(fid, 0))
        pos = len(self.b)
        self.b += struct.pack("<i", pos - vt) + bytes(off - 4)
        pending = []
        for fid, (kind, value) in fields.items():
            if kind in _SCALAR:
                struct.pack_into("<" + _SCALAR[kind][0], self.b, pos + slots[fid], value)
            else:
                pending.append((pos + slots[fid], kind, value))
        for at, kind, value in pending:
            target = self._child(kind, value)
            struct.pack_into("<I", self.b, at, target - at)
        return pos

    def _child(self, kind: str, value) -> int:
        if kind == "str":
            self._align(4)
            pos = len(self.b)
            data = value.encode("utf-8")
            self.b += struct.pack("<I", len(data)) + data + b"\0"
            return pos
        if kind in ("bytes", "structs"):
            data, count, alignment = (value[0], len(value[0]), value[1]) if kind == "bytes" else value
            self._align(4)
            while (len(self.b) + 4) % alignment:
                self.b += bytes(4)
            pos = len(self.b)
            self.b += struct.pack("<I", count) + bytes(data)
            return pos
        if kind == "table":
            return self.table(value)
        if kind == "tables":
            self._align(4)
            pos = len(self.b)
            self.b += struct.pack("<I", len(value)) + bytes(4 * len(value))
            for i, fields in enumerate(value):
                at = pos + 4 + 4 * i
                struct.pack_into("<I", self.b, at, self.table(fields) - at)
            return pos
        raise ValueError(kind)


# ------------------------------------------------------------------------------------------------
# The module
# ------------------------------------------------------------------------------------------------
@dataclass
class Import:
    full_name: str
    calling_convention: str        # e.g. "0rriCiD_v" (iree/vm/module.h)
    optional: bool = False


@dataclass
class Function:
    name: str                      # exported name ("" for internal-only functions)
    calling_convention: str
    bytecode: bytes
    i32_registers: int
    ref_registers: int
    blocks: int = 1


@dataclass
class Module:
    name: str
    version: int = 0
    types: List[str] = field(default_factory=list)
    dependencies: List[Tuple[str, int]] = field(default_factory=list)     # (module, minimum version)
    imports: List[Import] = field(default_factory=list)
    functions: List[Function] = field(default_factory=list)
    rodata: List[bytes] = field(default_factory=list)
    global_bytes: int = 0
    global_refs: int = 0
    bytecode_version: int = BYTECODE_VERSION


_FUNCTION_DESCRIPTOR = struct.Struct("<iiIhhhh")   # offset, length, requirements, reserved, blocks, i32 regs, ref regs


def write_module(m: Module, external_rodata: bool = False) -> bytes:
    """Serialises the module. With external_rodata the segments follow the FlatBuffer (64-byte
    aligned) instead of being embedded in it, as the compiler does for large constants."""
    code = bytearray()
    descriptors = bytearray()
    for f in m.functions:
        while len(code) % 8:
            code.append(0)
        descriptors += _FUNCTION_DESCRIPTOR.pack(len(code), len(f.bytecode), 0, 0, f.blocks, f.i32_registers, f.ref_registers)
        code += f.bytecode
    tail = bytearray()
    segments = []
    for data in m.rodata:
        if external_rodata:
            while len(tail) % SEGMENT_ALIGNMENT:
                tail.append(0)
            segments.append({3: ("u64", len(tail)), 4: ("u64", len(data))})
            tail += data
        else:
            segments.append({2: ("bytes", (data, SEGMENT_ALIGNMENT))})
    exported = [(i, f) for i, f in enumerate(m.functions) if f.name]
    root = {
        0: ("str", m.name),
        1: ("u32", m.version),
        4: ("tables", [{0: ("str", t)} for t in m.types]),
        5: ("tables", [{0: ("str", n), 1: ("u32", v)} for n, v in m.dependencies]),
        6: ("tables", [{0: ("str", i.full_name), 1: ("table", {0: ("str", i.calling_convention)}),
                        2: ("u32", 2 if i.optional else 1)} for i in m.imports]),
        7: ("tables", [{0: ("str", f.name), 1: ("i32", i)} for i, f in exported]),
        8: ("tables", [{0: ("str", f.calling_convention)} for f in m.functions]),
        9: ("tables", segments),
        11: ("table", {0: ("i32", m.global_bytes), 1: ("i32", m.global_refs)}),
        12: ("structs", (descriptors, len(m.functions), 4)),
        13: ("u32", m.bytecode_version),
        14: ("bytes", (code, 8)),
    }
    b = Builder()
    b.b += bytes(4) + b"IREE"
    struct.pack_into("<I", b.b, 0, b.table(root))
    flat = bytes(b.b)
    out = bytearray(struct.pack("<I", len(flat)) + flat)
    if tail:
        while len(out) % SEGMENT_ALIGNMENT:
            out.append(0)
        out += tail
    return bytes(out)


def read_module(contents: bytes) -> Module:
    """Parses a `.vmfb`; raises VmfbError with the status the reference's loader would give
    (runtime/src/iree/vm/bytecode/archive.c:60-140, verifier.c)."""
    base = 0
    if len(contents) >= 30 and struct.unpack_from("<I", contents, 0)[0] == ZIP_SIGNATURE:
        name_len, extra_len = struct.unpack_from("<HH", contents, 26)
        base = 30 + name_len + extra_len
        if base > len(contents):
            raise VmfbError("INVALID_ARGUMENT", "archive self-reports as a zip but does not have enough data to contain a module")
    if len(contents) - base < 16:
        raise VmfbError("INVALID_ARGUMENT", "FlatBuffer data is not present or less than 16 bytes")
    prefix = struct.unpack_from("<I", contents, base)[0]
    if prefix > len(contents) - base - 4:
        raise VmfbError("INVALID_ARGUMENT", "FlatBuffer length prefix out of bounds")
    flat = contents[base + 4:base + 4 + prefix]
    if flat[4:8] != b"IREE":
        raise VmfbError("INVALID_ARGUMENT", "FlatBuffer file identifier is not IREE")
    rodata_base = (base + 4 + prefix + SEGMENT_ALIGNMENT - 1) // SEGMENT_ALIGNMENT * SEGMENT_ALIGNMENT
    root = Table(flat, struct.unpack_from("<I", flat, 0)[0])
    name = root.string(0)
    if not name:
        raise VmfbError("INVALID_ARGUMENT", "module name missing")
    version = root.scalar(13, "I")
    if version >> 16 != BYTECODE_VERSION >> 16 or (version & 0xffff) > (BYTECODE_VERSION & 0xffff):
        raise VmfbError("INVALID_ARGUMENT", "bytecode version %d.%d is not supported (runtime is %d.%d)" % (
            version >> 16, version & 0xffff, BYTECODE_VERSION >> 16, BYTECODE_VERSION & 0xffff))
    m = Module(name, root.scalar(1, "I"), bytecode_version=version)
    m.types = [t.string(0) for t in root.tables(4)]
    m.dependencies = [(t.string(0), t.scalar(1, "I")) for t in root.tables(5)]
    for t in root.tables(6):
        sig = t.table(1)
        m.imports.append(Import(t.string(0), sig.string(0) if sig else "", t.scalar(2, "I", 1) == 2))
    state = root.table(11)
    if state:
        m.global_bytes, m.global_refs = state.scalar(0, "i"), state.scalar(1, "i")
    for seg in root.tables(9):
        data = seg.bytes_(2)
        if data is None:
            off, n = seg.scalar(3, "Q"), seg.scalar(4, "Q")
            if rodata_base + off + n > len(contents):
                raise VmfbError("OUT_OF_RANGE", "rodata segment lies outside the archive")
            data = bytes(contents[rodata_base + off:rodata_base + off + n])
        m.rodata.append(data)
    code = root.bytes_(14) or b""
    signatures = [t.string(0) or "" for t in root.tables(8)]
    start, count = root.vector(12)
    if count != len(signatures):
        raise VmfbError("INVALID_ARGUMENT", "function signatures and descriptors differ in count")
    exported = {t.scalar(1, "i"): t.string(0) for t in root.tables(7)}
    for i in range(count):
        off, n, _req, _res, blocks, i32s, refs = _FUNCTION_DESCRIPTOR.unpack_from(flat, start + i * _FUNCTION_DESCRIPTOR.size)
        if off < 0 or n < 0 or off + n > len(code):
            raise VmfbError("OUT_OF_RANGE", "function %d bytecode lies outside the bytecode data" % i)
        m.functions.append(Function(exported.get(i, ""), signatures[i], bytes(code[off:off + n]), i32s, refs, blocks))
    return m


# ------------------------------------------------------------------------------------------------
# Assembler
# ------------------------------------------------------------------------------------------------
class Assembler:
    """Emits bytecode for one function. i32 registers are plain ordinals (an i64 lives in the even
    pair r, r + 1); ref registers are written with the type bit."""

    def __init__(self):
        self.code = bytearray([OP["Block"]])
        self.blocks = 1
        self.i32_top = 0
        self.ref_top = 0

    def i32(self) -> int:
        r = self.i32_top
        self.i32_top += 1
        return r

    def i64(self) -> int:
        self.i32_top = (self.i32_top + 1) & ~1
        r = self.i32_top
        self.i32_top += 2
        return r

    def ref(self) -> int:
        r = self.ref_top
        self.ref_top += 1
        return r | REF_TYPE_BIT

    def _regs(self, regs):
        if len(self.code) % 2:
            self.code.append(0)
        self.code += struct.pack("<H", len(regs)) + b"".join(struct.pack("<H", r) for r in regs)

    def const_i32(self, value: int) -> int:
        r = self.i32()
        if value == 0:
            self.code += bytes([OP["ConstI32Zero"]]) + struct.pack("<H", r)
        else:
            self.code += bytes([OP["ConstI32"]]) + struct.pack("<iH", value, r)
        return r

    def const_i64(self, value: int) -> int:
        r = self.i64()
        if value == 0:
            self.code += bytes([OP["ConstI64Zero"]]) + struct.pack("<H", r)
        else:
            self.code += bytes([OP["ConstI64"]]) + struct.pack("<qH", value, r)
        return r

    def const_ref_zero(self) -> int:
        r = self.ref()
        self.code += bytes([OP["ConstRefZero"]]) + struct.pack("<H", r)
        return r

    def const_ref_rodata(self, ordinal: int) -> int:
        r = self.ref()
        self.code += bytes([OP["ConstRefRodata"]]) + struct.pack("<iH", ordinal, r)
        return r

    def call(self, import_ordinal: int, operands, results) -> None:
        self.code += bytes([OP["Call"]]) + struct.pack("<I", 0x80000000 | import_ordinal)
        self._regs(operands)
        self._regs(results)

    def call_variadic(self, import_ordinal: int, segment_sizes, operands, results) -> None:
        self.code += bytes([OP["CallVariadic"]]) + struct.pack("<I", 0x80000000 | import_ordinal)
        self._regs(segment_sizes)       # sizes themselves, not registers (dispatch.c:391-395)
        self._regs(operands)
        self._regs(results)

    def ret(self, operands) -> None:
        self.code += bytes([OP["Return"]])
        self._regs(operands)

    def function(self, name: str, calling_convention: str, argument_i32: int = 0, argument_refs: int = 0) -> Function:
        return Function(name, calling_convention, bytes(self.code), max(self.i32_top, argument_i32, 1),
                        max(self.ref_top, argument_refs, 1), self.blocks)
