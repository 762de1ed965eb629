"""Parameter archives (.irpa): Python face of ``iree_b200_parameter_*`` plus the command line of the
reference's ``iree-create-parameters`` tool (tools/iree-create-parameters-main.c).

    python -m iree_b200.parameters --output=weights.irpa --data=key0=4xf32=100.1 --splat=key2=i8=102
"""
from __future__ import annotations

import argparse
import ctypes as C
import sys
from typing import Dict, List, Optional

import numpy as np

from . import runtime as rt

STORAGE_SPLAT, STORAGE_FILE = 0, 1


class _Entry(C.Structure):
    _fields_ = [("key", C.c_void_p), ("key_length", C.c_uint64), ("metadata", C.c_void_p), ("metadata_length", C.c_uint64),
                ("length", C.c_uint64), ("storage_type", C.c_int32), ("pattern_length", C.c_uint8),
                ("pattern", C.c_uint8 * 16), ("file_offset", C.c_uint64)]


class _Source(C.Structure):
    _fields_ = [("key", C.c_char_p), ("metadata", C.c_void_p), ("metadata_length", C.c_uint64), ("storage_type", C.c_int32),
                ("length", C.c_uint64), ("data", C.c_void_p), ("pattern_length", C.c_uint8), ("pattern", C.c_uint8 * 16),
                ("alignment", C.c_uint64)]


class Entry:
    def __init__(self, raw: _Entry):
        self.key = C.string_at(raw.key, raw.key_length).decode()
        self.metadata = C.string_at(raw.metadata, raw.metadata_length) if raw.metadata_length else b""
        self.length = int(raw.length)
        self.storage_type = int(raw.storage_type)
        self.pattern = bytes(raw.pattern[:raw.pattern_length])
        self.file_offset = int(raw.file_offset)

    def __repr__(self):
        where = "splat %s" % self.pattern.hex() if self.storage_type == STORAGE_SPLAT else "file @%d" % self.file_offset
        return "<parameter %s: %d bytes, %s>" % (self.key, self.length, where)


class ParameterIndex:
    """An indexed archive (iree_io_parameter_index_t populated by iree_io_parse_irpa_index)."""

    def __init__(self, path: Optional[str] = None, data: Optional[bytes] = None):
        lib = rt.library()
        lib.iree_b200_parameter_index_count.restype = C.c_int64
        h = C.c_void_p()
        if path is not None:
            rt.check(lib.iree_b200_parameter_index_open(path.encode(), C.byref(h)))
        else:
            self._keep = C.create_string_buffer(data, len(data))
            rt.check(lib.iree_b200_parameter_index_parse(self._keep, C.c_size_t(len(data)), C.byref(h)))
        self.handle = h

    def close(self) -> None:
        if self.handle:
            rt.library().iree_b200_parameter_index_release(self.handle)
            self.handle = None

    def __len__(self) -> int:
        return int(rt.library().iree_b200_parameter_index_count(self.handle))

    def __getitem__(self, i: int) -> Entry:
        raw = _Entry()
        rt.check(rt.library().iree_b200_parameter_index_get(self.handle, C.c_int64(i), C.byref(raw)))
        return Entry(raw)

    def lookup(self, key: str) -> Entry:
        raw = _Entry()
        rt.check(rt.library().iree_b200_parameter_index_lookup(self.handle, key.encode(), C.byref(raw)))
        return Entry(raw)

    def read(self, key: str, dtype=np.uint8, shape=None, offset: int = 0) -> np.ndarray:
        """The parameter's bytes as a host array (splats expanded)."""
        e = self.lookup(key)
        n = e.length - offset if shape is None else int(np.prod(shape)) * np.dtype(dtype).itemsize
        out = np.empty(n, np.uint8)
        rt.check(rt.library().iree_b200_parameter_read(self.handle, key.encode(), C.c_uint64(offset), rt._vp(out),
                                                       C.c_uint64(n)))
        out = out.view(dtype)
        return out if shape is None else out.reshape(shape)

    def load(self, ctx: rt.Context, key: str, device_buffer, length: Optional[int] = None, offset: int = 0) -> None:
        """Parameter bytes [offset, offset + length) into device memory."""
        if length is None:
            length = self.lookup(key).length - offset
        rt.check(rt.library().iree_b200_parameter_load(ctx.handle, self.handle, key.encode(), C.c_uint64(offset),
                                                       rt._vp(device_buffer), C.c_uint64(length)))


def write_archive(path: str, entries: List[dict]) -> None:
    """entries: dicts with ``key`` and either ``data`` (ndarray / bytes) or ``splat`` (pattern bytes) +
    ``length``; optional ``metadata`` (bytes), ``alignment``; a data entry may give ``pattern`` +
    ``length`` instead of ``data``. Written in the order given."""
    arr = (_Source * len(entries))()
    keep = []
    for i, e in enumerate(entries):
        s = arr[i]
        s.key = e["key"].encode()
        md = e.get("metadata", b"")
        if md:
            buf = C.create_string_buffer(md, len(md))
            keep.append(buf)
            s.metadata, s.metadata_length = C.cast(buf, C.c_void_p), len(md)
        if "splat" in e:
            s.storage_type, s.length = STORAGE_SPLAT, int(e["length"])
            pat = bytes(e["splat"])
            s.pattern_length = len(pat)
            for j, b in enumerate(pat[:16]):
                s.pattern[j] = b
        else:
            s.storage_type = STORAGE_FILE
            s.alignment = int(e.get("alignment", 0))
            if "data" in e:
                data = np.ascontiguousarray(e["data"]).view(np.uint8).reshape(-1) if isinstance(e["data"], np.ndarray) \
                    else np.frombuffer(bytes(e["data"]), np.uint8)
                keep.append(data)
                s.data, s.length = data.ctypes.data, data.nbytes
            else:
                s.length = int(e["length"])
                pat = bytes(e.get("pattern", b""))
                s.pattern_length = len(pat)
                for j, b in enumerate(pat[:16]):
                    s.pattern[j] = b
    rt.check(rt.library().iree_b200_parameter_archive_write(path.encode(), C.c_int64(len(entries)), arr))


# ---- iree-create-parameters ---------------------------------------------------------------------------
_TYPES = {"i8": np.int8, "si8": np.int8, "ui8": np.uint8, "i16": np.int16, "si16": np.int16, "ui16": np.uint16,
          "i32": np.int32, "si32": np.int32, "ui32": np.uint32, "i64": np.int64, "si64": np.int64, "ui64": np.uint64,
          "f16": np.float16, "f32": np.float32, "f64": np.float64}


def parse_parameter_flag(text: str):
    """``name=shapextype=pattern`` -> (name, byte length, pattern bytes); an empty pattern means one
    zero byte (tools/iree-create-parameters-main.c:61-108)."""
    name, _, spec = text.partition("=")
    shape_type, _, contents = spec.partition("=")
    parts = shape_type.split("x")
    if parts[-1] == "bf16":
        dtype, bf16 = np.dtype(np.uint16), True
    elif parts[-1] in _TYPES:
        dtype, bf16 = np.dtype(_TYPES[parts[-1]]), False
    else:
        raise rt.IreeB200Error(3, "opaque and sub-byte aligned element types cannot currently be used as splats; "
                                  "use a bitcast type (2xi4=1xi8, etc)")
    count = 1
    for p in parts[:-1]:
        count *= int(p)
    if not contents:
        pattern = b"\x00"
    elif bf16:
        pattern = (np.array([float(contents)], np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
    elif dtype.kind == "f":
        pattern = np.array([float(contents)], dtype).tobytes()
    else:
        pattern = np.array([int(contents, 0)]).astype(dtype).tobytes()
    return name, count * dtype.itemsize, pattern


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="iree_b200.parameters", allow_abbrev=False,
                                 description="Creates IREE Parameter Archive (.irpa) files.")
    ap.add_argument("--splat", action="append", default=[], help="name=shapextype=pattern; no storage on disk")
    ap.add_argument("--data", action="append", default=[], help="name=shapextype=pattern; storage filled with the pattern")
    ap.add_argument("--alignment", type=int, default=64)
    ap.add_argument("--quiet", action="store_true")
    ap.add_argument("--output", required=True)
    args = ap.parse_args(argv)
    entries = []
    for text in args.splat:      # splats are declared first, then data, as the reference tool does
        name, length, pattern = parse_parameter_flag(text)
        entries.append({"key": name, "splat": pattern, "length": length})
    for text in args.data:
        name, length, pattern = parse_parameter_flag(text)
        entries.append({"key": name, "length": length, "pattern": pattern, "alignment": args.alignment})
    write_archive(args.output, entries)
    if not args.quiet:
        index = ParameterIndex(args.output)
        for i in range(len(index)):
            print(index[i])
        index.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
