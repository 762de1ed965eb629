"""Parameter archives (.irpa): the parser and writer against the reference's format.

Expected offsets, lengths and patterns are those of the reference's own parser test
(runtime/src/iree/io/formats/irpa/irpa_parser_test.cc:38-170) for archives built from the same
flag lists (testdata/generate_irpa_files.sh). When the reference checkout is present its own
fixture files are parsed too and re-written: the writer reproduces them byte for byte.
"""
import os
import struct

import numpy as np
import pytest

from iree_b200 import parameters as P
from iree_b200 import runtime as rt

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "irpa")
# same variable and default as oracle/Makefile
REFERENCE = os.path.join(os.environ.get("REFERENCE", "/root/reference"), "runtime/src/iree/io/formats/irpa/testdata")


def check_fixture(name, index, value_bytes=True):
    keys = [index[i].key for i in range(len(index))]
    if name == "empty":
        assert keys == []
    elif name == "single":
        assert keys == ["key0"]
        e = index.lookup("key0")
        assert (e.storage_type, e.file_offset, e.length, e.metadata) == (P.STORAGE_FILE, 192, 16, b"")
    elif name == "multiple":
        assert keys == ["key0", "key1"]
        e0, e1 = index.lookup("key0"), index.lookup("key1")
        assert (e0.storage_type, e0.file_offset, e0.length) == (P.STORAGE_FILE, 320, 16)
        assert (e1.storage_type, e1.file_offset, e1.length) == (P.STORAGE_FILE, 384, 5)
        assert (index.read("key1", np.int8) == 101).all()
    else:
        assert keys == ["key2", "key3", "key0", "key1"]          # splats are declared first
        e0, e1, e2, e3 = (index.lookup(k) for k in ("key0", "key1", "key2", "key3"))
        assert (e0.file_offset, e0.length, e1.file_offset, e1.length) == (512, 16, 576, 5)
        assert (e2.storage_type, e2.pattern, e2.length) == (P.STORAGE_SPLAT, bytes([102]), 1)
        assert (e3.storage_type, len(e3.pattern), e3.length) == (P.STORAGE_SPLAT, 8, 33554432)
        if value_bytes:
            assert e3.pattern == struct.pack("<q", 103)
            assert (index.read("key3", np.int64, shape=(1000,), offset=8 * 12345) == 103).all()
    with pytest.raises(rt.IreeB200Error) as err:
        index.lookup("missing")
    assert err.value.code_name == "NOT_FOUND"


@pytest.mark.parametrize("name", ["empty", "single", "multiple", "mixed"])
def test_committed_fixtures_parse_like_the_reference_parser_test(built, name):
    index = P.ParameterIndex(os.path.join(GOLDEN, name + ".irpa"))
    check_fixture(name, index)
    index.close()


@pytest.mark.parametrize("name", ["empty", "single", "multiple", "mixed"])
def test_reference_fixture_files_parse_and_are_reproduced_byte_for_byte(built, name, tmp_path):
    path = os.path.join(REFERENCE, name + ".irpa")
    if not os.path.exists(path):
        pytest.skip("reference checkout not present")
    index = P.ParameterIndex(path)
    check_fixture(name, index, value_bytes=False)   # the splat value bytes of that file are the tool's, not the format's
    entries = []
    for i in range(len(index)):
        e = index[i]
        if e.storage_type == P.STORAGE_SPLAT:
            entries.append({"key": e.key, "splat": e.pattern, "length": e.length})
        else:
            entries.append({"key": e.key, "data": index.read(e.key)})
    out = str(tmp_path / "again.irpa")
    P.write_archive(out, entries)
    assert open(out, "rb").read() == open(path, "rb").read()
    index.close()


def test_create_parameters_command_line_matches_the_reference_tool(built, tmp_path):
    """The fixture whose value bytes do not depend on the tool's number parsing."""
    ref = os.path.join(REFERENCE, "multiple.irpa")
    out = str(tmp_path / "multiple.irpa")
    assert P.main(["--quiet", "--output=" + out, "--data=key0=4xf32=100.1", "--data=key1=5xi8=101"]) == 0
    assert open(out, "rb").read() == open(os.path.join(GOLDEN, "multiple.irpa"), "rb").read()
    if os.path.exists(ref):
        assert open(out, "rb").read() == open(ref, "rb").read()


def test_data_round_trip_metadata_and_alignment(built, tmp_path):
    rng = np.random.default_rng(0)
    w = rng.integers(0, 256, (48, 100), dtype=np.uint8)
    s = rng.standard_normal((48, 3)).astype(np.float16)
    out = str(tmp_path / "model.irpa")
    P.write_archive(out, [{"key": "blk.0.wq", "data": w, "metadata": b"{\"shape\":[48,100]}"},
                          {"key": "blk.0.scales", "data": s, "alignment": 256},
                          {"key": "blk.0.zero", "splat": b"\x00\x3c", "length": 2 * 77}])
    index = P.ParameterIndex(out)
    assert len(index) == 3
    e = index.lookup("blk.0.wq")
    assert e.metadata == b"{\"shape\":[48,100]}" and e.length == w.nbytes and e.file_offset % 64 == 0
    assert np.array_equal(index.read("blk.0.wq", np.uint8, w.shape), w)
    assert np.array_equal(index.read("blk.0.scales", np.float16, s.shape), s)
    # alignment is relative to the storage segment, which starts at the first data entry (irpa_builder.c:289-300)
    assert (index.lookup("blk.0.scales").file_offset - e.file_offset) % 256 == 0
    assert (index.read("blk.0.zero", np.float16) == 1.0).all()
    assert np.array_equal(index.read("blk.0.wq", np.uint8, (100,), offset=100), w[1])      # ranged read
    with pytest.raises(rt.IreeB200Error) as err:
        index.read("blk.0.wq", np.uint8, (101,), offset=w.nbytes - 100)
    assert err.value.code_name == "OUT_OF_RANGE"
    index.close()


def test_header_chain(built, tmp_path):
    """Archives can be concatenated: next_header_offset links them (parameter_archive.h:84-87)."""
    a, b = str(tmp_path / "a.irpa"), str(tmp_path / "b.irpa")
    P.write_archive(a, [{"key": "first", "data": np.arange(10, dtype=np.int32)}])
    P.write_archive(b, [{"key": "second", "data": np.arange(7, dtype=np.int16)}, {"key": "third", "splat": b"\x07", "length": 9}])
    blob_a, blob_b = bytearray(open(a, "rb").read()), open(b, "rb").read()
    struct.pack_into("<Q", blob_a, 16, len(blob_a))          # next_header_offset of the first header
    index = P.ParameterIndex(data=bytes(blob_a) + blob_b)
    assert [index[i].key for i in range(len(index))] == ["first", "second", "third"]
    assert np.array_equal(index.read("first", np.int32), np.arange(10))
    assert np.array_equal(index.read("second", np.int16), np.arange(7))
    assert index.lookup("second").file_offset >= len(blob_a)
    index.close()


def test_parser_rejects_what_the_reference_rejects(built):
    good = bytearray(open(os.path.join(GOLDEN, "multiple.irpa"), "rb").read())

    def code(blob):
        with pytest.raises(rt.IreeB200Error) as err:
            P.ParameterIndex(data=bytes(blob))
        return err.value.code_name

    assert code(b"") == "INVALID_ARGUMENT"                                    # irpa_parser.c:268-272
    assert code(b"GGUF" + bytes(60)) == "INVALID_ARGUMENT"                    # magic, :276-281
    bad = bytearray(good); struct.pack_into("<H", bad, 4, 1)
    assert code(bad) == "UNIMPLEMENTED"                                       # major version, :309-313
    bad = bytearray(good); struct.pack_into("<H", bad, 6, 1)
    assert code(bad) == "UNIMPLEMENTED"                                       # newer minor, :163-168
    bad = bytearray(good); struct.pack_into("<Q", bad, 8, 96)
    assert code(bad) == "INVALID_ARGUMENT"                                    # header size, :171-175
    assert code(good[:60]) == "OUT_OF_RANGE"                                  # header underrun, :282-287
    bad = bytearray(good); struct.pack_into("<Q", bad, 40 + 8, 1 << 40)
    assert code(bad) == "OUT_OF_RANGE"                                        # entry segment beyond the file
    bad = bytearray(good); struct.pack_into("<Q", bad, 32, 50)
    assert code(bad) == "OUT_OF_RANGE"                                        # more entries than the table holds
    bad = bytearray(good); struct.pack_into("<I", bad, 96 + 8, 3)
    assert code(bad) == "UNIMPLEMENTED"                                       # external entries, :253-256
    bad = bytearray(good); struct.pack_into("<Q", bad, 96 + 20, 4000)
    assert code(bad) == "OUT_OF_RANGE"                                        # name outside the metadata segment
    skipped = bytearray(good); struct.pack_into("<I", skipped, 96 + 8, 0)
    index = P.ParameterIndex(data=bytes(skipped))                             # SKIP entries vanish, :246-247
    assert [index[i].key for i in range(len(index))] == ["key1"]
    index.close()


def test_writer_argument_errors(built, tmp_path):
    with pytest.raises(rt.IreeB200Error) as err:
        P.write_archive(str(tmp_path / "x.irpa"), [{"key": "k", "splat": b"\x01\x02\x03", "length": 9}])
    assert err.value.code_name == "INVALID_ARGUMENT"                          # irpa_builder.c:241-248
    with pytest.raises(rt.IreeB200Error):
        P.parse_parameter_flag("k=4xi4=1")


@pytest.mark.gpu
def test_parameters_reach_device_memory(ctx, tmp_path):
    rng = np.random.default_rng(1)
    w = rng.integers(0, 256, (1 << 21) + 13, dtype=np.uint8)
    out = str(tmp_path / "w.irpa")
    P.write_archive(out, [{"key": "w", "data": w}, {"key": "ones", "splat": np.float32(1.0).tobytes(), "length": 4 * 700001},
                          {"key": "bytes", "splat": b"\x5a", "length": 1000}])
    index = P.ParameterIndex(out)
    dw, do, db = ctx.alloc(w.nbytes), ctx.alloc(4 * 700001), ctx.alloc(1000)
    index.load(ctx, "w", dw)
    index.load(ctx, "ones", do)
    index.load(ctx, "bytes", db)
    assert np.array_equal(dw.download(np.uint8, w.shape), w)
    assert (do.download(np.float32, (700001,)) == 1.0).all()
    assert (db.download(np.uint8, (1000,)) == 0x5a).all()
    index.load(ctx, "w", dw, length=4096, offset=8192)                       # ranged load
    assert np.array_equal(dw.download(np.uint8, (4096,)), w[8192:8192 + 4096])
    index.close()
    for b in (dw, do, db):
        b.free()


@pytest.mark.gpu
def test_run_module_takes_weights_from_a_parameter_archive(ctx, tmp_path):
    """A W4A16 plan whose weights and scales are program parameters: the run-module front end loads
    them from `--parameters=model=...` and only the activations arrive as `--input`."""
    import oracle
    from iree_b200 import dispatch_gen as dg
    from iree_b200 import run_module, workloads
    M, N, K = 8, 256, 1024
    a, wq, s = workloads.c4_w4a16(M, N=N, K=K, seed=5)
    archive = str(tmp_path / "model.irpa")
    P.write_archive(archive, [{"key": "blk.0.wq", "data": wq}, {"key": "blk.0.scales", "data": s}])
    plan = dg.plan_w4a16("decode", M, N, K).bind_parameters({"wq": "model::blk.0.wq", "scales": "model::blk.0.scales"})
    index = P.ParameterIndex(archive)
    (out,) = run_module.execute_plan(ctx, plan, [a], {"model": index})
    want = oracle.w4a16(a, wq, s)
    assert np.allclose(out.astype(np.float32), want.astype(np.float32), rtol=1e-2, atol=1e-2)
    with pytest.raises(rt.IreeB200Error) as err:
        run_module.execute_plan(ctx, plan, [a], {})
    assert err.value.code_name == "NOT_FOUND"
    index.close()
    # the command line
    plan_path, a_path, out_path = str(tmp_path / "plan.json"), str(tmp_path / "a.npy"), str(tmp_path / "out.npy")
    open(plan_path, "w").write(plan.to_json())
    np.save(a_path, a)
    rc = run_module.main(["--device=cuda", "--module=" + plan_path, "--function=decode", "--parameters=model=" + archive,
                          "--input=%dx%dxf16=@%s" % (M, K, a_path), "--output=@" + out_path])
    assert rc == 0
    assert np.array_equal(np.load(out_path).view(np.uint16), out.view(np.uint16))
