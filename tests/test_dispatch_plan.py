"""The host plans (which exports run, with which bindings / constants / grids) that restate the
compiler plugin's lowering, and the iree-run-module-shaped CLI over them."""
import json
import os
import re

import numpy as np
import pytest

from iree_b200 import dispatch_gen as dg
from iree_b200 import run_module, workloads

ROOT = os.path.dirname(os.path.dirname(__file__))


def test_baseline_plans_pick_the_expected_exports():
    p = dg.baseline_plans()
    # 4096^3 has enough 256 x 256 tiles for the SM pairs: the CTA-pair exports, half-width right-hand boxes
    assert [d.export for d in p["c2_f16_4096"].dispatches] == ["b200_encode_tensormaps", "b200_matmul_pair_f16_f16"]
    assert p["c2_f16_4096"].dispatches[0].constants == [4096, 4096, 4096, 1, 0, 128, 2]
    gemm = p["c2_f16_4096"].dispatches[1]
    assert gemm.bindings == ["out", "workspace"] and gemm.constants == [4096, 4096, 4096, 1, 0, 256]
    assert gemm.grid == (148, 1, 1) and gemm.block == (256, 1, 1) and gemm.shared_memory == 230656
    assert [d.export for d in p["c2_f16_bmm"].dispatches] == ["b200_encode_tensormaps", "b200_matmul_f16_f16"]
    assert p["c3_w8a8_m4096"].dispatches[1].export == "b200_matmul_pair_i8_requant_f16"
    assert p["c1_i8_1024"].dispatches[1].export == "b200_matmul_i8_i32"
    assert p["c1_i8_1024"].dispatches[1].constants[-1] == 128          # 64 tiles of 128 x 128
    assert p["c3_w8a8_m16"].dispatches[1].bindings == ["out", "a_scale", "w_scale", "workspace"]
    assert p["c4_w4a16_m1"].dispatches[0].export == "b200_w4a16_decode_m8"
    assert p["c4_w4a16_m16"].dispatches[0].export == "b200_w4a16_decode_m16"
    assert p["c4_w4a16_m128"].dispatches[0].export == "b200_w4a16_gemm_wt"      # every M > 16 with an aligned result
    assert p["c4_w4a16_m128"].dispatches[0].grid == (86, 1, 1)                    # one 128-row activation tile x 86 weight tiles
    assert dg.plan_w4a16("odd", 100, 264, 256, ldo=270).dispatches[0].export == "b200_w4a16_gemm"   # pitch off the 16-byte grid
    assert p["c5_w4a16_m16"].dispatches[0].grid == (148, 1, 1)            # K = 8192: 74 tile walkers x 2 K slices
    assert p["c5_w4a16_m16"].transients[0]["host_tensor_maps"]["kind"] == "w4a16_decode"
    assert "host_tensor_maps" not in p["c4_w4a16_m16"].transients[0]      # one slice: plain bulk copies, no map
    assert p["c5_w4a16_m4096"].dispatches[0].export == "b200_w4a16_gemm_wt"
    assert p["c4_w4a16_m2048"].dispatches[0].constants == [2048, 11008, 4096, 11008, 0, 256, 0]


def _eval_constants(src):
    """`constexpr <type> kName = <integer expression>;` definitions of a C++ source, evaluated in order."""
    values = {}
    for name, expr in re.findall(r"constexpr\s+(?:u?int\d*_t|int|size_t)\s+(k\w+)\s*=\s*([^;]+);", src):
        expr = re.sub(r"/\*.*?\*/", "", expr)
        try:
            values[name] = int(eval(expr, {"__builtins__": {}}, dict(values)))
        except Exception:
            pass
    return values


def runtime_shared_memory_table(src):
    """export name -> dynamic shared memory bytes, from kEntries in the runtime library's source."""
    values = _eval_constants(src)
    table = {}
    for name, smem in re.findall(r'\{"(b200_[a-z0-9_]+)", \{[^}]*\}, (\w+)\}', src):
        table[name] = int(smem) if smem.isdigit() else values[smem]
    return table


def test_plugin_constants_match_the_runtime_export_table():
    """Every launch constant the compiler plugin bakes into its hal.dispatch.extern ops (threads per
    block, dynamic shared memory) must equal what the runtime library declares for the same export."""
    runtime = open(os.path.join(ROOT, "iree_b200", "csrc", "hal_b200.cc")).read()
    plugin = open(os.path.join(ROOT, "iree_b200", "compiler_plugin", "src", "RewriteContractionsPass.cpp")).read()
    smem = runtime_shared_memory_table(runtime)
    threads = {k: int({"kGemmThreads": "256"}.get(v, v)) for k, v in re.findall(r'\{"(b200_[a-z0-9_]+)", \{(\w+),', runtime)}
    consts = {}
    for decl in re.findall(r"constexpr int64_t ([^;]+);", plugin):
        for name, value in re.findall(r"(k\w+)\s*=\s*(\d+)", decl):
            consts[name] = int(value)
    expected = {"kGemmThreads": threads["b200_matmul_f16_f16"], "kGemmSmem": smem["b200_matmul_f16_f16"],
                "kW4GemmThreads": threads["b200_w4a16_gemm"], "kW4GemmSmem": smem["b200_w4a16_gemm"],
                "kW4WtSmem": smem["b200_w4a16_gemm_wt"], "kW4WtThreads": threads["b200_w4a16_gemm_wt"],
                "kDecodeThreads": threads["b200_w4a16_decode_m8"],
                "kDecodeSmemM8": smem["b200_w4a16_decode_m8"], "kDecodeSmemM16": smem["b200_w4a16_decode_m16"]}
    for name, value in expected.items():
        assert consts.get(name) == value, (name, consts.get(name), value)
    assert smem["b200_matmul_pair_f16_f16"] == smem["b200_matmul_f16_f16"]      # the pair exports share kGemmSmem
    # and the Python restatement of the same table
    assert (dg.GEMM_SMEM, dg.W4_SMEM, dg.W4_WT_SMEM) == (consts["kGemmSmem"], consts["kW4GemmSmem"], consts["kW4WtSmem"])
    assert dg.DECODE_SMEM == {8: consts["kDecodeSmemM8"], 16: consts["kDecodeSmemM16"]}
    assert (dg.W4_THREADS, dg.W4_WT_THREADS) == (consts["kW4GemmThreads"], consts["kW4WtThreads"])


def test_unaligned_shapes_go_to_the_generic_exports():
    plan = dg.plan_matmul("f", "i8", "acc", 123, 456, 789)
    assert [d.export for d in plan.dispatches] == ["b200_matmul_generic_i8_i32"] and not plan.transients
    assert dg.plan_w4a16("g", 3, 40, 512, group=64).dispatches[0].export == "b200_w4a16_generic"
    with pytest.raises(ValueError):
        dg.plan_matmul("f", "f16", "requant", 8, 8, 8)


def test_plan_limits_match_the_pipeline_layout():
    for plan in dg.baseline_plans().values():
        for d in plan.dispatches:
            assert len(d.bindings) <= 16 and len(d.constants) <= 64       # pipeline_layout.h:19-28
            assert all(-2 ** 31 <= c < 2 ** 31 for c in d.constants)
            assert d.shared_memory <= 232448


def test_export_table_matches_the_runtime_and_the_docs():
    src = open(os.path.join(ROOT, "iree_b200", "csrc", "hal_b200.cc")).read()
    entries = {k: {"kGemmThreads": "256"}.get(v, v) for k, v in re.findall(r'\{"(b200_[a-z0-9_]+)", \{(\w+),', src)}
    smem = runtime_shared_memory_table(src)
    for plan in dg.baseline_plans().values():
        for d in plan.dispatches:
            assert d.export in entries, d.export
            assert int(entries[d.export]) == d.block[0], d.export
            assert smem[d.export] == d.shared_memory, d.export
    doc = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    for name in ("b200_encode_tensormaps", "b200_matmul_i8_requant_f16", "b200_w4a16_gemm", "b200_w4a16_generic"):
        assert name in doc


def test_plan_json_round_trip_and_mlir_sketch():
    plan = dg.plan_matmul("mm", "f16", "cast", 256, 384, 512)
    again = dg.Plan.from_json(plan.to_json())
    assert again == plan
    text = dg.extern_mlir(plan)
    assert 'hal.dispatch.extern "b200_matmul_f16_f16"' in text and "push_constants = 6" in text
    assert '#hal.executable.object<{path = "b200_contraction.cubin"}>' in text


def test_tensor_flag_grammar(tmp_path):
    a = run_module.parse_tensor_flag("2x3xi8=1 2 3 4 5 6")
    assert a.dtype == np.int8 and a.tolist() == [[1, 2, 3], [4, 5, 6]]
    assert run_module.parse_tensor_flag("4xf16=2").tolist() == [2, 2, 2, 2]
    path = tmp_path / "x.npy"
    np.save(path, np.arange(6, dtype=np.int32).reshape(2, 3))
    assert run_module.parse_tensor_flag("2x3xi32=@%s" % path).tolist() == [[0, 1, 2], [3, 4, 5]]


@pytest.mark.gpu
@pytest.mark.parametrize("device_maps", [True, False])
def test_run_module_executes_plans_through_the_raw_kernel_abi(ctx, tmp_path, device_maps):
    """C1 and a small W4A16 decode dispatch driven only by push constants / descriptor sets /
    dispatch, i.e. by the kernel ABI the stock HAL CUDA driver uses."""
    import oracle
    a, b = workloads.c1_i8_matmul()
    plan = dg.plan_matmul("c1", "i8", "acc", 1024, 1024, 1024, device_tensor_maps=device_maps)
    (got,) = run_module.execute_plan(ctx, plan, [a, b])
    assert (got[:64] == oracle.matmul_port(oracle.TYPE_S8S8S32, a[:64], b)).all()      # the data-tiled CPU chain
    assert (got == a.astype(np.int32) @ b.astype(np.int32)).all()
    a16, wq, s = workloads.c4_w4a16(8, N=512, K=4096, seed=5)
    plan = dg.plan_w4a16("dec", 8, 512, 4096)
    (got,) = run_module.execute_plan(ctx, plan, [a16, wq.view(np.int8), s])
    np.testing.assert_allclose(got.astype(np.float32), oracle.w4a16(a16, wq, s).astype(np.float32), rtol=1e-2, atol=1e-2)


@pytest.mark.gpu
def test_run_module_cli(built, tmp_path):
    rng = np.random.default_rng(3)
    a = rng.integers(-4, 5, (256, 128)).astype(np.float16)
    b = rng.integers(-4, 5, (128, 384)).astype(np.float16)
    np.save(tmp_path / "a.npy", a); np.save(tmp_path / "b.npy", b)
    np.save(tmp_path / "want.npy", (a.astype(np.float32) @ b.astype(np.float32)).astype(np.float16))
    plan = dg.plan_matmul("mm", "f16", "cast", 256, 384, 128)
    (tmp_path / "plan.json").write_text(plan.to_json())
    argv = ["--device=cuda", "--module=%s" % (tmp_path / "plan.json"), "--function=mm",
            "--input=256x128xf16=@%s" % (tmp_path / "a.npy"), "--input=128x384xf16=@%s" % (tmp_path / "b.npy"),
            "--expected_output=256x384xf16=@%s" % (tmp_path / "want.npy")]
    assert run_module.main(argv) == 0
    np.save(tmp_path / "bad.npy", np.zeros((256, 384), np.float16))
    argv[-1] = "--expected_output=256x384xf16=@%s" % (tmp_path / "bad.npy")
    assert run_module.main(argv) == 1                                  # mismatch: non-zero exit code
    assert run_module.main(["--device=local-task", "--module=%s" % (tmp_path / "plan.json")]) == 2


# ---- the benchmark programs as MLIR text -------------------------------------------------------------
from iree_b200 import mlir_frontend as mf  # noqa: E402

PLUGIN_TESTS = os.path.join(ROOT, "iree_b200", "compiler_plugin", "test")


@pytest.mark.parametrize("config", ["c1", "c2", "c3", "c4", "c5"])
def test_config_mlir_lowers_to_the_baseline_plans(config):
    """Each committed config_*.mlir (the configuration written as linalg-on-tensors, in the op shapes
    dispatch formation groups) goes through the text matcher and must give, function by function,
    the plan that baseline_plans() states for that shape."""
    from dataclasses import asdict
    text = open(os.path.join(PLUGIN_TESTS, "config_%s.mlir" % config)).read()
    assert text.endswith(mf.config_mlir(config))            # the committed file is what the writer produces
    plans = mf.plans_from_mlir(text)
    by_function = {p.function: p for p in dg.baseline_plans().values()}
    expected = {f for f in by_function if f == config or f.startswith(config + "_")}
    assert set(plans) == expected and expected
    for f in expected:
        assert asdict(plans[f]) == asdict(by_function[f]), f


def test_text_matcher_refuses_what_the_pass_refuses():
    ok = mf.matmul_mlir("f", "i8", "requant", 16, 64, 128)
    assert mf.plans_from_mlir(ok)["f"].dispatches[-1].export == "b200_matmul_i8_requant_f16"
    # accumulating into something that is not a zero fill is left to the stock path
    assert mf.plans_from_mlir(ok.replace("arith.constant 0 : i32", "arith.constant 1 : i32")) == {}
    # a consumer that scales by w_scale[m] instead of w_scale[n] is not the requant epilogue: only the matmul is taken
    wrong = ok.replace("affine_map<(d0, d1) -> (d1)>", "affine_map<(d0, d1) -> (d0)>")
    assert mf.plans_from_mlir(wrong)["f"].dispatches[-1].export == "b200_matmul_i8_i32"
    w4 = mf.w4a16_mlir("g", 8, 64, 512)
    assert mf.plans_from_mlir(w4)["g"].dispatches[-1].export == "b200_w4a16_decode_m8"
    assert mf.plans_from_mlir(w4.replace("arith.extsi", "arith.extui")) == {}       # unsigned weights: a zero point would be needed
    assert mf.plans_from_mlir(w4.replace('"reduction", "reduction"', '"reduction", "parallel"')) == {}


@pytest.mark.gpu
def test_device_built_maps_of_the_w4a16_kernels_equal_the_host_encoded_ones(ctx):
    """The generic map builder (b200_encode_tensormap + the template table) against cuTensorMapEncodeTiled:
    every map the W4A16 kernels use must come out byte for byte as prepare() writes it, before any
    kernel is allowed to consume a device-built one."""
    import iree_b200 as ib
    for (M, N, K) in [(8, 512, 8192), (96, 272, 512), (512, 264, 512)]:
        a, wq, s = workloads.c4_w4a16(M, N=N, K=K, seed=8)
        da, dw, ds = ctx.to_device(a), ctx.to_device(wq), ctx.to_device(s)
        out = ctx.alloc(M * N * 2)
        host_ws, dev_ws = ctx.w4a16_workspace(N), ctx.w4a16_workspace(N)
        plan = dg.plan_w4a16("f", M, N, K, device_tensor_maps=True)
        kernel = plan.dispatches[-1]
        variant = {"b200_w4a16_decode_m8": ib.W4A16_DECODE, "b200_w4a16_gemm": ib.W4A16_GEMM,
                   "b200_w4a16_gemm_wt": ib.W4A16_GEMM_WT}[kernel.export]
        tile_n = kernel.constants[5] if variant == ib.W4A16_GEMM else 0
        ctx.w4a16_prepare(ib.W4A16Params(M, N, K, 128, N, 0, variant, tile_n), da, dw, ds, out, host_ws)
        import ctypes as C
        table = C.create_string_buffer(768)
        ib.runtime.check(ib.library().iree_b200_tensormap_templates(ctx.handle, table))
        templates = ctx.to_device(np.frombuffer(table.raw, np.uint8))
        buffers = {"a": da, "wq": dw, "scales": ds, "out": out, "templates": templates, "workspace": dev_ws}
        for d in plan.dispatches[:-1]:
            ctx.dispatch(d.export, [buffers[b] for b in d.bindings], d.constants, d.grid)
        ctx.synchronize()
        n = host_ws.nbytes if host_ws.nbytes < 2048 else 2048
        want, got = host_ws.download(np.uint8, (n,)), dev_ws.download(np.uint8, (n,))
        slots = {ib.W4A16_DECODE: [(0, 128), (448, 464)], ib.W4A16_GEMM: [(0, 256)],
                 ib.W4A16_GEMM_WT: [(0, 256), (512, 640)]}[variant]
        for lo, hi in slots:
            assert (want[lo:hi] == got[lo:hi]).all(), (kernel.export, lo, np.nonzero(want[lo:hi] != got[lo:hi])[0][:8])
        for b in (da, dw, ds, out, host_ws, dev_ws, templates):
            b.free()


@pytest.mark.gpu
@pytest.mark.parametrize("device_maps", [False, True])
def test_w4a16_plans_run_through_the_raw_kernel_abi(ctx, device_maps):
    """Decode with K > 4096 (weight map), the shared-memory-operand GEMM and the tensor-memory-operand
    GEMM, driven only by dispatches: with host-encoded maps, and with maps built on the device."""
    import oracle
    for (M, N, K) in [(8, 512, 8192), (96, 272, 512), (512, 264, 512)]:
        a, wq, s = workloads.c4_w4a16(M, N=N, K=K, seed=9)
        plan = dg.plan_w4a16("f", M, N, K, device_tensor_maps=device_maps)
        (got,) = run_module.execute_plan(ctx, plan, [a, wq.view(np.int8), s])
        np.testing.assert_allclose(got.astype(np.float32), oracle.w4a16(a, wq, s, threads=os.cpu_count() or 1).astype(np.float32),
                                   rtol=1e-2, atol=1e-2)


@pytest.mark.gpu
def test_benchmark_programs_from_mlir_text_run_on_the_gpu(ctx):
    """config_*.mlir -> text matcher -> plan -> run_module, for one shape of every configuration,
    against the CPU oracle (integer paths exactly)."""
    import oracle
    threads = os.cpu_count() or 1

    def plans(config):
        return mf.plans_from_mlir(open(os.path.join(PLUGIN_TESTS, "config_%s.mlir" % config)).read())
    a, b = workloads.c1_i8_matmul()
    (got,) = run_module.execute_plan(ctx, plans("c1")["c1"], [a, b])
    assert (got == oracle.matmul_ref(oracle.TYPE_S8S8S32, a, b, threads=threads)).all()
    a, w, sa, sw = workloads.c3_w8a8(16)
    (got,) = run_module.execute_plan(ctx, plans("c3")["c3_m16"], [a, w, sa, sw])
    assert (got == oracle.w8a8(a, w, sa, sw, use_ref=True, threads=threads)).all()
    a, wq, s = workloads.c4_w4a16(8)
    (got,) = run_module.execute_plan(ctx, plans("c4")["c4_m8"], [a.reshape(8, 32, 128), wq.view(np.int8), s])
    np.testing.assert_allclose(got.astype(np.float32), oracle.w4a16(a, wq, s, threads=threads).astype(np.float32), rtol=1e-2, atol=1e-2)
    a, wq, s = workloads.c5_w4a16_sharded(16)
    (got,) = run_module.execute_plan(ctx, plans("c5")["c5_m16"], [a.reshape(16, 64, 128), wq.view(np.int8), s])
    cols = np.arange(0, wq.shape[0], 13)
    np.testing.assert_allclose(got[:, cols].astype(np.float32), oracle.w4a16(a, wq[cols], s[cols], threads=threads).astype(np.float32),
                               rtol=1e-2, atol=1e-2)
