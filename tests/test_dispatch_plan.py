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
    assert [d.export for d in p["c2_f16_4096"].dispatches] == ["b200_encode_tensormaps", "b200_matmul_f16_f16"]
    gemm = p["c2_f16_4096"].dispatches[1]
    assert gemm.bindings == ["out", "workspace"] and gemm.constants == [4096, 4096, 4096, 1, 0, 256]
    assert gemm.grid == (148, 1, 1) and gemm.block == (256, 1, 1) and gemm.shared_memory == 197888
    assert p["c1_i8_1024"].dispatches[1].export == "b200_matmul_i8_i32"
    assert p["c1_i8_1024"].dispatches[1].constants[-1] == 128          # 64 tiles of 128 x 128
    assert p["c3_w8a8_m16"].dispatches[1].bindings == ["out", "a_scale", "w_scale", "workspace"]
    assert p["c4_w4a16_m1"].dispatches[0].export == "b200_w4a16_decode_m8"
    assert p["c4_w4a16_m16"].dispatches[0].export == "b200_w4a16_decode_m16"
    assert p["c4_w4a16_m128"].dispatches[0].export == "b200_w4a16_gemm"
    assert p["c5_w4a16_m16"].dispatches[0].grid == (148, 1, 1)            # K = 8192: two passes inside the kernel
    assert p["c5_w4a16_m4096"].dispatches[0].export == "b200_w4a16_gemm"


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
    for plan in dg.baseline_plans().values():
        for d in plan.dispatches:
            assert d.export in entries, d.export
            assert int(entries[d.export]) == d.block[0], d.export
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
