"""The command-buffer API beyond dispatch, through the C ABI on a GPU: begin / end, execution barriers,
fill and copy commands in stream mode and as graph nodes, pipeline layouts with several descriptor sets
(runtime/src/iree/hal/command_buffer.h:532-654, drivers/cuda/pipeline_layout.c:145-190)."""
import ctypes as C

import numpy as np
import pytest

import iree_b200 as ib
from iree_b200 import runtime as rt

pytestmark = pytest.mark.gpu


def test_begin_and_end_must_pair(ctx):
    ctx.begin()
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.begin()
    assert e.value.code_name == "FAILED_PRECONDITION"
    ctx.end()
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.end()
    assert e.value.code_name == "FAILED_PRECONDITION"


@pytest.mark.parametrize("graph", [False, True])
def test_fill_and_copy_commands(ctx, graph):
    """fill (1-, 2-, 4-byte patterns at offsets) then copy (ranges inside larger buffers), in recording
    order, in stream mode and as memset / memcpy nodes of a graph replayed twice."""
    n = 4096
    a, b = ctx.alloc(n).fill(0x11), ctx.alloc(n).fill(0x22)
    want_a = np.full(n, 0x11, np.uint8)
    want_a[16:16 + 256] = 0xAB
    want_a[512:512 + 128].view(np.uint16)[:] = 0xBEEF
    want_a[1024:1024 + 64].view(np.uint32)[:] = 0xDEADBEEF
    want_b = np.full(n, 0x22, np.uint8)
    want_b[100:100 + 2000] = want_a[8:8 + 2000]

    def record():
        ctx.begin()
        ctx.fill_buffer(a, 16, 256, bytes([0xAB]))
        ctx.fill_buffer(a, 512, 128, np.array([0xBEEF], np.uint16).tobytes())
        ctx.fill_buffer(a, 1024, 64, np.array([0xDEADBEEF], np.uint32).tobytes())
        ctx.execution_barrier()
        ctx.copy_buffer(a, 8, b, 100, 2000)
        ctx.end()

    if graph:
        ctx.begin_graph()
        record()
        g = ctx.end_graph()
        for _ in range(2):
            a.fill(0x11); b.fill(0x22)
            g.execute()
            ctx.synchronize()
            assert np.array_equal(a.download(np.uint8, (n,)), want_a)
            assert np.array_equal(b.download(np.uint8, (n,)), want_b)
        g.release()
    else:
        record()
        ctx.synchronize()
        assert np.array_equal(a.download(np.uint8, (n,)), want_a)
        assert np.array_equal(b.download(np.uint8, (n,)), want_b)
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.fill_buffer(a, 2, 8, np.array([1], np.uint32).tobytes())        # offset not aligned to the pattern
    assert e.value.code_name == "INVALID_ARGUMENT"
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.fill_buffer(a, 0, 9, bytes([1, 2, 3]))                           # no 3-byte patterns
    assert e.value.code_name == "INVALID_ARGUMENT"
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.copy_buffer(a, 0, a, 64, 128)                                    # overlapping ranges
    assert e.value.code_name == "INVALID_ARGUMENT"
    a.free(); b.free()


@pytest.mark.parametrize("graph", [False, True])
def test_dispatch_through_a_pipeline_layout_of_two_sets(ctx, graph):
    """The same export dispatched once with all bindings in set 0 and once through a pipeline layout whose
    sets hold one and two bindings: the kernel parameters are set 0's pointers, then set 1's, then the
    push constants. A fill and an execution barrier sit between dependent dispatches."""
    rng = np.random.default_rng(4)
    M, N, K = 48, 40, 24
    a = rng.integers(-3, 4, (M, K)).astype(np.float16)
    b = rng.integers(-3, 4, (K, N)).astype(np.float16)
    da, db = ctx.to_device(a), ctx.to_device(b)
    out0, out1 = ctx.alloc(M * N * 2).fill(0), ctx.alloc(M * N * 2).fill(0)
    grid = ((N + 15) // 16, (M + 15) // 16, 1)
    consts = [M, N, K, ib.RHS_KN]
    layout = ctx.pipeline_layout(4, [1, 2])

    def record():
        ctx.dispatch("b200_matmul_generic_f16_f16", [da, db, out0], consts, grid)
        ctx.execution_barrier()
        ctx.fill_buffer(out1, 0, M * N * 2, bytes([0x7F]))
        ctx.push_descriptor_set(0, [da])
        ctx.push_descriptor_set(1, [db, out1])
        ctx.dispatch_with_layout("b200_matmul_generic_f16_f16", layout, consts, grid)

    if graph:
        ctx.begin_graph()
        record()
        g = ctx.end_graph()
        g.execute()
        ctx.synchronize()
        g.release()
    else:
        record()
        ctx.synchronize()
    want = (a.astype(np.float32) @ b.astype(np.float32)).astype(np.float16)
    assert np.array_equal(out0.download(np.float16, (M, N)), want)
    assert np.array_equal(out1.download(np.float16, (M, N)), want)
    ctx.release_pipeline_layout(layout)
    with pytest.raises(ib.IreeB200Error) as e:
        ctx.pipeline_layout(65, [1])                                           # more push constants than the limit
    assert e.value.code_name == "INVALID_ARGUMENT"
    for x in (da, db, out0, out1):
        x.free()
