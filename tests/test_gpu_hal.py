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


def test_semaphores_and_queue_execute(ctx):
    """Timeline semaphores advanced by the device behind queued graphs and by the host; waits that the
    stream serves, a wait only the host can satisfy, the monotonic rule and a wait that runs out
    (hal/semaphore.h:60-140; iree_hal_device_queue_execute)."""
    import threading
    import time
    lib = ib.library()
    dev = ctx.device
    n = 1 << 20
    a, b = ctx.alloc(n).fill(0), ctx.alloc(n).fill(0)

    def graph_of(record):
        ctx.begin_graph()
        record()
        g = ctx.end_graph()
        return g

    g1 = graph_of(lambda: ctx.fill_buffer(a, 0, n, bytes([0x5A])))
    g2 = graph_of(lambda: ctx.copy_buffer(a, 0, b, 0, n))
    sem, host_sem = C.c_void_p(), C.c_void_p()
    rt.check(lib.iree_hal_b200_semaphore_create(dev, C.c_uint64(0), C.byref(sem)))
    rt.check(lib.iree_hal_b200_semaphore_create(dev, C.c_uint64(5), C.byref(host_sem)))

    def execute(waits, signals, graphs):
        ws = (C.c_void_p * max(len(waits), 1))(*[w[0].value for w in waits])
        wv = (C.c_uint64 * max(len(waits), 1))(*[w[1] for w in waits])
        ss = (C.c_void_p * max(len(signals), 1))(*[s[0].value for s in signals])
        sv = (C.c_uint64 * max(len(signals), 1))(*[s[1] for s in signals])
        gs = (C.c_void_p * max(len(graphs), 1))(*[g.handle.value for g in graphs])
        rt.check(lib.iree_hal_b200_device_queue_execute(dev, C.c_size_t(len(waits)), ws, wv, C.c_size_t(len(signals)), ss, sv,
                                                        C.c_size_t(len(graphs)), gs))

    # fill signals 1; the copy waits for 1 (served by the stream) and signals 2; a barrier submission signals 3
    execute([], [(sem, 1)], [g1])
    execute([(sem, 1)], [(sem, 2)], [g2])
    execute([(sem, 2)], [(sem, 3)], [])
    rt.check(lib.iree_hal_b200_semaphore_wait(sem, C.c_uint64(3), C.c_int64(5000)))
    value = C.c_uint64()
    rt.check(lib.iree_hal_b200_semaphore_query(sem, C.byref(value)))
    assert value.value == 3
    assert (b.download(np.uint8, (n,)) == 0x5A).all()

    # a wait only the host can satisfy: the submission is held until another thread signals
    a.fill(0); b.fill(0)
    t = threading.Thread(target=lambda: (time.sleep(0.05), rt.check(lib.iree_hal_b200_semaphore_signal(host_sem, C.c_uint64(6)))))
    t.start()
    execute([(host_sem, 6)], [(sem, 4)], [g1, g2])
    t.join()
    rt.check(lib.iree_hal_b200_semaphore_wait(sem, C.c_uint64(4), C.c_int64(5000)))
    assert (b.download(np.uint8, (n,)) == 0x5A).all()

    assert lib.iree_hal_b200_semaphore_signal(sem, C.c_uint64(4)) == 11            # OUT_OF_RANGE: values only grow
    assert lib.iree_hal_b200_semaphore_wait(sem, C.c_uint64(100), C.c_int64(30)) == 4  # DEADLINE_EXCEEDED
    with pytest.raises(ib.IreeB200Error) as e:
        execute([], [(sem, 2)], [])                                                # a signal below the payload
    assert e.value.code_name == "OUT_OF_RANGE"
    lib.iree_hal_b200_semaphore_retain(sem)
    lib.iree_hal_b200_semaphore_release(sem)
    rt.check(lib.iree_hal_b200_semaphore_query(sem, C.byref(value)))              # still alive: one reference left
    assert value.value == 4
    lib.iree_hal_b200_semaphore_release(sem)
    lib.iree_hal_b200_semaphore_release(host_sem)
    g1.release(); g2.release()
    a.free(); b.free()
