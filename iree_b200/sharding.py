"""N-sharding of a contraction over the ranks of one channel (host-side arithmetic only).

Weights (and their scales) are split along N into ``world`` contiguous row blocks, activations
are replicated, rank r computes output columns ``[r * N / world, (r + 1) * N / world)``, and one
all-gather through the channel delivers every slice to every rank. An all-gather concatenates
along the outermost dimension, so what arrives is ``[world, M, N / world]``; ``assemble`` turns
that into the row-major ``[M, N]`` result (the transposition IREE programs place around their
all-gather, compiler/src/iree/compiler/Dialect/Flow/Conversion/MeshToFlow/test/collectives.mlir:5-22).
"""
from __future__ import annotations

import numpy as np


def column_range(N: int, world: int, rank: int):
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank %d is not in a channel of %d" % (rank, world))
    if N % world:
        raise ValueError("N = %d does not divide over %d ranks" % (N, world))
    per = N // world
    return rank * per, (rank + 1) * per


def shard_weights(wq: np.ndarray, scales: np.ndarray, world: int, rank: int):
    """Row block of [N, ...] weight and scale tensors owned by `rank`."""
    n0, n1 = column_range(wq.shape[0], world, rank)
    return wq[n0:n1], scales[n0:n1]


def assemble(gathered: np.ndarray) -> np.ndarray:
    """[world, M, N/world] (all-gather order) -> [M, N] row-major."""
    world, M, n = gathered.shape
    return np.ascontiguousarray(np.transpose(gathered, (1, 0, 2)).reshape(M, world * n))


class PeerGather:
    """All-gather of per-rank blocks by peer copies (``iree_hal_b200_command_buffer_all_gather_peer_copies``).

    Every rank owns ``len(gather_buffers)`` receive buffers; their handles travel to the other ranks
    over the ``torch.distributed`` control plane once, each rank imports its peers' buffers, and
    from then on ``gather(k, send)`` puts this rank's block into slot ``rank`` of receive buffer k on
    every rank with the copy engines. One process per GPU, all on one node.
    """

    def __init__(self, ctx, channel, rank: int, world: int, gather_buffers):
        import ctypes as C
        import torch
        import torch.distributed as dist
        from . import runtime as rt
        self.ctx, self.channel, self.rank, self.world = ctx, channel, rank, world
        self.lib = rt.library()
        self._C, self._rt = C, rt
        n = len(gather_buffers)
        mine = torch.zeros(n * 64, dtype=torch.uint8)
        for k, buf in enumerate(gather_buffers):
            h = C.create_string_buffer(64)
            rt.check(self.lib.iree_hal_b200_buffer_export(ctx.device, C.c_void_p(buf.ptr), h))
            mine[k * 64:(k + 1) * 64] = torch.frombuffer(bytearray(h.raw), dtype=torch.uint8)
        everyone = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        self.imported = []
        self.tables = []
        for k, buf in enumerate(gather_buffers):
            table = (C.c_void_p * world)()
            for p in range(world):
                if p == rank:
                    table[p] = buf.ptr
                    continue
                ptr = C.c_void_p()
                raw = bytes(everyone[p][k * 64:(k + 1) * 64].numpy().tobytes())
                rt.check(self.lib.iree_hal_b200_buffer_import(ctx.device, raw, C.byref(ptr)))
                self.imported.append(ptr.value)
                table[p] = ptr.value
            self.tables.append(table)

    def gather(self, k: int, send_buffer, nbytes: int) -> None:
        C = self._C
        self._rt.check(self.lib.iree_hal_b200_command_buffer_all_gather_peer_copies(
            self.ctx.command_buffer, self.channel, C.c_void_p(send_buffer.ptr), C.c_size_t(nbytes), self.tables[k]))

    def close(self) -> None:
        for ptr in self.imported:
            self.lib.iree_hal_b200_buffer_unimport(self.ctx.device, self._C.c_void_p(ptr))
        self.imported = []


class PushGather:
    """N-sharded W4A16 dispatches that leave the full-width result on every rank without a collective
    (``iree_b200_w4a16_prepare_push / _run_push / _wait_arrivals``).

    Every rank owns ``buffers`` result buffers ``[M, N]`` f16 and as many arrival-word arrays; their
    handles travel over the ``torch.distributed`` control plane once and each rank imports its peers'.
    ``run(i, ...)`` dispatches this rank's column block of step i (the kernel's epilogue stores it into
    every rank's buffer ``i % buffers`` and then raises this rank's arrival word there) and enqueues
    the wait for all ranks' words on this rank. One process per GPU, all on one node.

    Reuse rule (two buffers are enough): step i + buffers overwrites what step i produced. A rank
    dispatches it only after its own wait of step i + buffers - 1, by which time every rank has
    finished step i + buffers - 1 and therefore everything it had ordered on its stream before that
    dispatch, which includes its readers of step i's result.
    """

    def __init__(self, ctx, channel, rank: int, world: int, M: int, N: int, buffers: int = 2):
        import ctypes as C
        import torch
        import torch.distributed as dist
        from . import runtime as rt
        self.ctx, self.rank, self.world, self.M, self.N = ctx, rank, world, M, N
        self.lib, self._rt, self._C = rt.library(), rt, C
        self.results = [ctx.alloc(M * N * 2).fill(0) for _ in range(buffers)]
        self.flags = [ctx.alloc(256).fill(0) for _ in range(buffers)]
        ctx.synchronize()
        self.uses = [0] * buffers
        owned = self.results + self.flags
        mine = torch.zeros(len(owned) * 64, dtype=torch.uint8)
        if world > 1:
            for k, buf in enumerate(owned):
                h = C.create_string_buffer(64)
                rt.check(self.lib.iree_hal_b200_buffer_export(ctx.device, C.c_void_p(buf.ptr), h))
                mine[k * 64:(k + 1) * 64] = torch.frombuffer(bytearray(h.raw), dtype=torch.uint8)
            everyone = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(everyone, mine)
        self.imported = []
        self.result_tables, self.flag_tables = [], []
        for k in range(buffers):
            for table_list, index, own in ((self.result_tables, k, self.results[k]),
                                           (self.flag_tables, buffers + k, self.flags[k])):
                table = []
                for p in range(world):
                    if p == rank:
                        table.append(own.ptr)
                        continue
                    ptr = C.c_void_p()
                    raw = bytes(everyone[p][index * 64:(index + 1) * 64].numpy().tobytes())
                    rt.check(self.lib.iree_hal_b200_buffer_import(ctx.device, raw, C.byref(ptr)))
                    self.imported.append(ptr.value)
                    table.append(ptr.value)
                table_list.append(table)

    def result(self, k: int):
        return self.results[k]

    def prepare(self, k: int, params, a, wq, scales, ws) -> None:
        """Writes the workspace of the dispatches that will target result buffer k with these operands."""
        self.ctx.w4a16_prepare_push(params, a, wq, scales, self.result_tables[k], self.flag_tables[k], self.rank, ws)

    def run(self, i: int, params, scales, ws) -> None:
        k = i % len(self.results)
        self.uses[k] += 1
        self.ctx.w4a16_run_push(params, scales, self.results[k], ws, self.world, self.rank, self.uses[k])
        self.ctx.w4a16_wait_arrivals(self.flags[k], ws, self.world, self.uses[k])

    def check(self) -> None:
        pass

    def close(self) -> None:
        self.ctx.synchronize()
        for ptr in self.imported:
            self.lib.iree_hal_b200_buffer_unimport(self.ctx.device, self._C.c_void_p(ptr))
        self.imported = []
        for b in self.results + self.flags:
            b.free()
        self.results, self.flags = [], []
