"""Worker of tests/test_gpu_multi.py: one rank of an all-gather by peer copies (run under torchrun)."""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import iree_b200 as ib  # noqa: E402
from iree_b200 import runtime as rt  # noqa: E402
from iree_b200.sharding import PeerGather  # noqa: E402


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    ctx = ib.Context(local)
    lib = ib.library()
    ident = C.create_string_buffer(128)
    if rank == 0:
        rt.check(lib.iree_hal_b200_channel_create_id(ident, C.c_size_t(128)))
    t = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        t[:] = torch.frombuffer(bytearray(ident.raw), dtype=torch.uint8)
    dist.broadcast(t, src=0)
    channel = C.c_void_p()
    rt.check(lib.iree_hal_b200_channel_create(ctx.device, bytes(t.numpy().tobytes()), C.c_size_t(128), C.c_int32(rank),
                                              C.c_int32(world), C.byref(channel)))
    n = 1 << 20  # int32 elements per rank and buffer
    rounds, buffers = 6, 2
    gathers = [ctx.alloc(world * n * 4).fill(0xEE) for _ in range(buffers)]
    send = ctx.alloc(n * 4)
    peer = PeerGather(ctx, channel, rank, world, gathers)
    ok = True
    for r in range(rounds):
        block = (np.arange(n, dtype=np.int32) * (rank + 1) + 1000 * r).astype(np.int32)
        send.upload(block)
        peer.gather(r % buffers, send, n * 4)
        rt.check(lib.iree_hal_b200_command_buffer_join_collectives(ctx.command_buffer))
        ctx.synchronize()
        got = gathers[r % buffers].download(np.int32, (world, n))
        for p in range(world):
            want = (np.arange(n, dtype=np.int32) * (p + 1) + 1000 * r).astype(np.int32)
            ok = ok and np.array_equal(got[p], want)
        dist.barrier()  # nobody overwrites `send` or a receive buffer while a peer still checks
    peer.close()
    # iree_hal_channel_split: one colour, keys in reverse rank order -> the same ranks in reverse; an
    # all-gather through the new channel is ordered by the new ranks. Then a split in which the last rank
    # passes no colour: it gets no channel, the others a channel without it.
    sub = C.c_void_p()
    rt.check(lib.iree_hal_b200_channel_split(channel, C.c_int32(0), C.c_int32(world - 1 - rank), C.byref(sub)))
    ok = ok and bool(sub.value) and lib.iree_hal_b200_channel_count(sub) == world
    ok = ok and lib.iree_hal_b200_channel_rank(sub) == world - 1 - rank
    word = ctx.to_device(np.array([100 + rank], np.int32))
    words = ctx.alloc(world * 4).fill(0)
    rt.check(lib.iree_hal_b200_command_buffer_all_gather(ctx.command_buffer, sub, C.c_int32(2), C.c_void_p(word.ptr),
                                                         C.c_void_p(words.ptr), C.c_size_t(1)))
    ctx.synchronize()
    ok = ok and np.array_equal(words.download(np.int32, (world,)), 100 + np.arange(world - 1, -1, -1, dtype=np.int32))
    lib.iree_hal_b200_channel_release(sub)
    sub2 = C.c_void_p()
    rt.check(lib.iree_hal_b200_channel_split(channel, C.c_int32(-1 if rank == world - 1 else 7), C.c_int32(rank), C.byref(sub2)))
    if rank == world - 1:
        ok = ok and not sub2.value
    else:
        ok = ok and bool(sub2.value) and lib.iree_hal_b200_channel_count(sub2) == world - 1
        ok = ok and lib.iree_hal_b200_channel_rank(sub2) == rank
        lib.iree_hal_b200_channel_release(sub2)
    # The other collective kinds through iree_hal_b200_command_buffer_collective (the reference's enum values).
    def collective(kind, reduction, param, send, recv, count, etype=2):
        rt.check(lib.iree_hal_b200_command_buffer_collective(
            ctx.command_buffer, channel, C.c_int32(kind), C.c_int32(reduction), C.c_int32(etype), C.c_uint32(param),
            C.c_void_p(send.ptr if send is not None else None), C.c_void_p(recv.ptr if recv is not None else None),
            C.c_size_t(count)))
        ctx.synchronize()
    m = 1024
    mine = (np.arange(m, dtype=np.int32) + 10 * rank).astype(np.int32)
    every = [(np.arange(m, dtype=np.int32) + 10 * p).astype(np.int32) for p in range(world)]
    src, dst = ctx.to_device(mine), ctx.alloc(m * 4 * world).fill(0)
    collective(1, 1, 0, src, dst, m)                                   # ALL_REDUCE, SUM
    ok = ok and np.array_equal(dst.download(np.int32, (m,)), sum(every))
    collective(1, 4, 0, src, dst, m)                                   # ALL_REDUCE, MAXIMUM
    ok = ok and np.array_equal(dst.download(np.int32, (m,)), every[-1])
    collective(3, 0, world - 1, src, dst, m)                           # BROADCAST from the last rank
    ok = ok and np.array_equal(dst.download(np.int32, (m,)), every[-1])
    dst.fill(0)
    collective(4, 1, 0, src, dst, m)                                   # REDUCE to rank 0
    if rank == 0:
        ok = ok and np.array_equal(dst.download(np.int32, (m,)), sum(every))
    collective(5, 1, 0, src, dst, m // world)                          # REDUCE_SCATTER: m / world elements per rank
    ok = ok and np.array_equal(dst.download(np.int32, (m // world,)), sum(every)[rank * (m // world):(rank + 1) * (m // world)])
    collective(2, 0, 0, src, dst, m)                                   # ALL_TO_ALL: m / world elements per peer
    want = np.concatenate([every[p][rank * (m // world):(rank + 1) * (m // world)] for p in range(world)])
    ok = ok and np.array_equal(dst.download(np.int32, (m,)), want)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    collective(8, 0, nxt | (prv << 16), src, dst, m)                   # SEND_RECV around the ring
    ok = ok and np.array_equal(dst.download(np.int32, (m,)), every[prv])
    if world == 2:
        dst.fill(0)
        if rank == 0:
            collective(6, 0, 1, src, None, m)                          # SEND to rank 1
        else:
            collective(7, 0, 0, None, dst, m)                          # RECV from rank 0
            ok = ok and np.array_equal(dst.download(np.int32, (m,)), every[0])
    f = ctx.to_device(np.full(m, 1.5 + rank, np.float32))
    fd = ctx.alloc(m * 4)
    collective(1, 5, 0, f, fd, m, etype=3)                             # ALL_REDUCE, AVERAGE, f32
    ok = ok and np.allclose(fd.download(np.float32, (m,)), 1.5 + (world - 1) / 2)
    lib.iree_hal_b200_channel_release(channel)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("PEER_GATHER_OK" if int(flag[0]) else "PEER_GATHER_MISMATCH", flush=True)
    ctx.close()
    return 0 if int(flag[0]) else 1


if __name__ == "__main__":
    sys.exit(main())
