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
