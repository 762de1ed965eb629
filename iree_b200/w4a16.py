"""Host-side helpers for the fused int4 dequant + matmul dispatch (``iree_b200_w4a16*``)."""
from __future__ import annotations

import numpy as np

from . import runtime as rt


def w4a16_numpy(ctx: rt.Context, a: np.ndarray, wq: np.ndarray, scales: np.ndarray, group: int = 128,
                variant: int = rt.W4A16_AUTO, tile_n: int = 0, out: np.ndarray = None, n_offset: int = 0) -> np.ndarray:
    """Host arrays in, host array out, through ``iree_b200_w4a16_host``.

    a [M, K] f16; wq [N, K/2] u8 (two int4 per byte, low nibble first); scales [N, K/group] f16.
    With ``out`` given (shape [M, ldo]) the N result columns land at ``n_offset``.
    """
    a = np.ascontiguousarray(a, np.float16)
    wq = np.ascontiguousarray(wq, np.uint8)
    scales = np.ascontiguousarray(scales, np.float16)
    M, K = a.shape
    N = wq.shape[0]
    assert wq.shape == (N, K // 2) and scales.shape == (N, K // group), (wq.shape, scales.shape)
    if out is None:
        out = np.empty((M, N), np.float16)
    assert out.dtype == np.float16 and out.flags.c_contiguous and out.shape[0] == M
    p = rt.W4A16Params(M, N, K, group, out.shape[1], n_offset, variant, tile_n)
    ctx.w4a16_host(p, a, wq, scales, out)
    return out
