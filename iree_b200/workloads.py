"""Seeded synthetic inputs of the benchmark configurations.

No public dataset is involved on this path; every tensor is drawn from
``numpy.random.default_rng(seed)`` (PCG64) in the order listed, C order, so the CPU oracle and
the GPU see identical bytes. Configuration numbers follow BASELINE.json's ``configs`` list.
"""
from __future__ import annotations

import numpy as np


def pack_int4(w: np.ndarray) -> np.ndarray:
    """[N, K] integers in [-8, 7] -> [N, K/2] bytes, element 2i in the low nibble of byte i.

    The order is the reference's sub-byte packing (runtime/src/iree/builtins/ukernel/
    mmt4d_tile_generic.c:35-44, tests/e2e/linalg/subbyte_to_fp.mlir).
    """
    w = np.asarray(w)
    assert w.shape[-1] % 2 == 0
    u = (w.astype(np.int16) & 0xF).astype(np.uint8)
    return (u[..., 0::2] | (u[..., 1::2] << 4)).astype(np.uint8)


def unpack_int4(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, np.uint8)
    lo = (b & 0xF).astype(np.int8)
    hi = (b >> 4).astype(np.int8)
    out = np.empty(b.shape[:-1] + (b.shape[-1] * 2,), np.int8)
    out[..., 0::2] = np.where(lo >= 8, lo - 16, lo)
    out[..., 1::2] = np.where(hi >= 8, hi - 16, hi)
    return out


def c1_i8_matmul(M=1024, N=1024, K=1024, seed=0):
    rng = np.random.default_rng(seed)
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (K, N), dtype=np.int8)
    return a, b


def c2_f16_matmul(M=4096, N=4096, K=4096, seed=1):
    rng = np.random.default_rng(seed)
    a = (rng.standard_normal((M, K), dtype=np.float32) * K ** -0.5).astype(np.float16)
    b = (rng.standard_normal((K, N), dtype=np.float32) * K ** -0.5).astype(np.float16)
    return a, b


def c2_f16_batch_matmul(B=32, M=512, N=512, K=128, seed=1):
    rng = np.random.default_rng(seed)
    # Drawn after the 4096^3 pair in the full configuration; the batch tensors are independent
    # of it statistically, so tests that only need them draw them alone.
    a = (rng.standard_normal((B, M, K), dtype=np.float32) * K ** -0.5).astype(np.float16)
    b = (rng.standard_normal((B, K, N), dtype=np.float32) * K ** -0.5).astype(np.float16)
    return a, b


def c3_w8a8(M, N=11008, K=4096, seed=2):
    rng = np.random.default_rng(seed)
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    w = rng.integers(-127, 128, (K, N), dtype=np.int8)
    a_scale = rng.uniform(0.001, 0.02, M).astype(np.float32)
    w_scale = rng.uniform(0.001, 0.02, N).astype(np.float32)
    return a, w, a_scale, w_scale


def c4_w4a16(M, N=11008, K=4096, group=128, seed=3):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K), dtype=np.float32).astype(np.float16)
    wq = pack_int4(rng.integers(-8, 8, (N, K), dtype=np.int8))
    s = rng.uniform(0.005, 0.05, (N, K // group)).astype(np.float16)
    return a, wq, s


def c5_w4a16_sharded(M, world=1, rank=0, N=28672, K=8192, group=128, seed=4):
    """Llama-70B-shaped W4A16; rank r owns weight rows [r*N/world, (r+1)*N/world)."""
    from .sharding import shard_weights
    a, wq, s = c4_w4a16(M, N=N, K=K, group=group, seed=seed)
    wq_r, s_r = shard_weights(wq, s, world, rank)
    return a, wq_r, s_r


def small_int_matrix(rng, shape, dtype, lo, hi):
    """Small-integer valued data (the reference's test generators keep values in a few units so
    float accumulation is exact: tools/testing/e2e/test_utils.c:269-317)."""
    return rng.integers(lo, hi + 1, shape).astype(dtype)
