"""Generates tests/golden/*.npz from the REFERENCE's own ukernels (oracle/_ref, compiled from
the reference sources by `make -C oracle`). Run in a checkout that has the reference:

    python tests/golden/make_golden.py

Each case stores the seeded inputs' recipe (seed, shape, value range), the tile the x86-64
data-tiling would choose, and the output of pack -> iree_uk_mmt4d -> unpack. Shapes follow
runtime/src/iree/builtins/ukernel/tools/mmt4d_test.c:449-504 and
tests/e2e/matmul/generate_e2e_matmul_tests.py:125-198 (small set); value ranges follow
tools/util.c:105-170 (small integers, so float results are exact).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

SHAPES = [(1, 1, 1), (1, 1, 2), (1, 1, 10), (1, 1, 1000), (2, 2, 2), (5, 7, 13),  # mmt4d_test.c
          (9, 9, 9), (6, 13, 3), (15, 37, 7), (81, 19, 41), (1, 10, 10), (10, 1, 10), (10, 10, 1),  # e2e small
          (123, 45, 78), (64, 128, 96)]


def inputs(kind, M, N, K, seed):
    rng = np.random.default_rng(seed)
    if kind == "s8s8s32":
        return (rng.integers(-128, 128, (M, K), dtype=np.int8), rng.integers(-128, 128, (K, N), dtype=np.int8))
    a = rng.integers(-8, 8, (M, K)).astype(np.float16)
    b = rng.integers(-8, 8, (K, N)).astype(np.float16)
    return a, b


def main():
    if not oracle.have_ref():
        oracle.build()
    assert oracle.have_ref(), "oracle/_ref is missing: the reference checkout is needed"
    out = {}
    for kind, t in (("s8s8s32", oracle.TYPE_S8S8S32), ("f16f16f32", oracle.TYPE_F16F16F32)):
        for i, (M, N, K) in enumerate(SHAPES):
            a, b = inputs(kind, M, N, K, 1000 + i)
            tile = oracle.x86_64_tile(t, M, N)
            for cpu_mode in (0, 1):  # generic tiles and the host's architecture tiles must agree
                r = oracle.matmul_ref(t, a, b, tile=tile, cpu_mode=cpu_mode)
                key = "%s_%dx%dx%d" % (kind, M, N, K)
                if key in out:
                    assert (out[key] == r).all(), key
                out[key] = r
            # accumulate flag
            acc0 = np.random.default_rng(77 + i).integers(-5, 5, (M, N)).astype(r.dtype)
            out[key + "_acc"] = oracle.matmul_ref(t, a, b, tile=tile, acc=acc0)
    np.savez_compressed(os.path.join(os.path.dirname(__file__), "matmul_ref.npz"), **out)
    # Nibble order fixture, values read off tests/e2e/linalg/subbyte_to_fp.mlir (i4 -> f32):
    # the tensor dense<[[0,1,2,3,4,5,6,7],[-8,-7,-6,-5,-4,-3,-2,-1]]> : tensor<2x8xi4> stored two
    # per byte with the lower index in the low nibble.
    print("wrote %d arrays" % len(out))


if __name__ == "__main__":
    main()
