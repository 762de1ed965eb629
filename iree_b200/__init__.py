"""B200 (sm_100a) drop-in for IREE's contraction dispatches.

The product is two artefacts built by :mod:`iree_b200.build`: a cubin holding the hand-written
kernels and ``libiree_b200.so``, the C ABI declared in ``include/iree_b200.h``. This package is
the thin Python host side over that ABI (:mod:`iree_b200.runtime`) plus the input generators of
the benchmark configurations (:mod:`iree_b200.workloads`). There is no CPU execution path:
without the built library or without a GPU every compute call raises.
"""
from .runtime import (Context, DeviceBuffer, IreeB200Error, MatmulParams, KIND_F16, KIND_BF16, KIND_I8,
                      EPILOGUE_CAST, EPILOGUE_ACCUMULATOR, EPILOGUE_REQUANT_F16, RHS_KN, RHS_NK,
                      FLAG_FORCE_GENERIC, FLAG_DEVICE_TENSORMAPS, FLAG_PAIR_CTAS, FLAG_SINGLE_CTA, WORKSPACE_BYTES, library, library_path,
                      cubin_path, last_error, W4A16Params, W4A16_AUTO, W4A16_DECODE, W4A16_GEMM, W4A16_GENERIC, W4A16_GEMM_WT, W4A16_DECODE_TC)

__all__ = ["Context", "DeviceBuffer", "IreeB200Error", "MatmulParams", "KIND_F16", "KIND_BF16", "KIND_I8",
           "EPILOGUE_CAST", "EPILOGUE_ACCUMULATOR", "EPILOGUE_REQUANT_F16", "RHS_KN", "RHS_NK",
           "FLAG_FORCE_GENERIC", "FLAG_DEVICE_TENSORMAPS", "FLAG_PAIR_CTAS", "FLAG_SINGLE_CTA", "WORKSPACE_BYTES", "library", "library_path",
           "cubin_path", "last_error", "W4A16Params", "W4A16_AUTO", "W4A16_DECODE", "W4A16_GEMM",
           "W4A16_GENERIC", "W4A16_GEMM_WT", "W4A16_DECODE_TC"]
