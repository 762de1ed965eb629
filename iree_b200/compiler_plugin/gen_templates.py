"""Writes src/TensorMapTemplates.inc: the tensor-map templates the rewrite pass embeds as a constant.

    python iree_b200/compiler_plugin/gen_templates.py [output path]

A template is an encoded 128-byte CUtensorMap that fixes element type, rank, swizzle and fill mode;
the device-side builders (exports b200_encode_tensormaps / b200_encode_tensormap) patch address,
extents, strides and box. Encoding needs the CUDA driver (cuTensorMapEncodeTiled), so this runs on
a machine with a GPU; the bytes do not depend on which one. Row order: IREE_B200_TEMPLATE_* of
include/iree_b200.h.
"""
import ctypes as C
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import iree_b200 as ib  # noqa: E402
from iree_b200 import runtime as rt  # noqa: E402

NAMES = ["f16, 128-byte swizzle, rank 3", "bf16, 128-byte swizzle, rank 3", "u8, 128-byte swizzle, rank 3",
         "u8, 64-byte swizzle, rank 3", "f16, no swizzle, rank 2", "u64, no swizzle, rank 2"]


def main() -> int:
    out = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "src", "TensorMapTemplates.inc")
    ctx = ib.Context(0)
    raw = C.create_string_buffer(128 * len(NAMES))
    rt.check(ib.library().iree_b200_tensormap_templates(ctx.handle, raw))
    ctx.close()
    lines = ["// Tensor-map templates (one encoded CUtensorMap per kind), written by gen_templates.py.",
             "// Rows follow IREE_B200_TEMPLATE_* of the runtime library's header.",
             "static const unsigned char kTensorMapTemplates[%d][128] = {" % len(NAMES)]
    for i, name in enumerate(NAMES):
        row = raw.raw[128 * i:128 * (i + 1)]
        lines.append("    {  // %d: %s" % (i, name))
        for k in range(0, 128, 16):
            lines.append("        " + ", ".join("0x%02x" % b for b in row[k:k + 16]) + ",")
        lines.append("    },")
    lines.append("};")
    with open(out, "w") as f:
        f.write("\n".join(lines) + "\n")
    print("wrote", out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
