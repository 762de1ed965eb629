"""Writes the parameter-archive fixtures of tests/test_parameters.py with this repository's own
writer, from the flag lists the reference uses for its parser fixtures
(runtime/src/iree/io/formats/irpa/testdata/generate_irpa_files.sh).

    python tests/golden/make_irpa_golden.py
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from iree_b200 import parameters  # noqa: E402

CASES = {
    "empty": [],
    "single": ["--data=key0=4xf32=100.1"],
    "multiple": ["--data=key0=4xf32=100.1", "--data=key1=5xi8=101"],
    "mixed": ["--data=key0=4xf32=100.1", "--data=key1=5xi8=101", "--splat=key2=i8=102", "--splat=key3=4096x1024xi64=103"],
}

if __name__ == "__main__":
    for name, flags in CASES.items():
        parameters.main(["--quiet", "--output=" + os.path.join(HERE, "irpa", name + ".irpa")] + flags)
        print("wrote", name)
