"""Regenerates tests/golden/types_kat.txt from the REFERENCE's own host codecs.

Run in a container where the reference tree is mounted:  python tests/golden/make_golden.py
It builds oracle/_ref/ref_types_kat (a printer compiled against the reference's
cccc/types.h, see oracle/Makefile), feeds it a fixed list of probe floats and stores its
text output.  The committed file is what the CPU tests pin the oracle against; the
reference tree is not needed to run those tests.
"""
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def probes() -> np.ndarray:
    edge = [
        0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00000, 0x7FFFFFFF, 0x00000001, 0x807FFFFF,
        0x3F800000, 0xBF800000, 0x3E800000, 0x3E7FFFFF, 0x3F400000, 0x3F3FFFFF, 0x3FA00000, 0x3FE00000, 0x40200000,
        0x40600000, 0x40A00000, 0x409FFFFF, 0x40C00000, 0x43E00000, 0x43DFFFFF, 0x43E00001, 0x43F00000, 0x44000000,
        0x47600000, 0x475FFFFF, 0x47600001, 0x47700000, 0x47800000, 0x38800000, 0x387FFFFF, 0x37800000, 0x37000000,
        0x36FFFFFF, 0x3C800000, 0x3C7FFFFF, 0x3B000000, 0x3AFFFFFF, 0x3A800000, 0x33800000, 0x7F7FFFFF, 0xFF7FFFFF,
    ]
    rng = np.random.default_rng(20240607)
    any_bits = rng.integers(0, 2**32, size=400, dtype=np.uint64).astype(np.uint32)
    # values in the ranges the codecs resolve: N(0,1)*{0.02, 1, 6, 448, 57344} and tiny ones
    vals = np.concatenate([
        rng.standard_normal(150) * s for s in (1e-5, 1e-3, 0.02, 1.0, 6.0, 448.0, 57344.0)
    ]).astype(np.float32)
    return np.concatenate([np.array(edge, np.uint32), any_bits, vals.view(np.uint32)])


def main() -> None:
    subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "ref"])
    exe = os.path.join(ROOT, "oracle", "_ref", "ref_types_kat")
    text = "\n".join(f"{int(p):08x}" for p in probes()) + "\n"
    out = subprocess.run([exe], input=text, capture_output=True, text=True, check=True).stdout
    with open(os.path.join(HERE, "types_kat.txt"), "w") as f:
        f.write(out)
    print("wrote", os.path.join(HERE, "types_kat.txt"), len(out), "bytes")


if __name__ == "__main__":
    main()
