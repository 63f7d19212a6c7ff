"""Writes tests/golden/reference_kernel_outputs.npz: what the reference's own kernels give on the cases
of tests/reference_cases.py.  Needs a GPU and the library that baseline/reference_kernels.py builds from
the reference's unmodified CUDA sources.

    python baseline/reference_kernels.py --build <reference checkout>
    python tests/golden/make_reference_kernel_outputs.py [--out FILE]

The inputs are not stored: every case makes them again from its seed.
"""
import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import reference_cases as RC                               # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "reference_kernel_outputs.npz"))
    a = ap.parse_args()
    out = {}
    for c in RC.all_cases():
        got = c.reference(c.make())
        for k, v in got.items():
            out[f"{c.name}/{k}"] = np.asarray(v)
        print("ran", c.name, flush=True)
    np.savez_compressed(a.out, **out)
    print("wrote", a.out, os.path.getsize(a.out), "bytes")


if __name__ == "__main__":
    main()
