"""Generates tests/golden/reference_outputs.npz.

Runs every case of cases.py through oracle/_ref/libogle_ref.so - the reference's
own shader and functor source compiled for the CPU - and stores the outputs.
Needs the reference tree at build time of that library; run from the repo root:

    make -C oracle ref && python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from oracle import oracle  # noqa: E402
import cases  # noqa: E402


def main():
    ref = oracle.load("reference")
    out = {}
    for name, make in sorted(cases.CASES.items()):
        out[name] = cases.run_case(ref, make())
        print(f"{name}: {out[name].shape}")
    path = os.path.join(HERE, "reference_outputs.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
