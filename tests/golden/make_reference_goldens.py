"""Collect the reference's own golden vectors for the energy+force path into one small fixture.

Reads (from a checkout of the reference): tests/test_data/{atat,dha,bb,water_64}.xyz and
tests/test_data/{atat,dha,bb,water}_{jaxmd,ase}.npz, i.e. the inputs and expected outputs of
tests/test_jaxmd.py:26-256 and tests/test_ase.py:9-142.  The water system is replicated 2x2x2 exactly as the
reference tests do (tests/test_jaxmd.py:195, tests/test_ase.py:62).

Usage: python make_reference_goldens.py /path/to/reference  ->  reference_goldens.npz (next to this script)
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle.so3lr_oracle import read_xyz  # noqa: E402

ref = sys.argv[1]
out = {}
for name in ("atat", "dha", "bb", "water"):
    Z, R, cell = read_xyz(os.path.join(ref, "tests/test_data", ("water_64" if name == "water" else name) + ".xyz"))
    if name == "water":
        Zs, Rs = [], []
        for a in range(2):
            for b in range(2):
                for c in range(2):
                    Zs.append(Z)
                    Rs.append(R + a * cell[0] + b * cell[1] + c * cell[2])
        Z, R, cell = np.concatenate(Zs), np.concatenate(Rs), cell * 2
        out[f"{name}_cell"] = cell
    out[f"{name}_Z"] = Z
    out[f"{name}_R"] = R
    for path in ("jaxmd", "ase"):
        g = np.load(os.path.join(ref, f"tests/test_data/{name}_{path}.npz"))
        out[f"{name}_energy_{path}"] = g["energy"]
        out[f"{name}_forces_{path}"] = g["forces"]
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_goldens.npz"), **out)
print({k: np.shape(v) for k, v in out.items()})
