"""Collect the reference's own golden vectors for the energy+force path into one small fixture.

Reads (from a checkout of the reference): tests/test_data/{atat,dha,bb,water_64}.xyz and
tests/test_data/{atat,dha,bb,water}_{jaxmd,ase}.npz, i.e. the inputs and expected outputs of
tests/test_jaxmd.py:26-256 and tests/test_ase.py:9-142.  The water system is replicated 2x2x2 exactly as the
reference tests do (tests/test_jaxmd.py:195, tests/test_ase.py:62).

The one vector the reference holds for the dipole and the Hirshfeld ratios is collected too: the printed float32 output of
`So3lr(calculate_forces=True, lr_cutoff=100)` for frame 49 of examples/data/ethanol.npz
(examples/evaluate_so3lr_on_dataset.ipynb, the cell `pprint(output)` after the 50-frame loop; the loop leaves its last frame in `output`).

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
# ethanol frame 49: inputs from the data file, expected outputs parsed from the notebook's stored cell output
import json
import re

eth = np.load(os.path.join(ref, "examples/data/ethanol.npz"))
out["ethanol_Z"] = eth["atomic_numbers"][49].astype(np.int32)
out["ethanol_R"] = eth["positions"][49].astype(np.float64)
nb = json.load(open(os.path.join(ref, "examples/evaluate_so3lr_on_dataset.ipynb")))
text = None
for cell in nb["cells"]:
    if "pprint(output)" in "".join(cell["source"]):
        text = "".join("".join(o.get("text", [])) for o in cell.get("outputs", []))
assert text is not None, "notebook cell with pprint(output) not found"


def _array(key):
    m = re.search(r"'%s': Array\((.*?), *dtype=float32\)" % key, text, re.S)
    return np.array(eval(m.group(1).replace("\n", " ")), dtype=np.float32)


out["ethanol_energy"] = _array("energy")[0]
out["ethanol_dipole_vec"] = _array("dipole_vec")[0]
out["ethanol_forces"] = _array("forces")[:9]
out["ethanol_hirshfeld_ratios"] = _array("hirshfeld_ratios")[:9]
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_goldens.npz"), **out)
print({k: np.shape(v) for k, v in out.items()})
