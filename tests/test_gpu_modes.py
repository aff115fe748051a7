"""The kernel variants that environment switches select (read once per process, hence child processes): every variant of
the attention kernels, the dense blocks and the first layer gives the same energies and forces as the default build-up.

  SO3LR_B200_ATTENTION = tcf | mma | simt  (default: tiled tcgen05 kernels in both directions)
  SO3LR_B200_DENSE     = mma | simt        (default: tcgen05 post-attention blocks and heads)
  SO3LR_B200_LAYER0    = generic           (default: per-element-pair tables)
"""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
from so3lr_b200 import workloads as W
from so3lr_b200.engine import System
g = np.load(sys.argv[1] + "/tests/golden/reference_goldens.npz")
out = {}
Z, R, cell = W.water_box(216, 18.7, 5)
s = System(Z, cell, cutoff_lr=9.0, damping=2.0, skin=0.5)
s.enable_virial(True)
o = s.compute(torch.tensor(np.asarray(R, dtype=np.float32), device="cuda"))
out["E_w"], out["F_w"], out["W_w"] = o["energy"].cpu().numpy(), o["forces"].cpu().numpy(), o["virial"].cpu().numpy()
Zm, Rm = g["bb_Z"], np.asarray(g["bb_R"] - g["bb_R"].mean(0), dtype=np.float32)
o = System(Zm, None, cutoff_lr=12.0, damping=2.0).compute(torch.tensor(Rm, device="cuda"))
out["E_m"], out["F_m"] = o["energy"].cpu().numpy(), o["forces"].cpu().numpy()
np.savez(sys.argv[2], **out)
"""


def _run(tmp_path, name, env):
    out = str(tmp_path / f"{name}.npz")
    e = dict(os.environ)
    for k in ("SO3LR_B200_ATTENTION", "SO3LR_B200_DENSE", "SO3LR_B200_LAYER0"):
        e.pop(k, None)
    e.update(env)
    subprocess.run([sys.executable, "-c", CHILD, ROOT, out], check=True, timeout=600, env=e)
    return np.load(out)


def test_kernel_variants_agree(tmp_path):
    ref = _run(tmp_path, "default", {})
    variants = {"attention_tcf": {"SO3LR_B200_ATTENTION": "tcf"}, "attention_mma": {"SO3LR_B200_ATTENTION": "mma"},
                "attention_simt": {"SO3LR_B200_ATTENTION": "simt"}, "dense_mma": {"SO3LR_B200_DENSE": "mma"},
                "dense_simt": {"SO3LR_B200_DENSE": "simt"},
                "layer0_generic": {"SO3LR_B200_LAYER0": "generic"}}
    for name, env in variants.items():
        got = _run(tmp_path, name, env)
        for k in ("E_w", "E_m"):
            assert abs(float(got[k].sum()) - float(ref[k].sum())) <= 2e-6 * abs(float(ref[k].sum())), (name, k)
        for k in ("F_w", "F_m"):
            assert np.abs(got[k] - ref[k]).max() <= 5e-5, (name, k, np.abs(got[k] - ref[k]).max())
        assert np.abs(got["W_w"] - ref["W_w"]).max() <= 2e-4 * np.abs(ref["W_w"]).max(), name
