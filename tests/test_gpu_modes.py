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


GRAPH_CHILD = r"""
import sys, numpy as np, torch
sys.path.insert(0, sys.argv[1])
from so3lr_b200 import workloads as W
from so3lr_b200.engine import System
Z, R, cell = W.water_box(216, 18.7, 5)
R = np.asarray(R, dtype=np.float32)
cellt = torch.tensor(np.asarray(cell, dtype=np.float32), device="cuda")
Rt = torch.tensor(R, device="cuda")
s = System(Z, cell, cutoff_lr=9.0, damping=2.0, lr_format="sparse")
def lists(which):
    _, cnt, _ = s.neighbor_list(Rt, which, 1)
    idx, cnt, _ = s.neighbor_list(Rt, which, cnt)
    i, j = idx[0].long(), idx[1].long()
    d = Rt[j] - Rt[i]
    f = d @ torch.linalg.inv(cellt)
    d = (f - torch.round(f)) @ cellt
    return i, j, d
i, j, d = lists(0)
il, jl, dl = lists(1)
out = {}
def forces(o, i, j, il, jl):
    F = torch.zeros_like(Rt)
    F.index_add_(0, i, o["g_edges"]); F.index_add_(0, j, -o["g_edges"])
    F.index_add_(0, il, o["g_edges_lr"]); F.index_add_(0, jl, -o["g_edges_lr"])
    return F
o = s.graph_eval(i, j, d, il, jl, dl)
out["E_sym"], out["F_sym"] = o["e_atom"].cpu().numpy(), forces(o, i, j, il, jl).cpu().numpy()
out["W_sym"] = (d[:, :, None] * o["g_edges"][:, None, :]).sum(0).cpu().numpy()
# one entry removed: the list is no longer symmetric, the exact scatter kernels must take over inside the same call
keep = torch.ones(i.numel(), dtype=torch.bool, device="cuda"); keep[i.numel() // 3] = False
o = s.graph_eval(i[keep], j[keep], d[keep], il, jl, dl)
out["E_asym"], out["G_asym"] = o["e_atom"].cpu().numpy(), o["g_edges"].cpu().numpy()
ref = s.compute(Rt)
out["E_ref"], out["F_ref"] = ref["energy"].cpu().numpy(), ref["forces"].cpu().numpy()
np.savez(sys.argv[2], **out)
"""


def test_graph_level_call_fast_and_scatter_paths_agree(tmp_path):
    """so3lr_b200_system_graph_eval on a symmetric list (tiled kernels, antisymmetrised per-entry cotangents) against the same
    call kept on the scatter kernels (exact per-entry cotangents): same energies, same forces after the featurizer's transpose,
    same strain derivative; both equal the fused positions -> forces call.  On a list with one entry removed both
    processes must run the scatter kernels and agree entry by entry."""
    def run(name, env):
        out = str(tmp_path / f"{name}.npz")
        e = dict(os.environ)
        for k in ("SO3LR_B200_ATTENTION", "SO3LR_B200_DENSE", "SO3LR_B200_LAYER0", "SO3LR_B200_GRAPH"):
            e.pop(k, None)
        e.update(env)
        subprocess.run([sys.executable, "-c", GRAPH_CHILD, ROOT, out], check=True, timeout=600, env=e)
        return np.load(out)
    fast, slow = run("fast", {}), run("scatter", {"SO3LR_B200_GRAPH": "scatter"})
    for got in (fast, slow):
        assert abs(float(got["E_sym"].sum()) - float(got["E_ref"].sum())) <= 2e-6 * abs(float(got["E_ref"].sum()))
        assert np.abs(got["F_sym"] - got["F_ref"]).max() <= 5e-5
    assert np.abs(fast["E_sym"] - slow["E_sym"]).max() <= 2e-5
    assert np.abs(fast["F_sym"] - slow["F_sym"]).max() <= 5e-5
    assert np.abs(fast["W_sym"] - slow["W_sym"]).max() <= 2e-4 * np.abs(slow["W_sym"]).max()
    assert np.abs(fast["E_asym"] - slow["E_asym"]).max() <= 2e-5
    assert np.abs(fast["G_asym"] - slow["G_asym"]).max() <= 5e-5
