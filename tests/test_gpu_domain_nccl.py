"""Two ranks on two GPUs over NCCL (skipped on a single-GPU box): same checks as the threaded test, real transport."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_nccl_run_matches_single_device(tmp_path):
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    out = str(tmp_path / "dd.npz")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dd_nccl_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                    "--master-port", "29517", worker, out], check=True, timeout=600, env=env)
    r = np.load(out)
    Z, R, cell = W.water_box(1000, 31.0, 21, jitter=0.02)
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=0.0)
    a = s.compute(torch.tensor(np.asarray(R, dtype=np.float32), device="cuda"))
    assert abs(float(r["E0"]) - float(a["energy"].sum())) <= 1e-5 * abs(float(r["E0"]))
    assert np.abs(r["F0"] - a["forces"].cpu().numpy()).max() <= 1e-4
    b = s.compute(torch.tensor(r["R1"], device="cuda"))
    assert abs(float(r["E1"]) - float(b["energy"].sum())) <= 1e-5 * abs(float(r["E1"]))
    assert np.abs(r["F1"] - b["forces"].cpu().numpy()).max() <= 1e-4
    assert int(r["rebuilds"]) >= 1
    s.set_kspace((32, 32, 32), 2.0, "pme")
    c = s.compute(torch.tensor(r["R1"], device="cuda"))
    assert abs(float(r["Ek"]) - float(c["energy"].sum())) <= 1e-5 * abs(float(r["Ek"]))
    assert np.abs(r["Fk"] - c["forces"].cpu().numpy()).max() <= 1e-4
