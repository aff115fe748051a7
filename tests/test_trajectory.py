"""Frame writer of the MD loop (so3lr_b200/trajectory.py) on host tensors: formats, subsets, error behaviour.
The reference's writers: so3lr/cli/so3lr_md.py:227-486."""
import os

import numpy as np
import pytest
import torch

from so3lr_b200.trajectory import FrameSink, read_extxyz


def _frames(n=7, k=5, seed=0):
    rng = np.random.default_rng(seed)
    return [dict(R=rng.normal(size=(n, 3)).astype(np.float32), P=rng.normal(size=(n, 3)).astype(np.float32),
                 q=rng.normal(size=n).astype(np.float32), h=rng.random(n).astype(np.float32), d=rng.normal(size=3).astype(np.float32),
                 box=np.diag([10.0 + i, 11.0, 12.0])) for i in range(k)]


def test_extxyz_round_trip_with_observables_and_subset(tmp_path):
    Z = np.array([8, 1, 1, 6, 7, 16, 17])
    fr = _frames()
    path = tmp_path / "traj" / "out.xyz"
    idx = [0, 3, 4, 6]
    with FrameSink(path, Z, "extxyz", observables=("partial_charges", "hirshfeld_ratios", "dipole_vec"), indices=idx, slots=2) as sink:
        for i, f in enumerate(fr):
            sink.append(torch.tensor(f["R"]), torch.tensor(f["P"]), f["box"],
                        dict(partial_charges=torch.tensor(f["q"]), hirshfeld_ratios=torch.tensor(f["h"]), dipole_vec=torch.tensor(f["d"])),
                        step=10 * (i + 1))
    assert sink.frames_written == len(fr)
    back = read_extxyz(path)
    assert len(back) == len(fr)
    for f, b in zip(fr, back):
        assert b["n"] == 4 and b["symbols"] == ["O", "C", "N", "Cl"]
        np.testing.assert_allclose(b["pos"], f["R"][idx], atol=1e-7)
        np.testing.assert_allclose(b["momenta"], f["P"][idx], atol=1e-7)
        np.testing.assert_allclose(b["charges"], f["q"][idx], atol=1e-7)
        np.testing.assert_allclose(b["hirsh_ratios"], f["h"][idx], atol=1e-7)
        np.testing.assert_allclose(b["cell"], f["box"])
        np.testing.assert_allclose([float(v) for v in b["info"]["dipole_vec"].split()], f["d"], atol=1e-7)
    assert [int(b["info"]["step"]) for b in back] == [10, 20, 30, 40, 50]
    # the oracle's xyz reader (lattice + positions) parses the same file
    from oracle.so3lr_oracle import read_xyz
    Z0, R0, cell0 = read_xyz(str(path))
    assert list(Z0) == [8, 6, 7, 17]
    np.testing.assert_allclose(R0, fr[0]["R"][idx], atol=1e-7)
    np.testing.assert_allclose(cell0, fr[0]["box"])


def test_npy_store_grows_frame_by_frame_and_is_memory_mappable(tmp_path):
    Z = np.ones(7, dtype=int)
    fr = _frames(k=9)
    d = tmp_path / "store"
    sink = FrameSink(d, Z, "npy", observables=("partial_charges", "dipole_vec"))
    for f in fr:
        sink.append(torch.tensor(f["R"]), torch.tensor(f["P"]), f["box"], dict(partial_charges=torch.tensor(f["q"]), dipole_vec=torch.tensor(f["d"])))
    sink.close()
    pos = np.load(d / "positions.npy", mmap_mode="r")
    assert pos.shape == (9, 7, 3) and pos.dtype == np.float32
    np.testing.assert_array_equal(pos, np.stack([f["R"] for f in fr]))
    np.testing.assert_array_equal(np.load(d / "momenta.npy"), np.stack([f["P"] for f in fr]))
    np.testing.assert_array_equal(np.load(d / "partial_charges.npy"), np.stack([f["q"] for f in fr]))
    np.testing.assert_array_equal(np.load(d / "dipole_vec.npy"), np.stack([f["d"] for f in fr]))
    np.testing.assert_allclose(np.load(d / "box.npy"), np.stack([f["box"] for f in fr]))


def test_existing_output_and_missing_observables_fail_loudly(tmp_path):
    Z = np.ones(3, dtype=int)
    p = tmp_path / "a.xyz"
    FrameSink(p, Z).close()
    with pytest.raises(RuntimeError, match="File exists"):
        FrameSink(p, Z)
    sink = FrameSink(p, Z, observables=("partial_charges",), exist_ok=True)
    with pytest.raises(KeyError):
        sink.append(torch.zeros(3, 3), torch.zeros(3, 3), None, {})
    sink.close()
    sink.close()                                   # idempotent
    with pytest.raises(RuntimeError, match="closed"):
        sink.append(torch.zeros(3, 3), torch.zeros(3, 3), None, dict(partial_charges=torch.zeros(3)))
    with pytest.raises(ValueError):
        FrameSink(tmp_path / "b", Z, fmt="hdf5")
