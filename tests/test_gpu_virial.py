"""Strain derivative of the energy (virial / stress) accumulated by the force kernels, against the oracle's autograd
derivative with respect to a homogeneous strain (float64).

Tolerances: float32 kernels; the virial is a sum of dR (x) f over all pairs, so its error scales with the force error
(1e-4 eV/A bar) times the interaction range times the square root of the pair count: 1e-5 of sum_i |R_i - <R>| |F_i| plus
2e-4 eV absolute is used (measured errors are printed by the asserts when they fail).
"""
import numpy as np
import pytest
import torch

from oracle import so3lr_oracle as O

pytestmark = pytest.mark.gpu


def _tol(R, F):
    return 2e-4 + 1e-5 * float((np.linalg.norm(R - R.mean(0), axis=1) * np.linalg.norm(F, axis=1)).sum())


@pytest.mark.parametrize("name", ["atat", "dha"])
def test_virial_of_molecules_matches_oracle(oracle_params, reference_goldens, name):
    from so3lr_b200.engine import System
    g = reference_goldens
    Z = g[f"{name}_Z"]
    R = np.asarray(g[f"{name}_R"] - g[f"{name}_R"].mean(0), dtype=np.float32)
    ref = O.energy_forces(oracle_params, R.astype(np.float64), Z, None, cutoff_lr=12.0, damping=2.0)
    s = System(Z, None, cutoff_lr=12.0, damping=2.0)
    plain = s.compute(torch.tensor(R, device="cuda"))["forces"].cpu().numpy()
    s.enable_virial(True)
    out = s.compute(torch.tensor(R, device="cuda"))
    W = out["virial"].cpu().numpy()
    assert "stress" not in out
    # forces do not change when the virial is on (up to the summation order of the long-range scatter)
    np.testing.assert_allclose(out["forces"].cpu().numpy(), plain, atol=5e-6)
    np.testing.assert_allclose(W, W.T, atol=1e-12)
    err = np.abs(W - ref["virial"]).max()
    assert err <= _tol(R, ref["forces"]), (err, _tol(R, ref["forces"]))
    # free space: dE/d eps = - sum_i R_i (x) F_i
    F = out["forces"].double().cpu().numpy()
    np.testing.assert_allclose(W, -(R.astype(np.float64)[:, :, None] * F[:, None, :]).sum(0), atol=5e-4)
    s.enable_virial(False)
    assert "virial" not in s.compute(torch.tensor(R, device="cuda"))


def test_virial_of_periodic_water_matches_oracle(oracle_params, reference_goldens):
    from so3lr_b200.engine import System
    g = reference_goldens
    Z, R, cell = g["water_Z"], np.asarray(g["water_R"], dtype=np.float32), g["water_cell"]
    ref = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=12.0, damping=2.0)
    vol = abs(np.linalg.det(cell))
    for skin in (0.0, 0.7):
        s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=skin)
        s.enable_virial(True)
        out = s.compute(torch.tensor(R, device="cuda"))
        W = out["virial"].cpu().numpy()
        err = np.abs(W - ref["virial"]).max()
        assert err <= _tol(R, ref["forces"]), (skin, err, _tol(R, ref["forces"]), np.abs(ref["virial"]).max())
        np.testing.assert_allclose(out["stress"].cpu().numpy(), W / vol, rtol=1e-12)
    # finite strain: the energy of the strained box changes by trace(W eps) to first order
    eps = 2e-4 * np.array([[1.0, 0.3, 0.0], [0.3, -0.5, 0.2], [0.0, 0.2, 0.7]])
    Es = []
    for sign in (+1, -1):
        A = np.eye(3) + sign * eps
        ss = System(Z, cell @ A.T, cutoff_lr=12.0, damping=2.0)
        Es.append(float(ss.compute(torch.tensor((R.astype(np.float64) @ A.T).astype(np.float32), device="cuda"))["energy"].sum()))
    dE = (Es[0] - Es[1]) / 2
    assert abs(dE - float((W * eps).sum())) < 2e-3 + 2e-3 * abs(dE), (dE, float((W * eps).sum()))


def test_virial_in_a_triclinic_cell(oracle_params):
    from so3lr_b200 import workloads as Wl
    from so3lr_b200.engine import System
    Z, R, cell = Wl.water_box(216, 18.7, 5, jitter=0.03)
    shear = np.array([[1.0, 0.0, 0.0], [0.18, 1.0, 0.0], [-0.1, 0.12, 1.0]])
    cell = np.asarray(cell, dtype=np.float64) @ shear
    R = (np.asarray(R, dtype=np.float64) @ shear).astype(np.float32)
    ref = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=8.0, damping=2.0)
    s = System(Z, cell, cutoff_lr=8.0, damping=2.0)
    s.enable_virial(True)
    W = s.compute(torch.tensor(R, device="cuda"))["virial"].cpu().numpy()
    err = np.abs(W - ref["virial"]).max()
    assert err <= _tol(R, ref["forces"]), (err, _tol(R, ref["forces"]))


def test_decomposed_virial_matches_single_device(reference_goldens):
    from so3lr_b200 import domain as D
    from so3lr_b200.engine import System
    from test_gpu_domain import _run_threads
    g = reference_goldens
    Z, R, cell = g["water_Z"], np.asarray(g["water_R"], dtype=np.float32), g["water_cell"]
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=0.5)
    s.enable_virial(True)
    W_ref = s.compute(torch.tensor(R, device="cuda"))["virial"].cpu().numpy()

    def fn(comm, rank):
        be = D.CudaBackend(cutoff_lr=12.0, damping=2.0, skin=0.5, device=0)
        be.enable_virial(True)
        dom = D.DomainSystem(comm, be, Z, R, cell, skin=0.5, cutoff_lr=12.0, device="cuda:0")
        dom.compute(check_rebuild=False)
        return dom.virial().cpu().numpy()

    for world in (2, 3):
        res = _run_threads(world, fn)
        for W in res:
            assert np.abs(W - W_ref).max() < 5e-3, np.abs(W - W_ref).max()
            np.testing.assert_array_equal(W, res[0])


class _Atoms:
    def __init__(self, Z, R, cell):
        self.Z, self.R, self.cell = Z, R, cell

    def get_atomic_numbers(self): return self.Z
    def get_positions(self): return self.R
    def get_cell(self): return self.cell
    def get_pbc(self): return np.array([self.cell is not None] * 3)


@pytest.mark.parametrize("calculate_stress", [True, False])
def test_ase_calculator_stress(reference_goldens, calculate_stress):
    """Mirror of the reference's tests/test_ase.py:145-172: Voigt stress of the 1536-atom water box, or NotImplementedError."""
    from so3lr_b200 import So3lrCalculator
    g = reference_goldens
    atoms = _Atoms(g["water_Z"], np.asarray(g["water_R"], dtype=np.float64), np.asarray(g["water_cell"], dtype=np.float64))
    calc = So3lrCalculator(calculate_stress=calculate_stress)
    if calculate_stress:
        stress = calc.get_stress(atoms)
        assert stress.shape == (6,)
        assert np.isfinite(stress).all() and np.abs(stress).max() < 0.1        # a liquid near ambient pressure: |stress| << 0.1 eV/A^3
        f = calc.get_forces(atoms)
        np.testing.assert_allclose(f, g["water_forces_jaxmd"], atol=5e-4)
    else:
        with pytest.raises(NotImplementedError):
            calc.get_stress(atoms)
