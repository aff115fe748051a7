"""The reciprocal-space (Ewald) oracle: known answers and the properties that pin it without a reference vector.
The reference's tests hold no vector for its k-space path (so3lr/cli/so3lr_md.py:1392-1428)."""
import math

import numpy as np
import pytest
import torch

from oracle import kspace_oracle as K
from oracle import so3lr_oracle as O


def test_madelung_constants_of_rock_salt_and_caesium_chloride():
    fcc = np.array([[0, 0, 0], [.5, .5, 0], [.5, 0, .5], [0, .5, .5]])
    R = np.concatenate([fcc, fcc + [.5, 0, 0]]) % 1.0
    q = np.array([1.0] * 4 + [-1.0] * 4)
    for s, n in ((0.12, 24), (0.2, 16)):                     # two splittings, one answer
        E = K.point_charge_ewald(R, q, np.eye(3), s, (n, n, n), 6 * s * math.sqrt(2))
        assert abs(-E / 4 * 0.5 - 1.7475645946) < 1e-9
    E = K.point_charge_ewald(np.array([[0, 0, 0], [.5, .5, .5]]), np.array([1.0, -1.0]), np.eye(3), 0.15, (20, 20, 20), 1.5)
    assert abs(-E * math.sqrt(3) / 2 - 1.76267477) < 1e-8


def test_grid_shape_and_indices():
    cell = np.diag([12.42, 12.42, 24.84])
    assert K.ewald_grid_shape(cell, 1.0) == (13, 13, 25)
    h = K.grid_indices((4, 5, 1))
    assert len(h) == 4 * 5 - 1
    assert h[:, 0].min() == -2 and h[:, 0].max() == 1 and h[:, 1].min() == -2 and h[:, 1].max() == 2 and (h[:, 2] == 0).all()


def test_reciprocal_energy_of_a_charged_triclinic_cell_does_not_depend_on_the_smearing():
    """Smeared charges in a neutralising background: pair part (erf-damped as in the model, minus the k-space part) summed
    directly over all images + reciprocal part (with its self and background terms) give the same total for every smearing."""
    rng = np.random.default_rng(7)
    cell = np.array([[7.0, 0.0, 0.0], [1.0, 6.5, 0.0], [0.5, -0.8, 7.5]])
    R = rng.random((9, 3)) @ cell
    q = rng.normal(size=9); q += (0.7 - q.sum()) / 9            # net charge 0.7
    sig = O.SIGMA_COULOMB / 2.0                                  # a narrower damping so that images converge quickly
    tot = []
    for s in (0.9, 1.2):
        a = 1.0 / (math.sqrt(2.0) * s)
        e = 0.0
        for n in np.ndindex(7, 7, 7):
            shift = (np.array(n) - 3) @ cell
            d = np.linalg.norm(R[None] + shift - R[:, None], axis=-1)
            m = d > 1e-9
            qq = (q[:, None] * q[None, :])[m]
            e += 0.5 * K.KE * np.sum(qq * np.array([(math.erf(x / sig) - math.erf(x * a)) / x for x in d[m]]))
        ek = K.reciprocal_energy(torch.tensor(R), torch.tensor(q), torch.tensor(cell), (36, 36, 36), s).sum().item()
        tot.append(e + ek)
    # the k = 0 components of the two parts add up to -ke pi sigma^2 Q^2 / (2 V) for every s: the pair part carries
    # +ke pi s^2 Q^2 / V of it in its direct sum, the reciprocal part's background term the opposite
    assert abs(tot[0] - tot[1]) < 1e-6 * abs(tot[0]) + 1e-6


def test_model_energy_and_forces_with_kspace_do_not_depend_on_the_smearing(oracle_params, reference_goldens):
    g = reference_goldens
    R, Z, cell = g["water_R"], g["water_Z"], g["water_cell"]
    n = 192                                                     # the first 64 molecules of the supercell in their own cell
    cell1 = cell / 2.0
    R, Z = R[:n], Z[:n]
    outs = []
    for s, lam in ((0.9, 0.55), (1.15, 0.7)):
        shape = K.ewald_grid_shape(cell1, lam)
        outs.append(O.energy_forces(oracle_params, R, Z, cell1, cutoff_lr=6.0, damping=2.0, k_grid=shape, k_smearing=s))
    assert abs(outs[0]["energy"] - outs[1]["energy"]) < 2e-5
    np.testing.assert_allclose(outs[0]["forces"], outs[1]["forces"], atol=2e-5)
    np.testing.assert_allclose(outs[0]["virial"], outs[1]["virial"], atol=5e-4)
    # only the electrostatic term changes when the split is switched on
    plain = O.energy_forces(oracle_params, R, Z, cell1, cutoff_lr=6.0, damping=2.0)
    for k in ("dispersion_energy", "zbl_repulsion", "partial_charges", "hirshfeld_ratios"):
        np.testing.assert_allclose(plain[k], outs[0][k], atol=1e-12)
    assert np.abs(plain["electrostatic_energy"] - outs[0]["electrostatic_energy"]).max() > 1e-3


def test_mesh_variant_converges_to_the_direct_sum_with_the_fourth_power_of_the_spacing():
    rng = np.random.default_rng(3)
    cell = np.array([[12.4, 0.0, 0.0], [1.0, 12.0, 0.0], [0.5, -0.7, 13.0]])
    R = rng.random((60, 3)) @ cell
    q = rng.normal(size=60); q -= q.mean()
    qt, ct, s = torch.tensor(q), torch.tensor(cell), 1.2

    def run(fn, shape):
        Rt = torch.tensor(R, requires_grad=True)
        eps = torch.zeros(3, 3, dtype=torch.float64, requires_grad=True)
        e = fn(Rt + Rt @ eps.T, qt, ct + ct @ eps.T, shape, s).sum()
        gR, gE = torch.autograd.grad(e, (Rt, eps))
        return e.item(), gR.numpy(), gE.numpy()

    e0, g0, v0 = run(K.reciprocal_energy, (40, 40, 40))
    err = []
    for n in (16, 32, 64):
        e, g, v = run(K.reciprocal_energy_mesh, (n, n, n))
        err.append((abs(e - e0), np.abs(g - g0).max(), np.abs(v - v0).max()))
    for a, b in zip(err[:-1], err[1:]):
        assert b[0] < a[0] / 10 and b[1] < a[1] / 8 and b[2] < a[2] / 8, err       # 16 per halving in the limit
    assert err[-1][0] < 2e-3 and err[-1][1] < 2e-3
    assert K.mesh_grid_shape(cell, 0.8) == (16, 16, 32) and K.mesh_grid_shape(np.eye(3) * 215.0, 1.0) == (256, 256, 256)
