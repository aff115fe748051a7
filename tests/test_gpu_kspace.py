"""Reciprocal-space (Ewald) Coulomb part on the device against the float64 oracle (oracle/kspace_oracle.py), through the C ABI
(System.set_kspace -> so3lr_b200_system_set_kspace) and through the reference-facing energy function (`k_grid`, `k_smearing`
keyword arguments, so3lr/jaxmd_utils.py:39-47).  The reference's tests hold no vector for this path; the oracle is pinned by the
Madelung constants and by the independence of the total from the smearing (tests/test_kspace_oracle.py).

Tolerances: the BASELINE float32 bars, E 1e-5 relative and F 1e-4 eV/A max-abs; virial as in test_gpu_virial.py.
"""
import numpy as np
import pytest
import torch

from oracle import kspace_oracle as K
from oracle import so3lr_oracle as O

pytestmark = pytest.mark.gpu


def _water192(g):
    return g["water_Z"][:192], np.asarray(g["water_R"][:192], dtype=np.float32), np.asarray(g["water_cell"], dtype=np.float64) / 2.0


def _vir_tol(R, F):
    return 2e-4 + 1e-5 * float((np.linalg.norm(R - R.mean(0), axis=1) * np.linalg.norm(F, axis=1)).sum())


def _check(out, ref, R):
    E = float(out["energy"].sum())
    assert abs(E - ref["energy"]) < 1e-5 * abs(ref["energy"]), (E, ref["energy"])
    dF = np.abs(out["forces"].cpu().numpy() - ref["forces"]).max()
    assert dF < 1e-4, dF
    np.testing.assert_allclose(out["partial_charges"].cpu().numpy(), ref["partial_charges"], atol=1e-5)
    if "virial" in out:
        err = np.abs(out["virial"].cpu().numpy() - ref["virial"]).max()
        assert err <= _vir_tol(R, ref["forces"]), (err, _vir_tol(R, ref["forces"]))


@pytest.mark.parametrize("smearing,lam", [(1.0, 0.6), (1.3, 0.8)])
def test_small_cell_matches_oracle(oracle_params, reference_goldens, smearing, lam):
    from so3lr_b200.engine import System
    Z, R, cell = _water192(reference_goldens)
    shape = K.ewald_grid_shape(cell, lam)
    ref = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=6.0, damping=2.0, k_grid=shape, k_smearing=smearing)
    s = System(Z, cell, cutoff_lr=6.0, damping=2.0)
    s.enable_virial(True)
    s.set_kspace(shape, smearing)
    out = s.compute(torch.tensor(R, device="cuda"))
    _check(out, ref, R)
    # electrostatic term alone (a periodic context orders its atoms spatially, so a pair's energy may be booked on the other atom
    # of the pair than in the oracle: compare the sum)
    ec = float(s.aux()["electrostatic_energy"].double().sum())
    assert abs(ec - ref["electrostatic_energy"].sum()) < 2e-4, (ec, ref["electrostatic_energy"].sum())
    # switched off again, the context returns to the truncated pair sum
    s.set_kspace(None)
    plain = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=6.0, damping=2.0)
    _check(s.compute(torch.tensor(R, device="cuda")), plain, R)


def test_periodic_water_with_skin_and_odd_grid_matches_oracle(oracle_params, reference_goldens):
    from so3lr_b200.engine import System
    g = reference_goldens
    Z, R, cell = g["water_Z"], np.asarray(g["water_R"], dtype=np.float32), np.asarray(g["water_cell"], dtype=np.float64)
    shape, smearing = (21, 20, 19), 2.4          # even and odd extents; 20 has the unpaired index -10
    ref = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=12.0, damping=2.0, k_grid=shape, k_smearing=smearing)
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=0.8)
    s.enable_virial(True)
    s.set_kspace(np.zeros(shape), torch.tensor([smearing]))
    Rt = torch.tensor(R, device="cuda")
    _check(s.compute(Rt), ref, R)
    # positions shifted by whole lattice vectors (unwrapped trajectories): same result, up to the rounding of the shifted
    # float32 positions themselves (4-8e-6 A at 50-75 A, times O-H force constants of ~50 eV/A^2)
    shift = np.zeros_like(R); shift[::3] += cell[0].astype(np.float32) * 2; shift[1::3] -= cell[2].astype(np.float32)
    out2 = s.compute(torch.tensor(R + shift, device="cuda"))
    assert abs(float(out2["energy"].sum()) - ref["energy"]) < 1e-5 * abs(ref["energy"])
    assert np.abs(out2["forces"].cpu().numpy() - ref["forces"]).max() < 1e-3


def test_total_does_not_depend_on_the_smearing_on_the_device(reference_goldens):
    from so3lr_b200.engine import System
    g = reference_goldens
    Z, R, cell = g["water_Z"], np.asarray(g["water_R"], dtype=np.float32), np.asarray(g["water_cell"], dtype=np.float64)
    res = []
    for smearing, lam in ((1.9, 1.0), (2.4, 1.25)):
        s = System(Z, cell, cutoff_lr=12.0, damping=2.0)
        s.set_kspace(K.ewald_grid_shape(cell, lam), smearing)
        out = s.compute(torch.tensor(R, device="cuda"))
        res.append((float(out["energy"].sum()), out["forces"].cpu().numpy()))
    assert abs(res[0][0] - res[1][0]) < 2e-5 * abs(res[0][0])
    assert np.abs(res[0][1] - res[1][1]).max() < 1e-4


def test_triclinic_cell_matches_oracle(oracle_params):
    from so3lr_b200 import workloads as Wl
    from so3lr_b200.engine import System
    Z, R, cell = Wl.water_box(216, 18.7, 5, jitter=0.03)
    shear = np.array([[1.0, 0.0, 0.0], [0.18, 1.0, 0.0], [-0.1, 0.12, 1.0]])
    cell = np.asarray(cell, dtype=np.float64) @ shear
    R = (np.asarray(R, dtype=np.float64) @ shear).astype(np.float32)
    shape, smearing = K.ewald_grid_shape(cell, 0.9), 1.5
    ref = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=8.0, damping=2.0, k_grid=shape, k_smearing=smearing)
    s = System(Z, cell, cutoff_lr=8.0, damping=2.0)
    s.enable_virial(True)
    s.set_kspace(shape, smearing)
    _check(s.compute(torch.tensor(R, device="cuda")), ref, R)


def test_energy_function_with_k_grid_matches_the_fused_entry(oracle_params, reference_goldens):
    """The reference-facing call: energy_fn(R, neighbor=, neighbor_lr=, box=, k_grid=, k_smearing=) and its force."""
    import so3lr_b200.api as A
    from so3lr_b200.engine import System
    Z, R, cell = _water192(reference_goldens)
    box = np.diag(cell).copy()
    smearing, shape = 1.0, A.get_kgrid_ewald_shape(cell, 0.6)
    assert shape == K.ewald_grid_shape(cell, 0.6)
    pot = A.make_potential_fn(lr_cutoff=6.0, coulomb_kspace_do_ewald=True)
    nfn, nfn_lr, energy_fn = A.to_jax_md(potential=pot, displacement_or_metric=None, box_size=box, species=Z)
    Rt = torch.tensor(R.astype(np.float64) / box, dtype=torch.float64)       # fractional coordinates, as the reference's MD uses
    nbrs, nbrs_lr = nfn.allocate(Rt, box=box), nfn_lr.allocate(Rt, box=box)
    kw = dict(neighbor=nbrs.idx, neighbor_lr=nbrs_lr.idx, box=box, k_grid=A.get_kgrid_ewald(cell, 0.6),
              k_smearing=torch.tensor([smearing]))
    E = float(energy_fn(Rt, **kw))
    F = A.force(energy_fn)(Rt, **kw).cpu().numpy()       # jax-md convention: the gradient w.r.t. fractional positions is the real-space one
    ref = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=6.0, damping=2.0, k_grid=shape, k_smearing=smearing)
    assert abs(E - ref["energy"]) < 1e-5 * abs(ref["energy"]), (E, ref["energy"])
    assert np.abs(F - ref["forces"]).max() < 1e-4
    # the route of the reference's NPT: the strain derivative as the gradient with respect to `perturbation`, which deforms the
    # displacements, the positions and the box (so3lr/jaxmd_utils.py:48-51)
    P = torch.eye(3, dtype=torch.float64, requires_grad=True)
    (gP,) = torch.autograd.grad(energy_fn(Rt, perturbation=P, **kw), P)
    err = np.abs(gP.cpu().numpy() - ref["virial"]).max()
    assert err <= 2 * _vir_tol(R, ref["forces"]), (err, _vir_tol(R, ref["forces"]))
    # the same potential without k_grid evaluates the truncated pair sum again
    kw2 = dict(neighbor=nbrs.idx, neighbor_lr=nbrs_lr.idx, box=box)
    plain = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=6.0, damping=2.0)
    assert abs(float(energy_fn(Rt, **kw2)) - plain["energy"]) < 1e-5 * abs(plain["energy"])
    # the reference's default k-space method is the mesh variant: same call, potential made without coulomb_kspace_do_ewald
    pot_pme = A.make_potential_fn(lr_cutoff=6.0)
    _, _, efn_pme = A.to_jax_md(potential=pot_pme, displacement_or_metric=None, box_size=box, species=Z)
    mesh = A.get_kgrid_mesh_shape(cell, 0.4)
    assert mesh == K.mesh_grid_shape(cell, 0.4) == (32, 32, 32)
    kwm = dict(kw, k_grid=A.get_kgrid_mesh(cell, 0.4))
    refm = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=6.0, damping=2.0, k_grid=mesh, k_smearing=smearing,
                           k_method="pme")
    Em, Fm = float(efn_pme(Rt, **kwm)), A.force(efn_pme)(Rt, **kwm).cpu().numpy()
    assert abs(Em - refm["energy"]) < 1e-5 * abs(refm["energy"]), (Em, refm["energy"])
    assert np.abs(Fm - refm["forces"]).max() < 1e-4
    # and the mesh result is the direct sum up to the interpolation error of this mesh (0.39 A between points at a smearing
    # of 1 A: 9e-3 eV and 1e-3 eV/A in the oracle)
    assert abs(Em - E) < 2e-2 and np.abs(Fm - F).max() < 3e-3
    with pytest.raises(NotImplementedError):
        A.make_potential_fn(lr_cutoff=6.0, coulomb_kspace_interp_nodes=5)


@pytest.mark.parametrize("case", ["water192", "water1536", "triclinic"])
def test_mesh_variant_matches_oracle(oracle_params, reference_goldens, case):
    from so3lr_b200 import workloads as Wl
    from so3lr_b200.engine import System
    g = reference_goldens
    if case == "water192":
        Z, R, cell = _water192(g)
        rc, smearing, shape, skin = 6.0, 1.0, (32, 32, 32), 0.0
    elif case == "water1536":
        Z, R, cell = g["water_Z"], np.asarray(g["water_R"], dtype=np.float32), np.asarray(g["water_cell"], dtype=np.float64)
        rc, smearing, shape, skin = 12.0, 2.4, (32, 30, 36), 0.8           # cuFFT takes any extents
    else:
        Z, R, cell = Wl.water_box(216, 18.7, 5, jitter=0.03)
        shear = np.array([[1.0, 0.0, 0.0], [0.18, 1.0, 0.0], [-0.1, 0.12, 1.0]])
        cell = np.asarray(cell, dtype=np.float64) @ shear
        R = (np.asarray(R, dtype=np.float64) @ shear).astype(np.float32)
        rc, smearing, shape, skin = 8.0, 1.5, (32, 32, 32), 0.0
    ref = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=rc, damping=2.0, k_grid=shape, k_smearing=smearing,
                          k_method="pme")
    s = System(Z, cell, cutoff_lr=rc, damping=2.0, skin=skin)
    s.enable_virial(True)
    s.set_kspace(shape, smearing, "pme")
    _check(s.compute(torch.tensor(R, device="cuda")), ref, R)
    # a second evaluation reuses the plans and the mesh
    _check(s.compute(torch.tensor(R, device="cuda")), ref, R)


def test_invalid_kspace_requests_fail_loudly(reference_goldens):
    from so3lr_b200._lib import So3lrB200Error
    from so3lr_b200.engine import System
    Z, R, cell = _water192(reference_goldens)
    with pytest.raises(So3lrB200Error):
        System(Z, None, cutoff_lr=6.0).set_kspace((8, 8, 8), 1.0)          # no cell
    with pytest.raises(So3lrB200Error):
        System(Z, cell, cutoff_lr=None).set_kspace((8, 8, 8), 1.0)         # no cutoff: nothing short-ranged to keep in the pair sum
    with pytest.raises(So3lrB200Error):
        System(Z, cell, cutoff_lr=6.0).set_kspace((8, 8, 8), 0.0)          # smearing must be positive
    with pytest.raises(So3lrB200Error):
        System(Z, cell, cutoff_lr=6.0).set_kspace((8, 2, 8), 1.0, "pme")   # four mesh points per axis at least


def test_nve_with_the_reciprocal_sum_conserves_energy_and_strained_cells_follow_the_virial():
    """The forces are the derivative of the energy the context reports (a short NVE run keeps their sum), and after
    rescale_cell the k vectors follow the cell: a finite strain changes the energy by trace(W eps)."""
    from so3lr_b200 import md
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    Z, R, cell = W.water_box(512, 24.9, 7, jitter=0.02)
    V, m = W.maxwell_boltzmann(Z, 300.0, 8)
    cell = np.asarray(cell, dtype=np.float64)
    s = System(Z, cell, cutoff_lr=10.0, damping=2.0, skin=0.5)
    s.set_kspace(K.ewald_grid_shape(cell, 1.0), 2.0)
    dof = 3.0 * len(Z)
    init_fn, apply_fn = md.nve(s, 0.25)
    state = init_fn(R, m, velocity=V)
    E0 = float(state.energy.sum()) + md.kinetic_energy(state)
    state = apply_fn(state, 120)
    assert abs(float(state.energy.sum()) + md.kinetic_energy(state) - E0) < 2e-3 * dof * 300.0 * 8.617333262e-5
    # strain
    s.enable_virial(True)
    Rf = np.asarray(R, dtype=np.float64)
    Wv = s.compute(torch.tensor(Rf.astype(np.float32), device="cuda"))["virial"].cpu().numpy()
    eps = 2e-4 * np.array([[1.0, 0.3, 0.0], [0.3, -0.5, 0.2], [0.0, 0.2, 0.7]])
    Es = []
    for sign in (+1, -1):
        A = np.eye(3) + sign * eps
        s.rescale_cell(cell @ A.T)
        Es.append(float(s.compute(torch.tensor((Rf @ A.T).astype(np.float32), device="cuda"))["energy"].sum()))
    dE = (Es[0] - Es[1]) / 2
    assert abs(dE - float((Wv * eps).sum())) < 2e-3 + 2e-3 * abs(dE), (dE, float((Wv * eps).sum()))


@pytest.mark.parametrize("method", ["ewald", "pme"])
def test_charged_cell_carries_the_background_term(oracle_params, reference_goldens, method):
    """A net charge: the charge embedding changes the features, the charges sum to the total charge, and the reciprocal part
    gains the neutralising-background term -ke pi s^2 Q^2 / V (energy and strain derivative)."""
    from so3lr_b200.engine import System
    Z, R, cell = _water192(reference_goldens)
    shape, smearing = ((32, 32, 32) if method == "pme" else K.ewald_grid_shape(cell, 0.6)), 1.0
    ref = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=6.0, damping=2.0, total_charge=[1.0],
                          k_grid=shape, k_smearing=smearing, k_method=method)
    s = System(Z, cell, cutoff_lr=6.0, damping=2.0, total_charge=[1.0])
    s.enable_virial(True)
    s.set_kspace(shape, smearing, method)
    out = s.compute(torch.tensor(R, device="cuda"))
    _check(out, ref, R)
    assert abs(float(out["partial_charges"].sum()) - 1.0) < 1e-4
    # the background term (ke pi s^2 Q^2 / V = 0.024 eV) is several times the energy tolerance at this size: a missing term would show
    assert K.KE * np.pi * smearing ** 2 / abs(np.linalg.det(cell)) > 5 * 1e-5 * abs(ref["energy"])
