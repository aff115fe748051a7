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
    # the same potential without k_grid evaluates the truncated pair sum again
    kw2 = dict(neighbor=nbrs.idx, neighbor_lr=nbrs_lr.idx, box=box)
    plain = O.energy_forces(oracle_params, R.astype(np.float64), Z, cell, cutoff_lr=6.0, damping=2.0)
    assert abs(float(energy_fn(Rt, **kw2)) - plain["energy"]) < 1e-5 * abs(plain["energy"])
    # the mesh variant is not part of the library: loud, not silent
    pot_pme = A.make_potential_fn(lr_cutoff=6.0)
    _, _, efn_pme = A.to_jax_md(potential=pot_pme, displacement_or_metric=None, box_size=box, species=Z)
    with pytest.raises(NotImplementedError):
        efn_pme(Rt, **kw)


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
