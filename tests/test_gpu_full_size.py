"""Size-independent properties of the energy+force path at the full sizes of the benchmark configurations, where the CPU
oracle cannot follow (the 999,999-atom and the 24,000-atom periodic water boxes).

What the physics guarantees for any correct implementation, with float32 tolerances stated beside each check:
  - the forces sum to zero (every pair term and every edge of the network is translation invariant);
  - a lattice translation of some atoms, a rigid shift of all atoms, a permutation of the atoms and a rotation of the whole
    cubic box by 90 degrees leave the energy unchanged and move the forces with the atoms;
  - a central finite difference of the energy along a random displacement field equals minus the projected forces;
  - velocity Verlet conserves the total energy.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _box(name):
    import bench
    from so3lr_b200 import workloads as W
    n_mol, box, seed = bench.WORKLOADS[name]
    # coordinates and the box edge on a grid of 2^-10 A (62.1 -> 62.0996, 215.0 stays): lattice translations, the rigid shift
    # below and the rotation are then exact in float32, so the checks compare like with like
    box = round(box * 1024.0) / 1024.0
    Z, R, cell = W.water_box(n_mol, box, seed)
    R = np.round(np.asarray(R, dtype=np.float64) * 1024.0) / 1024.0
    return Z, R.astype(np.float32), np.asarray(cell, dtype=np.float64), box


def _eval(Z, R, cell, skin=0.0):
    from so3lr_b200.engine import System
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=skin)
    out = s.compute(torch.tensor(R, device="cuda"))
    return float(out["energy"].sum()), out["forces"].cpu().numpy().astype(np.float64), out["partial_charges"].cpu().numpy(), s.stats()


@pytest.mark.parametrize("name", ["water_24k", "water_1m"])
def test_symmetries_at_full_size(name):
    Z, R, cell, box = _box(name)
    N = len(Z)
    E0, F0, q0, st0 = _eval(Z, R, cell)
    fmax = np.abs(F0).max()
    assert np.isfinite(F0).all() and np.isfinite(E0)
    # Newton's third law: each component of the total force is a sum of N numbers of size ~fmax with float32 rounding
    assert np.abs(F0.sum(0)).max() < 2e-6 * fmax * N ** 0.5 + 1e-3, (F0.sum(0), fmax)
    assert abs(float(q0.astype(np.float64).sum())) < 1e-5 * N ** 0.5 + 1e-3          # charge conservation, neutral box
    # expected list sizes for water at this density: 38.6 directed short-range edges and 363 ordered long-range pairs per atom
    # (the synthetic start is not equilibrated: about 40 edges)
    assert abs(st0["edges"] / N - 38.6) < 3.0 and abs(st0["pairs"] / N - 363.0) < 8.0, (st0["edges"] / N, st0["pairs"] / N)
    rng = np.random.default_rng(5)
    # 1. a rigid shift of everything plus lattice translations of a random third of the atoms (exact in float32 on this grid;
    # the minimum image subtracts the lattice vector from the displacement itself, so nothing is lost across the boundary)
    R1 = R.astype(np.float64) + np.array([3.25, -1.84375, 0.7705078125])      # multiples of 2^-10
    pick = rng.random(N) < 0.33
    R1[pick] += rng.integers(-2, 3, size=(int(pick.sum()), 3)) * box
    assert np.array_equal(R1.astype(np.float32).astype(np.float64), R1)
    E1, F1, _, st1 = _eval(Z, R1.astype(np.float32), cell)
    assert st1["edges"] == st0["edges"] and st1["pairs"] == st0["pairs"]
    assert abs(E1 - E0) < 2e-6 * abs(E0)
    assert np.abs(F1 - F0).max() < 2e-4 and np.sqrt(((F1 - F0) ** 2).mean()) < 2e-5, (np.abs(F1 - F0).max(), np.sqrt(((F1 - F0) ** 2).mean()))
    # 2. permutation of the atoms (molecules stay intact only by chance: the path may not depend on the order)
    perm = rng.permutation(N)
    E2, F2, _, st2 = _eval(Z[perm], R[perm], cell)
    assert st2["edges"] == st0["edges"] and st2["pairs"] == st0["pairs"]
    assert abs(E2 - E0) < 2e-6 * abs(E0)
    assert np.abs(F2 - F0[perm]).max() < 2e-4
    # 3. rotation of the cubic box by 90 degrees about z: (x, y, z) -> (-y, x, z)
    Q = np.array([[0.0, -1.0, 0.0], [1.0, 0.0, 0.0], [0.0, 0.0, 1.0]])
    E3, F3, _, _ = _eval(Z, (R.astype(np.float64) @ Q.T).astype(np.float32), cell)
    assert abs(E3 - E0) < 2e-6 * abs(E0)
    assert np.abs(F3 - F0 @ Q.T).max() < 2e-4
    # 4. the skin list gives the same numbers
    E4, F4, _, st4 = _eval(Z, R, cell, skin=1.0)
    assert st4["edges"] > st0["edges"]
    assert abs(E4 - E0) < 2e-6 * abs(E0) and np.abs(F4 - F0).max() < 2e-4


def test_forces_are_the_energy_gradient_at_24k():
    """Central difference of the total energy along a random displacement field against the projected forces.  The energy
    is a float64 sum of float32 per-atom energies (about 1e-7 relative each), so the field is scaled to move the energy by
    about 2 eV either way; the second-order error of the central difference stays below 1e-3 of that."""
    Z, R, cell, _ = _box("water_24k")
    rng = np.random.default_rng(9)
    E0, F0, _, _ = _eval(Z, R, cell)
    D = rng.normal(size=R.shape)
    D *= 2.0 / np.abs((F0 * D).sum())           # |dE| = 2 eV at unit step
    D = np.clip(D, -0.01, 0.01)                 # no atom moves more than 0.01 A
    slope = -(F0 * D).sum()
    Ep, _, _, _ = _eval(Z, (R.astype(np.float64) + D).astype(np.float32), cell)
    Em, _, _, _ = _eval(Z, (R.astype(np.float64) - D).astype(np.float32), cell)
    fd = (Ep - Em) / 2.0
    assert abs(fd - slope) < 0.01 * abs(slope) + 5e-3, (fd, slope)


def test_nve_energy_error_is_second_order_at_24k():
    """Velocity Verlet with forces that are the gradient of the energy: the energy error over a fixed time span falls by four
    when the step is halved.  (The synthetic start is far from equilibrium - stretched O-H bonds carry about 1 keV - so the
    error itself is several eV at dt = 0.25 fs; what is checked is how it scales.)"""
    from so3lr_b200 import md
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    Z, R, cell, _ = _box("water_24k")
    V, m = W.maxwell_boltzmann(Z, 300.0, 4)
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=1.0)
    err = {}
    for dt, steps in ((0.25, 32), (0.125, 64)):
        init_fn, apply_fn = md.nve(s, dt)
        state = init_fn(R, m, velocity=V)
        H0 = float(state.energy.sum()) + md.kinetic_energy(state)
        worst = 0.0
        for _ in range(4):
            state = apply_fn(state, steps // 4)
            worst = max(worst, abs(float(state.energy.sum()) + md.kinetic_energy(state) - H0))
        err[dt] = worst
    assert s.stats()["rebuilds"] >= 3                      # the skin test fired on the way
    assert err[0.125] < 0.4 * err[0.25] and err[0.25] < 5e-4 * abs(H0), err
