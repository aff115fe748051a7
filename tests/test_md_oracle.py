"""The oracle's MD step bodies (velocity Verlet, Nose-Hoover chain) checked through properties of the dynamics: the
reference holds no golden trajectory, so these pin the restatement on what the published algorithm guarantees."""
import numpy as np

from oracle import md_oracle as MD


def _springs(n=24, seed=5):
    rng = np.random.default_rng(seed)
    R0 = rng.uniform(0, 6, size=(n, 3))
    k = rng.uniform(1.0, 4.0, size=n)
    m = rng.uniform(1.0, 16.0, size=n)

    def force(R):
        d = R - R0
        # anharmonic wells coupled through the centre of mass distance so that energy flows between atoms
        c = d - d.mean(0)
        E = 0.5 * np.sum(k[:, None] * d * d) + 0.25 * np.sum(c ** 4)
        g = k[:, None] * d + (c ** 3 - (c ** 3).mean(0))
        return E, -g

    V = rng.normal(size=(n, 3)) * 0.01 / np.sqrt(m)[:, None]
    return force, R0 + rng.normal(size=(n, 3)) * 0.05, V, m


def test_nve_conserves_energy():
    force, R, V, m = _springs()
    E0, _ = force(R)
    H0 = E0 + MD.kinetic_energy(V, m)
    R1, V1, _, E1 = MD.nve(force, R, V, m, 0.25, 400)
    assert abs(E1 + MD.kinetic_energy(V1, m) - H0) < 2e-5 * abs(H0)


def test_nvt_conserves_the_extended_energy_and_reaches_the_target_temperature():
    force, R, V, m = _springs()
    kT, tau, dt = 0.05, 10.0, 0.25
    E, F = force(R)
    c = MD.nvt_init(V, m, kT, tau, 3)
    H0 = MD.nvt_invariant(c, E, V, m, kT)
    temps, drift = [], 0.0
    for step in range(6000):
        R, V, F, E = MD.nvt_step(force, c, R, V, F, m, dt, kT, 2, 3)
        if step % 50 == 0:
            drift = max(drift, abs(MD.nvt_invariant(c, E, V, m, kT) - H0))
        if step >= 2000:
            temps.append(2.0 * MD.kinetic_energy(V, m) / c.dof)
        # the kinetic energy the chain carries is the kinetic energy of the scaled velocities
        assert abs(c.ke - MD.kinetic_energy(V, m)) < 1e-9 * max(1.0, c.ke)
    assert drift < 1e-4 * c.dof * kT
    assert abs(np.mean(temps) / kT - 1.0) < 0.1


def test_suzuki_yoshida_weights_sum_to_one_and_one_factor_is_time_reversible():
    for k, w in MD.SY_WEIGHTS.items():
        assert len(w) == k and abs(sum(w) - 1.0) < 1e-12
    c = MD.Chain(3, 30, 0.7, 0.05, 8.0)
    c.p_xi[:] = [0.3, -0.2, 0.1]
    c.xi[:] = [0.01, 0.02, -0.03]
    ref = (c.xi.copy(), c.p_xi.copy(), c.ke)
    s1 = MD.chain_substep(c, 0.4, 0.05)
    s2 = MD.chain_substep(c, -0.4, 0.05)
    assert abs(s1 * s2 - 1.0) < 1e-12 and abs(c.ke - ref[2]) < 1e-12
    np.testing.assert_allclose(c.xi, ref[0], atol=1e-12)
    np.testing.assert_allclose(c.p_xi, ref[1], atol=1e-12)


def _soft_spheres(n_side=4, a=3.4, seed=2):
    """Periodic box of purely repulsive pairs (a phi = e0 (1 - r/rc)^4 bump): energy, forces and the strain derivative."""
    rng = np.random.default_rng(seed)
    g = np.stack(np.meshgrid(*[np.arange(n_side)] * 3, indexing="ij"), -1).reshape(-1, 3)
    R = (g + 0.5) * a + rng.normal(size=(len(g), 3)) * 0.1
    cell = np.eye(3) * n_side * a
    rc, e0 = 5.5, 0.4

    def force(R, cell):
        d = R[None, :, :] - R[:, None, :]                 # d[i, j] = R_j - R_i
        d -= np.round(d @ np.linalg.inv(cell)) @ cell
        r = np.linalg.norm(d, axis=-1) + np.eye(len(R)) * 1e3
        m = r < rc
        phi = np.where(m, e0 * (1 - r / rc) ** 4, 0.0)
        dphi = np.where(m, -4 * e0 / rc * (1 - r / rc) ** 3, 0.0)
        E = 0.5 * phi.sum()
        g = (dphi / r)[..., None] * d                     # dE_pair / d(d_ij)
        F = g.sum(1)                                      # F_i = + sum_j dphi * unit(d_ij)
        W = 0.5 * np.einsum("ija,ijb->ab", d, g)
        return E, F, W

    m = rng.uniform(10.0, 40.0, size=len(R))
    V = rng.normal(size=R.shape) * np.sqrt(0.03 * MD.ACC / m)[:, None]
    return force, R, V, m, cell


def test_soft_sphere_virial_is_the_strain_derivative():
    force, R, V, m, cell = _soft_spheres()
    E, F, W = force(R, cell)
    h = 1e-6
    for eps in (np.eye(3), np.array([[0, 1.0, 0], [0, 0, 0], [0, 0, 0]])):
        A = np.eye(3) + h * eps
        B = np.eye(3) - h * eps
        dE = (force(R @ A.T, cell @ A.T)[0] - force(R @ B.T, cell @ B.T)[0]) / (2 * h)
        assert abs(dE - (W * eps).sum()) < 1e-6 * max(1.0, abs(dE))
    # forces are minus the position gradient
    R2 = R.copy(); R2[3, 1] += h
    R3 = R.copy(); R3[3, 1] -= h
    assert abs(-(force(R2, cell)[0] - force(R3, cell)[0]) / (2 * h) - F[3, 1]) < 1e-6


def test_npt_conserves_its_invariant_and_relaxes_towards_the_target_pressure():
    force, R, V, m, cell = _soft_spheres()
    kT, dt, tau_t, tau_b = 0.03, 1.0, 50.0, 400.0
    s = MD.NPTState(R, V, m, cell, kT, tau_t, tau_b, 3, force)

    def pressure_of(s):
        return (2.0 * MD.kinetic_energy(s.V, s.m) - np.trace(s.virial)) / (3.0 * s.volume())

    p0 = pressure_of(s)
    target = 0.5 * p0                      # the compressed start must expand
    H0 = MD.npt_invariant(s, kT, target)
    vol0, drift, ps = s.volume(), 0.0, []
    for step in range(4000):
        MD.npt_step(force, s, dt, kT, target, 2, 3)
        if step % 40 == 0:
            drift = max(drift, abs(MD.npt_invariant(s, kT, target) - H0))
        if step >= 2000:
            ps.append(pressure_of(s))
    assert drift < 2e-4 * 3 * s.N * kT, drift
    assert s.volume() > 1.05 * vol0
    assert abs(np.mean(ps) / target - 1.0) < 0.15, (np.mean(ps), target)
