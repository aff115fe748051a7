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
