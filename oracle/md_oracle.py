"""CPU restatement (float64 numpy) of the MD step bodies the reference drives: velocity Verlet (NVE) and velocity Verlet
under a Nose-Hoover chain thermostat (NVT).

TEST INFRASTRUCTURE ONLY: imported by tests/ and by nothing in the product path.

PARITY UNPINNED: the reference holds no golden vectors for a trajectory or for a thermostat state; its integrators live
in a third-party dependency that is absent from the reference checkout (jax-md, pinned in the reference's
pyproject.toml:23 as the branch kabylda/jax-md@main, no commit).  What follows restates the published algorithm
(Martyna, Tuckerman, Tobias, Klein, Mol. Phys. 87, 1117 (1996): Nose-Hoover chain propagated with a Suzuki-Yoshida
factorisation, half a thermostat step either side of velocity Verlet) in the form jax_md.simulate.nvt_nose_hoover uses
it, anchored on the reference's own call sites:

  so3lr/cli/so3lr_md.py:1047-1075   create_nhc_fn -> jax_md.simulate.nvt_nose_hoover(energy_fn, shift, dt, kT, thermostat_kwargs)
  so3lr/cli/so3lr_md.py:1698-1707   chain_length / chain_steps / sy_steps / tau = dt * nhc_thermo
  so3lr/cli/so3lr_cli.py:114-116    defaults 3 / 2 / (3) / 100
  so3lr/cli/so3lr_md.py:1011-1045   create_nve_fn -> jax_md.simulate.nve
  so3lr/cli/so3lr_md.py:912-916     kinetic energy of the state; temperature = 2 KE / (dof kB), dof = 3 N (no constraint removed)

Units: Angstrom, fs, amu, eV.  One amu A^2/fs^2 is 1/ACC eV with ACC = 9.648533212331e-3.
"""
from __future__ import annotations

import numpy as np

ACC = 9.648533212331e-3          # eV / (amu A^2 / fs^2) inverse: a [A/fs^2] = ACC * F [eV/A] / m [amu]
KB = 8.617333262e-5              # eV / K

# Suzuki-Yoshida weights by number of factors (each set sums to 1).
SY_WEIGHTS = {
    1: [1.0],
    3: [0.828981543588751, -0.657963087177502, 0.828981543588751],
    5: [0.2967324292201065, 0.2967324292201065, -0.186929716880426, 0.2967324292201065, 0.2967324292201065],
    7: [0.784513610477560, 0.235573213359357, -1.17767998417887, 1.31518632068391, -1.17767998417887, 0.235573213359357,
        0.784513610477560],
}


def kinetic_energy(V, m):
    """0.5 sum m v^2 in eV (V in A/fs, m in amu)."""
    return 0.5 * float(np.sum(m[:, None] * V * V)) / ACC


class Chain:
    """Thermostat chain state: positions xi, momenta p_xi (eV fs), masses Q (eV fs^2), the kinetic energy it last saw."""

    def __init__(self, chain_length, dof, ke, kT, tau):
        self.L = int(chain_length)
        self.xi = np.zeros(self.L)
        self.p_xi = np.zeros(self.L)
        self.dof = float(dof)
        self.tau = float(tau)
        self.ke = float(ke)
        self.set_mass(kT)

    def set_mass(self, kT):
        self.Q = kT * self.tau ** 2 * np.ones(self.L)
        self.Q[0] *= self.dof


def chain_substep(c: Chain, delta, kT):
    """One factor of the chain propagator over the time delta; returns the factor the particle momenta are scaled by."""
    L, M = c.L, c.L - 1
    p, Q = c.p_xi, c.Q
    d2, d4, d8 = delta / 2, delta / 4, delta / 8
    if L == 1:
        G = 2.0 * c.ke - c.dof * kT
        p[0] += d4 * G
    else:
        G = p[M - 1] ** 2 / Q[M - 1] - kT
        p[M] += d4 * G
        for m in range(M - 1, 0, -1):
            G = p[m - 1] ** 2 / Q[m - 1] - kT
            s = np.exp(-d8 * p[m + 1] / Q[m + 1])
            p[m] = s * (s * p[m] + d4 * G)
        G = 2.0 * c.ke - c.dof * kT
        s = np.exp(-d8 * p[1] / Q[1])
        p[0] = s * (s * p[0] + d4 * G)
    scale = np.exp(-d2 * p[0] / Q[0])
    c.ke *= scale ** 2
    c.xi += d2 * p / Q
    G = 2.0 * c.ke - c.dof * kT
    if L == 1:
        p[0] += d4 * G
    else:
        for m in range(M):
            s = np.exp(-d8 * p[m + 1] / Q[m + 1])
            p[m] = s * (s * p[m] + d4 * G)
            G = p[m] ** 2 / Q[m] - kT
        p[M] += d4 * G
    return scale


def chain_half_step(c: Chain, dt, kT, chain_steps, sy_steps):
    """The thermostat half of an MD step: chain_steps x sy_steps factors over dt / chain_steps each (weighted)."""
    w = SY_WEIGHTS[sy_steps]
    total = 1.0
    for i in range(chain_steps * sy_steps):
        total *= chain_substep(c, dt / chain_steps * w[i % sy_steps], kT)
    return total


def velocity_verlet(force_fn, R, V, F, m, dt):
    a = ACC / m[:, None]
    V = V + 0.5 * dt * a * F
    R = R + dt * V
    E, F = force_fn(R)
    V = V + 0.5 * dt * a * F
    return R, V, F, E


def nve(force_fn, R, V, m, dt, n_steps):
    E, F = force_fn(R)
    for _ in range(n_steps):
        R, V, F, E = velocity_verlet(force_fn, R, V, F, m, dt)
    return R, V, F, E


def nvt_init(V, m, kT, tau, chain_length):
    return Chain(chain_length, 3 * len(m), kinetic_energy(V, m), kT, tau)


def nvt_step(force_fn, c: Chain, R, V, F, m, dt, kT, chain_steps, sy_steps):
    c.set_mass(kT)
    V = V * chain_half_step(c, dt, kT, chain_steps, sy_steps)
    R, V, F, E = velocity_verlet(force_fn, R, V, F, m, dt)
    c.ke = kinetic_energy(V, m)
    V = V * chain_half_step(c, dt, kT, chain_steps, sy_steps)
    return R, V, F, E


def nvt_invariant(c: Chain, E_pot, V, m, kT):
    """Conserved quantity of the thermostatted dynamics: E_pot + KE + sum p_xi^2 / (2Q) + dof kT xi_0 + kT sum_{k>0} xi_k."""
    H = E_pot + kinetic_energy(V, m)
    H += float(np.sum(c.p_xi ** 2 / (2.0 * c.Q))) + c.dof * kT * c.xi[0] + kT * float(np.sum(c.xi[1:]))
    return H


# ----------------------------------------------------------------------------------------------------------------------
# NPT: isotropic Martyna-Tobias-Klein barostat with Nose-Hoover chains on the particles and on the box, in the form
# jax_md.simulate.npt_nose_hoover integrates it (created at so3lr/cli/so3lr_md.py:1078-1107 with the thermostat settings
# of :1698-1707 and the barostat's tau = dt * nhc_baro, :1709-1711; the box after a step is read back at :1270-1282).
# The box coordinate is eps = (1/3) ln(V / V0); its momentum p_eps has the mass W = 3 (N + 1) kT tau_b^2.
# Positions are Cartesian here and scale with the box.  force_fn(R, cell) -> (E, F, virial) with virial = dE/d strain (3x3).
# ----------------------------------------------------------------------------------------------------------------------
BAR = 6.241509074e-7             # eV / A^3 per bar


def sinhx_x(x):
    """sinh(x)/x by its series (the step's arguments are ~1e-4)."""
    x2 = x * x
    return 1 + x2 / 6 + x2 ** 2 / 120 + x2 ** 3 / 5040 + x2 ** 4 / 362880 + x2 ** 5 / 39916800


class NPTState:
    def __init__(self, R, V, m, cell0, kT, tau_t, tau_b, chain_length, force_fn):
        self.R, self.V, self.m = np.array(R, dtype=np.float64), np.array(V, dtype=np.float64), np.array(m, dtype=np.float64)
        self.cell0 = np.array(cell0, dtype=np.float64)
        self.V0 = abs(np.linalg.det(self.cell0))
        self.N = len(self.m)
        self.eps, self.p_eps = 0.0, 0.0
        self.tau_b = float(tau_b)
        self.W = 3.0 * (self.N + 1) * kT * self.tau_b ** 2
        self.thermostat = Chain(chain_length, 3 * self.N, kinetic_energy(self.V, self.m), kT, tau_t)
        self.barostat = Chain(chain_length, 1, 0.0, kT, tau_b)
        self.E, self.F, self.virial = force_fn(self.R, self.cell())

    def volume(self):
        return self.V0 * np.exp(3.0 * self.eps)

    def cell(self):
        return self.cell0 * np.exp(self.eps)


def npt_step(force_fn, s: NPTState, dt, kT, pressure, chain_steps, sy_steps):
    """One step; pressure in eV/A^3."""
    N, a = s.N, ACC / s.m[:, None]
    alpha = 1.0 + 1.0 / N
    s.barostat.set_mass(kT)
    s.thermostat.set_mass(kT)
    s.W = 3.0 * (N + 1) * kT * s.tau_b ** 2
    s.p_eps *= chain_half_step(s.barostat, dt, kT, chain_steps, sy_steps)
    s.V = s.V * chain_half_step(s.thermostat, dt, kT, chain_steps, sy_steps)

    def box_force():
        ke2 = 2.0 * kinetic_energy(s.V, s.m)
        return alpha * ke2 - np.trace(s.virial) - 3.0 * pressure * s.volume()

    def kick():
        x = alpha * (s.p_eps / s.W) * dt / 2
        s.V = s.V * np.exp(-x) + (dt / 2) * a * s.F * sinhx_x(x / 2) * np.exp(-x / 2)

    s.p_eps += dt / 2 * box_force()
    kick()
    v_eps = s.p_eps / s.W
    s.eps += v_eps * dt
    x = v_eps * dt
    s.R = s.R * np.exp(x) + dt * s.V * np.exp(x / 2) * sinhx_x(x / 2)
    s.E, s.F, s.virial = force_fn(s.R, s.cell())
    kick()
    s.p_eps += dt / 2 * box_force()
    s.thermostat.ke = kinetic_energy(s.V, s.m)
    s.barostat.ke = s.p_eps ** 2 / (2.0 * s.W)
    s.V = s.V * chain_half_step(s.thermostat, dt, kT, chain_steps, sy_steps)
    s.p_eps *= chain_half_step(s.barostat, dt, kT, chain_steps, sy_steps)
    return s


def npt_invariant(s: NPTState, kT, pressure):
    """Conserved quantity of the NPT dynamics: E_pot + KE + p_eps^2 / 2W + P V + both chains' energies."""
    H = s.E + kinetic_energy(s.V, s.m) + s.p_eps ** 2 / (2.0 * s.W) + pressure * s.volume()
    for c in (s.thermostat, s.barostat):
        H += float(np.sum(c.p_xi ** 2 / (2.0 * c.Q))) + c.dof * kT * c.xi[0] + kT * float(np.sum(c.xi[1:]))
    return H
