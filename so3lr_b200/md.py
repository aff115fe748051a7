"""Host-side mirror of the integrator factories the reference builds its MD loops from.

The reference calls jax_md.simulate.nve / nvt_nose_hoover, which return an (init_fn, apply_fn) pair working on a state
record (so3lr/cli/so3lr_md.py:1011-1075), and steps the pair inside lax.fori_loop together with the two neighbor-list
updates (so3lr/cli/so3lr_md.py:1115-1222, 1815-1822).  Here the pair drives so3lr_b200_system_nve / _nvt: positions,
velocities, forces and the thermostat chain stay on the device, the skin test and list rebuilds happen inside the library's
force evaluation, and apply_fn takes the number of steps to run before it returns (the body of the reference's inner loop).

Units: Angstrom, fs, amu, eV (kT in eV: kT = KB * T).  The reference converts its inputs with jax-md's metal unit system
(so3lr/cli/so3lr_md.py:124-161); a time of 1 ps there is 1000 fs here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .engine import BAR, System, nhc_state, npt_state  # noqa: F401

KB = 8.617333262e-5               # eV / K
ACC_UNIT = 9.648533212331e-3      # eV / (A amu) -> A / fs^2


@dataclass
class MDState:
    """Counterpart of jax-md's NVEState / NVTNoseHooverState: everything a step needs, resident on the device."""
    position: torch.Tensor          # (n, 3) float32
    velocity: torch.Tensor          # (n, 3) float32, A / fs
    force: torch.Tensor             # (n, 3) float32, eV / A
    mass: torch.Tensor              # (n,) float32, amu
    chain: Optional[torch.Tensor]   # thermostat chain (None for NVE), see so3lr_b200.engine.nhc_state
    energy: Optional[torch.Tensor] = None     # potential energy per graph after the last step
    box: Optional[np.ndarray] = None          # NPT: the current cell (3,3), lattice vectors as rows
    reference_box: Optional[np.ndarray] = None

    @property
    def momentum(self):
        return self.velocity * self.mass[:, None]


def kinetic_energy(state: MDState) -> float:
    """0.5 sum m v^2 in eV (jax_md.quantity.kinetic_energy, used at so3lr/cli/so3lr_md.py:912-916)."""
    v = state.velocity.double()
    return float(0.5 * (state.mass.double() * (v * v).sum(1)).sum() / ACC_UNIT)


def temperature(state: MDState) -> float:
    """Kinetic temperature in K with 3 n degrees of freedom (jax_md.quantity.temperature, so3lr/cli/so3lr_md.py:979-982)."""
    return 2.0 * kinetic_energy(state) / (3.0 * state.mass.numel() * KB)


def _init_state(system: System, R, mass, velocity, kT, seed, chain):
    dev = system.device
    R = torch.as_tensor(np.asarray(R, dtype=np.float32) if not torch.is_tensor(R) else R).to(dev, torch.float32).contiguous().clone()
    m = torch.as_tensor(np.asarray(mass, dtype=np.float32) if not torch.is_tensor(mass) else mass).to(dev, torch.float32)
    m = m.expand(R.shape[0]).contiguous() if m.dim() == 0 or m.numel() == 1 else m.contiguous()
    if velocity is None:
        # Maxwell-Boltzmann draw at kT with the centre-of-mass motion removed (jax-md's initialize_momenta)
        g = torch.Generator(device="cpu").manual_seed(int(seed))
        v = torch.randn(R.shape, generator=g, dtype=torch.float64) * torch.sqrt(kT * ACC_UNIT / m.double().cpu())[:, None]
        v -= (v * m.double().cpu()[:, None]).sum(0) / m.double().sum().cpu()
        V = v.to(dev, torch.float32).contiguous()
    else:
        V = torch.as_tensor(np.asarray(velocity, dtype=np.float32) if not torch.is_tensor(velocity) else velocity)
        V = V.to(dev, torch.float32).contiguous().clone()
    out = system.compute(R)
    return MDState(R, V, out["forces"].clone(), m, chain, out["energy"].clone())


def nve(system: System, dt: float):
    """(init_fn, apply_fn) for velocity Verlet; dt in fs.  Mirrors create_nve_fn (so3lr/cli/so3lr_md.py:1011-1045)."""

    def init_fn(R, mass, velocity=None, kT=0.0, seed=0):
        return _init_state(system, R, mass, velocity, kT, seed, None)

    def apply_fn(state: MDState, n_steps: int = 1):
        state.energy = system.nve(n_steps, dt, state.mass, state.position, state.velocity, state.force)
        return state

    return init_fn, apply_fn


def nvt_nose_hoover(system: System, dt: float, kT: float, chain_length: int = 3, chain_steps: int = 2, sy_steps: int = 3,
                    tau: Optional[float] = None):
    """(init_fn, apply_fn) for velocity Verlet under a Nose-Hoover chain; dt and tau in fs, kT in eV, tau = 100 dt when
    not given (the reference passes tau = dt * nhc_thermo, so3lr/cli/so3lr_md.py:1698-1707).  Mirrors create_nhc_fn
    (so3lr/cli/so3lr_md.py:1047-1075)."""
    tau = 100.0 * dt if tau is None else float(tau)

    def init_fn(R, mass, velocity=None, seed=0):
        return _init_state(system, R, mass, velocity, kT, seed, nhc_state(system.device))

    def apply_fn(state: MDState, n_steps: int = 1, kT: float = kT):
        state.energy = system.nvt(n_steps, dt, kT, tau, state.mass, state.position, state.velocity, state.force, state.chain,
                                  chain_length=chain_length, chain_steps=chain_steps, sy_steps=sy_steps)
        return state

    apply_fn.settings = dict(chain_length=chain_length, chain_steps=chain_steps, sy_steps=sy_steps, tau=tau, kT=kT, dt=dt)
    return init_fn, apply_fn


def nvt_nose_hoover_invariant(state: MDState, kT: float, tau: float, chain_length: int = 3) -> float:
    """Conserved quantity of the thermostatted dynamics in eV (jax_md.simulate.nvt_nose_hoover_invariant, used at
    so3lr/cli/so3lr_md.py:931-939): E_pot + KE + sum p_xi^2 / 2Q + dof kT xi_0 + kT sum_{k>0} xi_k."""
    c = state.chain.cpu().numpy()
    L = chain_length
    dof = 3.0 * state.mass.numel()
    Q = kT * tau ** 2 * np.ones(L)
    Q[0] *= dof
    xi, p = c[2:2 + L], c[10:10 + L]
    return float(state.energy.sum()) + kinetic_energy(state) + float(np.sum(p * p / (2 * Q))) + dof * kT * xi[0] + kT * float(xi[1:].sum())


def npt_nose_hoover(system: System, dt: float, pressure: float, kT: float, barostat_kwargs: Optional[dict] = None,
                    thermostat_kwargs: Optional[dict] = None):
    """(init_fn, apply_fn) for the isotropic Martyna-Tobias-Klein barostat with Nose-Hoover chains on particles and box;
    dt and the taus in fs, kT in eV, pressure in eV/A^3 (BAR converts).  The kwargs carry chain_length / chain_steps /
    sy_steps / tau as the reference passes them (so3lr/cli/so3lr_md.py:1698-1711); tau defaults to 100 dt (thermostat) and
    1000 dt (barostat).  Both chains share the thermostat's chain_length / chain_steps / sy_steps.  Mirrors create_npt_nhc_fn
    (so3lr/cli/so3lr_md.py:1089-1107); the cell of `system` follows the box, read it with npt_box(state)."""
    tk = dict(chain_length=3, chain_steps=2, sy_steps=3, tau=100.0 * dt)
    tk.update(thermostat_kwargs or {})
    bk = dict(tk, tau=1000.0 * dt)
    bk.update(barostat_kwargs or {})
    if any(bk[k] != tk[k] for k in ("chain_length", "chain_steps", "sy_steps")):
        raise NotImplementedError("the two chains share their length and factorisation")

    def init_fn(R, box, mass, velocity=None, seed=0):
        system.enable_virial(True)
        system.set_cell(box)
        state = _init_state(system, R, mass, velocity, kT, seed, npt_state(system.device))
        state.box = np.asarray(box, dtype=np.float64).reshape(3, 3).copy()
        state.reference_box = state.box.copy()
        return state

    def apply_fn(state: MDState, n_steps: int = 1, kT: float = kT, pressure: float = pressure):
        state.energy, state.box = system.npt(n_steps, dt, kT, pressure, tk["tau"], bk["tau"], state.mass, state.position,
                                             state.velocity, state.force, state.chain, state.reference_box,
                                             chain_length=tk["chain_length"], chain_steps=tk["chain_steps"], sy_steps=tk["sy_steps"])
        return state

    apply_fn.settings = dict(thermostat=tk, barostat=bk, kT=kT, pressure=pressure, dt=dt)
    return init_fn, apply_fn


def npt_box(state: MDState) -> np.ndarray:
    """The cell after the latest step (jax_md.simulate.npt_box, used at so3lr/cli/so3lr_md.py:1270)."""
    return state.box


def pressure(system: System, state: MDState) -> float:
    """Instantaneous pressure in eV/A^3: (2 KE - trace of the virial) / (3 V), from the latest evaluation."""
    vol = abs(float(np.linalg.det(state.box)))
    return (2.0 * kinetic_energy(state) - float(torch.trace(system.virial()))) / (3.0 * vol)


def npt_nose_hoover_invariant(state: MDState, kT: float, pressure: float, tau_t: float, tau_b: float, chain_length: int = 3) -> float:
    """Conserved quantity of the NPT dynamics in eV (jax_md.simulate.npt_nose_hoover_invariant, so3lr/cli/so3lr_md.py:940-949)."""
    c = state.chain.cpu().numpy()
    L, n = chain_length, state.mass.numel()
    vol = abs(float(np.linalg.det(state.box)))
    W = 3.0 * (n + 1) * kT * tau_b ** 2
    H = float(state.energy.sum()) + kinetic_energy(state) + c[37] ** 2 / (2.0 * W) + pressure * vol
    for off, dof, tau in ((0, 3.0 * n, tau_t), (18, 1.0, tau_b)):
        Q = kT * tau ** 2 * np.ones(L)
        Q[0] *= dof
        xi, p = c[off + 2:off + 2 + L], c[off + 10:off + 10 + L]
        H += float(np.sum(p * p / (2 * Q))) + dof * kT * xi[0] + kT * float(xi[1:].sum())
    return H


OBSERVABLES = ("partial_charges", "hirshfeld_ratios", "dipole_vec", "electrostatic_energy", "dispersion_energy", "zbl_repulsion")


def run_cycles(system: System, apply_fn, state: MDState, cycles: int, steps_per_cycle: int, sink=None, observables=(),
               on_cycle=None):
    """The outer loop of the reference's MD driver (so3lr/cli/so3lr_md.py:1815-1921): `cycles` times `steps_per_cycle` steps;
    after every cycle the frame (positions, momenta, box) goes to `sink` (so3lr_b200.trajectory.FrameSink) together with the
    requested observables, which -- as in the reference's obs_fn (so3lr/cli/so3lr_md.py:1345-1390) -- come from one more
    evaluation of the energy function with its auxiliary outputs.  Nothing here waits for the device unless the sink's ring
    of buffers is full; `on_cycle(cycle, state)` is called after each cycle (logging, restart files)."""
    for name in observables:
        if name not in OBSERVABLES:
            raise ValueError(f"Observable '{name}' is not recognized")
    for cycle in range(cycles):
        state = apply_fn(state, steps_per_cycle)
        if sink is not None:
            obs = {}
            if observables:
                out = system.compute(state.position)
                aux = system.aux() if any(k.endswith("_energy") or k == "zbl_repulsion" for k in observables) else {}
                for k in observables:
                    obs[k] = out[k][0] if k == "dipole_vec" else (out[k] if k in out else aux[k])
            sink.append(state.position, state.momentum, state.box if state.box is not None else system._cell, obs,
                        step=(cycle + 1) * steps_per_cycle)
        if on_cycle is not None:
            on_cycle(cycle, state)
    return state


def save_state(state: MDState, box, cycle: int, path_to_save, ensemble: str = "nvt"):
    """Restart file of an MD run, one .npz (so3lr/cli/so3lr_md.py:2286-2345): position, momentum, force, mass, box, the cycle
    number and the ensemble's extra state -- the thermostat chain for 'nvt', the barostat / chains record for 'npt' (both are the
    flat device records of so3lr_b200.engine.nhc_state / npt_state).  Waits for the device."""
    ens = ensemble.lower()
    if ens not in ("nve", "nvt", "npt"):
        raise ValueError("ensemble must be 'nve', 'nvt' or 'npt'")
    cpu = lambda t: np.asarray(t.detach().cpu())
    d = dict(position=cpu(state.position), momentum=cpu(state.momentum), force=cpu(state.force), mass=cpu(state.mass),
             box=np.zeros(3) if box is None else np.asarray(box, dtype=np.float64), step=int(cycle), ensemble=ens)
    if ens in ("nvt", "npt"):
        if state.chain is None:
            raise ValueError(f"an '{ens}' state carries its thermostat record in state.chain")
        d["chain"] = cpu(state.chain)
    if ens == "npt" and state.reference_box is not None:
        d["reference_box"] = np.asarray(state.reference_box, dtype=np.float64)
    np.savez(path_to_save, **d)


class RestartInNewEnsembleError(RuntimeError):
    """The restart file was written by another ensemble (so3lr/cli/so3lr_md.py:2369-2372 raises an error of this name)."""


def load_state(path_to_load, ensemble: str = "nvt", device="cuda"):
    """(state, box, cycle) from a file written by save_state; raises RestartInNewEnsembleError when the file belongs to another
    ensemble (so3lr/cli/so3lr_md.py:2348-2440)."""
    z = np.load(path_to_load, allow_pickle=False)
    ens = ensemble.lower()
    if str(z["ensemble"]) != ens:
        raise RestartInNewEnsembleError(f"restart file holds an '{z['ensemble']}' state, asked for '{ens}'")
    dev = torch.device(device)
    t = lambda a, dt=torch.float32: torch.as_tensor(np.asarray(a)).to(dev, dt).contiguous()
    mass = t(z["mass"])
    chain = t(z["chain"], torch.float64) if "chain" in z.files else None
    box = np.asarray(z["box"], dtype=np.float64)
    state = MDState(t(z["position"]), (t(z["momentum"]) / mass[:, None]).contiguous(), t(z["force"]), mass, chain, None,
                    box if box.shape == (3, 3) else None,
                    np.asarray(z["reference_box"], dtype=np.float64) if "reference_box" in z.files else None)
    return state, (None if not box.any() else box), int(z["step"])
