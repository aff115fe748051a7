"""MD step bodies on the device (velocity Verlet, Nose-Hoover chain) against the oracle's float64 integrators.

Tolerances: the chain itself runs in double on the device -> 1e-12 relative against the oracle's chain; a trajectory of a
few steps with float32 positions, velocities and forces -> positions 2e-5 A, velocities 2e-6 A/fs (measured ~1e-6 / 1e-7).
"""
import numpy as np
import pytest
import torch

from oracle import md_oracle as MD
from oracle import so3lr_oracle as O

pytestmark = pytest.mark.gpu

KT300 = 300.0 * MD.KB


@pytest.mark.parametrize("chain_length,chain_steps,sy_steps", [(3, 2, 3), (1, 1, 1), (5, 3, 5), (8, 1, 7), (2, 4, 3)])
def test_chain_kernel_matches_oracle(chain_length, chain_steps, sy_steps):
    from so3lr_b200.engine import nhc_half_steps, nhc_state
    rng = np.random.default_rng(chain_length * 100 + sy_steps)
    dof, kT, tau, dt = 3 * 500.0, KT300, 50.0, 0.5
    chain = nhc_state("cuda:0")
    c = MD.Chain(chain_length, dof, 0.0, kT, tau)
    total = 1.0
    for it in range(40):
        # kinetic energies away from equipartition so that the chain is driven
        parts = rng.uniform(0.2, 1.8, size=7) * 0.5 * dof * kT / 7 * (0.5 if it % 3 else 1.6)
        ke = torch.tensor(parts, dtype=torch.float64, device="cuda")
        n_half = 1 + it % 2
        fresh = it % 4 != 3
        nhc_half_steps(chain, n_half, dt, kT, tau, dof, ke, chain_length=chain_length, chain_steps=chain_steps, sy_steps=sy_steps,
                       fresh_scale=fresh)
        c.ke = float(parts.sum())
        s = 1.0
        for _ in range(n_half):
            s *= MD.chain_half_step(c, dt, kT, chain_steps, sy_steps)
        total = s if fresh else total * s
        got = chain.cpu().numpy()
        assert abs(got[1] / total - 1.0) < 1e-12
        assert abs(got[0] / c.ke - 1.0) < 1e-12
        np.testing.assert_allclose(got[2:2 + chain_length], c.xi, rtol=1e-10, atol=1e-14)
        np.testing.assert_allclose(got[10:10 + chain_length], c.p_xi, rtol=1e-10, atol=1e-12)
    # without partials the chain continues from the kinetic energy it holds
    nhc_half_steps(chain, 1, dt, kT, tau, dof, None, chain_length=chain_length, chain_steps=chain_steps, sy_steps=sy_steps)
    s = MD.chain_half_step(c, dt, kT, chain_steps, sy_steps)
    got = chain.cpu().numpy()
    assert abs(got[1] / s - 1.0) < 1e-12 and abs(got[0] / c.ke - 1.0) < 1e-12


def test_chain_settings_are_checked():
    from so3lr_b200.engine import nhc_half_steps, nhc_state
    chain = nhc_state("cuda:0")
    for kw in (dict(chain_length=0), dict(chain_length=9), dict(sy_steps=2), dict(sy_steps=9), dict(chain_steps=0)):
        with pytest.raises(RuntimeError):
            nhc_half_steps(chain, 1, 0.5, KT300, 50.0, 300.0, None, **kw)
    with pytest.raises(RuntimeError):
        nhc_half_steps(chain, 1, 0.5, -1.0, 50.0, 300.0, None)


def _molecule(g, name):
    Z = g[f"{name}_Z"]
    R = np.asarray(g[f"{name}_R"] - g[f"{name}_R"].mean(0), dtype=np.float32)
    masses = {1: 1.008, 6: 12.011, 7: 14.007, 8: 15.999, 16: 32.06}
    m = np.array([masses[int(z)] for z in Z], dtype=np.float32)
    rng = np.random.default_rng(21)
    V = (rng.normal(size=R.shape) * np.sqrt(KT300 * MD.ACC / m)[:, None]).astype(np.float32)
    return Z, R, V, m


def test_nvt_and_nve_trajectories_match_oracle(oracle_params, reference_goldens):
    from so3lr_b200.engine import System, nhc_state
    Z, R, V, m = _molecule(reference_goldens, "atat")
    dt, tau, steps = 0.5, 10.0, 6       # a short tau so that the thermostat visibly acts within the few steps

    def force(X):
        ref = O.energy_forces(oracle_params, X, Z, None, cutoff_lr=12.0, damping=2.0)
        return ref["energy"], ref["forces"]

    s = System(Z, None, cutoff_lr=12.0, damping=2.0)
    md = torch.tensor(m, device="cuda")
    # NVT, in two calls so that the chain is carried between them
    Rd, Vd = torch.tensor(R, device="cuda"), torch.tensor(V * 1.5, device="cuda")     # hotter than the target
    Fd = s.compute(Rd)["forces"].clone()
    chain = nhc_state("cuda:0")
    s.nvt(2, dt, KT300, tau, md, Rd, Vd, Fd, chain)
    E = s.nvt(steps - 2, dt, KT300, tau, md, Rd, Vd, Fd, chain)
    Ro, Vo, mo = R.astype(np.float64), V.astype(np.float64) * 1.5, m.astype(np.float64)
    Eo, Fo = force(Ro)
    c = MD.nvt_init(Vo, mo, KT300, tau, 3)
    scale_seen = 1.0
    for _ in range(steps):
        ke0 = c.ke
        Ro, Vo, Fo, Eo = MD.nvt_step(force, c, Ro, Vo, Fo, mo, dt, KT300, 2, 3)
        scale_seen = min(scale_seen, c.ke / max(ke0, 1e-30))
    got = chain.cpu().numpy()
    assert np.abs(Rd.cpu().numpy() - Ro).max() < 2e-5
    assert np.abs(Vd.cpu().numpy() - Vo).max() < 2e-6
    assert np.abs(Fd.cpu().numpy() - Fo).max() < 1e-4
    assert abs(float(E.sum()) - Eo) < 1e-5 * abs(Eo)
    assert got[1] == 1.0 and abs(got[0] / c.ke - 1.0) < 1e-5
    np.testing.assert_allclose(got[2:5], c.xi, rtol=1e-4, atol=1e-9)
    np.testing.assert_allclose(got[10:13], c.p_xi, rtol=1e-4, atol=1e-7)
    assert abs(c.xi[0]) > 1e-4          # the thermostat did act
    # NVE
    Rd, Vd = torch.tensor(R, device="cuda"), torch.tensor(V, device="cuda")
    Fd = s.compute(Rd)["forces"].clone()
    s.nve(steps, dt, md, Rd, Vd, Fd)
    Ro, Vo, Fo, Eo = MD.nve(force, R.astype(np.float64), V.astype(np.float64), mo, dt, steps)
    assert np.abs(Rd.cpu().numpy() - Ro).max() < 2e-5
    assert np.abs(Vd.cpu().numpy() - Vo).max() < 2e-6


def test_nvt_water_box_conserves_extended_energy_and_cools_towards_target():
    """Size-independent properties on a periodic box, through the (init_fn, apply_fn) pair the reference's MD loop is
    written against: the thermostat's conserved quantity stays put while heat is drawn from a start twice as hot as the
    target."""
    from so3lr_b200 import md
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    Z, R, cell = W.water_box(512, 24.9, 7, jitter=0.02)
    V, m = W.maxwell_boltzmann(Z, 600.0, 8)
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=0.5)
    dt, tau, dof = 0.25, 25.0, 3.0 * len(Z)
    init_fn, apply_fn = md.nvt_nose_hoover(s, dt, KT300, chain_length=3, chain_steps=2, sy_steps=3, tau=tau)
    state = init_fn(R, m, velocity=V)
    assert abs(md.temperature(state) - 600.0) < 30.0
    H0 = md.nvt_nose_hoover_invariant(state, KT300, tau)
    for _ in range(4):
        state = apply_fn(state, 30)
    H1, ke_nvt = md.nvt_nose_hoover_invariant(state, KT300, tau), md.kinetic_energy(state)
    assert abs(H1 - H0) < 2e-3 * dof * KT300, (H0, H1)      # float32 positions and forces
    assert abs(float(state.chain[0]) / ke_nvt - 1.0) < 1e-5 and float(state.chain[1]) == 1.0
    assert float(state.chain[2]) > 0 and float(state.chain[10]) > 0     # the first thermostat has been taking heat up
    # NVE from the same factory shape and the same start: total energy stays put, and without the thermostat the box
    # (which starts far from equilibrium and heats up either way) ends hotter
    init_fn, apply_fn = md.nve(s, dt)
    state = init_fn(R, m, velocity=V)
    E0 = float(state.energy.sum()) + md.kinetic_energy(state)
    state = apply_fn(state, 120)
    ke_nve = md.kinetic_energy(state)
    assert abs(float(state.energy.sum()) + ke_nve - E0) < 2e-3 * dof * KT300
    assert ke_nvt < 0.97 * ke_nve, (ke_nvt, ke_nve)


def test_decomposed_nvt_tracks_single_device():
    from so3lr_b200 import domain as D
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System, nhc_state
    from test_gpu_domain import _run_threads
    Z, R, cell = W.water_box(512, 24.9, 11, jitter=0.02)
    R = np.asarray(R, dtype=np.float32)
    V, m = W.maxwell_boltzmann(Z, 450.0, 12)
    V = np.asarray(V, dtype=np.float32)
    skin, dt, tau, steps = 0.5, 0.5, 20.0, 12
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=skin)
    Rd, Vd = torch.tensor(R, device="cuda"), torch.tensor(V, device="cuda")
    md = torch.tensor(np.asarray(m, dtype=np.float32), device="cuda")
    Fd = s.compute(Rd)["forces"].clone()
    chain = nhc_state("cuda:0")
    s.nvt(steps, dt, KT300, tau, md, Rd, Vd, Fd, chain)
    ref_chain = chain.cpu().numpy()

    def fn(comm, rank):
        be = D.CudaBackend(cutoff_lr=12.0, damping=2.0, skin=skin, device=0)
        dom = D.DomainSystem(comm, be, Z, R, cell, skin=skin, cutoff_lr=12.0, velocities=V, masses=m, device="cuda:0")
        dom.compute(check_rebuild=False)
        ch = be.nhc_state()
        dom.nvt(steps, dt, KT300, tau, ch)
        return dom.gather_global(dom.R[: dom.n0]).cpu().numpy(), dom.gather_global(dom.V).cpu().numpy(), ch.cpu().numpy()

    res = _run_threads(2, fn)
    np.testing.assert_array_equal(res[0][2], res[1][2])          # both ranks hold the same chain, bit for bit
    Rdd, Vdd, ch = res[0]
    d = Rdd - Rd.cpu().numpy()
    d -= np.round(d / 24.9) * 24.9
    assert np.abs(d).max() < 1e-3 and np.median(np.abs(d)) < 2e-5, (np.abs(d).max(), np.median(np.abs(d)))
    assert np.median(np.abs(Vdd - Vd.cpu().numpy())) < 2e-6
    np.testing.assert_allclose(ch[2:5], ref_chain[2:5], rtol=1e-3, atol=1e-8)
    np.testing.assert_allclose(ch[10:13], ref_chain[10:13], rtol=1e-3, atol=1e-5)


def test_npt_trajectory_matches_oracle(oracle_params):
    """A few NPT steps of the 192-atom water box against the oracle's float64 integrator driven by the oracle's energy, forces
    and strain derivative.  Short time constants so that box and chains move visibly within the few steps."""
    from so3lr_b200 import md
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    Z, R, cell = W.water_box(64, 12.42, 1000)
    R = np.asarray(R, dtype=np.float32)
    cell = np.asarray(cell, dtype=np.float64)
    V, m = W.maxwell_boltzmann(Z, 300.0, 3)
    V, m = np.asarray(V, dtype=np.float32), np.asarray(m, dtype=np.float32)
    dt, tau_t, tau_b, steps, lr = 0.5, 10.0, 40.0, 5, 5.5
    P_target = 1000.0 * md.BAR

    def force(X, c):
        ref = O.energy_forces(oracle_params, X, Z, c, cutoff_lr=lr, damping=2.0)
        return ref["energy"], ref["forces"], ref["virial"]

    s = System(Z, cell, cutoff_lr=lr, damping=2.0, skin=0.3)
    init_fn, apply_fn = md.npt_nose_hoover(s, dt, P_target, KT300, barostat_kwargs=dict(tau=tau_b), thermostat_kwargs=dict(tau=tau_t))
    state = init_fn(R, cell, m, velocity=V)
    state = apply_fn(state, 2)
    state = apply_fn(state, steps - 2)          # the state is carried between calls
    o = MD.NPTState(R.astype(np.float64), V.astype(np.float64), m.astype(np.float64), cell, KT300, tau_t, tau_b, 3, force)
    for _ in range(steps):
        MD.npt_step(force, o, dt, KT300, P_target, 2, 3)
    c = state.chain.cpu().numpy()
    assert abs(o.eps) > 1e-7                                     # the box did move
    assert abs(c[36] - o.eps) < 2e-3 * abs(o.eps) + 1e-9, (c[36], o.eps)
    assert abs(c[37] - o.p_eps) < 2e-3 * abs(o.p_eps), (c[37], o.p_eps)
    np.testing.assert_allclose(md.npt_box(state), o.cell(), rtol=2e-6)
    assert np.abs(state.position.cpu().numpy() - o.R).max() < 5e-5
    assert np.abs(state.velocity.cpu().numpy() - o.V).max() < 3e-6
    assert abs(float(state.energy.sum()) - o.E) < 1e-5 * abs(o.E)
    np.testing.assert_allclose(c[2:5], o.thermostat.xi, rtol=1e-3, atol=1e-9)
    np.testing.assert_allclose(c[10:13], o.thermostat.p_xi, rtol=1e-3, atol=1e-6)
    np.testing.assert_allclose(c[20:23], o.barostat.xi, rtol=1e-2, atol=1e-9)
    np.testing.assert_allclose(c[28:31], o.barostat.p_xi, rtol=1e-2, atol=1e-6)
    assert c[1] == 1.0 and abs(c[42] / o.volume() - 1.0) < 1e-6


def test_npt_water_box_conserves_its_invariant_and_moves_towards_the_target_pressure():
    from so3lr_b200 import md
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    Z, R, cell = W.water_box(512, 24.9, 7, jitter=0.02)
    cell = np.asarray(cell, dtype=np.float64)
    V, m = W.maxwell_boltzmann(Z, 300.0, 8)
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=0.5)
    dt, tau_t, tau_b = 0.25, 25.0, 100.0
    init_fn, apply_fn = md.npt_nose_hoover(s, dt, 0.0, KT300, barostat_kwargs=dict(tau=tau_b), thermostat_kwargs=dict(tau=tau_t))
    state = init_fn(R, cell, m, velocity=V)
    p0 = md.pressure(s, state)
    target = p0 - np.sign(p0) * 2000.0 * md.BAR           # 2 kbar towards zero from where the start happens to be
    init_fn, apply_fn = md.npt_nose_hoover(s, dt, target, KT300, barostat_kwargs=dict(tau=tau_b), thermostat_kwargs=dict(tau=tau_t))
    state = init_fn(R, cell, m, velocity=V)
    H0 = md.npt_nose_hoover_invariant(state, KT300, target, tau_t, tau_b)
    vol0 = abs(np.linalg.det(state.box))
    state = apply_fn(state, 4)
    # pressure above the target pushes the box outwards, below it inwards (the first steps; the pressure of this
    # unequilibrated start swings by tens of kbar within a few fs afterwards)
    assert float(state.chain[37]) * np.sign(p0 - target) > 0
    assert (abs(np.linalg.det(md.npt_box(state))) - vol0) * np.sign(p0 - target) > 0
    for _ in range(4):
        state = apply_fn(state, 24)
    H1 = md.npt_nose_hoover_invariant(state, KT300, target, tau_t, tau_b)
    dof = 3.0 * len(Z)
    assert abs(H1 - H0) < 2e-3 * dof * KT300, (H0, H1)
    assert abs(abs(np.linalg.det(md.npt_box(state))) / vol0 - 1.0) > 1e-4        # the box keeps moving
    # the context's cell followed the box: a fresh context at the final cell gives the same energy and forces
    chk = System(Z, md.npt_box(state), cutoff_lr=12.0, damping=2.0).compute(state.position)
    assert abs(float(chk["energy"].sum()) - float(state.energy.sum())) < 1e-5 * abs(float(state.energy.sum()))
    assert np.abs(chk["forces"].cpu().numpy() - state.force.cpu().numpy()).max() < 2e-4


def test_decomposed_npt_tracks_single_device():
    from so3lr_b200 import domain as D
    from so3lr_b200 import md
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System, npt_state
    from test_gpu_domain import _run_threads
    Z, R, cell = W.water_box(512, 24.9, 11, jitter=0.02)
    R, cell = np.asarray(R, dtype=np.float32), np.asarray(cell, dtype=np.float64)
    V, m = W.maxwell_boltzmann(Z, 300.0, 12)
    V, m = np.asarray(V, dtype=np.float32), np.asarray(m, dtype=np.float32)
    skin, dt, tau_t, tau_b, steps = 0.5, 0.5, 20.0, 60.0, 10
    P_target = 1000.0 * md.BAR
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=skin)
    s.enable_virial(True)
    Rd, Vd = torch.tensor(R, device="cuda"), torch.tensor(V, device="cuda")
    mdv = torch.tensor(m, device="cuda")
    Fd = s.compute(Rd)["forces"].clone()
    st = npt_state("cuda:0")
    _, cell_ref = s.npt(steps, dt, KT300, P_target, tau_t, tau_b, mdv, Rd, Vd, Fd, st, cell)
    ref = st.cpu().numpy()
    assert abs(ref[36]) > 1e-6                     # the box moved

    def fn(comm, rank):
        be = D.CudaBackend(cutoff_lr=12.0, damping=2.0, skin=skin, device=0)
        be.enable_virial(True)
        dom = D.DomainSystem(comm, be, Z, R, cell, skin=skin, cutoff_lr=12.0, velocities=V, masses=m, device="cuda:0")
        dom.compute(check_rebuild=False)
        state = be.npt_state()
        dom.npt(4, dt, KT300, P_target, tau_t, tau_b, state, cell)
        _, c = dom.npt(steps - 4, dt, KT300, P_target, tau_t, tau_b, state, cell)
        return dom.gather_global(dom.R[: dom.n0]).cpu().numpy(), dom.gather_global(dom.V).cpu().numpy(), state.cpu().numpy(), c

    res = _run_threads(2, fn)
    np.testing.assert_array_equal(res[0][2], res[1][2])          # both ranks hold the same box and chains, bit for bit
    Rdd, Vdd, stt, c = res[0]
    assert abs(stt[36] - ref[36]) < 1e-3 * abs(ref[36]) + 1e-9, (stt[36], ref[36])
    assert abs(stt[37] - ref[37]) < 2e-3 * abs(ref[37]), (stt[37], ref[37])
    np.testing.assert_allclose(c, cell_ref, rtol=1e-6)
    d = Rdd - Rd.cpu().numpy()
    d -= np.round(d / c[0, 0]) * c[0, 0]
    assert np.abs(d).max() < 1e-3 and np.median(np.abs(d)) < 2e-5, (np.abs(d).max(), np.median(np.abs(d)))
    assert np.median(np.abs(Vdd - Vd.cpu().numpy())) < 2e-6
    np.testing.assert_allclose(stt[2:5], ref[2:5], rtol=1e-3, atol=1e-8)
    assert stt[1] == 1.0


def test_deferred_skin_test_gives_the_same_trajectory():
    """so3lr_b200_system_defer_skin_test: the rebuild decision is read one step late (no host wait per step) and the trigger
    distance is lowered by the margin.  Lists built earlier or later hold the same pairs inside the cutoff, so the trajectory
    equals the default mode's up to the order of float32 sums, and the lists are still rebuilt on the way."""
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    Z, R, cell = W.water_box(64, 12.42, 1000)
    V, m = W.maxwell_boltzmann(Z, 300.0, 3)
    res = []
    for deferred in (False, True):
        s = System(Z, cell, cutoff_lr=6.0, damping=2.0, skin=0.6)
        if deferred:
            s.defer_skin_test(True, margin=0.05)
        Rd = torch.tensor(R, dtype=torch.float32, device="cuda")
        Vd = torch.tensor(V, dtype=torch.float32, device="cuda")
        md = torch.tensor(m, dtype=torch.float32, device="cuda")
        Fd = s.compute(Rd)["forces"].clone()
        s.nve(120, 0.5, md, Rd, Vd, Fd)
        torch.cuda.synchronize()
        res.append((Rd.cpu().numpy(), Fd.cpu().numpy(), s.stats()["rebuilds"]))
    (R0, F0, n0), (R1, F1, n1) = res
    assert n0 >= 2 and n1 >= 2                       # both modes rebuild their lists on the way
    assert np.abs(R1 - R0).max() < 2e-3 and np.abs(F1 - F0).max() < 5e-2      # chaotic growth of float32 differences over 120 steps
    assert np.median(np.abs(R1 - R0)) < 2e-5


def test_md_loop_writes_frames_and_observables_without_waiting_for_the_device(tmp_path):
    """The outer loop of the reference's MD driver (cycles of steps, a frame and the observables after each cycle,
    so3lr/cli/so3lr_md.py:1815-1921) with the asynchronous frame writer: what lands in the files is the state at the end of each
    cycle, although the integrator goes on overwriting the positions in place while the copies are in flight."""
    from so3lr_b200 import md
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    from so3lr_b200.trajectory import FrameSink, read_extxyz
    Z, R, cell = W.water_box(216, 18.7, 5, jitter=0.03)
    V, m = W.maxwell_boltzmann(Z, 300.0, 6)
    s = System(Z, cell, cutoff_lr=8.0, damping=2.0, skin=0.5)
    init_fn, apply_fn = md.nve(s, 0.5)
    snaps = []
    obs = ("partial_charges", "hirshfeld_ratios", "dipole_vec", "electrostatic_energy")
    for fmt in ("extxyz", "npy"):
        state = init_fn(R, m, velocity=V)
        snaps.clear()
        path = tmp_path / ("traj." + fmt)
        with FrameSink(path, Z, fmt, observables=obs, slots=2) as sink:
            md.run_cycles(s, apply_fn, state, cycles=5, steps_per_cycle=4, sink=sink, observables=obs,
                          on_cycle=lambda c, st: snaps.append((st.position.clone(), st.momentum.clone())))
        assert sink.frames_written == 5
        want_R = np.stack([a.cpu().numpy() for a, _ in snaps])
        want_P = np.stack([b.cpu().numpy() for _, b in snaps])
        assert np.abs(want_R[1] - want_R[0]).max() > 1e-3            # the atoms did move between the frames
        if fmt == "extxyz":
            fr = read_extxyz(path)
            got_R, got_P = np.stack([f["pos"] for f in fr]), np.stack([f["momenta"] for f in fr])
            q, h = fr[-1]["charges"], fr[-1]["hirsh_ratios"]
            dip = np.array([float(v) for v in fr[-1]["info"]["dipole_vec"].split()])
            np.testing.assert_allclose(fr[0]["cell"], np.asarray(cell))
            assert [int(f["info"]["step"]) for f in fr] == [4, 8, 12, 16, 20]
            tol = 2e-7 * np.abs(want_R).max() + 1e-8                 # eight decimals in the text file
        else:
            got_R, got_P = np.load(path / "positions.npy"), np.load(path / "momenta.npy")
            q, h, dip = np.load(path / "partial_charges.npy")[-1], np.load(path / "hirshfeld_ratios.npy")[-1], np.load(path / "dipole_vec.npy")[-1]
            assert np.load(path / "electrostatic_energy.npy").shape == (5, len(Z)) and np.load(path / "box.npy").shape == (5, 3, 3)
            tol = 0.0
        np.testing.assert_allclose(got_R, want_R, atol=tol + 1e-7)
        np.testing.assert_allclose(got_P, want_P, atol=1e-6)
        ref = s.compute(snaps[-1][0])
        np.testing.assert_allclose(q, ref["partial_charges"].cpu().numpy(), atol=1e-6)
        np.testing.assert_allclose(h, ref["hirshfeld_ratios"].cpu().numpy(), atol=1e-6)
        # sum_i q_i R_i over 648 atoms up to 18.7 A from the origin: a uniform charge offset of 1e-7 (float32 rounding of the charge
        # conservation, which differs between two evaluations with different atom orderings) moves it by 6e-4
        np.testing.assert_allclose(dip, ref["dipole_vec"][0].cpu().numpy(), atol=2e-3)


def test_md_steps_replayed_from_a_cuda_graph_match_plain_launches():
    """Between two list rebuilds the force evaluation of a small structure is replayed from a CUDA graph when the caller's stream
    can be captured; on the legacy default stream the same steps run as plain launches.  Same trajectory either way."""
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    Z, R, cell = W.water_box(216, 18.7, 5, jitter=0.03)
    V, m = W.maxwell_boltzmann(Z, 300.0, 6)

    def run(stream, steps=14):
        s = System(Z, cell, cutoff_lr=8.0, damping=2.0, skin=0.6)
        s.defer_skin_test(True, 0.05)
        with torch.cuda.stream(stream):
            Rd = torch.tensor(np.asarray(R, dtype=np.float32), device="cuda")
            Vd = torch.tensor(np.asarray(V, dtype=np.float32), device="cuda")
            md_ = torch.tensor(np.asarray(m, dtype=np.float32), device="cuda")
            Fd = s.compute(Rd)["forces"].clone()
            E = s.nve(steps, 0.5, md_, Rd, Vd, Fd)
        stream.synchronize()
        return Rd.cpu().numpy(), Fd.cpu().numpy(), float(E.sum()), s.stats(), s.graph_replays()

    Ra, Fa, Ea, sa, ra = run(torch.cuda.Stream())
    Rb, Fb, Eb, sb, rb = run(torch.cuda.default_stream())
    assert rb == 0 and ra >= 8, (ra, rb)                 # replays on the side stream (the first two steps capture), none on the default one
    assert sa["launches"] == sb["launches"] and sa["rebuilds"] == sb["rebuilds"]
    np.testing.assert_allclose(Ra, Rb, atol=2e-5)        # atomics reorder sums: float32 roundoff over 14 steps
    np.testing.assert_allclose(Fa, Fb, atol=2e-4)
    assert abs(Ea - Eb) < 1e-5 * abs(Eb)
