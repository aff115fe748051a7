"""Host-side logic of the domain decomposition on CPU ranks (gloo, world size 2 and 3) with a stand-in model.

The stand-in has the same dependency structure as the real evaluation phases: a per-atom quantity from the short-range
neighbourhood ("raw charge"), a global conservation constraint, a pair term that couples the charges over the long
range, and forces obtained by differentiating each rank's share of the energy.  The decomposed result must equal
the single-domain result of the same stand-in: energy, forces in the caller's atom order, and it must stay equal after
atoms have moved far enough to trigger re-partitioning (atoms migrate between ranks).
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle import md_oracle as MD
from so3lr_b200 import domain as D

RC_SR, RC_LR = 4.5, 9.0


def _min_image(d, cell):
    inv = torch.linalg.inv(cell)
    s = d @ inv
    return d - torch.round(s) @ cell


class ToyBackend:
    """Stand-in with the dependency structure of the real evaluation: two message-passing layers over the 4.5 A shell
    (x_{l+1}[i] = x_l[i] + sum_j psi(r_ij) tanh(x_l[j])), a per-atom energy x_L^2, raw charges tanh(x_L) made neutral
    globally, and a pair term sum_{i<j} q_i q_j chi(r_ij) over the long range.  Implements the backend protocol of
    so3lr_b200.domain: everything is evaluated for the owned atoms only, by gathering from owned and ghost rows."""
    num_layers = 2

    def set_atoms(self, Z_local, counts, cell_local):
        self.n0, self.n1, self.n = [int(v) for v in counts]
        self.cell = torch.tensor(np.asarray(cell_local), dtype=torch.float64)
        self.x = [torch.ones(self.n, 1, dtype=torch.float64) for _ in range(self.num_layers + 1)]
        self.G = torch.zeros(self.n, 1, dtype=torch.float64)

    @staticmethod
    def psi(r):
        return torch.where(r < RC_SR, (1 - r / RC_SR) ** 3, torch.zeros_like(r))

    @staticmethod
    def dpsi(r):
        return torch.where(r < RC_SR, -3 * (1 - r / RC_SR) ** 2 / RC_SR, torch.zeros_like(r))

    @staticmethod
    def chi(r):
        return torch.where(r < RC_LR, (1 - r / RC_LR) ** 3 / (1 + r), torch.zeros_like(r))

    @staticmethod
    def dchi(r):
        return torch.where(r < RC_LR, -3 * (1 - r / RC_LR) ** 2 / RC_LR / (1 + r) - (1 - r / RC_LR) ** 3 / (1 + r) ** 2,
                           torch.zeros_like(r))

    # reciprocal-space stand-in: E_k = 1/2 sum_k g(k) |S(k)|^2 over a few k vectors of the whole cell, S(k) = sum_i q_i exp(i k r_i)
    kvec = None

    @staticmethod
    def k_vectors(shape, smearing, cell):
        h = np.stack(np.meshgrid(*[np.arange(-(n // 2), (n + 1) // 2) for n in shape], indexing="ij"), -1).reshape(-1, 3)
        h = h[(h != 0).any(1)]
        k = 2 * np.pi * torch.tensor(h, dtype=torch.float64) @ torch.linalg.inv(torch.as_tensor(np.asarray(cell), dtype=torch.float64)).T
        k2 = (k * k).sum(-1)
        return k, torch.exp(-0.5 * smearing ** 2 * k2) / k2

    def set_kspace(self, shape, smearing, method, cell_global, total_charge):
        self.kset = None if shape is None else (shape, smearing)
        self.kvec = None
        if shape is not None:
            self.kspace_cell(cell_global)

    def kspace_cell(self, cell_global):
        self.kvec, self.kg = self.k_vectors(self.kset[0], self.kset[1], cell_global)

    def kspace_accumulate(self):
        th = self.Rown @ self.kvec.T
        q = self.q_all[: self.n0]
        self.S = torch.cat([(q[:, None] * torch.cos(th)).sum(0), (q[:, None] * torch.sin(th)).sum(0)])
        return self.S

    def kspace_finish(self, add_strain):
        K = len(self.kvec)
        Sr, Si = self.S[:K], self.S[K:]
        th = self.Rown @ self.kvec.T
        c, s = torch.cos(th), torch.sin(th)
        q = self.q_all[: self.n0]
        phi = ((c * Sr[None, :] + s * Si[None, :]) * self.kg[None, :]).sum(1)
        self.e_k_half = 0.5 * (q * phi).sum()
        self.gq = self.gq + phi
        self.F -= q[:, None] * (((c * Si[None, :] - s * Sr[None, :]) * self.kg[None, :]) @ self.kvec)
        return self.gq.sum().reshape(1)

    def begin(self, R_local):
        n0 = self.n0
        R = R_local.detach().to(torch.float64)
        self.Rown = R[:n0]
        self.e_k_half = 0.0
        self.d = _min_image(R[None, :, :] - R[:n0, None, :], self.cell)          # (n0, n, 3): R_j - R_i
        r = self.d.norm(dim=-1)
        r[torch.arange(n0), torch.arange(n0)] = 1e3
        self.r = r
        self.F = torch.zeros(n0, 3, dtype=torch.float64)
        for x in self.x:
            x.fill_(1.0)

    def layer_forward(self, l):
        n0 = self.n0
        msg = (self.psi(self.r) * torch.tanh(self.x[l][:, 0])[None, :]).sum(1)
        self.x[l + 1][:n0, 0] = self.x[l][:n0, 0] + msg

    def feature_rows(self, l):
        return [self.x[l]]

    def heads(self):
        xL = self.x[-1][: self.n0, 0]
        return torch.tanh(xL).float(), xL.abs().float()

    def pair(self, q_local, h_local):
        n0 = self.n0
        q = q_local.detach().to(torch.float64)
        self.q_all = q
        chi = self.chi(self.r)
        self.e_pair_half = 0.5 * (q[:n0, None] * q[None, :] * chi).sum()
        self.gq = (q[None, :] * chi).sum(1)                                        # dE/dq_i over all pairs of i
        s = (q[:n0, None] * q[None, :] * self.dchi(self.r) / self.r)[..., None] * self.d
        self.F += s.sum(1)                                                         # F_i = +dE_ij/d(R_j - R_i)
        return self.gq.sum().reshape(1)

    def heads_backward(self, gq_sum_all, n_all):
        n0 = self.n0
        xL = self.x[-1][:n0, 0]
        gq_raw = self.gq - gq_sum_all / n_all
        self.g = 2 * xL + gq_raw * (1 - torch.tanh(xL) ** 2)                        # cotangent of x_L, owned atoms
        return ((xL ** 2).sum() + self.e_pair_half + self.e_k_half).reshape(1)

    def layer_backward_post(self, l):
        self.G.zero_()
        self.G[: self.n0, 0] = self.g

    def cotangent_rows(self):
        return [self.G]

    def layer_backward_attn(self, l):
        n0 = self.n0
        G, x = self.G[:, 0], self.x[l][:, 0]
        t = torch.tanh(x)
        psi, dpsi = self.psi(self.r), self.dpsi(self.r)
        # both directions of every edge, gathered towards the owned atom i
        self.g = G[:n0] + (psi * G[None, :]).sum(1) * (1 - t[:n0] ** 2)
        coef = dpsi * (G[:n0, None] * t[None, :] + G[None, :] * t[:n0, None]) / self.r   # dE/dr_ij / r
        self.F += (coef[..., None] * self.d).sum(1)

    def forces(self):
        return self.F.float()

    # thermostat chain with the layout of the device one: [0] kinetic energy, [1] waiting scale, [2:10] xi, [10:18] p_xi
    def nhc_state(self):
        c = torch.zeros(18, dtype=torch.float64)
        c[1] = 1.0
        return c

    def nhc_half_steps(self, chain, n_half, dt_fs, kT, tau_fs, dof, kinetic_energy, chain_length=3, chain_steps=2, sy_steps=3):
        c = MD.Chain(chain_length, dof, float(kinetic_energy.sum()), kT, tau_fs)
        c.xi[:] = chain[2:2 + chain_length].numpy()
        c.p_xi[:] = chain[10:10 + chain_length].numpy()
        scale = 1.0
        for _ in range(n_half):
            scale *= MD.chain_half_step(c, dt_fs, kT, chain_steps, sy_steps)
        chain[0], chain[1] = c.ke, scale
        chain[2:2 + chain_length] = torch.from_numpy(c.xi)
        chain[10:10 + chain_length] = torch.from_numpy(c.p_xi)


def _serial_reference(R, cell, kspace=None):
    R = torch.tensor(R, dtype=torch.float64, requires_grad=True)
    c = torch.tensor(cell, dtype=torch.float64)
    d = _min_image(R[None] - R[:, None], c)
    r = d.norm(dim=-1) + torch.eye(len(R), dtype=torch.float64) * 1e3
    x = torch.ones(len(R), dtype=torch.float64)
    for _ in range(ToyBackend.num_layers):
        x = x + (ToyBackend.psi(r) * torch.tanh(x)[None, :]).sum(1)
    q = torch.tanh(x)
    q = q - q.mean()
    E = (x ** 2).sum() + 0.5 * (q[:, None] * q[None, :] * ToyBackend.chi(r)).sum()
    if kspace is not None:
        k, g = ToyBackend.k_vectors(kspace[0], kspace[1], cell)
        th = R @ k.T
        E = E + 0.5 * (g * ((q[:, None] * torch.cos(th)).sum(0) ** 2 + (q[:, None] * torch.sin(th)).sum(0) ** 2)).sum()
    F = -torch.autograd.grad(E, R)[0]
    return E.item(), F.numpy()


def _problem(seed=3, n=160, box=(46.0, 19.0, 19.5)):
    rng = np.random.default_rng(seed)
    cell = np.diag(box)
    R = rng.uniform(0, 1, size=(n, 3)) * np.array(box)
    return R.astype(np.float32), cell


NVT_STEPS, NVT_DT, NVT_KT, NVT_TAU = 6, 0.5, 0.5, 20.0
KSPACE = ((5, 3, 4), 3.0)


def _nvt_problem():
    R, _ = _problem()
    rng = np.random.default_rng(11)
    m = rng.uniform(1.0, 16.0, size=len(R)).astype(np.float32)
    V = (rng.normal(size=R.shape) * 0.05 / np.sqrt(m)[:, None]).astype(np.float32)
    return R, V, m


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    R, cell = _problem()
    Z = np.ones(len(R), np.int32)
    V = np.zeros_like(R)
    dom = D.DomainSystem(D.DistComm(), ToyBackend(), Z, R, cell, skin=1.0, cutoff_lr=RC_LR, velocities=V, masses=np.ones(len(R)))
    E, _ = dom.compute(check_rebuild=False)
    res = {"E0": float(E), "F0": dom.global_forces().numpy(), "n_own": dom.n0, "n_local": dom.n_local}
    # move every atom by a known displacement larger than skin/2 along the decomposed axis: re-partition + migration
    shift = np.zeros(3, np.float32); shift[dom.geo.axis] = 3.7
    dom.R[: dom.n0] += torch.tensor(shift)
    E1, _ = dom.compute()
    res.update(E1=float(E1), F1=dom.global_forces().numpy(), rebuilds=dom.n_rebuilds, R1=dom.gather_global(dom.R[: dom.n0]).numpy())
    # host-buffer entry point: all positions in, total energy and all forces out
    E2, F2 = dom.compute_host(R)
    E3, F3 = dom.compute_host(R + 0.01)          # small move: no re-partitioning, same forces
    res.update(E2=E2, F2=F2.copy(), E3=E3, F3=F3.copy(), rebuilds_host=dom.n_rebuilds)
    # thermostatted steps: every rank advances its own copy of the chain with the all-reduced kinetic energy
    Rt, Vt, mt = _nvt_problem()
    dom = D.DomainSystem(D.DistComm(), ToyBackend(), Z, Rt, cell, skin=1.0, cutoff_lr=RC_LR, velocities=Vt, masses=mt)
    dom.compute(check_rebuild=False)
    chain = dom.backend.nhc_state()
    dom.nvt(NVT_STEPS, NVT_DT, NVT_KT, NVT_TAU, chain)
    res.update(Rt=dom.gather_global(dom.R[: dom.n0]).numpy(), Vt=dom.gather_global(dom.V).numpy(), chain=chain.numpy().copy())
    # reciprocal-space part: the ranks' shares of the structure factors are summed over the ranks (the one exchange of that part)
    dom = D.DomainSystem(D.DistComm(), ToyBackend(), Z, R, cell, skin=1.0, cutoff_lr=RC_LR, velocities=V, masses=np.ones(len(R)))
    dom.set_kspace(KSPACE[0], KSPACE[1], "ewald")
    Ek, _ = dom.compute(check_rebuild=False)
    res.update(Ek=float(Ek), Fk=dom.global_forces().numpy())
    dom.set_kspace(None)
    res.update(Ek_off=float(dom.compute(check_rebuild=False)[0]))
    if rank == 0:
        torch.save(res, out)
    dist.barrier()
    dist.destroy_process_group()


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


@pytest.mark.parametrize("world", [2, 3])
def test_decomposed_toy_model_matches_single_domain(tmp_path, world):
    out = str(tmp_path / "res.pt")
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    res = torch.load(out, weights_only=False)
    R, cell = _problem()
    E0, F0 = _serial_reference(R, cell)
    assert abs(res["E0"] - E0) < 1e-6 * max(1.0, abs(E0))
    np.testing.assert_allclose(res["F0"], F0, atol=2e-5)
    assert res["rebuilds"] == 2
    R1 = R.copy(); R1[:, 0] += 3.7
    E1, F1 = _serial_reference(R1, cell)
    assert abs(res["E1"] - E1) < 1e-6 * max(1.0, abs(E1))
    np.testing.assert_allclose(res["F1"], F1, atol=2e-5)
    assert abs(res["E2"] - E0) < 1e-6 * max(1.0, abs(E0)) and abs(res["E3"] - E0) < 1e-5 * max(1.0, abs(E0))
    np.testing.assert_allclose(res["F2"], F0, atol=2e-5)
    np.testing.assert_allclose(res["F3"], F0, atol=1e-4)
    assert res["rebuilds_host"] == 3
    Ek, Fk = _serial_reference(R, cell, KSPACE)
    assert abs(Ek - E0) > 1e-3 and abs(res["Ek"] - Ek) < 1e-6 * max(1.0, abs(Ek)) and abs(res["Ek_off"] - E0) < 1e-6 * max(1.0, abs(E0))
    np.testing.assert_allclose(res["Fk"], Fk, atol=2e-5)
    # thermostatted trajectory against the serial integrator of the oracle with the serial forces
    Rt, Vt, mt = _nvt_problem()
    force = lambda X: _serial_reference(X, cell)
    Rs, Vs, ms = Rt.astype(np.float64), Vt.astype(np.float64), mt.astype(np.float64)
    _, Fs = force(Rs)
    c = MD.nvt_init(Vs, ms, NVT_KT, NVT_TAU, 3)
    for _ in range(NVT_STEPS):
        Rs, Vs, Fs, _ = MD.nvt_step(force, c, Rs, Vs, Fs, ms, NVT_DT, NVT_KT, 2, 3)
    dt_ = res["Rt"] - Rs
    dt_[:, 0] -= np.round(dt_[:, 0] / cell[0, 0]) * cell[0, 0]
    np.testing.assert_allclose(dt_, 0, atol=2e-5)
    np.testing.assert_allclose(res["Vt"], Vs, atol=2e-6, rtol=1e-5)
    np.testing.assert_allclose(res["chain"][2:5], c.xi, rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(res["chain"][10:13], c.p_xi, rtol=1e-4, atol=1e-7)
    assert res["chain"][1] == 1.0
    # positions come back in the caller's order, wrapped into the cell along the decomposed axis
    d = res["R1"] - R1
    d[:, 0] -= np.round(d[:, 0] / cell[0, 0]) * cell[0, 0]
    np.testing.assert_allclose(d, 0, atol=1e-4)


def test_slab_selection_holds_every_partner_of_an_owned_atom():
    R, cell = _problem(seed=5, n=400)
    geo = D.SlabDecomposition(cell, 3, skin=1.0, cutoff_lr=RC_LR)
    Rt = torch.tensor(R)
    Rw, s = geo.wrap(Rt)
    owner = geo.owner(s)
    total_owned = 0
    for rank in range(3):
        idx, shift, cls = geo.selection(rank, Rw, s)
        n0 = int((cls == 0).sum())
        total_owned += n0
        assert (cls[:-1] <= cls[1:]).all()                           # owned first, then short-range ghosts, then the rest
        assert (owner[idx[:n0]] == rank).all()
        Rl = Rw[idx].double() + shift[:, None].double() * torch.tensor(cell[geo.axis])
        own_pos = Rl[:n0]
        have = {}
        for g, k, c in zip(idx.tolist(), shift.tolist(), cls.tolist()):
            have[(g, k)] = c
        # every atom image within the short-range (long-range) list radius of an owned atom is present locally, and the
        # short-range ones are classed as feature-carrying ghosts (brute force over images)
        for k in (-1, 0, 1):
            img = Rw.double() + k * torch.tensor(cell[geo.axis])
            d = (img[None] - own_pos[:, None])
            d[..., 1] -= torch.round(d[..., 1] / cell[1, 1]) * cell[1, 1]
            d[..., 2] -= torch.round(d[..., 2] / cell[2, 2]) * cell[2, 2]
            dist = d.norm(dim=-1)
            for g in torch.nonzero((dist < geo.lr_radius).any(0)).squeeze(1).tolist():
                assert (g, k) in have
            for g in torch.nonzero((dist < geo.shell).any(0)).squeeze(1).tolist():
                assert have[(g, k)] <= 1
    assert total_owned == len(R)


# ---- independent structures over ranks: partition logic and result gathering (no GPU: a stand-in evaluator) ----
class _FakeSystem:
    def __init__(self, Z, cell, **kw):
        self.Z = Z
        gs = kw.get("graph_start")
        self.gs = np.array([0, len(Z)]) if gs is None else np.asarray(gs)

    def compute_host(self, R):
        e = np.array([float((self.Z[a:b] * R[a:b, 0]).sum()) for a, b in zip(self.gs[:-1], self.gs[1:])])
        return dict(energy=e, forces=-R * self.Z[:, None], partial_charges=R[:, 1].copy(), hirshfeld_ratios=R[:, 2].copy(),
                    dipole_vec=np.zeros((len(e), 3), np.float32))


def _batch_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from so3lr_b200 import batch as B
    from so3lr_b200 import workloads as W
    dist.init_process_group("gloo", rank=rank, world_size=world)
    Z, R, gs = W.molecule_batch(23, seed=1001)
    sb = B.ShardedBatch(Z, gs, world, rank, system_factory=_FakeSystem)
    res = B.gather_results(sb.compute_host(R), world)
    if rank == 0:
        torch.save(res, out)
    dist.barrier()
    dist.destroy_process_group()


def test_graph_shards_cover_the_batch_and_are_balanced(tmp_path):
    from so3lr_b200 import batch as B
    from so3lr_b200 import workloads as W
    Z, R, gs = W.molecule_batch(23, seed=1001)
    for world in (1, 2, 3, 8, 40):
        ranges = [B.shard_graphs(gs, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == 23
        assert all(a[1] == b[0] for a, b in zip(ranges[:-1], ranges[1:]))
        if world <= 8:
            atoms = [gs[b] - gs[a] for a, b in ranges]
            assert max(atoms) - min(atoms) <= 2 * 40            # within two molecules of each other
    out = str(tmp_path / "b.pt")
    mp.spawn(_batch_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out, weights_only=False)
    ref = _FakeSystem(Z, None, graph_start=gs).compute_host(R.astype(np.float32))
    np.testing.assert_allclose(res["energy"], ref["energy"], rtol=1e-6)
    np.testing.assert_allclose(res["forces"], ref["forces"])
