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

from so3lr_b200 import domain as D

RC_SR, RC_LR = 4.5, 9.0


def _min_image(d, cell):
    inv = torch.linalg.inv(cell)
    s = d @ inv
    return d - torch.round(s) @ cell


class ToyBackend:
    """E = sum_i a_i^2 + sum_{i<j} q_i q_j chi(r_ij), a_i = sum_j psi(r_ij) over the 4.5 A shell, q_i = tanh(a_i) shifted
    so that the charges sum to zero.  Implements the forward / pair / backward protocol of so3lr_b200.domain backends."""

    def __init__(self):
        self.n_set = 0

    def set_atoms(self, Z_local, shells, cell_local):
        self.shells = [int(v) for v in shells]
        self.cell = torch.tensor(np.asarray(cell_local), dtype=torch.float64)
        self.n_set += 1

    @staticmethod
    def psi(r):
        return torch.where(r < RC_SR, (1 - r / RC_SR) ** 3, torch.zeros_like(r))

    @staticmethod
    def chi(r):
        return torch.where(r < RC_LR, (1 - r / RC_LR) ** 3 / (1 + r), torch.zeros_like(r))

    def forward(self, R_local):
        n0 = self.shells[0]
        self.R = R_local.detach().to(torch.float64).requires_grad_(True)
        d = _min_image(self.R[None, :, :] - self.R[:n0, None, :], self.cell)
        r = d.norm(dim=-1)
        mask = torch.ones_like(r, dtype=torch.bool)
        mask[torch.arange(n0), torch.arange(n0)] = False
        self.r = torch.where(mask, r, torch.full_like(r, 1e3))
        self.a = self.psi(self.r).sum(1)
        self.q_raw = torch.tanh(self.a)
        return self.q_raw.detach().float(), self.a.detach().abs().float()

    def pair(self, q_local, h_local):
        n0 = self.shells[0]
        self.q_in = q_local.detach().to(torch.float64)
        qi = self.q_in[:n0].clone().requires_grad_(True)
        # derivatives that land on the owned atom, full weight; partner values are constants
        e_side = (qi[:, None] * self.q_in[None, :] * self.chi(self.r)).sum()
        self.gq, = torch.autograd.grad(e_side, qi, retain_graph=True)
        self.e_side = e_side
        return self.gq.sum().reshape(1)

    def backward(self, gq_sum_all, n_all):
        n0 = self.shells[0]
        gq_raw = self.gq - gq_sum_all / n_all
        # owned energy: a_i^2 + half of every pair the atom takes part in
        E_own = (self.a ** 2).sum() + 0.5 * self.e_side.detach()
        # gradient w.r.t. local positions: network part (through a and through q_raw with its cotangent) + pair geometry
        qi_const = self.q_in[:n0]
        pair_geom = (qi_const[:, None] * self.q_in[None, :] * self.chi(self.r)).sum()   # i-side: d/dR_i of all pairs of i
        # d(pair_geom)/dR_j for ghosts j must not be counted here (the owner of j does it): subtract by detaching R_j
        Rj = self.R.detach()
        d2 = _min_image(Rj[None, :, :] - self.R[:n0, None, :], self.cell)
        r2 = d2.norm(dim=-1)
        mask = torch.ones_like(r2, dtype=torch.bool)
        mask[torch.arange(n0), torch.arange(n0)] = False
        r2 = torch.where(mask, r2, torch.full_like(r2, 1e3))
        pair_i_side = (qi_const[:, None] * self.q_in[None, :] * self.chi(r2)).sum()
        loss = (self.a ** 2).sum() + (self.q_raw * gq_raw.detach()).sum() + pair_i_side
        g, = torch.autograd.grad(loss, self.R)
        return (-g).float(), E_own.reshape(1)


def _serial_reference(R, cell):
    R = torch.tensor(R, dtype=torch.float64, requires_grad=True)
    c = torch.tensor(cell, dtype=torch.float64)
    d = _min_image(R[None] - R[:, None], c)
    r = d.norm(dim=-1) + torch.eye(len(R), dtype=torch.float64) * 1e3
    a = ToyBackend.psi(r).sum(1)
    q = torch.tanh(a)
    q = q - q.mean()
    E = (a ** 2).sum() + 0.5 * (q[:, None] * q[None, :] * ToyBackend.chi(r)).sum()
    F = -torch.autograd.grad(E, R)[0]
    return E.item(), F.numpy()


def _problem(seed=3, n=160, box=(46.0, 19.0, 19.5)):
    rng = np.random.default_rng(seed)
    cell = np.diag(box)
    R = rng.uniform(0, 1, size=(n, 3)) * np.array(box)
    return R.astype(np.float32), cell


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
    # positions come back in the caller's order, wrapped into the cell along the decomposed axis
    d = res["R1"] - R1
    d[:, 0] -= np.round(d[:, 0] / cell[0, 0]) * cell[0, 0]
    np.testing.assert_allclose(d, 0, atol=1e-4)


def test_slab_selection_covers_every_neighbour_within_three_shells():
    R, cell = _problem(seed=5, n=400)
    geo = D.SlabDecomposition(cell, 3, skin=1.0, cutoff_lr=RC_LR)
    Rt = torch.tensor(R)
    Rw, s = geo.wrap(Rt)
    owner = geo.owner(s)
    total_owned = 0
    for rank in range(3):
        idx, shift, shell = geo.selection(rank, Rw, s)
        n0 = int((shell == 0).sum())
        total_owned += n0
        assert (shell[:-1] <= shell[1:]).all()                       # owned first, then shell by shell
        assert (owner[idx[:n0]] == rank).all()
        Rl = Rw[idx].double() + shift[:, None].double() * torch.tensor(cell[geo.axis])
        # every atom image within 4.5 + skin of an owned atom is present locally (brute force over images)
        own_pos = Rl[:n0]
        for k in (-1, 0, 1):
            img = Rw.double() + k * torch.tensor(cell[geo.axis])
            d = (img[None] - own_pos[:, None])
            d[..., 1] -= torch.round(d[..., 1] / cell[1, 1]) * cell[1, 1]
            d[..., 2] -= torch.round(d[..., 2] / cell[2, 2]) * cell[2, 2]
            need = torch.nonzero((d.norm(dim=-1) < geo.shell).any(0)).squeeze(1)
            have = set(zip(idx.tolist(), shift.tolist()))
            assert all((int(g), k) in have for g in need)
    assert total_owned == len(R)
