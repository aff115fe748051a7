"""Spatial domain decomposition of one large periodic structure over several GPUs (one process per GPU).

The box is cut into slabs along the lattice direction with the largest perpendicular width.  Every rank owns the atoms
of its slab and keeps copies ("ghosts") of the atoms within the long-range list radius (12 A + skin) of it; the ghosts
within one short-range shell (4.5 A + skin) additionally receive the per-layer features of their owners.  The library
evaluates a rank's owned atoms layer by layer (so3lr_b200_dd_*); this module moves rows between the ranks:

  per step      positions of all ghosts                          owner -> holder   (send/recv)
                features x, ev after layers 0 and 1              owner -> holder   (send/recv, short-range ghosts)
                sum of raw partial charges                       all-reduce        (charge conservation)
                charges and Hirshfeld ratios of all ghosts       owner -> holder   (send/recv)
                sum of dE/dq                                     all-reduce        (reverse of the charge conservation)
                cotangents of each layer's attention outputs     owner -> holder   (send/recv, short-range ghosts, 3 x)
  per rebuild   all positions and velocities                     all-reduce of the scattered owned rows; every rank then
                                                                 selects its own atoms and ghosts, so atoms migrate
                                                                 without extra messages

Every kernel of this path gathers towards an owned atom (both directions of an edge are evaluated by the owner of the
receiving end), so no rank computes on behalf of a ghost and no forces travel: the work per rank is that of its owned
atoms, and the traffic is a few hundred bytes per ghost atom and layer over NVLink.

The reference has no multi-device path; the radii follow from its cutoffs (so3lr/potential.py:17-29).
The numerical work is behind a small backend interface so that the bookkeeping can be tested on CPU ranks (gloo) with
a stand-in model; `CudaBackend` is the real one.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Dict, List, Optional

import numpy as np
import torch

CUTOFF_SR = 4.5
ACC_UNIT = 9.648533212331e-3      # eV / (A amu) -> A / fs^2


# ----------------------------------------------------------------------------------------------------------------
# communicators
# ----------------------------------------------------------------------------------------------------------------
class DistComm:
    """torch.distributed (NCCL on GPUs, gloo on CPU): one process per rank."""

    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()

    def exchange(self, sends: Dict[int, torch.Tensor], recvs: Dict[int, torch.Tensor]):
        """Send sends[p] to rank p and fill recvs[p] from rank p (every pair of ranks calls this with matching sizes)."""
        ops = []
        for p, t in sends.items():
            if t.numel():
                ops.append(self.dist.P2POp(self.dist.isend, t.contiguous(), p))
        for p, t in recvs.items():
            if t.numel():
                ops.append(self.dist.P2POp(self.dist.irecv, t, p))
        if ops:
            for w in self.dist.batch_isend_irecv(ops):
                w.wait()

    def all_reduce_sum(self, t):
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return t

    def all_reduce_max(self, t):
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t


class ThreadWorld:
    """Ranks as threads of one process (all on one device): the same driver code, used to test several domains on one GPU."""

    def __init__(self, world):
        self.world = world
        self.barrier = threading.Barrier(world)
        self.box: Dict = {}
        self.lock = threading.Lock()

    def comm(self, rank):
        return ThreadComm(self, rank)


class ThreadComm:
    def __init__(self, world: ThreadWorld, rank: int):
        self.w, self.rank, self.world = world, rank, world.world

    def _sync(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.w.barrier.wait()

    def exchange(self, sends, recvs):
        with self.w.lock:
            for p, t in sends.items():
                self.w.box[("x", self.rank, p)] = t.clone()
        self._sync()
        for p, t in recvs.items():
            if t.numel():
                t.copy_(self.w.box[("x", p, self.rank)])
        self._sync()

    def _reduce(self, t, op):
        with self.w.lock:
            self.w.box[("r", self.rank)] = t.clone()
        self._sync()
        parts = [self.w.box[("r", r)] for r in range(self.world)]
        out = torch.stack(parts).sum(0) if op == "sum" else torch.stack(parts).amax(0)
        self._sync()
        t.copy_(out)
        return t

    def all_reduce_sum(self, t):
        return self._reduce(t, "sum")

    def all_reduce_max(self, t):
        return self._reduce(t, "max")


# ----------------------------------------------------------------------------------------------------------------
# geometry of the decomposition
# ----------------------------------------------------------------------------------------------------------------
def _spread3(v):
    v = v & 0x3FF
    v = (v | (v << 16)) & 0x030000FF
    v = (v | (v << 8)) & 0x0300F00F
    v = (v | (v << 4)) & 0x030C30C3
    v = (v | (v << 2)) & 0x09249249
    return v


class SlabDecomposition:
    """Slabs along one lattice direction of a periodic cell (rows = lattice vectors)."""

    def __init__(self, cell, world: int, skin: float, cutoff_lr: float, axis: Optional[int] = None):
        self.cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        self.inv = np.linalg.inv(self.cell)
        widths = 1.0 / np.linalg.norm(self.inv, axis=0)
        self.axis = int(np.argmax(widths)) if axis is None else int(axis)
        self.width = float(widths[self.axis])
        self.world = int(world)
        self.shell = CUTOFF_SR + skin                        # short-range list radius
        self.lr_radius = max(cutoff_lr + skin, self.shell)   # long-range list radius = halo width
        self.sf = self.shell / self.width                    # both in fractional units along the axis
        self.reach = self.lr_radius / self.width
        if self.reach > 1.0:
            raise ValueError("the cell is thinner than the halo along the decomposed direction")
        self.bounds = np.arange(self.world + 1, dtype=np.float64) / self.world
        self.ext = 1.0 / self.world + 2 * self.reach + (self.lr_radius + 1.0) / self.width

    def rescale(self, factor: float):
        """The cell grows by `factor` in every direction (isotropic barostat); the slab boundaries and the halo stay what
        they are in fractional coordinates until the next partition recomputes them from the new widths."""
        self.cell = self.cell * float(factor)
        self.inv = np.linalg.inv(self.cell)
        self.width *= float(factor)
        self.sf = self.shell / self.width
        self.reach = self.lr_radius / self.width
        if self.reach > 1.0:
            raise ValueError("the cell is thinner than the halo along the decomposed direction")
        self.ext = 1.0 / self.world + 2 * self.reach + (self.lr_radius + 1.0) / self.width

    def local_cell(self):
        c = self.cell.copy()
        c[self.axis] = self.cell[self.axis] * self.ext
        return c

    def wrap(self, R):
        """Positions wrapped into [0, 1) along the decomposed direction and that fractional coordinate (float64;
        identical on all ranks because they hold identical R)."""
        inv_col = torch.tensor(self.inv[:, self.axis], dtype=torch.float64, device=R.device)
        a_vec = torch.tensor(self.cell[self.axis], dtype=torch.float64, device=R.device)
        s = R.to(torch.float64) @ inv_col
        k = torch.floor(s)
        Rw = (R.to(torch.float64) - k[:, None] * a_vec).to(torch.float32)
        s = Rw.to(torch.float64) @ inv_col
        return Rw, s.clamp_(0.0, 1.0 - 1e-12)      # float32 rounding may leave s a hair outside [0, 1)

    def owner(self, s):
        b = torch.tensor(self.bounds, dtype=torch.float64, device=s.device)
        return (torch.searchsorted(b, s, right=True) - 1).clamp_(0, self.world - 1)

    def selection(self, rank: int, R, s):
        """Atoms of `rank` in its local order: (global index, image shift along the axis, class), class 0 = owned,
        1 = ghost within the short-range shell of the slab, 2 = ghost within the long-range radius only."""
        dev = R.device
        lo, hi = float(self.bounds[rank]), float(self.bounds[rank + 1])
        own = self.owner(s) == rank
        idx = [torch.nonzero(own).squeeze(1)]
        shift = [torch.zeros_like(idx[0])]
        shell = [torch.zeros_like(idx[0])]
        reach = self.reach
        for k in (-1, 0, 1):
            sp = s + k
            for side in (0, 1):
                d = (lo - sp) if side == 0 else (sp - hi)
                m = (d > 0) & (d <= reach) if side == 0 else (d >= 0) & (d < reach)
                if k == 0:
                    m &= ~own
                g = torch.nonzero(m).squeeze(1)
                idx.append(g)
                shift.append(torch.full_like(g, k))
                shell.append(torch.where(d[g] <= self.sf, 1, 2).to(torch.int64))
        idx, shift, shell = torch.cat(idx), torch.cat(shift), torch.cat(shell)
        # order: shell, then a Morton curve over cells of one shell width (keeps neighbours close in memory)
        a_vec = torch.tensor(self.cell[self.axis], dtype=torch.float64, device=dev)
        Rl = R[idx].to(torch.float64) + shift[:, None].to(torch.float64) * a_vec
        sl = Rl @ torch.tensor(self.inv, dtype=torch.float64, device=dev)
        sl[:, self.axis] = sl[:, self.axis] - (lo - reach)
        for k in range(3):
            if k != self.axis:
                sl[:, k] = sl[:, k] - torch.floor(sl[:, k])
        widths = torch.tensor(1.0 / np.linalg.norm(self.inv, axis=0), dtype=torch.float64, device=dev)
        cells = torch.floor(sl * widths / self.shell).to(torch.int64).clamp_(0, 1023)
        key = _spread3(cells[:, 0]) | (_spread3(cells[:, 1]) << 1) | (_spread3(cells[:, 2]) << 2)
        order = torch.argsort(shell * (1 << 32) + key, stable=True)
        return idx[order], shift[order], shell[order]


# ----------------------------------------------------------------------------------------------------------------
# backends
# ----------------------------------------------------------------------------------------------------------------
class CudaBackend:
    """One rank's evaluation phases through the C ABI (so3lr_b200_dd_*).

    Backend interface used by DomainSystem (a CPU stand-in implements the same methods in the tests):
      num_layers; set_atoms(Z_local, counts, cell_local); begin(R_local); layer_forward(l); feature_rows(l) -> list of
      (n_local, d) tensors viewing the layer-l features; heads() -> (q_raw, h) of the owned atoms; pair(q_local, h_local)
      -> sum of dE/dq over owned atoms; heads_backward(gq_sum_all, n_all) -> energy of the owned atoms;
      layer_backward_post(l); cotangent_rows() -> list of (n_local, d) tensors; layer_backward_attn(l); forces() -> (n0, 3);
      for the thermostat: nhc_state() -> chain tensor, nhc_half_steps(chain, n_half, dt, kT, tau, dof, kinetic_energy, ...).
    """
    num_layers = 3

    def __init__(self, cutoff_lr=12.0, damping=2.0, skin=1.0, device=0):
        from .engine import Model
        self.cutoff_lr, self.damping, self.skin = cutoff_lr, damping, skin
        self.device = torch.device("cuda", device)
        self.model = Model.default(device)
        self.sys = None
        self.capacity = 0
        self.want_virial = False
        self.kspace = None          # (grid shape, smearing, method, cell of the whole structure, total charge)

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _call(self, name, *args):
        from ._lib import check, lib
        check(getattr(lib, "so3lr_b200_" + name)(self.sys._h, *args), name)

    def _buffer(self, which, layer):
        from ._lib import check, lib
        from .engine import _from_ptr
        ptr, rf = C.c_void_p(), C.c_int()
        check(lib.so3lr_b200_dd_buffer(self.sys._h, which, layer, C.byref(ptr), C.byref(rf)), "dd_buffer")
        return _from_ptr(ptr.value, self.capacity * rf.value, self.device).view(self.capacity, rf.value)[: self.n]

    def set_atoms(self, Z_local, counts, cell_local):
        from .engine import System, _ptr
        n = int(Z_local.numel())
        if n > self.capacity:
            self.sys = None
            self.capacity = int(1.2 * n) + 1024
            self.sys = System(np.ones(self.capacity, np.int32), np.asarray(cell_local), cutoff_lr=self.cutoff_lr, damping=self.damping,
                              skin=self.skin, lr_format="sparse", model=self.model)
            if self.want_virial:
                self.sys.enable_virial(True)
            self._apply_kspace()
        self.n, self.counts = n, [int(v) for v in counts]
        sh = np.asarray([self.counts[0], self.counts[1], self.counts[1], n], dtype=np.int32)
        c9 = np.ascontiguousarray(np.asarray(cell_local, dtype=np.float32).reshape(9))
        Zl = Z_local.to(self.device, torch.int32).contiguous()
        torch.cuda.current_stream(self.device).synchronize()
        self._call("dd_set_atoms", n, _ptr(sh), _ptr(Zl), _ptr(c9))
        self._x = [self._buffer(0, l) for l in range(4)]
        self._ev = [self._buffer(1, l) for l in range(4)]
        self._g = [self._buffer(2, 0), self._buffer(3, 0)]

    # ---- reciprocal-space Coulomb part: every rank holds the whole mesh (or all structure factors) ----
    def set_kspace(self, k_grid, k_smearing, method, cell_global, total_charge):
        self.kspace = None if k_grid is None else (k_grid, k_smearing, method, np.asarray(cell_global, dtype=np.float64).copy(),
                                                   float(total_charge))
        if self.sys is not None:
            self._apply_kspace()

    def _apply_kspace(self):
        if self.kspace is None:
            self.sys.set_kspace(None)
            return
        shape, smearing, method, cell, qtot = self.kspace
        self.sys.set_kspace(shape, smearing, method)
        self.kspace_cell(cell)

    def kspace_cell(self, cell_global):
        from .engine import _ptr
        shape, smearing, method, _, qtot = self.kspace
        self.kspace = (shape, smearing, method, np.asarray(cell_global, dtype=np.float64).copy(), qtot)
        c9 = np.ascontiguousarray(np.asarray(cell_global, dtype=np.float32).reshape(9))
        self._call("dd_kspace_cell", _ptr(c9), C.c_float(qtot))

    def kspace_accumulate(self):
        """The owned atoms' share of the charge mesh / structure factors: a flat float32 view to be summed over the ranks in place."""
        from .engine import _from_ptr, _ptr
        ptr, nf = C.c_void_p(), C.c_int64()
        self._call("dd_kspace_accumulate", self._stream(), _ptr(self._R), _ptr(self._q), C.byref(ptr), C.byref(nf))
        return _from_ptr(ptr.value, nf.value, self.device)

    def kspace_finish(self, add_strain):
        from .engine import _ptr
        s = torch.zeros(1, dtype=torch.float64, device=self.device)
        self._call("dd_kspace_finish", self._stream(), _ptr(self._R), _ptr(self._q), 1 if add_strain else 0, _ptr(s))
        return s

    def enable_virial(self, on=True):
        self.want_virial = bool(on)
        if self.sys is not None:
            self.sys.enable_virial(on)

    def virial(self):
        """Share of the owned atoms in dE/d eps, (3,3) float64."""
        return self.sys.virial()

    def rescale_cell(self, cell_local):
        self.sys.rescale_cell(cell_local)

    def npt_state(self):
        from .engine import npt_state
        return npt_state(self.device)

    def npt_box_step(self, which, state, *args, **kw):
        from .engine import npt_box_step
        npt_box_step(which, state, *args, **kw)

    def nhc_state(self):
        from .engine import nhc_state
        return nhc_state(self.device)

    def nhc_half_steps(self, chain, n_half, dt_fs, kT, tau_fs, dof, kinetic_energy, **kw):
        from .engine import nhc_half_steps
        nhc_half_steps(chain, n_half, dt_fs, kT, tau_fs, dof, kinetic_energy, **kw)

    def begin(self, R_local):
        from .engine import _ptr
        self._R = R_local.contiguous()
        self._call("dd_begin", self._stream(), _ptr(self._R))

    def layer_forward(self, l):
        self._call("dd_layer_forward", self._stream(), int(l))

    def feature_rows(self, l):
        return [self._x[l], self._ev[l]]

    def heads(self):
        from .engine import _ptr
        n0 = self.counts[0]
        q, h = torch.empty(n0, device=self.device), torch.empty(n0, device=self.device)
        self._call("dd_heads", self._stream(), _ptr(q), _ptr(h))
        return q, h

    def pair(self, q_local, h_local):
        from .engine import _ptr
        s = torch.zeros(1, dtype=torch.float64, device=self.device)
        self._q, self._h = q_local.contiguous(), h_local.contiguous()
        self._call("dd_pair", self._stream(), _ptr(self._R), _ptr(self._q), _ptr(self._h), _ptr(s))
        return s

    def heads_backward(self, gq_sum_all, n_all):
        from .engine import _ptr
        E = torch.zeros(1, dtype=torch.float64, device=self.device)
        self._gq_sum = gq_sum_all
        self._call("dd_heads_backward", self._stream(), _ptr(gq_sum_all), C.c_int64(int(n_all)), _ptr(E))
        return E

    def layer_backward_post(self, l):
        self._call("dd_layer_backward_post", self._stream(), int(l))

    def cotangent_rows(self):
        return self._g

    def layer_backward_attn(self, l):
        self._call("dd_layer_backward_attn", self._stream(), int(l))

    def forces(self):
        from .engine import _ptr
        F = torch.empty(self.counts[0], 3, device=self.device)
        self._call("dd_forces", self._stream(), _ptr(F))
        return F

    def stats(self):
        return self.sys.stats()

    # ---- halo packing: one launch gathers (scatters) the rows of all arrays of an exchange ----
    def _rows_call(self, name, tensors, idx, buf):
        from ._lib import check, lib
        k = len(tensors)
        ptrs = (C.c_void_p * k)(*[t.data_ptr() for t in tensors])
        widths = (C.c_int * k)(*[int(t.shape[1]) for t in tensors])
        check(getattr(lib, name)(self._stream(), k, ptrs, widths, C.c_void_p(idx.data_ptr()), C.c_int64(idx.numel()),
                                 C.c_void_p(buf.data_ptr())), name)

    def pack_rows(self, tensors, idx):
        """buf[r] = the rows idx[r] of `tensors` ((n, w_t) float32, contiguous) side by side."""
        buf = torch.empty((idx.numel(), sum(int(t.shape[1]) for t in tensors)), dtype=torch.float32, device=self.device)
        if idx.numel():
            self._rows_call("so3lr_b200_pack_rows", tensors, idx, buf)
        return buf

    def unpack_rows(self, tensors, idx, buf):
        if idx.numel():
            self._rows_call("so3lr_b200_unpack_rows", tensors, idx, buf)


# ----------------------------------------------------------------------------------------------------------------
# the driver of one rank
# ----------------------------------------------------------------------------------------------------------------
class DomainSystem:
    """One rank's share of a periodic structure of `n_all` atoms.

    At construction every rank passes the same global arrays (atomic numbers, positions, optionally velocities and
    masses); afterwards each rank keeps only its own atoms and ghosts.  `compute()` returns the total energy and the
    forces on the owned atoms; `nve()` integrates the owned atoms; `compute_host()` is the host-buffer call;
    `gather_global()` reassembles arrays in the caller's atom order.
    """

    def __init__(self, comm, backend, atomic_numbers, positions, cell, *, skin=1.0, cutoff_lr=12.0, total_charge=0.0,
                 velocities=None, masses=None, device=None):
        self.comm, self.backend = comm, backend
        self.rank, self.world = comm.rank, comm.world
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.geo = SlabDecomposition(cell, self.world, skin, cutoff_lr)
        self.skin = skin
        self.total_charge = float(total_charge)
        self.Z_all = torch.as_tensor(np.asarray(atomic_numbers), dtype=torch.int32, device=self.device)
        self.n_all = int(self.Z_all.numel())
        self.m_all = None if masses is None else torch.as_tensor(np.asarray(masses), dtype=torch.float32, device=self.device)
        R = torch.as_tensor(np.asarray(positions), dtype=torch.float32, device=self.device)
        V = None if velocities is None else torch.as_tensor(np.asarray(velocities), dtype=torch.float32, device=self.device)
        self.n_rebuilds = 0
        self.kspace = None
        self._partition(R, V)

    def set_kspace(self, k_grid=None, k_smearing=None, method="pme"):
        """Reciprocal-space Coulomb part (System.set_kspace) for the decomposed structure; `k_grid=None` switches it off."""
        if not hasattr(self.backend, "set_kspace"):
            raise NotImplementedError("this backend has no reciprocal-space part")
        if k_grid is None:
            self.kspace = None
            self.backend.set_kspace(None, None, None, self.geo.cell, self.total_charge)
            return
        shape = tuple(int(v) for v in (k_grid.shape if hasattr(k_grid, "shape") else k_grid))
        s = float(np.asarray(k_smearing.detach().cpu() if torch.is_tensor(k_smearing) else k_smearing, dtype=np.float64).reshape(-1)[0])
        self.kspace = (shape, s, method)
        self.backend.set_kspace(shape, s, method, self.geo.cell, self.total_charge)

    # ---- partition / halo plans (all ranks hold identical R_all here) ----
    def _peers(self):
        """Ranks whose slab lies within the halo of mine (periodic), myself included (own periodic images)."""
        geo, out = self.geo, []
        for p in range(self.world):
            gap = min((p - self.rank) % self.world, (self.rank - p) % self.world)
            if p == self.rank or (gap - 1) / self.world < geo.reach + 1e-9:
                out.append(p)
        return out

    def _partition(self, R_all, V_all):
        geo, dev = self.geo, self.device
        R_in = R_all
        R_all, s = geo.wrap(R_all)
        self.wrap_vec = R_in - R_all          # lattice translation that brought every atom into the cell
        owner_all = geo.owner(s)
        peers = self._peers()
        sel = {p: geo.selection(p, R_all, s) for p in peers}
        idx, shift, cls = sel[self.rank]
        self.gid, self.shift = idx, shift
        self.n0, self.n1, self.n_local = int((cls == 0).sum()), int((cls <= 1).sum()), int(cls.numel())
        a_vec = torch.tensor(geo.cell[geo.axis], dtype=torch.float32, device=dev)
        self.shift_vec = shift[:, None].to(torch.float32) * a_vec
        self.R = (R_all[idx] + self.shift_vec).contiguous()
        self.R_ref = self.R[: self.n0].clone()
        self.V = None if V_all is None else V_all[idx[: self.n0]].contiguous()
        self.m = None if self.m_all is None else self.m_all[idx[: self.n0]].contiguous()
        # plans: recv_slots[p] = my ghost slots owned by p (my order); send_slots[p] = my owned slots that p holds as ghosts
        # (p's order).  The *_sr variants cover the short-range ghosts only (a prefix of each list, since ghosts are
        # ordered by class).
        slot_of_gid = torch.full((self.n_all,), -1, dtype=torch.int64, device=dev)
        slot_of_gid[idx[: self.n0]] = torch.arange(self.n0, device=dev)
        ghost_owner = owner_all[idx[self.n0:]]
        self.recv_slots, self.send_slots, self.recv_sr, self.send_sr = {}, {}, {}, {}
        for p in peers:
            r = torch.nonzero(ghost_owner == p).squeeze(1) + self.n0
            self.recv_slots[p] = r
            self.recv_sr[p] = r[r < self.n1]
            pidx, _, pcls = sel[p]
            n0p = int((pcls == 0).sum())
            pg, pc = pidx[n0p:], pcls[n0p:]
            mine = owner_all[pg] == self.rank
            self.send_slots[p] = slot_of_gid[pg[mine]]
            self.send_sr[p] = slot_of_gid[pg[mine & (pc == 1)]]
        self.backend.set_atoms(self.Z_all[idx], [self.n0, self.n1, self.n_local], geo.local_cell())
        self.n_rebuilds += 1

    # ---- halo traffic ----
    def _halo_fill(self, tensors, sr_only=False):
        """Fill the ghost rows of each (n_local, d) tensor from the owners' rows (rows [0, n0) are the owned ones)."""
        send_slots = self.send_sr if sr_only else self.send_slots
        recv_slots = self.recv_sr if sr_only else self.recv_slots
        ev = None
        if getattr(self, "time_halo", False) and self.device.type == "cuda":      # device time of the exchanges, for the benchmark
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
            self._halo_events.append(ev)
        width = [t.shape[1] for t in tensors]
        me = self.rank
        fused = (hasattr(self.backend, "pack_rows") and len(tensors) <= 4
                 and all(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() for t in tensors))
        if fused:       # one gather launch per peer into the send buffer, one scatter launch per peer out of the receive buffer
            be = self.backend
            sends = {p: be.pack_rows(tensors, sl) for p, sl in send_slots.items() if p != me}
            recvs = {p: torch.empty((sl.numel(), sum(width)), dtype=torch.float32, device=self.device)
                     for p, sl in recv_slots.items() if p != me}
            self.comm.exchange(sends, recvs)
            for p, buf in recvs.items():
                be.unpack_rows(tensors, recv_slots[p], buf)
            if recv_slots[me].numel():                      # own periodic images
                be.unpack_rows(tensors, recv_slots[me], be.pack_rows(tensors, send_slots[me]))
        else:
            sends = {p: torch.cat([t[sl] for t in tensors], 1) for p, sl in send_slots.items() if p != me}
            recvs = {p: torch.empty((sl.numel(), sum(width)), dtype=tensors[0].dtype, device=self.device)
                     for p, sl in recv_slots.items() if p != me}
            self.comm.exchange(sends, recvs)
            for p, buf in recvs.items():
                o = 0
                for t, w in zip(tensors, width):
                    t[recv_slots[p]] = buf[:, o:o + w]
                    o += w
            for t in tensors:                                   # own periodic images
                t[recv_slots[me]] = t[send_slots[me]]
        if ev is not None:
            ev[1].record()

    def _mark(self, name):
        """Device-side time stamps of the step's phases (benchmark only): the time between two marks covers the kernels, the
        messages and any wait for a neighbouring rank that fall between them."""
        if getattr(self, "time_phases", False) and self.device.type == "cuda":
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._phase_events.append((name, e))

    # ---- evaluation ----
    def defer_skin_test(self, on=True, margin=0.05):
        """Read the skin test one step late: the largest squared displacement of step k is all-reduced on the device, copied to
        pinned memory asynchronously and looked at when step k + 1 starts, so no rank waits for its device (or for the slowest
        rank's host) inside a step.  The trigger distance is lowered to skin / 2 - margin so the lists cover the extra step
        (margin >= the largest displacement of an atom in one step)."""
        self._defer, self._margin, self._pending = bool(on), float(margin), None

    def _skin_value(self):
        d2 = (self.R[: self.n0] - self.R_ref).square().sum(1).amax().reshape(1) if self.n0 else torch.zeros(1, device=self.device)
        return self.comm.all_reduce_max(d2.to(torch.float32))

    def _maybe_rebuild(self):
        thr = 0.5 * self.skin
        if getattr(self, "_defer", False) and self.skin > 0 and self.device.type == "cuda":
            thr = max(thr - self._margin, 0.0)
            cur = self._skin_value()
            if getattr(self, "_pin_d2", None) is None:
                self._pin_d2 = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
                self._ev_d2 = [torch.cuda.Event() for _ in range(2)]
                self._slot = 0
            k = self._slot
            self._pin_d2[k].copy_(cur, non_blocking=True)
            self._ev_d2[k].record()
            prev, self._pending, self._slot = self._pending, k, k ^ 1
            if prev is None:
                return False
            self._ev_d2[prev].synchronize()              # a whole step old
            d2 = float(self._pin_d2[prev])
        else:
            d2 = float(self._skin_value())      # the step's one host read
        if not np.isfinite(d2):
            raise RuntimeError("non-finite positions")
        if d2 > thr ** 2 or self.skin <= 0:
            self._pending = None
            import time
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            t0 = time.perf_counter()
            R_all = self.gather_global(self.R[: self.n0])
            V_all = None if self.V is None else self.gather_global(self.V)
            self._partition(R_all, V_all)
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            self.t_repartition = getattr(self, "t_repartition", 0.0) + time.perf_counter() - t0
            return True
        return False

    def repartition(self):
        """Re-select owned atoms and ghosts from the current positions now (what the skin test triggers by itself)."""
        R_all = self.gather_global(self.R[: self.n0])
        V_all = None if self.V is None else self.gather_global(self.V)
        self._partition(R_all, V_all)

    def compute(self, check_rebuild=True):
        """Total energy (float64 tensor, all ranks) and forces on the owned atoms (n0, 3)."""
        self._mark("step_start")
        if check_rebuild:
            self._maybe_rebuild()
        self._mark("skin_test_repartition")
        # ghost positions follow their owners
        self.R[self.n0:] = 0.0
        self._halo_fill([self.R])
        self.R[self.n0:] += self.shift_vec[self.n0:]
        self._mark("halo_positions")
        return self._evaluate()

    def compute_host(self, R_all_host):
        """The call of a host application that keeps all positions in host memory: (n_all, 3) float32 positions in the
        caller's atom order go in (every rank passes the same array), total energy and (n_all, 3) forces come back as
        numpy arrays.  Each rank uploads the positions, picks its own atoms and ghosts (no position halo exchange is
        needed), evaluates, and the forces are assembled over the ranks."""
        Rh = torch.as_tensor(np.ascontiguousarray(R_all_host, dtype=np.float32))
        if self.device.type == "cuda":
            if getattr(self, "_pin", None) is None or self._pin.shape != Rh.shape:
                self._pin = torch.empty_like(Rh).pin_memory()
                self._pin_F = torch.empty_like(Rh).pin_memory()
            self._pin.copy_(Rh)
            R_all = self._pin.to(self.device, non_blocking=True)
        else:
            R_all = Rh.clone()
        ref = getattr(self, "_R_all_ref", None)
        moved = True
        if ref is not None and self.skin > 0:
            moved = bool(((R_all - ref).square().sum(1).amax() > (0.5 * self.skin) ** 2).item())   # identical on all ranks
        if moved:
            self._R_all_ref = R_all.clone()
            self._partition(R_all, None)
        else:
            self.R = (R_all[self.gid] - self.wrap_vec[self.gid] + self.shift_vec).contiguous()
        E, _ = self._evaluate()
        F_all = self.global_forces()
        if self.device.type == "cuda":
            self._pin_F.copy_(F_all, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            return float(E), self._pin_F.numpy()
        return float(E), F_all.numpy()

    def _evaluate(self):
        be, L = self.backend, self.backend.num_layers
        be.begin(self.R)
        self._mark("lists_zbl")
        for l in range(L):
            be.layer_forward(l)
            self._mark(f"layer{l}_forward")
            if l + 1 < L:
                self._halo_fill(be.feature_rows(l + 1), sr_only=True)
                self._mark(f"halo_features{l + 1}")
        q_raw, h = be.heads()
        qsum = self.comm.all_reduce_sum(q_raw.sum(dtype=torch.float64).reshape(1))
        q = q_raw + ((self.total_charge - qsum) / self.n_all).to(torch.float32)
        qh = torch.zeros(self.n_local, 2, device=self.device)
        qh[: self.n0, 0], qh[: self.n0, 1] = q, h
        self._mark("heads_charge_sum")
        self._halo_fill([qh])
        self._mark("halo_charges")
        gq_own = be.pair(qh[:, 0].contiguous(), qh[:, 1].contiguous())
        self._mark("pair_terms")
        if self.kspace is not None:
            # every rank spreads its own atoms, the meshes (or structure factors) are summed over the ranks, and every rank
            # transforms the whole mesh and reads it at its own atoms
            buf = be.kspace_accumulate()
            tot = self.comm.all_reduce_sum(buf)
            if tot.data_ptr() != buf.data_ptr():
                buf.copy_(tot)
            gq_own = be.kspace_finish(add_strain=self.rank == 0)
            self._mark("kspace")
        gq_sum = self.comm.all_reduce_sum(gq_own)
        E_own = be.heads_backward(gq_sum, self.n_all)
        self._mark("heads_backward")
        for l in reversed(range(L)):
            be.layer_backward_post(l)
            self._mark(f"layer{l}_backward_dense")
            self._halo_fill(be.cotangent_rows(), sr_only=True)
            self._mark(f"halo_cotangents{l}")
            be.layer_backward_attn(l)
            self._mark(f"layer{l}_backward_attention")
        self.F = be.forces()
        self.E = self.comm.all_reduce_sum(E_own)
        self._mark("forces_energy_sum")
        self.q, self.h = q, h
        return self.E, self.F

    def nve(self, n_steps, dt_fs):
        """Velocity Verlet on the owned atoms (forces of the current positions must be in self.F)."""
        for _ in range(n_steps):
            s = (0.5 * dt_fs * ACC_UNIT / self.m)[:, None]
            self.V += s * self.F
            self.R[: self.n0] += dt_fs * self.V
            self.compute()
            s = (0.5 * dt_fs * ACC_UNIT / self.m)[:, None]      # ownership may have changed
            self.V += s * self.F
        return self.E

    def virial(self):
        """dE/d eps (3,3) float64 of the latest evaluation, summed over the ranks (backend.enable_virial() first)."""
        return self.comm.all_reduce_sum(self.backend.virial().reshape(9).clone()).reshape(3, 3)

    def kinetic_energy(self):
        """Kinetic energy of all atoms (eV) as a one-element float64 tensor, identical on every rank."""
        v = self.V.double()
        ke = 0.5 * (self.m.double() * (v * v).sum(1)).sum().reshape(1) / ACC_UNIT
        return self.comm.all_reduce_sum(ke)

    def nvt(self, n_steps, dt_fs, kT, tau_fs, chain, chain_length=3, chain_steps=2, sy_steps=3):
        """Velocity Verlet under a Nose-Hoover chain thermostat on the owned atoms (forces of the current positions must be
        in self.F).  Every rank carries the same chain (`chain` from backend.nhc_state()) and advances it with the all-reduced
        kinetic energy, so the ranks scale their velocities by the same factor without a further exchange.  Mirrors
        jax_md.simulate.nvt_nose_hoover as driven by so3lr/cli/so3lr_md.py:1047-1075."""
        if n_steps <= 0:
            return self.E
        dof = 3.0 * self.n_all
        kw = dict(chain_length=chain_length, chain_steps=chain_steps, sy_steps=sy_steps)
        self.backend.nhc_half_steps(chain, 1, dt_fs, kT, tau_fs, dof, self.kinetic_energy(), **kw)
        for step in range(n_steps):
            self.V *= chain[1].to(self.V.dtype)
            s = (0.5 * dt_fs * ACC_UNIT / self.m)[:, None]
            self.V += s * self.F
            self.R[: self.n0] += dt_fs * self.V
            self.compute()
            s = (0.5 * dt_fs * ACC_UNIT / self.m)[:, None]      # ownership may have changed
            self.V += s * self.F
            # the second half step of this MD step and the first of the next act back to back on the velocities
            self.backend.nhc_half_steps(chain, 1 if step == n_steps - 1 else 2, dt_fs, kT, tau_fs, dof, self.kinetic_energy(), **kw)
        self.V *= chain[1].to(self.V.dtype)
        chain[1] = 1.0
        return self.E

    def npt(self, n_steps, dt_fs, kT, pressure, tau_t_fs, tau_b_fs, state, cell0, chain_length=3, chain_steps=2, sy_steps=3):
        """NPT steps (isotropic Martyna-Tobias-Klein barostat, Nose-Hoover chains on particles and box) on the owned atoms.
        Every rank carries the same box-and-chains `state` (backend.npt_state()) and advances it with the all-reduced kinetic
        energy and virial, so all ranks rescale box, positions and velocities alike.  `cell0` is the reference cell of the
        box coordinate; backend.enable_virial() and a compute() must precede the first call.  Returns the energy and the
        cell after the last step.  Mirrors jax_md.simulate.npt_nose_hoover as driven by so3lr/cli/so3lr_md.py:1089-1107,
        1254-1282."""
        cell0 = np.asarray(cell0, dtype=np.float64).reshape(3, 3)
        V0 = abs(float(np.linalg.det(cell0)))
        kw = dict(chain_length=chain_length, chain_steps=chain_steps, sy_steps=sy_steps)
        args = (self.n_all, dt_fs, kT, pressure, tau_t_fs, tau_b_fs, V0)
        if getattr(self, "_virial_all", None) is None:
            self._virial_all = self.virial().contiguous()
        for step in range(n_steps):
            self.backend.npt_box_step("pre", state, *args, self._virial_all, self.kinetic_energy() if step == 0 else None, **kw)
            acc = (ACC_UNIT / self.m)[:, None]
            c1, c2 = state[38].to(self.V.dtype), state[39].to(self.V.dtype)
            self.V = self.V * (state[1].to(self.V.dtype) * c1) + (c2 * acc) * self.F
            # the box moves by ~1e-6 per step: add the increment (r1 - 1) R instead of multiplying by r1 in float32
            Ro = self.R[: self.n0]
            self.R[: self.n0] = Ro + (Ro * (state[40] - 1.0).to(self.R.dtype) + state[41].to(self.R.dtype) * self.V)
            # the new cell on the host: the step's one extra host read
            scale = float(torch.exp(state[36]))
            self.geo.rescale(scale * np.cbrt(V0 / abs(np.linalg.det(self.geo.cell))))
            a_vec = torch.tensor(self.geo.cell[self.geo.axis], dtype=torch.float32, device=self.device)
            self.shift_vec = self.shift[:, None].to(torch.float32) * a_vec
            self.backend.rescale_cell(self.geo.local_cell())
            if self.kspace is not None:
                self.backend.kspace_cell(self.geo.cell)
            self.compute()
            self._virial_all = self.virial().contiguous()
            acc = (ACC_UNIT / self.m)[:, None]              # ownership may have changed
            self.V = self.V * state[38].to(self.V.dtype) + (state[39].to(self.V.dtype) * acc) * self.F
            self.backend.npt_box_step("post", state, *args, self._virial_all, self.kinetic_energy(), **kw)
        self.V = self.V * state[1].to(self.V.dtype)
        state[1] = 1.0
        return self.E, self.geo.cell.copy()

    # ---- reassembly ----
    def gather_global(self, owned_rows):
        """Global (n_all, ...) array in the caller's atom order from the owned rows of every rank (a sum of disjoint
        scatters, hence exact and identical on all ranks)."""
        g = torch.zeros((self.n_all,) + owned_rows.shape[1:], dtype=owned_rows.dtype, device=self.device)
        g[self.gid[: self.n0]] = owned_rows
        return self.comm.all_reduce_sum(g)

    def global_forces(self):
        return self.gather_global(self.F)
