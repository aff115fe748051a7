"""Thin object layer over the C ABI: `Model` (weights on one device) and `System` (one evaluation context).

torch is used only to own device memory and streams; every number is produced by libso3lr_b200.so.
"""
import ctypes as C
import os

import numpy as np
import torch

from . import _lib
from ._lib import Options, check, lib

_PARAMS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "params", "so3lr_v1.npz")


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        return C.c_void_p(t.data_ptr())
    return t.ctypes.data_as(C.c_void_p)


def load_blob(path=None):
    return np.ascontiguousarray(np.load(path or _PARAMS)["blob"], dtype=np.float32)


class Model:
    """Pretrained SO3LR weights uploaded to one CUDA device (handle of so3lr_b200_model_create)."""
    _cache = {}

    def __init__(self, device=0, blob=None):
        if not torch.cuda.is_available():
            raise RuntimeError("so3lr_b200 needs a CUDA device (sm_100a); there is no CPU path")
        self.device = int(device)
        torch.cuda.init()
        b = load_blob() if blob is None else np.ascontiguousarray(blob, dtype=np.float32)
        h = C.c_void_p()
        check(lib.so3lr_b200_model_create(_ptr(b), b.size, self.device, C.byref(h)), "model_create")
        self._h = h

    @classmethod
    def default(cls, device=0):
        if device not in cls._cache:
            cls._cache[device] = cls(device)
        return cls._cache[device]

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib.so3lr_b200_model_destroy(h)
            self._h = None


class System:
    """Evaluation context: atoms (optionally several graphs), neighbor lists and workspaces.

    cell: None or (3,3) with lattice vectors as rows [Angstrom].  cutoff_lr None: no long-range cutoff.
    lr_format: 'ordered_sparse' (so3lr/potential.py:22) or 'sparse' (so3lr/base_calculator.py:31).
    """

    def __init__(self, atomic_numbers, cell=None, *, cutoff_lr=12.0, damping=2.0, skin=0.0, lr_format="ordered_sparse",
                 graph_start=None, total_charge=None, num_unpaired=None, lr_list_cutoff=None, model=None, device=0):
        self.model = model or Model.default(device)
        self.device = torch.device("cuda", self.model.device)
        Z = np.ascontiguousarray(atomic_numbers, dtype=np.int32)
        self.n = int(Z.size)
        gs = None if graph_start is None else np.ascontiguousarray(graph_start, dtype=np.int32)
        self.n_graphs = 1 if gs is None else int(gs.size - 1)
        tq = None if total_charge is None else np.ascontiguousarray(total_charge, dtype=np.float32).reshape(-1)
        ts = None if num_unpaired is None else np.ascontiguousarray(num_unpaired, dtype=np.float32).reshape(-1)
        c9 = None if cell is None else np.ascontiguousarray(np.asarray(cell, dtype=np.float32).reshape(9))
        opt = Options(float(cutoff_lr) if cutoff_lr else -1.0, float(damping) if damping else -1.0, float(skin),
                      1 if lr_format == "sparse" else 0, float(lr_list_cutoff) if lr_list_cutoff else -1.0)
        h = C.c_void_p()
        check(lib.so3lr_b200_system_create(self.model._h, self.n, _ptr(Z), self.n_graphs, _ptr(gs), _ptr(tq), _ptr(ts),
                                           _ptr(c9), C.byref(opt), C.byref(h)), "system_create")
        self._h = h
        self._cell = None if cell is None else np.asarray(cell, dtype=np.float64).reshape(3, 3)
        self._virial = False
        self.kspace = None

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib.so3lr_b200_system_destroy(h)
            self._h = None

    def set_cell(self, cell):
        c9 = np.ascontiguousarray(np.asarray(cell, dtype=np.float32).reshape(9))
        check(lib.so3lr_b200_system_set_cell(self._h, _ptr(c9)), "set_cell")
        self._cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)

    def defer_skin_test(self, on=True, margin=0.05):
        """Read the skin-test flag one step late (no host wait per step); lists are rebuilt at skin / 2 - margin instead."""
        check(lib.so3lr_b200_system_defer_skin_test(self._h, 1 if on else 0, float(margin)), "defer_skin_test")

    def enable_virial(self, on=True):
        """Also accumulate the strain derivative of the energy (single-structure contexts); compute() then returns
        'virial' (3,3) float64 = dE/d eps in eV and, for a periodic cell, 'stress' = virial / volume in eV/A^3."""
        check(lib.so3lr_b200_system_enable_virial(self._h, 1 if on else 0), "enable_virial")
        self._virial = bool(on)

    def virial(self, stream=None):
        """dE/d eps (3,3) float64 of the latest evaluation."""
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.stream(s):      # the result is allocated on the stream the kernels run on
            w = torch.empty(3, 3, dtype=torch.float64, device=self.device)
        check(lib.so3lr_b200_system_virial(self._h, C.c_void_p(s.cuda_stream), _ptr(w)), "virial")
        return w

    def compute(self, positions, stream=None):
        """positions: float32 CUDA tensor (n,3).  Returns dict of CUDA tensors (async on `stream`, default: the current one).
        Temporaries and outputs are created under `stream`, so the caching allocator ties their lifetime to the stream the
        kernels are enqueued on; a caller that passes another stream orders it against the producer of `positions` itself."""
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        n, g = self.n, self.n_graphs
        with torch.cuda.stream(s):
            R = positions.to(self.device, torch.float32).contiguous()
            out = dict(forces=torch.empty(n, 3, device=self.device), e_atom=torch.empty(n, device=self.device),
                       energy=torch.empty(g, dtype=torch.float64, device=self.device),
                       partial_charges=torch.empty(n, device=self.device), hirshfeld_ratios=torch.empty(n, device=self.device),
                       dipole_vec=torch.empty(g, 3, device=self.device))
            if R.data_ptr() == positions.data_ptr():
                positions.record_stream(s)
        check(lib.so3lr_b200_system_compute(self._h, C.c_void_p(s.cuda_stream), _ptr(R), _ptr(out["forces"]), _ptr(out["e_atom"]),
                                            _ptr(out["energy"]), _ptr(out["partial_charges"]), _ptr(out["hirshfeld_ratios"]),
                                            _ptr(out["dipole_vec"])), "system_compute")
        if getattr(self, "_virial", False):
            out["virial"] = self.virial(s)
            if self._cell is not None:
                with torch.cuda.stream(s):
                    out["stress"] = out["virial"] / abs(float(np.linalg.det(self._cell)))
        return out

    def compute_host(self, positions, want_aux=True):
        """positions: numpy float32 (n,3) on the host; results are numpy arrays (host<->device copies inside)."""
        R = np.ascontiguousarray(positions, dtype=np.float32)
        n, g = self.n, self.n_graphs
        F = np.empty((n, 3), np.float32); E = np.empty(g, np.float64)
        q = np.empty(n, np.float32) if want_aux else None
        h = np.empty(n, np.float32) if want_aux else None
        d = np.empty((g, 3), np.float32) if want_aux else None
        check(lib.so3lr_b200_system_compute_host(self._h, _ptr(R), _ptr(F), _ptr(E), _ptr(q), _ptr(h), _ptr(d)), "compute_host")
        return dict(forces=F, energy=E, partial_charges=q, hirshfeld_ratios=h, dipole_vec=d)

    def aux(self):
        """Per-atom ZBL / Coulomb / dispersion energies of the last evaluation (copies)."""
        ps = [C.c_void_p() for _ in range(3)]
        check(lib.so3lr_b200_system_aux(self._h, *[C.byref(p) for p in ps]), "aux")
        out = {}
        for name, p in zip(("zbl_repulsion", "electrostatic_energy", "dispersion_energy"), ps):
            out[name] = _from_ptr(p.value, self.n, self.device).clone()
        return out

    def kspace_vectors(self):
        """Number of k vectors the reciprocal sum runs over (both members of every pair (k, -k) counted; mesh points of the
        mesh variant) or None."""
        if self.kspace is None:
            return None
        n1, n2, n3 = self.kspace[0]
        return n1 * n2 * n3 - 1

    def stats(self):
        v = [C.c_int64() for _ in range(4)]
        check(lib.so3lr_b200_system_stats(self._h, *[C.byref(x) for x in v]), "stats")
        return dict(rebuilds=v[0].value, edges=v[1].value, pairs=v[2].value, launches=v[3].value)

    def graph_replays(self):
        """Evaluations that were replayed from a CUDA graph so far (see so3lr_b200_system_graph_replays)."""
        v = C.c_int64()
        check(lib.so3lr_b200_system_graph_replays(self._h, C.byref(v)), "graph_replays")
        return v.value

    def valid_edges(self):
        """Short-range list entries inside the cutoff at the latest evaluation (synchronises the device)."""
        v = C.c_int64()
        check(lib.so3lr_b200_system_valid_edges(self._h, C.byref(v)), "valid_edges")
        return v.value

    def profile(self, enable=True):
        check(lib.so3lr_b200_system_profile(self._h, 1 if enable else 0), "profile")

    def profile_read(self):
        """{group: (total_ms, launches)} since profile(True); synchronises the device."""
        ms = (C.c_float * 16)(); cnt = (C.c_int64 * 16)(); names = (C.c_char_p * 16)()
        ng = lib.so3lr_b200_system_profile_read(self._h, 16, ms, cnt, names)
        return {names[g].decode(): (float(ms[g]), int(cnt[g])) for g in range(ng)}

    def neighbor_list(self, positions, which, capacity):
        """jax-md style (2, capacity) int32 index array padded with n, plus (count, overflow)."""
        R = positions.to(self.device, torch.float32).contiguous()
        idx = torch.empty(2, capacity, dtype=torch.int32, device=self.device)
        cnt, ovf = C.c_int64(), C.c_int()
        s = torch.cuda.current_stream(self.device)
        check(lib.so3lr_b200_system_export_list(self._h, C.c_void_p(s.cuda_stream), _ptr(R), int(which), _ptr(idx), int(capacity),
                                                C.byref(cnt), C.byref(ovf)), "export_list")
        return idx, cnt.value, bool(ovf.value)

    def set_kspace(self, k_grid=None, k_smearing=None, method="ewald"):
        """Switch the reciprocal-space Coulomb part on: `k_grid` is the grid shape (n1, n2, n3) or an array of that shape,
        `k_smearing` the Gaussian width in Angstrom (the `k_grid` / `k_smearing` arguments of the reference's energy function,
        so3lr/jaxmd_utils.py:39-47); `method` 'ewald' sums over the k vectors of the index grid, 'pme' interpolates on a mesh of
        that shape with cubic B-splines (so3lr/potential.py:11-12).  `k_grid=None` switches it off.  One periodic structure with
        a long-range cutoff only."""
        if k_grid is None:
            check(lib.so3lr_b200_system_set_kspace(self._h, 0, 0.0, 0, 0, 0), "set_kspace")
            self.kspace = None
            return
        shape = tuple(int(v) for v in (k_grid.shape if hasattr(k_grid, "shape") else k_grid))
        if len(shape) != 3:
            raise ValueError("k_grid must have three dimensions")
        if k_smearing is None:
            raise ValueError("k_smearing is needed with k_grid")
        s = float(np.asarray(k_smearing.detach().cpu() if torch.is_tensor(k_smearing) else k_smearing, dtype=np.float64).reshape(-1)[0])
        if method not in ("ewald", "pme"):
            raise ValueError("method must be 'ewald' or 'pme'")
        check(lib.so3lr_b200_system_set_kspace(self._h, 1 if method == "ewald" else 2, s, *shape), "set_kspace")
        self.kspace = (shape, s, method)

    def graph_eval(self, idx_i, idx_j, edges, idx_i_lr, idx_j_lr, edges_lr, g_e_atom=None, positions=None):
        """`positions` (n, 3): required while the reciprocal-space part is on; the result then holds `g_positions`, the gradient
        of that part with respect to the positions at fixed charges, and `kspace_strain`, its strain derivative at fixed fractional
        coordinates (xx yy zz yz xz xy)."""
        dev = self.device
        t = lambda a, dt: a.to(dev, dt).contiguous()
        idx_i, idx_j, idx_i_lr, idx_j_lr = (t(a, torch.int32) for a in (idx_i, idx_j, idx_i_lr, idx_j_lr))
        edges, edges_lr = t(edges, torch.float32), t(edges_lr, torch.float32)
        ge = None if g_e_atom is None else t(g_e_atom, torch.float32)
        n = self.n
        out = dict(e_atom=torch.empty(n, device=dev), g_edges=torch.zeros_like(edges), g_edges_lr=torch.zeros_like(edges_lr),
                   partial_charges=torch.empty(n, device=dev), hirshfeld_ratios=torch.empty(n, device=dev))
        s = torch.cuda.current_stream(dev)
        if getattr(self, "kspace", None) is not None:
            if positions is None or ge is not None:
                raise ValueError("with the reciprocal-space part on, graph_eval needs `positions` and a uniform upstream cotangent")
            R = t(positions, torch.float32)
            out["g_positions"] = torch.empty(n, 3, device=dev)
            out["kspace_strain"] = torch.empty(6, device=dev)
            check(lib.so3lr_b200_system_graph_eval_kspace(self._h, C.c_void_p(s.cuda_stream), edges.shape[0], _ptr(idx_i), _ptr(idx_j),
                                                          _ptr(edges), edges_lr.shape[0], _ptr(idx_i_lr), _ptr(idx_j_lr), _ptr(edges_lr),
                                                          _ptr(R), _ptr(out["e_atom"]), _ptr(out["g_edges"]), _ptr(out["g_edges_lr"]),
                                                          _ptr(out["g_positions"]), _ptr(out["kspace_strain"]), _ptr(out["partial_charges"]),
                                                          _ptr(out["hirshfeld_ratios"])), "graph_eval_kspace")
            return out
        check(lib.so3lr_b200_system_graph_eval(self._h, C.c_void_p(s.cuda_stream), edges.shape[0], _ptr(idx_i), _ptr(idx_j), _ptr(edges),
                                               edges_lr.shape[0], _ptr(idx_i_lr), _ptr(idx_j_lr), _ptr(edges_lr), _ptr(ge),
                                               _ptr(out["e_atom"]), _ptr(out["g_edges"]), _ptr(out["g_edges_lr"]),
                                               _ptr(out["partial_charges"]), _ptr(out["hirshfeld_ratios"])), "graph_eval")
        return out

    def nve(self, n_steps, dt_fs, masses, positions, velocities, forces):
        """In-place velocity-Verlet steps on device tensors; returns the per-graph energy of the last step."""
        E = torch.empty(self.n_graphs, dtype=torch.float64, device=self.device)
        s = torch.cuda.current_stream(self.device)
        check(lib.so3lr_b200_system_nve(self._h, C.c_void_p(s.cuda_stream), int(n_steps), float(dt_fs), _ptr(masses), _ptr(positions),
                                        _ptr(velocities), _ptr(forces), _ptr(E)), "nve")
        return E


    def nvt(self, n_steps, dt_fs, kT, tau_fs, masses, positions, velocities, forces, chain, chain_length=3, chain_steps=2,
            sy_steps=3):
        """In-place velocity-Verlet steps under a Nose-Hoover chain thermostat (kT in eV, tau in fs); `chain` comes from
        nhc_state() and carries the thermostat between calls.  Returns the per-graph energy of the last step."""
        E = torch.empty(self.n_graphs, dtype=torch.float64, device=self.device)
        s = torch.cuda.current_stream(self.device)
        check(lib.so3lr_b200_system_nvt(self._h, C.c_void_p(s.cuda_stream), int(n_steps), float(dt_fs), float(kT), float(tau_fs),
                                        int(chain_length), int(chain_steps), int(sy_steps), _ptr(masses), _ptr(positions),
                                        _ptr(velocities), _ptr(forces), _ptr(chain), _ptr(E)), "nvt")
        return E


    def rescale_cell(self, cell):
        """New, slightly rescaled cell; the neighbor lists are kept (the positions must have moved with the cell)."""
        c9 = np.ascontiguousarray(np.asarray(cell, dtype=np.float32).reshape(9))
        check(lib.so3lr_b200_system_rescale_cell(self._h, _ptr(c9)), "rescale_cell")
        self._cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)

    def npt(self, n_steps, dt_fs, kT, pressure, tau_t_fs, tau_b_fs, masses, positions, velocities, forces, state, cell0,
            chain_length=3, chain_steps=2, sy_steps=3):
        """In-place NPT steps (isotropic barostat with Nose-Hoover chains; pressure in eV/A^3); `state` comes from npt_state()
        and `cell0` is the reference cell the box coordinate refers to.  The virial must be enabled and the latest evaluation
        must be the one of `positions`.  Returns (per-graph energy of the last step, the cell after it)."""
        E = torch.empty(self.n_graphs, dtype=torch.float64, device=self.device)
        c0 = np.ascontiguousarray(np.asarray(cell0, dtype=np.float32).reshape(9))
        cout = np.empty(9, np.float32)
        s = torch.cuda.current_stream(self.device)
        check(lib.so3lr_b200_system_npt(self._h, C.c_void_p(s.cuda_stream), int(n_steps), float(dt_fs), float(kT), float(pressure),
                                        float(tau_t_fs), float(tau_b_fs), int(chain_length), int(chain_steps), int(sy_steps),
                                        _ptr(masses), _ptr(positions), _ptr(velocities), _ptr(forces), _ptr(state), _ptr(c0),
                                        _ptr(cout), _ptr(E)), "npt")
        self._cell = cout.astype(np.float64).reshape(3, 3)
        return E, self._cell.copy()


NHC_STATE_DOUBLES = 18
NHC_MAX_CHAIN = 8
NPT_STATE_DOUBLES = 44
BAR = 6.241509074e-7              # eV / A^3 per bar


def npt_box_step(which, state, n_atoms, dt_fs, kT, pressure, tau_t_fs, tau_b_fs, V0, virial, kinetic_energy, chain_length=3,
                 chain_steps=2, sy_steps=3):
    """so3lr_b200_npt_pre (`which` = "pre") / so3lr_b200_npt_post ("post") on `state`: the box-and-chains part of an NPT step.
    `virial` (3,3) and `kinetic_energy` (1,) are float64 CUDA tensors holding totals over all ranks."""
    fn = lib.so3lr_b200_npt_pre if which == "pre" else lib.so3lr_b200_npt_post
    assert virial.is_cuda and virial.dtype == torch.float64 and virial.is_contiguous()
    assert kinetic_energy is None or (kinetic_energy.is_cuda and kinetic_energy.dtype == torch.float64)
    with torch.cuda.device(state.device):
        s = torch.cuda.current_stream(state.device)
        check(fn(C.c_void_p(s.cuda_stream), _ptr(state), int(n_atoms), float(dt_fs), float(kT), float(pressure), float(tau_t_fs),
                 float(tau_b_fs), int(chain_length), int(chain_steps), int(sy_steps), float(V0), _ptr(virial), _ptr(kinetic_energy)),
              "npt_" + which)


def npt_state(device):
    """A zeroed NPT state on `device`: [0:18] thermostat chain, [18:36] barostat chain, [36] eps = ln(V/V0)/3, [37] its
    momentum, [38:42] step coefficients, [42] volume."""
    st = torch.empty(NPT_STATE_DOUBLES, dtype=torch.float64, device=device)
    with torch.cuda.device(st.device):
        s = torch.cuda.current_stream(st.device)
        check(lib.so3lr_b200_npt_init(C.c_void_p(s.cuda_stream), _ptr(st)), "npt_init")
    return st


def nhc_state(device):
    """A zeroed thermostat chain on `device`: [0] kinetic energy (eV), [1] momentum scale not yet applied, [2:10] chain
    positions, [10:18] chain momenta (eV fs)."""
    chain = torch.empty(NHC_STATE_DOUBLES, dtype=torch.float64, device=device)
    with torch.cuda.device(chain.device):
        s = torch.cuda.current_stream(chain.device)
        check(lib.so3lr_b200_nhc_init(C.c_void_p(s.cuda_stream), _ptr(chain)), "nhc_init")
    return chain


def nhc_half_steps(chain, n_half_steps, dt_fs, kT, tau_fs, dof, kinetic_energy=None, chain_length=3, chain_steps=2, sy_steps=3,
                   fresh_scale=True):
    """Advances `chain` by half thermostat steps.  `kinetic_energy` (float64 CUDA tensor, eV; its entries are summed) replaces
    the kinetic energy the chain holds.  The momentum scale of the half steps lands in chain[1]."""
    ke = kinetic_energy
    assert ke is None or (ke.is_cuda and ke.dtype == torch.float64 and ke.is_contiguous())
    with torch.cuda.device(chain.device):
        s = torch.cuda.current_stream(chain.device)
        check(lib.so3lr_b200_nhc_half_steps(C.c_void_p(s.cuda_stream), _ptr(chain), int(chain_length), int(chain_steps), int(sy_steps),
                                            float(dt_fs), float(tau_fs), float(kT), float(dof), int(n_half_steps),
                                            1 if fresh_scale else 0, _ptr(ke), 0 if ke is None else int(ke.numel())), "nhc_half_steps")


def _from_ptr(ptr, n, device):
    """float32 CUDA tensor viewing `n` floats at a raw device address."""
    iface = {"shape": (n,), "typestr": "<f4", "data": (int(ptr), False), "version": 2}

    class _W:
        __cuda_array_interface__ = iface

    return torch.as_tensor(_W(), device=device)


NOALLOC_MAX_ATOMS = 16384


def neighbor_list_noalloc(positions, cell, r_cutoff, ordered, idx, count, overflow, stream=None):
    """Pair list through so3lr_b200_neighbor_list_noalloc, the entry point for callers that cannot allocate GPU memory
    (for instance a handler running inside XLA, whose allocator already owns the device's memory).  Every buffer is the
    caller's: positions (n,3) float32 CUDA, idx (2,capacity) int32 CUDA, count (1,) int64 CUDA, overflow (1,) int32
    CUDA; cell is None or a host (3,3) array with lattice vectors as rows.  At most NOALLOC_MAX_ATOMS atoms.  The
    call only enqueues work; calls on one device must not overlap because they share one fixed scratch array."""
    assert positions.is_cuda and positions.dtype == torch.float32 and positions.is_contiguous()
    assert idx.is_cuda and idx.dtype == torch.int32 and idx.is_contiguous() and idx.shape[0] == 2
    assert count.is_cuda and count.dtype == torch.int64 and overflow.is_cuda and overflow.dtype == torch.int32
    c9 = None if cell is None else np.ascontiguousarray(np.asarray(cell, dtype=np.float32).reshape(9))
    with torch.cuda.device(positions.device):
        s = stream if stream is not None else torch.cuda.current_stream(positions.device)
        check(lib.so3lr_b200_neighbor_list_noalloc(C.c_void_p(s.cuda_stream), int(positions.shape[0]), _ptr(positions), _ptr(c9),
                                                   float(r_cutoff), 1 if ordered else 0, _ptr(idx), int(idx.shape[1]), _ptr(count),
                                                   _ptr(overflow)), "neighbor_list_noalloc")
