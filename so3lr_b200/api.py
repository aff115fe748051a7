"""Host-side mirror of the reference's public interface for the energy+force path.

Same names, argument meaning and error behaviour as so3lr/__init__.py:3-7 of the reference:

    So3lrPotential  <- so3lr/potential.py:7-29        (MLFFPotentialSparse.create_from_workdir)
    Graph           <- so3lr/graph.py:3-36
    to_jax_md       <- so3lr/jaxmd_utils.py:80-143    (+ neighbor_list_featurizer :11-77)
    So3lr           <- so3lr/base_calculator.py:8-124 (make_so3lr)
    So3lrCalculator <- so3lr/ase_utils.py:7-28        (mlffCalculatorSparse)
    neighbor_list   <- jax_md.partition.neighbor_list as called at so3lr/jaxmd_utils.py:96-121

Arrays are torch tensors (CUDA) where the reference uses jax arrays; differentiation goes through
torch.autograd where the reference uses jax.grad.  Every number comes from libso3lr_b200.so; this file only
moves pointers, gathers endpoints and applies the minimum-image convention exactly like the reference's
featurizer does in JAX.
"""
from __future__ import annotations

from collections import namedtuple
from typing import Optional

import numpy as np
import torch

from .engine import Model, System

CUTOFF_SR = 4.5

_GraphBase = namedtuple("_GraphBase", (
    "positions", "edges", "nodes", "centers", "others", "mask", "total_charge", "num_unpaired_electrons", "edges_lr",
    "idx_i_lr", "idx_j_lr", "cell", "k_grid", "k_smearing", "theory_mask", "residue_segments", "residue_charge"))


class Graph(_GraphBase):
    """Boundary record handed to the potential (field for field so3lr/graph.py:3-24)."""

    def __new__(cls, positions, edges, nodes, centers, others, mask, total_charge, num_unpaired_electrons, edges_lr,
                idx_i_lr, idx_j_lr, cell, k_grid=None, k_smearing=None, theory_mask=None, residue_segments=None,
                residue_charge=None):
        return super().__new__(cls, positions, edges, nodes, centers, others, mask, total_charge, num_unpaired_electrons,
                               edges_lr, idx_i_lr, idx_j_lr, cell, k_grid, k_smearing, theory_mask, residue_segments,
                               residue_charge)


def _dev(device=None):
    return torch.device("cuda", 0) if device is None else torch.device(device)


# ------------------------------------------------------------------------------------------------------------
# potential
# ------------------------------------------------------------------------------------------------------------
class _GraphEnergy(torch.autograd.Function):
    """e_atom(edges, edges_lr).  Forward also produces the gradients for a uniform cotangent (the `.sum()` the
    reference takes, so3lr/jaxmd_utils.py:141); a non-uniform cotangent triggers one re-evaluation."""

    @staticmethod
    def forward(ctx, edges, edges_lr, system, idx_i, idx_j, idx_i_lr, idx_j_lr, aux_out, positions=None, cell=None):
        out = system.graph_eval(idx_i, idx_j, edges, idx_i_lr, idx_j_lr, edges_lr, positions=positions)
        ctx.system = system
        ctx.lists = (idx_i, idx_j, idx_i_lr, idx_j_lr)
        ctx.has_positions = positions is not None
        gp = out["g_positions"] if positions is not None else edges.new_zeros(0)
        gc = edges.new_zeros(0)
        if positions is not None and cell is not None:
            # reciprocal part E(positions X, cell C): its strain derivative at fixed fractional coordinates is
            # W = g^T X + G^T C with g = dE/dX, G = dE/dC, so the cell's own cotangent is G = C^-T (W - g^T X)^T
            w = out["kspace_strain"].double()
            W = torch.stack([torch.stack([w[0], w[5], w[4]]), torch.stack([w[5], w[1], w[3]]), torch.stack([w[4], w[3], w[2]])])
            X = positions.double()
            gc = (torch.linalg.inv(cell.double().to(X.device)).T @ (W - gp.double().T @ X).T).to(cell.dtype)
        ctx.save_for_backward(edges, edges_lr, out["g_edges"], out["g_edges_lr"], gp, gc)
        aux_out.update(partial_charges=out["partial_charges"], hirshfeld_ratios=out["hirshfeld_ratios"])
        return out["e_atom"]

    @staticmethod
    def backward(ctx, g):
        edges, edges_lr, ge, gel, gp, gc = ctx.saved_tensors
        g = g.contiguous()
        lo, hi = torch.aminmax(g)
        if bool(lo == hi):
            c = lo.to(ge.dtype)
            return (ge * c, gel * c, None, None, None, None, None, None, (gp * c if ctx.has_positions else None),
                    (gc * c.to(gc.dtype) if gc.numel() else None))
        if ctx.has_positions:
            raise NotImplementedError("the reciprocal-space energy is differentiated for a uniform cotangent (its sum) only")
        out = ctx.system.graph_eval(ctx.lists[0], ctx.lists[1], edges, ctx.lists[2], ctx.lists[3], edges_lr, g_e_atom=g)
        return out["g_edges"], out["g_edges_lr"], None, None, None, None, None, None, None, None


class So3lrPotentialB200:
    """Callable with the interface of mlff's MLFFPotentialSparse as the reference uses it
    (so3lr/jaxmd_utils.py:99,113,138-141): attributes `cutoff`, `long_range_cutoff`; `pot(graph)` -> per-atom
    energies, `pot(graph, has_aux=True)` -> (energies, aux dict)."""

    MAX_CACHED_SYSTEMS = 4      # evaluation contexts kept per potential (each holds every per-atom workspace of its system)

    def __init__(self, lr_cutoff=12.0, dispersion_energy_cutoff_lr_damping=2.0, neighborlist_format_lr="ordered_sparse",
                 dtype=np.float32, device=None, coulomb_kspace_do_ewald=False, coulomb_kspace_interp_nodes=4):
        """`dtype` is the dtype of the returned energies and gradients, as in the reference where it "determines the output
        dtype" of float32 parameters (tests/test_jaxmd.py:210-212): float32 or float64.  The kernels compute in float32 either
        way; with float64 the float32 results are widened, so they carry float32 accuracy (1e-7 relative on energies)."""
        if np.dtype(dtype) not in (np.dtype(np.float32), np.dtype(np.float64)):
            raise ValueError("dtype must be float32 or float64")
        self.dtype = torch.float64 if np.dtype(dtype) == np.dtype(np.float64) else torch.float32
        self.cutoff = CUTOFF_SR
        self.long_range_cutoff = lr_cutoff
        self.damping = dispersion_energy_cutoff_lr_damping
        self.neighborlist_format_lr = neighborlist_format_lr
        self.device = _dev(device)
        # a graph that carries k_grid / k_smearing is evaluated with the Ewald sum over the index grid when this is set, else with
        # particle-mesh Ewald on a mesh of that shape (so3lr/potential.py:11-12); the mesh variant has four interpolation nodes
        if int(coulomb_kspace_interp_nodes) != 4:
            raise NotImplementedError("the mesh variant interpolates with four nodes per axis (cubic B-splines) only")
        self.coulomb_kspace_do_ewald = bool(coulomb_kspace_do_ewald)
        self._systems = {}

    def system_for(self, species, cell=None, graph_start=None, total_charge=None, num_unpaired=None):
        Z = np.ascontiguousarray(species.detach().cpu().numpy() if torch.is_tensor(species) else species, dtype=np.int32)
        n_graphs = 1 if graph_start is None else len(graph_start) - 1

        def per_graph(v):
            if v is None:
                return None
            a = np.asarray(torch.as_tensor(v).detach().cpu(), dtype=np.float32).reshape(-1)
            a = np.broadcast_to(a, (n_graphs,)) if a.size == 1 else a[:n_graphs]
            return None if not a.any() else np.ascontiguousarray(a)

        tq, ts = per_graph(total_charge), per_graph(num_unpaired)
        key = (Z.tobytes(), None if graph_start is None else np.asarray(graph_start).tobytes(),
               None if tq is None else tq.tobytes(), None if ts is None else ts.tobytes())
        s = self._systems.pop(key, None)
        if s is None:
            s = System(Z, None, cutoff_lr=self.long_range_cutoff, damping=self.damping, lr_format=self.neighborlist_format_lr,
                       graph_start=graph_start, total_charge=tq, num_unpaired=ts, device=self.device.index or 0)
        self._systems[key] = s                      # most recently used last
        while len(self._systems) > self.MAX_CACHED_SYSTEMS:
            self._systems.pop(next(iter(self._systems)))
        return s

    def __call__(self, graph: Graph, has_aux: bool = False):
        kspace = graph.k_grid is not None
        if kspace:
            if graph.k_smearing is None or graph.positions is None or graph.cell is None:
                raise ValueError("k-space electrostatics needs Graph.k_smearing, Graph.positions and Graph.cell")
        s = self.system_for(graph.nodes, total_charge=graph.total_charge, num_unpaired=graph.num_unpaired_electrons)
        if kspace:
            cell = np.asarray(graph.cell.detach().cpu(), dtype=np.float64).reshape(3, 3)
            if s._cell is None or not np.array_equal(s._cell, cell):
                s.set_cell(cell)
            shape = tuple(int(v) for v in graph.k_grid.shape)
            sm = float(np.asarray(torch.as_tensor(graph.k_smearing).detach().cpu(), dtype=np.float64).reshape(-1)[0])
            method = "ewald" if self.coulomb_kspace_do_ewald else "pme"
            if s.kspace != (shape, sm, method):
                s.set_kspace(shape, sm, method)
        elif s.kspace is not None:
            s.set_kspace(None)
        edges, edges_lr = graph.edges, graph.edges_lr
        idx_i, idx_j, idx_i_lr, idx_j_lr = graph.centers, graph.others, graph.idx_i_lr, graph.idx_j_lr
        # the kernels want lists grouped by centre; jax-md style lists already are
        perm = perm_lr = None
        if idx_i.numel() > 1 and bool((idx_i[1:] < idx_i[:-1]).any()):
            perm = torch.sort(idx_i, stable=True).indices
            idx_i, idx_j, edges = idx_i[perm], idx_j[perm], edges[perm]
        if idx_i_lr.numel() > 1 and bool((idx_i_lr[1:] < idx_i_lr[:-1]).any()):
            perm_lr = torch.sort(idx_i_lr, stable=True).indices
            idx_i_lr, idx_j_lr, edges_lr = idx_i_lr[perm_lr], idx_j_lr[perm_lr], edges_lr[perm_lr]
        aux = {}
        e = _GraphEnergy.apply(edges.to(self.device, torch.float32), edges_lr.to(self.device, torch.float32), s, idx_i, idx_j,
                               idx_i_lr, idx_j_lr, aux,
                               graph.positions.to(self.device, torch.float32) if kspace else None,
                               graph.cell.to(self.device) if kspace else None).to(self.dtype)
        if not has_aux:
            return e
        aux.update(s.aux())
        aux = {k: (v.to(self.dtype) if torch.is_tensor(v) and v.is_floating_point() else v) for k, v in aux.items()}
        if graph.positions is not None:
            aux["dipole_vec"] = (aux["partial_charges"][:, None] * graph.positions).sum(0)
        return e, aux


def make_potential_fn(lr_cutoff=12.0, dispersion_energy_cutoff_lr_damping=2.0, dtype=np.float32, coulomb_kspace_do_ewald=False,
                      coulomb_kspace_interp_nodes=4, **kwargs):
    """so3lr/potential.py:7-29.  For graphs that carry `k_grid` / `k_smearing`: `coulomb_kspace_do_ewald=True` selects the Ewald
    sum over the index grid, the default the particle-mesh variant with `coulomb_kspace_interp_nodes` = 4 nodes per axis."""
    return So3lrPotentialB200(lr_cutoff, dispersion_energy_cutoff_lr_damping, "ordered_sparse", dtype, kwargs.get("device"),
                              coulomb_kspace_do_ewald=coulomb_kspace_do_ewald, coulomb_kspace_interp_nodes=coulomb_kspace_interp_nodes)


def get_kgrid_ewald_shape(cell, lr_wavelength):
    """Shape of the k-vector index grid for a resolution `lr_wavelength` (Angstrom): one index per `lr_wavelength` of each lattice
    vector's length (argument convention of `jaxpme.kspace.get_kgrid_ewald` as called at so3lr/cli/so3lr_md.py:1421-1423)."""
    c = np.asarray(cell.detach().cpu() if torch.is_tensor(cell) else cell, dtype=np.float64).reshape(3, 3)
    lam = float(np.asarray(lr_wavelength.detach().cpu() if torch.is_tensor(lr_wavelength) else lr_wavelength).reshape(-1)[0])
    return tuple(int(max(1, np.ceil(np.linalg.norm(c[d]) / lam - 1e-9))) for d in range(3))


def get_kgrid_ewald(cell, lr_wavelength):
    """An array whose SHAPE is the index grid (the only property of `k_grid` that the evaluation reads)."""
    return torch.zeros(get_kgrid_ewald_shape(cell, lr_wavelength))


def get_kgrid_mesh_shape(cell, mesh_spacing):
    """Mesh of the particle-mesh variant: the power of two per lattice vector that brings the distance between mesh points to
    `mesh_spacing` (Angstrom) or below (argument convention of `jaxpme.kspace.get_kgrid_mesh`, so3lr/cli/so3lr_md.py:1424-1427)."""
    c = np.asarray(cell.detach().cpu() if torch.is_tensor(cell) else cell, dtype=np.float64).reshape(3, 3)
    h = float(np.asarray(mesh_spacing.detach().cpu() if torch.is_tensor(mesh_spacing) else mesh_spacing).reshape(-1)[0])
    return tuple(int(2 ** max(2, int(np.ceil(np.log2(np.linalg.norm(c[d]) / h) - 1e-9)))) for d in range(3))


def get_kgrid_mesh(cell, mesh_spacing):
    return torch.zeros(get_kgrid_mesh_shape(cell, mesh_spacing))


# ------------------------------------------------------------------------------------------------------------
# neighbor lists with the jax-md calling convention
# ------------------------------------------------------------------------------------------------------------
class NeighborList:
    """What the reference reads from a jax-md neighbor list: `.idx` (2, capacity) int32 padded with N,
    `.did_buffer_overflow`, `.update(R, box=...)` (so3lr/cli/so3lr_md.py:862-876, :1143-1152)."""

    def __init__(self, fn, idx, count, overflow, reference_position):
        self._fn, self.idx, self.count, self.did_buffer_overflow = fn, idx, count, overflow
        self.reference_position = reference_position

    @property
    def capacity(self):
        return self.idx.shape[1]

    def update(self, R, **kwargs):
        return self._fn._update(self, R, kwargs.get("box", self._fn.box))


class NeighborFn:
    def __init__(self, box, r_cutoff, dr_threshold, capacity_multiplier, fractional_coordinates, ordered, species_len=None,
                 device=None):
        self.box, self.r_cutoff, self.dr_threshold = box, float(r_cutoff), float(dr_threshold)
        self.capacity_multiplier, self.fractional, self.ordered = float(capacity_multiplier), fractional_coordinates, ordered
        self.device = _dev(device)
        self._sys = None
        self._cell_key = None

    def _cell(self, box):
        if box is None:
            return None
        b = torch.as_tensor(box, dtype=torch.float64).cpu().numpy()
        if b.ndim == 0 or b.shape == (1,):
            return np.eye(3) * float(b.reshape(-1)[0])
        if b.shape == (3,):
            return np.diag(b)
        return b.T.copy()   # jax-md boxes hold lattice vectors as columns

    def _cartesian(self, R, box):
        R = (torch.as_tensor(R) if not torch.is_tensor(R) else R.detach()).to(self.device)
        cell = self._cell(box)
        if cell is not None and self.fractional:
            R = R.double() @ torch.tensor(cell, dtype=torch.float64, device=self.device)
        return R.float().contiguous(), cell

    def _system(self, n, cell):
        key = (n, None if cell is None else cell.tobytes())
        if self._sys is None or self._cell_key != key:
            if self._sys is not None and self._cell_key[0] == n and cell is not None and self._cell_key[1] is not None:
                self._sys.set_cell(cell)
            else:
                # list radius = r_cutoff + dr_threshold; the same context serves either list through its long-range slot
                self._sys = System(np.ones(n, np.int32), cell, cutoff_lr=self.r_cutoff, damping=None, skin=self.dr_threshold,
                                   lr_format="ordered_sparse" if self.ordered else "sparse", device=self.device.index or 0)
            self._cell_key = key
        return self._sys

    def allocate(self, R, **kwargs):
        box = kwargs.get("box", self.box)
        Rc, cell = self._cartesian(R, box)
        s = self._system(Rc.shape[0], cell)
        _, count, _ = s.neighbor_list(Rc, 1, 1)
        cap = max(int(count * self.capacity_multiplier) + 1, 1)
        idx, count, ovf = s.neighbor_list(Rc, 1, cap)
        return NeighborList(self, idx, count, ovf, Rc)

    def _update(self, nbrs, R, box):
        """jax-md's update protocol: the list is kept while no atom has moved further than dr_threshold / 2 since it was
        built, also when the box has changed meanwhile (an NPT run rescales it every step, so3lr/cli/so3lr_md.py:1270-1282:
        the Cartesian positions carry the rescaling, so the same test covers it); otherwise it is rebuilt into the same
        capacity and an overflow is flagged, never raised."""
        Rc, cell = self._cartesian(R, box)
        n = Rc.shape[0]
        same_kind = self._sys is not None and self._cell_key[0] == n and (cell is None) == (self._cell_key[1] is None)
        if self.dr_threshold > 0 and same_kind and nbrs.reference_position.shape == Rc.shape:
            moved = (Rc - nbrs.reference_position).square().sum(-1).max() > (0.5 * self.dr_threshold) ** 2
            if not bool(moved):
                if cell is not None and self._cell_key[1] != cell.tobytes():
                    self._sys.rescale_cell(cell)
                    self._cell_key = (n, cell.tobytes())
                return nbrs
        s = self._system(n, cell)
        idx, count, ovf = s.neighbor_list(Rc, 1, nbrs.capacity)
        return NeighborList(self, idx, count, ovf or nbrs.did_buffer_overflow, Rc)


def neighbor_list(displacement_or_metric, box, r_cutoff, dr_threshold=0.0, capacity_multiplier=1.25, buffer_size_multiplier=1.25,
                  minimum_cell_size_multiplier=1.0, fractional_coordinates=False, format=1, disable_cell_list=False, **kwargs):
    """Positional signature of the jax-md fork's partition.neighbor_list (so3lr/jaxmd_utils.py:96-121).
    format 1 = Sparse (both directions), 2 = OrderedSparse (i < j).  The multipliers that size jax-md's cell
    buffers have no counterpart here (rows are counted exactly) and are ignored, as is `disable_cell_list`."""
    fmt = int(getattr(format, "value", format))
    if fmt not in (1, 2):
        raise ValueError("only Sparse (1) and OrderedSparse (2) neighbor list formats are supported")
    return NeighborFn(box, r_cutoff, dr_threshold, capacity_multiplier, fractional_coordinates, fmt == 2, device=kwargs.get("device"))


# ------------------------------------------------------------------------------------------------------------
# jax-md style adapter
# ------------------------------------------------------------------------------------------------------------
def _min_image(dR, cell_t):
    if cell_t is None:
        return dR
    s = dR.detach() @ torch.linalg.inv(cell_t)
    return dR - torch.round(s) @ cell_t


class _Transform(torch.autograd.Function):
    """Fractional -> Cartesian positions with jax-md's convention for the derivative (jax_md.space.transform has a custom
    JVP whose tangent is dR + transform(dbox, R)): the gradient with respect to fractional positions is the real-space one,
    which is why the reference compares `quantity.force(energy_fn)(R0_fractional, ...)` with forces in eV/A directly
    (tests/test_jaxmd.py:86-101)."""

    @staticmethod
    def forward(ctx, R, cell_t):
        return R @ cell_t

    @staticmethod
    def backward(ctx, g):
        return g, None


def neighbor_list_featurizer(displacement_fn, species, fractional_coordinates=True, device=None, total_charge=0.0):
    """so3lr/jaxmd_utils.py:11-77 (and its CLI twin with `total_charge`, so3lr/cli/so3lr_md.py:606-685): endpoints gather,
    minimum-image displacement, Graph assembly.  Positions and box keep the precision they are given in (float64 positions in
    a 1000 A box lose nothing); the displacements are handed to the float32 kernels.  `perturbation` (a scalar or a 3x3
    matrix) deforms every displacement, dR -> perturbation dR, as jax-md's displacement functions do with that keyword; it is
    differentiable, which is how the reference's NPT obtains the strain derivative of the energy (jaxmd_utils.py:48-51)."""
    dev = _dev(device)
    species_t = torch.as_tensor(np.asarray(species), dtype=torch.int32, device=dev)

    def featurize(R, neighbor, neighbor_lr, **kwargs):
        R = torch.as_tensor(R, device=dev) if not torch.is_tensor(R) else R.to(dev)
        if R.dtype not in (torch.float32, torch.float64):
            R = R.float()
        n = R.shape[0]
        box = kwargs.get("box")
        cell_t = None
        if box is not None:
            b = torch.as_tensor(box, dtype=R.dtype, device=dev)
            if b.shape == (3, 3):
                cell_t = b.T
            elif b.shape == (3,):
                cell_t = torch.diag(b)
            elif b.shape == (1,) or b.ndim == 0:
                cell_t = torch.eye(3, dtype=R.dtype, device=dev) * b.reshape(-1)[0]
            else:
                raise ValueError(f"Invalid box shape {tuple(b.shape)}. Expected (3, 3), (3,), or (1,).")
        k_grid, k_smearing = kwargs.get("k_grid"), kwargs.get("k_smearing")
        pert = kwargs.get("perturbation")
        if k_grid is not None and cell_t is None:
            raise ValueError("k-space electrostatics needs `box`")
        Rc = _Transform.apply(R, cell_t) if (cell_t is not None and fractional_coordinates) else R
        neighbor, neighbor_lr = torch.as_tensor(neighbor, device=dev), torch.as_tensor(neighbor_lr, device=dev)
        idx_i, idx_j = neighbor[0].long(), neighbor[1].long()
        idx_i_lr, idx_j_lr = neighbor_lr[0].long(), neighbor_lr[1].long()
        cl = lambda a: a.clamp(max=n - 1)   # JAX gathers clamp the padding index N to N-1
        # the kernels take dR = R_j - R_i; the energy does not depend on the sign convention
        dR = _min_image(Rc[cl(idx_j)] - Rc[cl(idx_i)], cell_t)
        dR_lr = _min_image(Rc[cl(idx_j_lr)] - Rc[cl(idx_i_lr)], cell_t)
        positions = Rc if k_grid is not None else None
        if pert is not None:
            p = pert if torch.is_tensor(pert) else torch.as_tensor(pert)
            p = p.to(device=dev, dtype=dR.dtype)
            if p.ndim == 0 or p.numel() == 1:
                dR, dR_lr = dR * p.reshape(()), dR_lr * p.reshape(())
                if positions is not None:     # positions and box are deformed with the displacements (jaxmd_utils.py:48-51)
                    positions, cell_t = positions * p.reshape(()), cell_t * p.reshape(())
            else:
                dR, dR_lr = dR @ p.T, dR_lr @ p.T
                if positions is not None:
                    positions = positions @ p.T
                if cell_t is not None:
                    cell_t = cell_t @ p.T
        return Graph(positions=positions, k_grid=k_grid, k_smearing=k_smearing, nodes=species_t, edges=dR.float(), centers=neighbor[0], others=neighbor[1], mask=None,
                     total_charge=torch.tensor([float(total_charge)]), num_unpaired_electrons=torch.zeros(1), edges_lr=dR_lr.float(),
                     idx_i_lr=neighbor_lr[0], idx_j_lr=neighbor_lr[1], cell=cell_t)

    return featurize


def force(energy_fn):
    """jax_md.quantity.force: R, **kwargs -> -dE/dR (README.md:241, tests/test_jaxmd.py:81 of the reference)."""

    def force_fn(R, **kwargs):
        Rg = (torch.as_tensor(R) if not torch.is_tensor(R) else R).detach().clone().requires_grad_(True)
        E = energy_fn(Rg, **kwargs)
        (g,) = torch.autograd.grad(E, Rg)
        return -g

    return force_fn


def to_jax_md(potential, displacement_or_metric, box_size, species=None, dr_threshold: float = 0.0, capacity_multiplier: float = 1.25,
              buffer_size_multiplier_sr: float = 1.25, buffer_size_multiplier_lr: float = 1.25,
              minimum_cell_size_multiplier_sr: float = 1.0, minimum_cell_size_multiplier_lr: float = 1.0,
              disable_cell_list: bool = False, fractional_coordinates: bool = True, total_charge: float = 0.0, **neighbor_kwargs):
    """so3lr/jaxmd_utils.py:80-143 (with the `total_charge` of the CLI's variant, so3lr/cli/so3lr_md.py:690-782): returns
    (neighbor_fn, neighbor_fn_lr, energy_fn)."""
    neighbor_fn = neighbor_list(displacement_or_metric, box_size, potential.cutoff, dr_threshold, capacity_multiplier,
                                buffer_size_multiplier_sr, minimum_cell_size_multiplier_sr,
                                fractional_coordinates=fractional_coordinates, format=1, disable_cell_list=disable_cell_list,
                                **neighbor_kwargs)
    neighbor_fn_lr = neighbor_list(displacement_or_metric, box_size, potential.long_range_cutoff, dr_threshold, capacity_multiplier,
                                   buffer_size_multiplier_lr, minimum_cell_size_multiplier_lr,
                                   fractional_coordinates=fractional_coordinates, format=2, disable_cell_list=disable_cell_list,
                                   **neighbor_kwargs)
    featurizer = neighbor_list_featurizer(displacement_or_metric, species, fractional_coordinates=fractional_coordinates,
                                          device=potential.device, total_charge=total_charge)

    def energy_fn(R, neighbor, neighbor_lr, has_aux=False, **energy_fn_kwargs):
        graph = featurizer(R, neighbor, neighbor_lr, **energy_fn_kwargs)
        if has_aux:
            return potential(graph, has_aux=True)
        return potential(graph).sum()

    return neighbor_fn, neighbor_fn_lr, energy_fn


# ------------------------------------------------------------------------------------------------------------
# batched calculator
# ------------------------------------------------------------------------------------------------------------
def make_so3lr(lr_cutoff=12.0, dispersion_energy_cutoff_lr_damping=2.0, calculate_forces=True, workdir=None, device=None):
    """so3lr/base_calculator.py:8-124.  Returns so3lr_fn(inputs) -> outputs with keys energy (n_graph,),
    forces (n_node,3), dipole_vec (n_graph,3), hirshfeld_ratios (n_node,), partial_charges (n_node,).
    `inputs` carries the same keys the reference passes to model.apply (positions, atomic_numbers, idx_i, idx_j,
    idx_i_lr, idx_j_lr, cell, total_charge, num_unpaired_electrons, batch_segments, node_mask, graph_mask);
    long-range lists hold both directions ('sparse', :31)."""
    if workdir is not None:
        raise NotImplementedError("custom checkpoints (orbax workdir) are not supported; the packed default weights are used")
    dev = _dev(device)
    pot = So3lrPotentialB200(lr_cutoff, dispersion_energy_cutoff_lr_damping, "sparse", np.float32, dev)

    def so3lr_fn(inputs):
        R = torch.as_tensor(inputs["positions"], dtype=torch.float32, device=dev)
        n = R.shape[0]
        Z = np.asarray(torch.as_tensor(inputs["atomic_numbers"]).cpu(), dtype=np.int32)
        bs = inputs.get("batch_segments")
        gm = inputs.get("graph_mask")
        if bs is None:
            assert gm is None
            bs_np, n_graphs = np.zeros(n, np.int64), 1
            gm_t = torch.ones(1, dtype=torch.bool, device=dev)
        else:
            bs_np = np.asarray(torch.as_tensor(bs).cpu(), dtype=np.int64)
            gm_t = torch.as_tensor(gm, device=dev).bool()
            n_graphs = int(gm_t.shape[0])
        if np.any(np.diff(bs_np) < 0):
            raise ValueError("batch_segments must be non-decreasing (atoms of one graph contiguous)")
        graph_start = np.searchsorted(bs_np, np.arange(n_graphs + 1)).astype(np.int32)
        s = pot.system_for(Z, graph_start=graph_start if n_graphs > 1 else None, total_charge=inputs.get("total_charge"),
                           num_unpaired=inputs.get("num_unpaired_electrons"))
        cell = inputs.get("cell")
        cell_t = None
        if cell is not None:
            c = torch.as_tensor(cell, dtype=torch.float32, device=dev)
            if c.ndim == 3:
                if c.shape[0] != 1 and bool((c - c[:1]).abs().max() > 0):
                    raise NotImplementedError("one cell per batch is supported")
                c = c[0]
            if bool(c.abs().sum() > 0):
                cell_t = c
        ii, jj = torch.as_tensor(inputs["idx_i"], device=dev).long(), torch.as_tensor(inputs["idx_j"], device=dev).long()
        il, jl = torch.as_tensor(inputs["idx_i_lr"], device=dev).long(), torch.as_tensor(inputs["idx_j_lr"], device=dev).long()
        cl = lambda a: a.clamp(max=n - 1)

        def sort_by_centre(a, b):
            if a.numel() > 1 and bool((a[1:] < a[:-1]).any()):
                p = torch.sort(a, stable=True).indices
                return a[p], b[p]
            return a, b

        ii, jj = sort_by_centre(ii, jj)
        il, jl = sort_by_centre(il, jl)
        dR = _min_image(R[cl(jj)] - R[cl(ii)], cell_t)
        dRl = _min_image(R[cl(jl)] - R[cl(il)], cell_t)
        nm = inputs.get("node_mask")
        node_mask = torch.ones(n, dtype=torch.bool, device=dev) if nm is None else torch.as_tensor(nm, device=dev).bool()
        # cotangent of the masked energy sum (base_calculator.py:91)
        ge = gm_t[torch.as_tensor(bs_np, device=dev)].float() * node_mask.float()
        out = s.graph_eval(ii.int(), jj.int(), dR, il.int(), jl.int(), dRl, g_e_atom=ge)
        bs_t = torch.as_tensor(bs_np, device=dev)
        e_atom = out["e_atom"] * node_mask
        energy = torch.zeros(n_graphs, device=dev).index_add_(0, bs_t, e_atom) * gm_t
        q = out["partial_charges"] * node_mask
        h = out["hirshfeld_ratios"] * node_mask
        dip = torch.zeros(n_graphs, 3, device=dev).index_add_(0, bs_t, q[:, None] * R) * gm_t[:, None]
        res = dict(energy=energy, dipole_vec=dip, hirshfeld_ratios=h, partial_charges=q)
        if calculate_forces:
            F = torch.zeros(n, 3, device=dev)
            vi, vl = (ii < n) & (jj < n), (il < n) & (jl < n)
            F.index_add_(0, cl(ii), out["g_edges"] * vi[:, None]); F.index_add_(0, cl(jj), -out["g_edges"] * vi[:, None])
            F.index_add_(0, cl(il), out["g_edges_lr"] * vl[:, None]); F.index_add_(0, cl(jl), -out["g_edges_lr"] * vl[:, None])
            res["forces"] = F
        return res

    return so3lr_fn


# ------------------------------------------------------------------------------------------------------------
# ASE-style calculator
# ------------------------------------------------------------------------------------------------------------
try:  # pragma: no cover - ase is optional
    from ase.calculators.calculator import Calculator as _AseCalculator, all_changes as _all_changes
except Exception:  # ase not installed: a duck-typed stand-in with the same entry points
    _AseCalculator = object
    _all_changes = ()


class So3lrCalculatorB200(_AseCalculator):
    """so3lr/ase_utils.py:7-28.  `get_potential_energy(atoms)` / `get_forces(atoms)`; `atoms` needs
    get_positions(), get_atomic_numbers(), get_cell(), get_pbc().  With calculate_stress=True `get_stress(atoms)` returns the
    stress of a periodic cell in Voigt order (xx, yy, zz, yz, xz, xy), eV/A^3; without it get_stress raises NotImplementedError
    as the reference does (tests/test_ase.py:145-172).  The Hessian is not provided."""
    implemented_properties = ["energy", "forces", "charges", "hirshfeld_ratios", "dipole", "stress"]

    def __init__(self, lr_cutoff=12.0, dispersion_energy_cutoff_lr_damping=2.0, calculate_stress=False, calculate_hessian=False,
                 dtype=np.float32, skin=0.0, device=None, **kwargs):
        if _AseCalculator is not object:
            super().__init__(**kwargs)
        if calculate_hessian:
            raise NotImplementedError("the Hessian is not provided by so3lr_b200")
        self.calculate_stress = bool(calculate_stress)
        if np.dtype(dtype) not in (np.dtype(np.float32), np.dtype(np.float64)):
            raise ValueError("dtype must be float32 or float64")
        self.dtype = np.dtype(dtype)        # results are float32 computations, returned in this dtype
        self.lr_cutoff, self.damping, self.skin = lr_cutoff, dispersion_energy_cutoff_lr_damping, skin
        self.device = _dev(device)
        self._sys, self._key = None, None
        self.results = {}

    def _evaluate(self, atoms):
        Z = np.asarray(atoms.get_atomic_numbers(), dtype=np.int32)
        pbc = np.asarray(atoms.get_pbc()).any()
        cell = np.asarray(atoms.get_cell(), dtype=np.float64) if pbc else None
        info = getattr(atoms, "info", None) or {}
        charge = float(info.get("charge", 0.0))
        unpaired = float(info.get("multiplicity", 1.0)) - 1.0
        key = (Z.tobytes(), None if cell is None else cell.tobytes(), charge, unpaired)
        if self._key != key:
            if self._sys is not None and self._key[0] == key[0] and cell is not None and self._key[1] is not None and self._key[2:] == key[2:]:
                self._sys.set_cell(cell)
            else:
                self._sys = System(Z, cell, cutoff_lr=self.lr_cutoff, damping=self.damping, skin=self.skin,
                                   total_charge=[charge] if charge else None, num_unpaired=[unpaired] if unpaired else None,
                                   device=self.device.index or 0)
                if self.calculate_stress:
                    self._sys.enable_virial(True)
            self._key = key
        out = self._sys.compute_host(np.asarray(atoms.get_positions(), dtype=np.float32))
        self.results = dict(energy=float(out["energy"].sum()), forces=out["forces"].astype(np.float64),
                            charges=out["partial_charges"].astype(self.dtype), hirshfeld_ratios=out["hirshfeld_ratios"].astype(self.dtype),
                            dipole=out["dipole_vec"][0].astype(self.dtype))
        if self.calculate_stress and cell is not None:
            w = self._sys.virial().cpu().numpy() / abs(np.linalg.det(cell))
            self.results["stress"] = np.array([w[0, 0], w[1, 1], w[2, 2], w[1, 2], w[0, 2], w[0, 1]])
        return self.results

    def calculate(self, atoms=None, properties=("energy",), system_changes=_all_changes):
        if _AseCalculator is not object:
            super().calculate(atoms, properties, system_changes)
        self._evaluate(atoms if atoms is not None else self.atoms)

    def get_potential_energy(self, atoms=None, **kw):
        return self._evaluate(atoms)["energy"]

    def get_forces(self, atoms=None, **kw):
        return self._evaluate(atoms)["forces"]

    def get_stress(self, atoms=None, **kw):
        if not self.calculate_stress:
            raise NotImplementedError("create the calculator with calculate_stress=True")
        res = self._evaluate(atoms)
        if "stress" not in res:
            raise NotImplementedError("stress needs a periodic cell")
        return res["stress"]


def make_ase_calculator(lr_cutoff=12.0, dispersion_energy_cutoff_lr_damping=2.0, calculate_stress=False, calculate_hessian=False,
                        dtype=np.float32, **kwargs):
    return So3lrCalculatorB200(lr_cutoff, dispersion_energy_cutoff_lr_damping, calculate_stress, calculate_hessian, dtype, **kwargs)
