"""CPU oracle for the reciprocal-space (Ewald and particle-mesh Ewald) part of the electrostatic energy.  TEST INFRASTRUCTURE ONLY.

The reference switches its long-range Coulomb term to a real-space + reciprocal-space split when the energy function is
called with `k_grid` and `k_smearing` (so3lr/jaxmd_utils.py:39-47,70-71; so3lr/cli/so3lr_md.py:1392-1428 builds the grid
with `jaxpme.kspace.get_kgrid_ewald(cell, lr_wavelength)`; so3lr/potential.py:11-12,24-25 selects Ewald or the mesh
variant).  The arithmetic lives in the un-vendored dependencies `jax-pme` (fbruenig/jax-pme@main, pyproject.toml:25) and
`mlff` (`coulomb_erf_shifted_force_smooth_pme`, imported at so3lr/cli/tune_ewald.py:10); neither source is in the reference
tree and the reference's tests hold no vector for this path, so parity with the reference is UNPINNED.  What is restated here
is the published Ewald summation for Gaussian-smeared charges:

    erf(r / sigma) / r  =  [erf(r / sigma) - erf(r / (sqrt(2) s))] / r   (short-ranged: stays in the pair sum)
                         +  erf(r / (sqrt(2) s)) / r                      (summed over all periodic images in k-space)

    E_k = ke / (2 V) sum_{k != 0} (4 pi / k^2) exp(-s^2 k^2 / 2) |S(k)|^2  -  ke sum_i q_i^2 / (sqrt(2 pi) s)
          -  ke pi s^2 Q^2 / V,            S(k) = sum_i q_i exp(i k r_i),  Q = sum_i q_i

with the k vectors on the FFT-frequency index grid whose shape is the shape of `k_grid`.  The split is exact for any
smearing s, which the tests use (the total must not depend on s), together with the Madelung constants of the rock-salt
and caesium-chloride lattices as known answers.  The mesh variant (smooth particle-mesh Ewald with cubic B-splines, at the
end of this file) is checked against the direct sum: it converges to it with the fourth power of the mesh spacing.

Nothing in the product path may import this module.
"""
from __future__ import annotations

import math

import numpy as np
import torch

KE = 14.399645351950548                         # so3lr/cli/tune_ewald.py:163


def ewald_grid_shape(cell, lr_wavelength):
    """Shape of the k-vector index grid for a resolution `lr_wavelength` (Angstrom): one index per `lr_wavelength` of each
    lattice vector's length (the argument convention of so3lr/cli/so3lr_md.py:1421-1423)."""
    cell = np.asarray(cell, dtype=np.float64)
    return tuple(int(max(1, math.ceil(np.linalg.norm(cell[d]) / float(lr_wavelength) - 1e-9))) for d in range(3))


def grid_indices(shape):
    """Integer triples (h1, h2, h3) of the FFT-frequency grid of the given shape, origin removed: (K, 3) int64."""
    axes = [np.rint(np.fft.fftfreq(n, 1.0 / n)).astype(np.int64) for n in shape]
    h = np.stack(np.meshgrid(*axes, indexing="ij"), -1).reshape(-1, 3)
    return h[(h != 0).any(1)]


def reciprocal_energy(R, q, cell, shape, smearing):
    """Per-atom reciprocal-space energies (eV), differentiable torch code.

    R (N,3) Cartesian positions, q (N,) charges, cell (3,3) lattice vectors as rows (all torch, same dtype); the
    energy of atom i is q_i phi_i / 2 minus its self term minus its share of the neutralising background.
    """
    dt = R.dtype
    h = torch.as_tensor(grid_indices(shape), dtype=dt)
    inv = torch.linalg.inv(cell)
    vol = torch.abs(torch.linalg.det(cell))
    kvec = 2 * math.pi * h @ inv.T                      # k = 2 pi (h1 b1 + h2 b2 + h3 b3), b = columns of cell^-1
    k2 = (kvec * kvec).sum(-1)
    g = 4 * math.pi / k2 * torch.exp(-0.5 * smearing ** 2 * k2)
    theta = R @ kvec.T                                  # (N, K)
    c, s = torch.cos(theta), torch.sin(theta)
    sr, si = (q[:, None] * c).sum(0), (q[:, None] * s).sum(0)
    phi = KE / vol * ((c * sr[None, :] + s * si[None, :]) * g[None, :]).sum(-1)
    qtot = q.sum()
    return 0.5 * q * phi - KE * q * q / (math.sqrt(2 * math.pi) * smearing) - KE * math.pi * smearing ** 2 * q * qtot / vol


def pair_kernel_longrange(r, smearing):
    """erf(r / (sqrt(2) s)) / r: the part of a pair interaction that the reciprocal sum already holds."""
    return torch.erf(r / (math.sqrt(2.0) * smearing)) / r


def point_charge_ewald(R, q, cell, smearing, shape, real_cutoff):
    """Total electrostatic energy (units of ke = 1) of periodic POINT charges: complementary-error-function pair sum over
    all images inside `real_cutoff` plus the reciprocal sum above.  Used with the Madelung known answers only."""
    R = np.asarray(R, dtype=np.float64); q = np.asarray(q, dtype=np.float64); cell = np.asarray(cell, dtype=np.float64)
    n = len(R)
    reach = [int(math.ceil(real_cutoff / np.linalg.norm(cell[d]))) + 1 for d in range(3)]
    e_real = 0.0
    for a in range(-reach[0], reach[0] + 1):
        for b in range(-reach[1], reach[1] + 1):
            for c in range(-reach[2], reach[2] + 1):
                shift = a * cell[0] + b * cell[1] + c * cell[2]
                d = R[None, :, :] + shift[None, None, :] - R[:, None, :]
                r = np.linalg.norm(d, axis=-1)
                m = (r > 1e-12) & (r < real_cutoff)
                qq = q[:, None] * q[None, :]
                e_real += 0.5 * np.sum(qq[m] * np.array([math.erfc(x / (math.sqrt(2.0) * smearing)) for x in r[m]]) / r[m])
    e_k = reciprocal_energy(torch.tensor(R), torch.tensor(q), torch.tensor(cell), shape, smearing).sum().item() / KE
    return e_real + e_k


# ----------------------------------------------------------------------------------------------------------
# mesh variant (smooth particle-mesh Ewald, Essmann et al., J. Chem. Phys. 103, 8577 (1995)), cubic B-splines = 4 nodes per axis
# (the reference's `coulomb_kspace_interp_nodes=4`, so3lr/potential.py:12; its own mesh code is in the absent jax-pme)
# ----------------------------------------------------------------------------------------------------------
def mesh_grid_shape(cell, mesh_spacing):
    """Power-of-two mesh with at most `mesh_spacing` (Angstrom) between points along each lattice vector."""
    cell = np.asarray(cell, dtype=np.float64)
    return tuple(int(2 ** max(2, math.ceil(math.log2(np.linalg.norm(cell[d]) / float(mesh_spacing)) - 1e-9))) for d in range(3))


def _bspline4(t):
    """Weights M4(t + j), j = 0..3, of the four mesh points m0 - j around a scaled coordinate m0 + t (t in [0, 1))."""
    return torch.stack([t ** 3 / 6, (-3 * t ** 3 + 3 * t ** 2 + 3 * t + 1) / 6, (3 * t ** 3 - 6 * t ** 2 + 4) / 6, (1 - t) ** 3 / 6], -1)


def reciprocal_energy_mesh(R, q, cell, shape, smearing):
    """Per-atom reciprocal-space energies with the structure factors interpolated on a mesh of the given shape.  Same
    arguments and per-atom bookkeeping as `reciprocal_energy`; converges to it as the mesh is refined."""
    dt = R.dtype
    n = [int(v) for v in shape]
    inv = torch.linalg.inv(cell)
    vol = torch.abs(torch.linalg.det(cell))
    f = R @ inv
    f = f - torch.floor(f).detach()
    u = f * torch.tensor(n, dtype=dt)
    m0 = torch.floor(u).detach()
    w = _bspline4(u - m0)                                            # (N, 3, 4)
    j = torch.arange(4)
    k = [(m0[:, d].long()[:, None] - j[None, :]) % n[d] for d in range(3)]
    idx = ((k[0][:, :, None, None] * n[1] + k[1][:, None, :, None]) * n[2] + k[2][:, None, None, :]).reshape(len(R), 64)
    w3 = (w[:, 0, :, None, None] * w[:, 1, None, :, None] * w[:, 2, None, None, :]).reshape(len(R), 64)
    Q = torch.zeros(n[0] * n[1] * n[2], dtype=dt).index_add(0, idx.reshape(-1), (q[:, None] * w3).reshape(-1)).reshape(n)
    Fq = torch.fft.fftn(Q)
    mm = [torch.as_tensor(np.rint(np.fft.fftfreq(nd, 1.0 / nd)), dtype=dt) for nd in n]
    h = torch.stack(torch.meshgrid(*mm, indexing="ij"), -1)           # (n1, n2, n3, 3) signed mesh frequencies
    kvec = 2 * math.pi * h @ inv.T
    k2 = (kvec * kvec).sum(-1)
    k2 = torch.where(k2 == 0, torch.ones_like(k2), k2)
    origin = torch.ones(n, dtype=dt); origin[0, 0, 0] = 0.0
    g = 4 * math.pi / k2 * torch.exp(-0.5 * smearing ** 2 * k2) * origin
    b = [9.0 / (2.0 + torch.cos(2 * math.pi * mm[d] / n[d])) ** 2 for d in range(3)]
    c = KE / vol * g * b[0][:, None, None] * b[1][None, :, None] * b[2][None, None, :]
    pot = torch.fft.ifftn(c * Fq).real * (n[0] * n[1] * n[2])          # unnormalised inverse transform
    phi = (w3 * pot.reshape(-1)[idx]).sum(-1)
    qtot = q.sum()
    return 0.5 * q * phi - KE * q * q / (math.sqrt(2 * math.pi) * smearing) - KE * math.pi * smearing ** 2 * q * qtot / vol
