"""CPU oracle for the reciprocal-space (Ewald) part of the electrostatic energy.  TEST INFRASTRUCTURE ONLY.

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
and caesium-chloride lattices as known answers.

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
