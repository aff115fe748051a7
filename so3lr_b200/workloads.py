"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark configurations
(periodic water boxes, batches of small organic molecules).  The reference measures on user-supplied structure
files; these generators stand in for them."""
from __future__ import annotations

import numpy as np

MASS = {1: 1.008, 6: 12.011, 7: 14.007, 8: 15.999, 16: 32.06}
KB_EV = 8.617333262e-5
# (eV / amu)^(1/2) in Angstrom / fs
_VEL_UNIT = 0.0982269478846


def _random_rotations(rng, n):
    q = rng.normal(size=(n, 4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    a, b, c, d = q.T
    return np.stack([np.stack([a * a + b * b - c * c - d * d, 2 * (b * c - a * d), 2 * (b * d + a * c)], -1),
                     np.stack([2 * (b * c + a * d), a * a - b * b + c * c - d * d, 2 * (c * d - a * b)], -1),
                     np.stack([2 * (b * d - a * c), 2 * (c * d + a * b), a * a - b * b - c * c + d * d], -1)], -2)


def water_box(n_molecules: int, box: float, seed: int, jitter: float = 0.05):
    """`n_molecules` rigid-geometry H2O (O-H 0.9572 A, H-O-H 104.52 deg) on a cubic grid in a cubic cell of edge `box`,
    each with a seeded uniform-random orientation, plus Gaussian jitter.  Returns Z (3n,), R (3n,3), cell (3,3).
    Atoms are ordered molecule by molecule along the grid (x fastest)."""
    rng = np.random.default_rng(seed)
    g = int(np.ceil(n_molecules ** (1.0 / 3.0) - 1e-9))
    while g ** 3 < n_molecules:
        g += 1
    sites = np.stack(np.meshgrid(np.arange(g), np.arange(g), np.arange(g), indexing="ij"), -1).reshape(-1, 3)
    sites = sites[:, ::-1]          # x fastest
    if g ** 3 > n_molecules:
        keep = np.sort(rng.choice(g ** 3, n_molecules, replace=False))
        sites = sites[keep]
    centres = (sites + 0.5) * (box / g)
    half = np.deg2rad(104.52) / 2
    mol = np.array([[0.0, 0.0, 0.0], [0.9572 * np.sin(half), 0.9572 * np.cos(half), 0.0],
                    [-0.9572 * np.sin(half), 0.9572 * np.cos(half), 0.0]])
    mol = mol - mol.mean(0)
    rot = _random_rotations(rng, n_molecules)
    R = centres[:, None, :] + np.einsum("nij,aj->nai", rot, mol)
    R = R + rng.normal(scale=jitter, size=R.shape)
    Z = np.tile(np.array([8, 1, 1], dtype=np.int32), n_molecules)
    return Z, R.reshape(-1, 3), np.eye(3) * box


def maxwell_boltzmann(Z, temperature: float, seed: int):
    """Velocities in Angstrom/fs at `temperature` K with zero total momentum."""
    rng = np.random.default_rng(seed)
    m = np.array([MASS[int(z)] for z in Z])
    v = rng.normal(size=(len(Z), 3)) * np.sqrt(KB_EV * temperature / m)[:, None] * _VEL_UNIT
    v -= (v * m[:, None]).sum(0) / m.sum()
    return v, m


def molecule(rng, n_atoms: int):
    """One neutral molecule of about `n_atoms` atoms: a self-avoiding random walk of C/N/O/S heavy atoms
    (0.70/0.12/0.15/0.03), bonds U(1.2,1.55) A, angles U(105,120) deg, capped with H at 1.09 A up to valence
    4/3/2/2 while the atom budget lasts."""
    valence = {6: 4, 7: 3, 8: 2, 16: 2}
    n_heavy = max(2, int(round(n_atoms / 2.6)))
    Zs, Rs, bonds = [], [], []
    for k in range(n_heavy):
        z = int(rng.choice([6, 7, 8, 16], p=[0.70, 0.12, 0.15, 0.03]))
        if 0 < k < n_heavy - 1 and valence[z] < 2:
            z = 6
        for _ in range(200):
            if k == 0:
                pos = np.zeros(3)
            else:
                b = rng.uniform(1.2, 1.55)
                if k == 1:
                    d = rng.normal(size=3)
                else:
                    prev = Rs[k - 1] - Rs[k - 2]
                    prev /= np.linalg.norm(prev)
                    ang = np.deg2rad(rng.uniform(105, 120))
                    perp = np.cross(prev, rng.normal(size=3))
                    perp /= np.linalg.norm(perp)
                    d = -np.cos(ang) * prev + np.sin(ang) * perp
                pos = Rs[k - 1] + b * d / np.linalg.norm(d)
            if all(np.linalg.norm(pos - r) > 1.9 for r in Rs[:-1]) or k < 2:
                break
        Zs.append(z)
        Rs.append(pos)
        bonds.append(0)
        if k > 0:
            bonds[k] += 1
            bonds[k - 1] += 1
    n_h = n_atoms - n_heavy
    heavy = list(range(n_heavy))
    Zh, Rh = [], []
    order = [k for k in heavy for _ in range(valence[Zs[k]])]
    rng.shuffle(order)
    for k in order:
        if n_h <= 0:
            break
        if bonds[k] >= valence[Zs[k]]:
            continue
        for _ in range(100):
            d = rng.normal(size=3)
            d /= np.linalg.norm(d)
            pos = Rs[k] + 1.09 * d
            others = [r for i, r in enumerate(Rs) if i != k] + Rh
            if all(np.linalg.norm(pos - r) > 1.5 for r in others):
                Zh.append(1)
                Rh.append(pos)
                bonds[k] += 1
                n_h -= 1
                break
    Z = np.array(Zs + Zh, dtype=np.int32)
    R = np.array(Rs + Rh)
    return Z, R - R.mean(0)


def molecule_batch(n_molecules: int, seed: int, lo: int = 10, hi: int = 40):
    """Concatenated batch of independent molecules; returns Z, R, graph_start (n_molecules + 1)."""
    rng = np.random.default_rng(seed)
    Zs, Rs, start = [], [], [0]
    for _ in range(n_molecules):
        Z, R = molecule(rng, int(rng.integers(lo, hi + 1)))
        Zs.append(Z)
        Rs.append(R)
        start.append(start[-1] + len(Z))
    return np.concatenate(Zs), np.concatenate(Rs), np.array(start, dtype=np.int32)
