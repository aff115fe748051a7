"""Seeded synthetic inputs with the shapes, sizes and value distributions of the benchmark configurations
(periodic water boxes, batches of small organic molecules).  The reference measures on user-supplied structure
files; these generators stand in for them."""
from __future__ import annotations

import numpy as np

MASS = {1: 1.008, 6: 12.011, 7: 14.007, 8: 15.999, 11: 22.990, 16: 32.06, 17: 35.45}
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


class _Hash:
    """Points in cubic bins of edge `h` for the overlap checks of the polymer builder."""

    def __init__(self, h):
        self.h, self.bins = h, {}

    def _key(self, p):
        return tuple(np.floor(p / self.h).astype(int))

    def add(self, p):
        self.bins.setdefault(self._key(p), []).append(p)

    def remove(self, p):
        b = self.bins[self._key(p)]
        for k, q in enumerate(b):
            if q is p:
                del b[k]
                return

    def clear_of(self, p, dmin, skip=()):
        k = self._key(p)
        for a in (-1, 0, 1):
            for b in (-1, 0, 1):
                for c in (-1, 0, 1):
                    for q in self.bins.get((k[0] + a, k[1] + b, k[2] + c), ()):
                        if any(q is s for s in skip):
                            continue
                        if np.dot(q - p, q - p) < dmin * dmin:
                            return False
        return True


def polymer(rng, n_atoms: int, bond: float = 1.5, angle_deg: float = 109.5, radius: float = 32.0):
    """A neutral H-capped random-walk polymer of about `n_atoms` atoms: a self-avoiding walk of C/N/O backbone atoms
    (0.70/0.15/0.15) with `bond` A bonds and `angle_deg` bond angles, kept inside a sphere of `radius` A around its start
    (a free walk of this length would not fit the box), capped with H at 1.09 A up to valence 4/3/2."""
    valence = {6: 4, 7: 3, 8: 2}
    n_heavy = int(round(n_atoms / 2.6))
    ang = np.deg2rad(angle_deg)
    grid = _Hash(2.0)
    Zs, Rs = [], []
    while len(Rs) < n_heavy:
        k = len(Rs)
        z = int(rng.choice([6, 7, 8], p=[0.70, 0.15, 0.15]))
        pos = None
        for _ in range(200):
            if k == 0:
                cand = np.zeros(3)
            elif k == 1:
                d = rng.normal(size=3)
                cand = Rs[0] + bond * d / np.linalg.norm(d)
            else:
                prev = Rs[k - 1] - Rs[k - 2]
                prev /= np.linalg.norm(prev)
                perp = np.cross(prev, rng.normal(size=3))
                perp /= np.linalg.norm(perp)
                cand = Rs[k - 1] + bond * (-np.cos(ang) * prev + np.sin(ang) * perp)
            if np.linalg.norm(cand) > radius:
                continue
            if k < 2 or grid.clear_of(cand, 1.9, skip=(Rs[k - 1],)):
                pos = cand
                break
        if pos is None:      # boxed in: take back the last few steps and walk on from there
            for _ in range(min(8, len(Rs) - 2)):
                grid.remove(Rs.pop())
                Zs.pop()
            continue
        Zs.append(z)
        Rs.append(pos)
        grid.add(pos)
    bonds = np.zeros(n_heavy, dtype=int)
    bonds[1:] += 1
    bonds[:-1] += 1
    n_h = n_atoms - n_heavy
    Zh, Rh = [], []
    order = [k for k in range(n_heavy) for _ in range(valence[Zs[k]])]
    rng.shuffle(order)
    for k in order:
        if n_h <= 0:
            break
        if bonds[k] >= valence[Zs[k]]:
            continue
        for _ in range(60):
            d = rng.normal(size=3)
            cand = Rs[k] + 1.09 * d / np.linalg.norm(d)
            if grid.clear_of(cand, 1.5, skip=(Rs[k],)):
                Zh.append(1)
                Rh.append(cand)
                grid.add(cand)
                bonds[k] += 1
                n_h -= 1
                break
    Z = np.array(Zs + Zh, dtype=np.int32)
    R = np.array(Rs + Rh)
    return Z, R - R.mean(0)


def solvated_polymer(box: float = 100.0, n_polymer_atoms: int = 5000, seed: int = 1003, salt_molar: float = 0.15, clearance: float = 2.5,
                     polymer_radius: float | None = None):
    """Synthetic solvated biopolymer: the polymer of `polymer` centred in a cubic water box of edge `box` at the density of
    `water_box`; waters with an atom within `clearance` A of a polymer atom are removed; then randomly chosen waters are replaced
    by Na+ / Cl- (at the oxygen position) at `salt_molar` mol/L.  Returns Z, R, cell; about 100,000 atoms for the defaults
    (elements H, C, N, O, Na, Cl; zero total charge)."""
    from scipy.spatial import cKDTree
    rng = np.random.default_rng(seed)
    if polymer_radius is None:
        polymer_radius = 0.32 * box
    Zp, Rp = polymer(rng, n_polymer_atoms, radius=polymer_radius)
    Rp = Rp + 0.5 * box
    n_water = int(round(333333 / 215.0 ** 3 * box ** 3))
    Zw, Rw, cell = water_box(n_water, box, seed + 17)
    Rw = Rw.reshape(n_water, 3, 3)
    tree = cKDTree(Rp)
    near = tree.query(Rw.reshape(-1, 3), distance_upper_bound=clearance)[0].reshape(n_water, 3)
    keep = ~np.isfinite(near).any(1)
    Rw = Rw[keep]
    n_pairs = int(round(salt_molar * 6.02214076e23 * box ** 3 * 1e-27))
    ions = rng.choice(len(Rw), 2 * n_pairs, replace=False)
    is_ion = np.zeros(len(Rw), dtype=bool)
    is_ion[ions] = True
    Zi = np.array([11] * n_pairs + [17] * n_pairs, dtype=np.int32)
    Ri = Rw[ions, 0, :]
    Rw = Rw[~is_ion]
    Z = np.concatenate([Zp, np.tile(np.array([8, 1, 1], dtype=np.int32), len(Rw)), Zi])
    R = np.concatenate([Rp, Rw.reshape(-1, 3), Ri])
    return Z, R, cell
