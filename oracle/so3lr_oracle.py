"""CPU oracle for the SO3LR energy + force path.  TEST INFRASTRUCTURE ONLY.

This file restates, in float64 torch on the CPU, the arithmetic that the reference package executes when
`potential(graph)` / `model.apply(params, inputs)` is called (so3lr/jaxmd_utils.py:130-141,
so3lr/base_calculator.py:57-122).  That arithmetic lives in the un-vendored dependency `mlff`
(git branch `v1.0_dev_import`, pinned in the reference's pyproject.toml:21), whose source is not part of the
reference tree; the restatement follows the published SO3krates / SO3LR method, the parameter tree
so3lr/params/params.pkl, so3lr/params/hyperparameters.yaml:130-166 and the in-repo call contracts
(so3lr/cli/tune_ewald.py:121-158 for dispersion, :893-927 for the Coulomb call).

Parity is PINNED: `tests/test_oracle_golden.py` checks this file against every golden vector of the
reference's own test-suite (tests/test_data/{atat,dha,bb,water}_{jaxmd,ase}.npz): energies agree to
<= 5e-5 eV absolute (2e-8 relative) and forces to <= 2e-6 eV/A on the float64 jax-md goldens.

Nothing in the product path may import this module; only tests, the smoke check and the CPU-baseline
leg of the benchmark do.
"""
from __future__ import annotations

import math
import os
from typing import Dict, Optional

import numpy as np
import torch

# ----------------------------------------------------------------------------------------------------------
# constants (hyperparameters.yaml:130-166 unless noted)
# ----------------------------------------------------------------------------------------------------------
NUM_LAYERS = 3
NUM_FEATURES = 128
NUM_HEADS = 4
HEAD_DIM = 32
DEGREES = (1, 2, 3, 4)
M_TOT = 24
NUM_RBF = 32
CUTOFF_SR = 4.5
AVG_NUM_NEIGHBORS = 13.168995780096482          # hyperparameters.yaml:2
# exponential-Bernstein decay constant; the reference holds it as a float32 number
RBF_GAMMA = float(np.float32(0.9448630629184640))
LN_EPS = 1e-6
KE = 14.399645351950548                         # so3lr/cli/tune_ewald.py:163
SIGMA_COULOMB = 4.0                             # electrostatic_energy_scale
CUTON_FRACTION = 0.45                           # so3lr/cli/tune_ewald.py:896
DISPERSION_SCALE = 1.2                          # dispersion_energy_scale
BOHR = 0.5291772105638411
HARTREE = 27.211386024367243
FINE_STRUCTURE = 0.0072973525693
ZBL_SWITCH_OFF = 1.5
# free-atom polarisabilities / C6 coefficients (atomic units), Z = 1..18
ALPHA_FREE = (4.5, 1.38, 164.2, 38.0, 21.0, 12.0, 7.4, 5.4, 3.8, 2.67, 162.7, 71.0, 60.0, 37.0, 25.0, 19.6, 15.0, 11.1)
C6_FREE = (6.5, 1.46, 1387.0, 214.0, 99.5, 46.6, 24.2, 15.6, 9.52, 6.38, 1556.0, 627.0, 528.0, 305.0, 185.0, 134.0, 94.6, 64.3)
GAMMA_CUBIC = (-0.00433008, 0.24428889, 0.04125273, -0.00078893)   # b0..b3 of the QDO width fit

_SEG = torch.tensor(sum([[i] * (2 * l + 1) for i, l in enumerate(DEGREES)], []))
_DTYPE = [torch.float64]


def set_dtype(dtype):
    """Arithmetic type of the oracle: torch.float64 (parity checks) or torch.float32 (CPU timing baseline)."""
    _DTYPE[0] = dtype


def _dt():
    return _DTYPE[0]


def _inv_w():
    return torch.tensor([1.0 / math.sqrt(2 * l + 1) for l in DEGREES], dtype=_dt())

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_BLOB = os.path.join(_HERE, "..", "so3lr_b200", "params", "so3lr_v1.npz")


def load_params(path: str = DEFAULT_BLOB) -> Dict[str, torch.Tensor]:
    """Flat blob -> {flax key path: float64 tensor}.  Key paths are those of so3lr/params/params.pkl."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "_pack_params", os.path.join(_HERE, "..", "so3lr_b200", "params", "pack_params.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    blob = np.load(path)["blob"]
    return {k: torch.tensor(v, dtype=_dt()) for k, v in mod.unpack(blob).items()}


# ----------------------------------------------------------------------------------------------------------
# neighbor lists (replaces jax_md.partition.neighbor_list as called at so3lr/jaxmd_utils.py:96-121)
# ----------------------------------------------------------------------------------------------------------
def min_image(dR: np.ndarray, cell: Optional[np.ndarray]) -> np.ndarray:
    """Minimum-image displacement for a cell whose ROWS are the lattice vectors.  float32 in, float32 out.
    k = rint(dR @ inv(cell)); dR = dR - k @ cell  (the same operation order as the CUDA kernels and as the float64 path of
    energy_forces: the lattice translation is subtracted from dR itself, which keeps dR's precision across the boundary)."""
    if cell is None:
        return dR
    cell = np.asarray(cell, dtype=np.float32)
    inv = np.linalg.inv(cell.astype(np.float64)).astype(np.float32)
    k = np.rint((dR[..., 0:1] * inv[0] + dR[..., 1:2] * inv[1]) + dR[..., 2:3] * inv[2])
    return dR - ((k[..., 0:1] * cell[0] + k[..., 1:2] * cell[1]) + k[..., 2:3] * cell[2])


def neighbor_list(R: np.ndarray, cell: Optional[np.ndarray], cutoff: float, ordered: bool = False, chunk: int = 512):
    """All pairs with |min_image(R_j - R_i)| < cutoff, self excluded, as (idx_i, idx_j) sorted by (i, j).
    `ordered=True` keeps i < j only (jax-md OrderedSparse, so3lr/jaxmd_utils.py:119); otherwise both
    directions (Sparse, :105).  Distances are evaluated in float32 exactly as the CUDA builder does:
    d2 = (dx*dx + dy*dy) + dz*dz, test d2 < cutoff*cutoff."""
    R = np.asarray(R, dtype=np.float32)
    n = len(R)
    rc2 = np.float32(cutoff) * np.float32(cutoff)
    I, J = [], []
    for s in range(0, n, chunk):
        d = R[None, :, :] - R[s:s + chunk, None, :]
        d = min_image(d, cell)
        d2 = (d[..., 0] * d[..., 0] + d[..., 1] * d[..., 1]) + d[..., 2] * d[..., 2]
        ii, jj = np.nonzero(d2 < rc2)
        ii = ii + s
        keep = (ii < jj) if ordered else (ii != jj)
        I.append(ii[keep])
        J.append(jj[keep])
    return np.concatenate(I).astype(np.int32), np.concatenate(J).astype(np.int32)


# ----------------------------------------------------------------------------------------------------------
# building blocks
# ----------------------------------------------------------------------------------------------------------
def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.nn.functional.softplus(x)


def dense(x, P, name):
    return x @ P[name + "/kernel"] + P[name + "/bias"]


def layer_norm(x, P, name):
    m = x.mean(-1, keepdim=True)
    v = ((x - m) ** 2).mean(-1, keepdim=True)
    return (x - m) / torch.sqrt(v + LN_EPS) * P[name + "/scale"] + P[name + "/bias"]


def bernstein_rbf(d):
    """32 exponential Bernstein polynomials b_k = C(31,k) x^k (1-x)^(31-k), x = exp(-gamma d)."""
    K = NUM_RBF
    k = torch.arange(K, dtype=_dt())
    logb = torch.tensor([math.lgamma(K) - math.lgamma(i + 1) - math.lgamma(K - i) for i in range(K)], dtype=_dt())
    ar = -RBF_GAMMA * d[:, None]
    return torch.exp(logb + k * ar + (K - 1 - k) * torch.log(-torch.expm1(ar)))


def phys_cutoff(d, rc=CUTOFF_SR):
    u = d / rc
    return torch.where(d < rc, 1 - 6 * u ** 5 + 15 * u ** 4 - 10 * u ** 3, torch.zeros_like(d))


def real_sph_harm(u):
    """Orthonormal real spherical harmonics l = 1..4 of unit vectors, (E, 24), m = -l..l inside each l."""
    x, y, z = u[:, 0], u[:, 1], u[:, 2]
    pi = math.pi
    s = math.sqrt
    o = []
    c1 = s(3 / (4 * pi))
    o += [c1 * y, c1 * z, c1 * x]
    o += [0.5 * s(15 / pi) * x * y, 0.5 * s(15 / pi) * y * z, 0.25 * s(5 / pi) * (3 * z * z - 1),
          0.5 * s(15 / pi) * x * z, 0.25 * s(15 / pi) * (x * x - y * y)]
    o += [0.25 * s(35 / (2 * pi)) * y * (3 * x * x - y * y), 0.5 * s(105 / pi) * x * y * z,
          0.25 * s(21 / (2 * pi)) * y * (5 * z * z - 1), 0.25 * s(7 / pi) * (5 * z ** 3 - 3 * z),
          0.25 * s(21 / (2 * pi)) * x * (5 * z * z - 1), 0.25 * s(105 / pi) * (x * x - y * y) * z,
          0.25 * s(35 / (2 * pi)) * x * (x * x - 3 * y * y)]
    o += [0.75 * s(35 / pi) * x * y * (x * x - y * y), 0.75 * s(35 / (2 * pi)) * y * z * (3 * x * x - y * y),
          0.75 * s(5 / pi) * x * y * (7 * z * z - 1), 0.75 * s(5 / (2 * pi)) * y * z * (7 * z * z - 3),
          (3 / 16) * s(1 / pi) * (35 * z ** 4 - 30 * z * z + 3), 0.75 * s(5 / (2 * pi)) * x * z * (7 * z * z - 3),
          (3 / 8) * s(5 / pi) * (x * x - y * y) * (7 * z * z - 1), 0.75 * s(35 / (2 * pi)) * x * z * (x * x - 3 * y * y),
          (3 / 16) * s(35 / pi) * (x * x * (x * x - 3 * y * y) - y * y * (3 * x * x - y * y))]
    return torch.stack(o, -1)


def degree_invariants(ev):
    """Per-degree contraction to l=0: sum_m chi_lm^2 / sqrt(2l+1), (n, 24) -> (n, 4)."""
    out = torch.zeros(ev.shape[0], 4, dtype=ev.dtype)
    return out.index_add(1, _SEG, ev * ev) * _inv_w()


def _smooth_sigma(x):
    safe = torch.where(x > 0, x, torch.ones_like(x))
    return torch.where(x > 0, torch.exp(-1.0 / safe), torch.zeros_like(x))


def switching_fn(x, x_on, x_off):
    """1 for x <= x_on, 0 for x >= x_off, C-infinity in between."""
    c = (x - x_on) / (x_off - x_on)
    return _smooth_sigma(1 - c) / (_smooth_sigma(1 - c) + _smooth_sigma(c))


# ----------------------------------------------------------------------------------------------------------
# the network
# ----------------------------------------------------------------------------------------------------------
def charge_spin_embed(P, prefix, Z, psi, batch_segments, num_graphs):
    """Charge / spin embedding (feature_embeddings_{1,2}); identically zero for psi = 0."""
    p = prefix + "/ChargeSpinEmbedSparse_0/"
    q = P[p + "Embed_0/embedding"][Z]
    idx = (psi < 0).long()
    k = P[p + "Embed_1/embedding"][idx][batch_segments]
    v = P[p + "Embed_2/embedding"][idx][batch_segments]
    y = softplus((q * k).sum(-1) / math.sqrt(NUM_FEATURES))
    den = torch.zeros(num_graphs, dtype=y.dtype).index_add(0, batch_segments, y)
    a = psi[batch_segments] * y / den[batch_segments]
    e = a[:, None] * v
    # bias-free pre-activation residual block
    t = silu(e) @ P[p + "Residual_0/layers_0/kernel"]
    t = silu(t) @ P[p + "Residual_0/layers_1/kernel"]
    return e + t


def so3krates_layer(P, l, x, ev, rbf, Y, cut, idx_i, idx_j, record=None):
    N = x.shape[0]
    a = f"layers_{l}/attention_block/"
    w1 = dense(silu(dense(rbf, P, a + "radial_filter1_layer_1")), P, a + "radial_filter1_layer_2")
    w2 = dense(silu(dense(rbf, P, a + "radial_filter2_layer_1")), P, a + "radial_filter2_layer_2")
    s = degree_invariants(ev[idx_j] - ev[idx_i])
    w1 = w1 + dense(silu(dense(s, P, a + "spherical_filter1_layer_1")), P, a + "spherical_filter1_layer_2")
    w2 = w2 + dense(silu(dense(s, P, a + "spherical_filter2_layer_1")), P, a + "spherical_filter2_layer_2")
    xh = x.reshape(N, NUM_HEADS, HEAD_DIM)

    def proj(name):
        return torch.einsum("hij,nhj->nhi", P[a + name], xh)

    q1, k1, v1, q2, k2 = proj("Wq1"), proj("Wk1"), proj("Wv1"), proj("Wq2"), proj("Wk2")
    scale = (cut / AVG_NUM_NEIGHBORS)[:, None]
    a1 = (q1[idx_i] * w1.reshape(-1, 4, 32) * k1[idx_j]).sum(-1) * scale
    a2 = (q2[idx_i] * w2.reshape(-1, 4, 32) * k2[idx_j]).sum(-1) * scale
    x_att = torch.zeros(N, 4, 32, dtype=x.dtype).index_add(0, idx_i, a1[:, :, None] * v1[idx_j]).reshape(N, 128)
    ev_att = torch.zeros(N, M_TOT, dtype=x.dtype).index_add(0, idx_i, a2[:, _SEG] * Y)
    xa = x + x_att
    ev1 = ev + ev_att
    x1 = layer_norm(xa, P, f"layers_{l}/layer_normalization_1")
    y = dense(silu(dense(silu(x1), P, f"layers_{l}/res_mlp_1_layer_1")), P, f"layers_{l}/res_mlp_1_layer_2")
    x2 = x1 + y
    yx = dense(torch.cat([x2, degree_invariants(ev1)], -1), P, f"layers_{l}/exchange_block/mlp_layer_2")
    x3 = x2 + yx[:, :128]
    ev2 = ev1 + yx[:, 128:][:, _SEG] * ev1
    x4 = layer_norm(x3, P, f"layers_{l}/layer_normalization_2")
    if record is not None:
        record[f"l{l}_q1"] = q1.reshape(N, 128); record[f"l{l}_k1"] = k1.reshape(N, 128)
        record[f"l{l}_v1"] = v1.reshape(N, 128); record[f"l{l}_q2"] = q2.reshape(N, 128)
        record[f"l{l}_k2"] = k2.reshape(N, 128)
        record[f"l{l}_xa"] = xa; record[f"l{l}_ev1"] = ev1; record[f"l{l}_x2"] = x2
        record[f"l{l}_x3"] = x3; record[f"l{l}_x4"] = x4; record[f"l{l}_ev2"] = ev2
    return x4, ev2


def zbl_energy(P, Zf, d, cut, idx_i, N):
    z = "observables_0/zbl_repulsion/"
    a = [softplus(P[z + f"a{k}"])[0] for k in range(1, 5)]
    c = [softplus(P[z + f"c{k}"])[0] for k in range(1, 5)]
    csum = sum(c)
    c = [ck / csum for ck in c]
    p = softplus(P[z + "p"])[0]
    dd = softplus(P[z + "d"])[0]
    return a, c, p, dd


def coulomb_pair(d, cutoff_lr, k_smearing=None):
    """erf-damped Coulomb kernel chi(r) (without ke q_i q_j).  With a cutoff: potential-shifted below the
    switch-on radius, blended smoothly into the force-shifted form towards the cutoff, zero beyond.
    With `k_smearing` s the part erf(r / (sqrt(2) s)) / r, which the reciprocal-space sum holds, is taken out of the
    pair function before it is shifted and blended (the role of `coulomb_erf_shifted_force_smooth_pme`,
    so3lr/cli/tune_ewald.py:612-614; its exact blending is in the absent mlff source, so this form is unpinned)."""
    sig = SIGMA_COULOMB
    a = None if k_smearing is None else 1.0 / (math.sqrt(2.0) * float(k_smearing))

    def pot(r):
        v = torch.erf(r / sig) / r
        return v if a is None else v - torch.erf(r * a) / r

    if cutoff_lr is None:
        return pot(d)
    rc = torch.tensor(float(cutoff_lr), dtype=d.dtype)

    def dpot(r):
        v = (2 * r * torch.exp(-(r / sig) ** 2) / (math.sqrt(math.pi) * sig) - torch.erf(r / sig)) / r ** 2
        if a is not None:
            v = v - (2 * r * a * torch.exp(-(r * a) ** 2) / math.sqrt(math.pi) - torch.erf(r * a)) / r ** 2
        return v

    f = switching_fn(d, CUTON_FRACTION * cutoff_lr, cutoff_lr)
    shifted = pot(d) - pot(rc)
    chi = f * shifted + (1 - f) * (shifted - dpot(rc) * (d - rc))
    return torch.where(d < rc, chi, torch.zeros_like(chi))


def dispersion_pair(d, Zi, Zj, hi, hj, cutoff_lr, damping):
    """QDO-damped C6/C8/C10 pair dispersion in eV (so3lr/cli/tune_ewald.py:121-158)."""
    alpha = torch.tensor(ALPHA_FREE, dtype=d.dtype)
    c6 = torch.tensor(C6_FREE, dtype=d.dtype)
    ai, aj = alpha[Zi - 1] * hi, alpha[Zj - 1] * hj
    ci, cj = c6[Zi - 1] * hi * hi, c6[Zj - 1] * hj * hj
    a_ij = (ai + aj) / 2
    c6_ij = 2 * ci * cj * aj * ai / (ai ** 2 * cj + aj ** 2 * ci)
    b0, b1, b2, b3 = GAMMA_CUBIC
    rv = FINE_STRUCTURE ** (-4.0 / 21) * a_ij ** (1.0 / 7)
    sg = b3 * rv ** 3 + b2 * rv ** 2 + b1 * rv + b0
    gam = 0.5 / sg ** 2
    Rb = d / BOHR
    c8 = 5 / gam * c6_ij
    c10 = 245 / 8 / gam ** 2 * c6_ij
    p = DISPERSION_SCALE * 2 * 2.54 * a_ij ** (1.0 / 7)
    e = -c6_ij / (Rb ** 6 + p ** 6) - c8 / (Rb ** 8 + p ** 8) - c10 / (Rb ** 10 + p ** 10)
    e = e * HARTREE
    if cutoff_lr is not None and damping is not None:
        e = e * switching_fn(d, cutoff_lr - damping, cutoff_lr)
    return e


def energy_from_graph(P, Z, dR, idx_i, idx_j, dR_lr, idx_i_lr, idx_j_lr, *, lr_format="ordered_sparse",
                      cutoff_lr: Optional[float] = 12.0, damping: Optional[float] = 2.0,
                      total_charge=None, num_unpaired=None, batch_segments=None, num_graphs=1, record=None, kspace=None):
    """Per-atom energies and auxiliary outputs from the Graph-level inputs of so3lr/graph.py:3-24.

    `kspace` = dict(positions (N,3), cell (3,3), grid (n1,n2,n3), smearing, method 'ewald' | 'pme') switches the Coulomb term to the
    real-space + reciprocal-space split of oracle/kspace_oracle.py (Graph fields positions, cell, k_grid, k_smearing).

    dR (E,3) displacement of each short-range edge (idx_i = centre, idx_j = neighbour), dR_lr (P,3) of each
    long-range pair.  `lr_format`: 'ordered_sparse' (each pair once, so3lr/potential.py:22) or 'sparse'
    (both directions, energy halved, so3lr/base_calculator.py:31).  Edges whose endpoint index is >= N or
    whose length is 0 are padding and contribute nothing (so3lr/jaxmd_utils.py:12-21 pads with N).
    """
    N = len(Z)
    Z = torch.as_tensor(np.asarray(Z).astype(np.int64))
    idx_i = torch.as_tensor(np.asarray(idx_i).astype(np.int64)); idx_j = torch.as_tensor(np.asarray(idx_j).astype(np.int64))
    idx_i_lr = torch.as_tensor(np.asarray(idx_i_lr).astype(np.int64)); idx_j_lr = torch.as_tensor(np.asarray(idx_j_lr).astype(np.int64))
    if batch_segments is None:
        batch_segments = torch.zeros(N, dtype=torch.int64)
    else:
        batch_segments = torch.as_tensor(np.asarray(batch_segments).astype(np.int64))
    tq = torch.zeros(num_graphs, dtype=_dt()) if total_charge is None else torch.as_tensor(total_charge, dtype=_dt()).reshape(-1)
    ts = torch.zeros(num_graphs, dtype=_dt()) if num_unpaired is None else torch.as_tensor(num_unpaired, dtype=_dt()).reshape(-1)

    # drop padding
    d_all = dR.norm(dim=-1)
    keep = (idx_i < N) & (idx_j < N) & (d_all > 0) & (d_all < CUTOFF_SR)
    dR, idx_i, idx_j = dR[keep], idx_i[keep], idx_j[keep]
    d = dR.norm(dim=-1)
    u = dR / d[:, None]
    rbf = bernstein_rbf(d)
    cut = phys_cutoff(d)
    Y = real_sph_harm(u)

    x = P["feature_embeddings_0/Embed_0/embedding"][Z]
    x = x + charge_spin_embed(P, "feature_embeddings_1", Z, tq, batch_segments, num_graphs)
    x = x + charge_spin_embed(P, "feature_embeddings_2", Z, ts, batch_segments, num_graphs)
    x = x / math.sqrt(3.0)
    ev = torch.zeros(N, M_TOT, dtype=_dt())
    if record is not None:
        record["x0"] = x
    for l in range(NUM_LAYERS):
        x, ev = so3krates_layer(P, l, x, ev, rbf, Y, cut, idx_i, idx_j, record)

    o = "observables_0/"
    e_nn = dense(silu(dense(x, P, o + "energy_dense_regression")), P, o + "energy_dense_final")[:, 0]
    e_nn = e_nn * P[o + "atomic_scales"][Z] + P[o + "energy_offset"][Z]

    # ZBL repulsion on the short-range edges
    a, c, p, dd = zbl_energy(P, None, None, None, None, None)
    zi, zj = Z[idx_i].to(_dt()), Z[idx_j].to(_dt())
    rzd = d * (zi ** p + zj ** p) * dd
    phi = sum(ck * torch.exp(-ak * rzd) for ak, ck in zip(a, c))
    e_zbl_edge = 0.5 * KE * cut * zi * zj / d * phi * switching_fn(d, 0.0, ZBL_SWITCH_OFF)
    e_zbl = torch.zeros(N, dtype=_dt()).index_add(0, idx_i, e_zbl_edge)

    # partial charges with per-graph charge conservation
    pc = o + "electrostatic_energy/partial_charges/"
    qt = P[pc + "Embed_0/embedding"][Z][:, 0] + dense(silu(dense(x, P, pc + "charge_dense_regression_vec")), P, pc + "charge_dense_final_vec")[:, 0]
    qsum = torch.zeros(num_graphs, dtype=_dt()).index_add(0, batch_segments, qt)
    cnt = torch.zeros(num_graphs, dtype=_dt()).index_add(0, batch_segments, torch.ones(N, dtype=_dt()))
    q = qt + ((tq - qsum) / cnt.clamp(min=1))[batch_segments]

    # Hirshfeld ratios
    h_ = "observables_2/"
    kk = dense(silu(dense(x, P, h_ + "hirshfeld_ratios_dense_regression")), P, h_ + "hirshfeld_ratios_dense_final")
    hr = torch.abs(P[h_ + "Embed_0/embedding"][Z][:, 0] + (P[h_ + "Embed_1/embedding"][Z] * kk).sum(-1) / math.sqrt(64.0))

    # long-range pair terms
    dl_all = dR_lr.norm(dim=-1)
    keep = (idx_i_lr < N) & (idx_j_lr < N) & (dl_all > 0)
    dl, il, jl = dl_all[keep], idx_i_lr[keep], idx_j_lr[keep]
    fac = 0.5 if lr_format == "sparse" else 1.0
    e_c_pair = fac * KE * q[il] * q[jl] * coulomb_pair(dl, cutoff_lr, None if kspace is None else kspace["smearing"])
    e_d_pair = fac * dispersion_pair(dl, Z[il], Z[jl], hr[il], hr[jl], cutoff_lr, damping)
    if cutoff_lr is not None:
        e_d_pair = torch.where(dl < cutoff_lr, e_d_pair, torch.zeros_like(e_d_pair))
    e_c = torch.zeros(N, dtype=_dt()).index_add(0, il, e_c_pair)
    e_d = torch.zeros(N, dtype=_dt()).index_add(0, il, e_d_pair)
    if kspace is not None:
        from oracle.kspace_oracle import reciprocal_energy, reciprocal_energy_mesh
        fn = reciprocal_energy_mesh if kspace.get("method", "ewald") == "pme" else reciprocal_energy
        e_c = e_c + fn(kspace["positions"], q, kspace["cell"], kspace["grid"], float(kspace["smearing"]))

    e_atom = e_nn + e_zbl + e_c + e_d
    aux = dict(partial_charges=q, hirshfeld_ratios=hr, zbl_repulsion=e_zbl, electrostatic_energy=e_c,
               dispersion_energy=e_d, e_nn=e_nn, x_final=x, batch_segments=batch_segments)
    return e_atom, aux


def energy_forces(P, R, Z, cell=None, *, cutoff_lr: Optional[float] = 12.0, damping: Optional[float] = 2.0,
                  lr_format="ordered_sparse", lr_neighbor_cutoff: Optional[float] = None, total_charge=None,
                  num_unpaired=None, batch_segments=None, num_graphs=1, record=None, lists=None, k_grid=None,
                  k_smearing=None, k_method="ewald"):
    """Positions -> total energy, forces and aux outputs, the composition used by
    so3lr/jaxmd_utils.py:130-141 + jax_md.quantity.force and by so3lr/base_calculator.py:95-122.

    R (N,3) Cartesian in Angstrom, cell None (free space) or 3x3 with lattice vectors as rows.
    Neighbor lists are built here (short range 4.5 A, long range `cutoff_lr`) unless `lists` provides
    (idx_i, idx_j, idx_i_lr, idx_j_lr).  For several graphs pass `batch_segments`; lists are then
    restricted to pairs inside one graph.  `k_grid` (an index-grid shape or an array of that shape) and `k_smearing`
    switch on the reciprocal-space Coulomb part (one periodic structure); `k_method` 'ewald' sums over the index grid,
    'pme' interpolates on a mesh of that shape.
    """
    R = np.asarray(R, dtype=np.float64)
    N = len(R)
    if lists is None:
        rl = lr_neighbor_cutoff if lr_neighbor_cutoff is not None else cutoff_lr
        idx_i, idx_j = neighbor_list(R, cell, CUTOFF_SR, ordered=False)
        idx_i_lr, idx_j_lr = neighbor_list(R, cell, rl, ordered=(lr_format == "ordered_sparse"))
        if batch_segments is not None:
            bs = np.asarray(batch_segments)
            m = bs[idx_i] == bs[idx_j]; idx_i, idx_j = idx_i[m], idx_j[m]
            m = bs[idx_i_lr] == bs[idx_j_lr]; idx_i_lr, idx_j_lr = idx_i_lr[m], idx_j_lr[m]
    else:
        idx_i, idx_j, idx_i_lr, idx_j_lr = lists
    Rt = torch.tensor(R, dtype=_dt(), requires_grad=True)
    # homogeneous strain r -> (1 + eps) r applied to every displacement (the `perturbation` of so3lr/jaxmd_utils.py:48-51);
    # dE/d eps at eps = 0 is the virial, stress = virial / volume
    eps = torch.zeros(3, 3, dtype=_dt(), requires_grad=True)
    ii, jj = torch.as_tensor(idx_i.astype(np.int64)), torch.as_tensor(idx_j.astype(np.int64))
    il, jl = torch.as_tensor(idx_i_lr.astype(np.int64)), torch.as_tensor(idx_j_lr.astype(np.int64))

    def disp(a, b):
        dR = Rt[b] - Rt[a]
        if cell is not None:
            c = torch.tensor(np.asarray(cell, dtype=np.float64), dtype=_dt())
            s = dR.detach() @ torch.linalg.inv(c)
            dR = dR - torch.round(s) @ c
        return dR + dR @ eps.T

    kspace = None
    if k_grid is not None:
        c0 = torch.tensor(np.asarray(cell, dtype=np.float64), dtype=_dt())
        shape = tuple(int(v) for v in (k_grid.shape if hasattr(k_grid, "shape") else k_grid))
        kspace = dict(positions=Rt + Rt @ eps.T, cell=c0 + c0 @ eps.T, grid=shape, smearing=float(np.asarray(k_smearing).reshape(-1)[0]),
                      method=k_method)
    e_atom, aux = energy_from_graph(P, Z, disp(ii, jj), idx_i, idx_j, disp(il, jl), idx_i_lr, idx_j_lr,
                                    lr_format=lr_format, cutoff_lr=cutoff_lr, damping=damping,
                                    total_charge=total_charge, num_unpaired=num_unpaired,
                                    batch_segments=batch_segments, num_graphs=num_graphs, record=record, kspace=kspace)
    E = e_atom.sum()
    gR, gE = torch.autograd.grad(E, (Rt, eps))
    F = -gR
    bs = aux["batch_segments"]
    q = aux["partial_charges"].detach()
    dip = torch.zeros(num_graphs, 3, dtype=_dt()).index_add(0, bs, q[:, None] * Rt.detach())
    e_graph = torch.zeros(num_graphs, dtype=_dt()).index_add(0, bs, e_atom.detach())
    out = dict(energy=E.item(), energy_per_graph=e_graph.numpy(), forces=F.numpy(), e_atom=e_atom.detach().numpy(),
               partial_charges=q.numpy(), hirshfeld_ratios=aux["hirshfeld_ratios"].detach().numpy(),
               dipole_vec=dip.numpy(), zbl_repulsion=aux["zbl_repulsion"].detach().numpy(),
               electrostatic_energy=aux["electrostatic_energy"].detach().numpy(),
               dispersion_energy=aux["dispersion_energy"].detach().numpy(),
               num_edges=len(idx_i), num_pairs=len(idx_i_lr), virial=gE.numpy())
    return out


# ----------------------------------------------------------------------------------------------------------
# small readers used by the tests (the reference uses ase.io.read, tests/test_jaxmd.py:35)
# ----------------------------------------------------------------------------------------------------------
_SYMBOLS = {"H": 1, "C": 6, "N": 7, "O": 8, "F": 9, "P": 15, "S": 16, "Cl": 17}


def read_xyz(path):
    lines = open(path).read().split("\n")
    n = int(lines[0])
    import re
    m = re.search(r'Lattice="([^"]+)"', lines[1])
    cell = np.array([float(v) for v in m.group(1).split()]).reshape(3, 3) if m else None
    Z, R = [], []
    for ln in lines[2:2 + n]:
        s = ln.split()
        Z.append(_SYMBOLS[s[0]])
        R.append([float(v) for v in s[1:4]])
    return np.array(Z, dtype=np.int32), np.array(R, dtype=np.float64), cell
