"""Host-callable pieces of the device math (same source as the kernels) against the CPU oracle. No GPU needed."""
import ctypes as C
import math

import numpy as np
import pytest
import torch

from oracle import so3lr_oracle as O

from so3lr_b200 import _lib
lib = _lib.lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def test_library_exports_every_declared_symbol():
    import os, re
    hdr = open(os.path.join(os.path.dirname(__file__), "..", "include", "so3lr_b200.h")).read()
    declared = set(re.findall(r"\b(so3lr_b200_[a-z0-9_]+)\s*\(", hdr))
    declared -= {"so3lr_b200_model", "so3lr_b200_system", "so3lr_b200_options"}
    assert declared, "no declarations parsed"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/so3lr_b200.h but not exported"
    assert lib.so3lr_b200_version() >= 100


def test_spherical_harmonics_and_vjp():
    rng = np.random.default_rng(0)
    for _ in range(20):
        v = rng.normal(size=3); v /= np.linalg.norm(v)
        y = np.zeros(24, np.float32)
        lib.so3lr_b200_host_sph_harm(*[float(c) for c in v], _p(y))
        u = torch.tensor(v[None], dtype=torch.float64, requires_grad=True)
        yt = O.real_sph_harm(u)[0]
        np.testing.assert_allclose(y, yt.detach().numpy(), atol=3e-6)
        g = rng.normal(size=24).astype(np.float32)
        g3 = np.zeros(3, np.float32)
        lib.so3lr_b200_host_sph_harm_vjp(*[float(c) for c in v], _p(g), _p(g3))
        (yt * torch.tensor(g, dtype=torch.float64)).sum().backward()
        np.testing.assert_allclose(g3, u.grad[0].numpy(), atol=2e-5)
    # per-degree norm of orthonormal harmonics: sum_m Y_lm^2 = (2l+1)/(4 pi)
    s = [float((y[a:b] ** 2).sum()) for a, b in ((0, 3), (3, 8), (8, 15), (15, 24))]
    np.testing.assert_allclose(s, [(2 * l + 1) / (4 * math.pi) for l in (1, 2, 3, 4)], rtol=1e-5)


@pytest.mark.parametrize("cutoff,damping", [(12.0, 2.0), (-1.0, -1.0), (1000.0, 2.0)])
def test_pair_terms_match_oracle(cutoff, damping):
    rng = np.random.default_rng(1)
    for _ in range(40):
        r = float(rng.uniform(0.8, 11.9))
        zi, zj = (int(z) for z in rng.choice([1, 6, 7, 8, 9, 15, 16, 17], 2))
        qi, qj = (float(v) for v in rng.normal(0, 0.4, 2))
        hi, hj = (float(v) for v in rng.uniform(0.5, 1.1, 2))
        out = np.zeros(8, np.float32)
        lib.so3lr_b200_host_pair_terms(r, zi, zj, qi, qj, hi, hj, cutoff, damping, _p(out))
        rt = torch.tensor([r], dtype=torch.float64, requires_grad=True)
        ht = torch.tensor([hi, hj], dtype=torch.float64, requires_grad=True)
        cl = cutoff if cutoff > 0 else None
        dm = damping if damping > 0 else None
        ec = O.KE * qi * qj * O.coulomb_pair(rt, cl)[0]
        ed = O.dispersion_pair(rt, torch.tensor([zi]), torch.tensor([zj]), ht[0:1], ht[1:2], cl, dm)[0]
        dec, = torch.autograd.grad(ec, rt, retain_graph=True)
        ded_r, ded_h = torch.autograd.grad(ed, [rt, ht])
        np.testing.assert_allclose(out[0], ec.item(), rtol=2e-5, atol=2e-6)
        np.testing.assert_allclose(out[1], dec.item(), rtol=1e-4, atol=2e-6)
        np.testing.assert_allclose(out[3], ed.item(), rtol=5e-5, atol=1e-7)
        np.testing.assert_allclose(out[4], ded_r.item(), rtol=2e-4, atol=1e-7)
        np.testing.assert_allclose(out[5:7], ded_h.numpy(), rtol=2e-4, atol=1e-7)
        # the hand-derived form the pair kernels use
        o4 = np.zeros(4, np.float32)
        lib.so3lr_b200_host_dispersion_fast(r, zi, zj, hi, hj, cutoff, damping, _p(o4))
        np.testing.assert_allclose(o4[0], ed.item(), rtol=5e-5, atol=1e-7)
        np.testing.assert_allclose(o4[1], ded_r.item(), rtol=2e-4, atol=1e-7)
        np.testing.assert_allclose(o4[2:4], ded_h.numpy(), rtol=2e-4, atol=1e-7)


def test_zbl_matches_oracle(oracle_params):
    blob = np.load(O.DEFAULT_BLOB)["blob"].astype(np.float32)
    a, c, p, dd = O.zbl_energy(oracle_params, None, None, None, None, None)
    for r in (0.3, 0.7, 0.96, 1.09, 1.3, 1.49, 1.6):
        for zi, zj in ((8, 1), (6, 6), (1, 1), (17, 6)):
            out = np.zeros(2, np.float32)
            lib.so3lr_b200_host_zbl(_p(blob), r, zi, zj, _p(out))
            d = torch.tensor([r], dtype=torch.float64, requires_grad=True)
            rzd = d * (zi ** p + zj ** p) * dd
            phi = sum(ck * torch.exp(-ak * rzd) for ak, ck in zip(a, c))
            e = (0.5 * O.KE * O.phys_cutoff(d) * zi * zj / d * phi * O.switching_fn(d, 0.0, O.ZBL_SWITCH_OFF))[0]
            de, = torch.autograd.grad(e, d)
            np.testing.assert_allclose(out[0], e.item(), rtol=3e-5, atol=1e-6)
            np.testing.assert_allclose(out[1], de.item(), rtol=2e-4, atol=2e-5)


def test_radial_filter_table_function(oracle_params):
    """The tabulated radial filter (+ folded spherical-filter constants) equals the direct evaluation."""
    blob = np.load(O.DEFAULT_BLOB)["blob"].astype(np.float32)
    P = oracle_params
    for layer in range(3):
        for r in (0.5, 0.96, 1.5, 2.7, 4.2):
            w = np.zeros(256); dw = np.zeros(256)
            lib.so3lr_b200_host_radial_filter(_p(blob), layer, r, _p(w), _p(dw))
            d = torch.tensor([r], dtype=torch.float64, requires_grad=True)
            rbf = O.bernstein_rbf(d)
            a = f"layers_{layer}/attention_block/"
            ws = []
            for f in (1, 2):
                wr = O.dense(O.silu(O.dense(rbf, P, a + f"radial_filter{f}_layer_1")), P, a + f"radial_filter{f}_layer_2")[0]
                wr = wr + P[a + f"spherical_filter{f}_layer_2/bias"]
                if layer == 0:
                    wr = wr + O.silu(P[a + f"spherical_filter{f}_layer_1/bias"]) @ P[a + f"spherical_filter{f}_layer_2/kernel"]
                ws.append(wr)
            wt = torch.cat(ws)
            np.testing.assert_allclose(w, wt.detach().numpy(), atol=1e-9)
            g = torch.autograd.grad(wt[7] + wt[200], d)[0].item()
            np.testing.assert_allclose(dw[7] + dw[200], g, rtol=1e-8, atol=1e-9)


def test_radial_filter_chebyshev_expansion():
    """The 64-term Chebyshev expansion that the tiled attention kernels contract on the tensor cores reproduces the radial
    filters and their r-derivatives over the whole cutoff range (largest |w| is 6-12, largest |dw/dr| 28-51)."""
    blob = np.load(O.DEFAULT_BLOB)["blob"].astype(np.float32)
    for layer in (1, 2):
        worst = worst_d = 0.0
        for r in np.concatenate([np.linspace(0.02, 4.49, 60), [0.9572, 1.09, 1.5139, 2.76]]):
            w = np.zeros(256); dw = np.zeros(256); wc = np.zeros(256); dwc = np.zeros(256)
            lib.so3lr_b200_host_radial_filter(_p(blob), layer, float(r), _p(w), _p(dw))
            lib.so3lr_b200_host_radial_filter_chebyshev(_p(blob), layer, float(r), _p(wc), _p(dwc))
            worst = max(worst, np.abs(w - wc).max())
            worst_d = max(worst_d, np.abs(dw - dwc).max())
        assert worst < 1e-6, (layer, worst)
        assert worst_d < 5e-4, (layer, worst_d)


@pytest.mark.parametrize("smearing", [0.0, 1.0, 2.4])
def test_coulomb_pair_function_with_the_reciprocal_part_taken_out_matches_oracle(smearing):
    """The pair function the long-range kernels evaluate when the Ewald sum is on (smearing > 0), value and slope."""
    out = np.zeros(2, dtype=np.float32)
    for cutoff in (6.0, 12.0):
        for r in (0.9, 2.3, 4.0, 5.5, 5.99, 7.7, 11.2):
            lib.so3lr_b200_host_coulomb_chi(r, cutoff, smearing, _p(out))
            rt = torch.tensor([r], dtype=torch.float64, requires_grad=True)
            chi = O.coulomb_pair(rt, cutoff, smearing if smearing > 0 else None)[0]
            (dchi,) = torch.autograd.grad(chi, rt)
            assert abs(out[0] - chi.item()) < 2e-7 + 2e-6 * abs(chi.item()), (cutoff, r, out[0], chi.item())
            assert abs(out[1] - dchi.item()) < 2e-7 + 5e-6 * abs(dchi.item()), (cutoff, r, out[1], dchi.item())


@pytest.mark.parametrize("shape", [(1, 1, 2), (4, 5, 1), (16, 16, 16), (17, 33, 64), (21, 20, 19), (52, 52, 52), (83, 83, 83), (3, 130, 7)])
def test_ewald_tiles_count_every_index_once(shape):
    """Half of the index grid is kept (one member of every pair (k, -k) with weight 2, unpaired indices of even extents with
    weight 1): the weights must add up to the number of non-zero index triples, the groups of the structure-factor kernel must
    cover every tile exactly once with runs of at most four adjacent tiles, and the row masks must agree with the weights."""
    counts = np.zeros(4, dtype=np.int64)
    wsum = C.c_double()
    assert lib.so3lr_b200_host_kspace_tiles(*shape, _p(counts), C.byref(wsum)) == 0
    n1, n2, n3 = shape
    assert wsum.value == n1 * n2 * n3 - 1
    assert counts[3] == 0 and 1 <= counts[2] <= 4 and counts[1] <= counts[0]
    assert counts[0] * 256 >= (n1 * n2 * n3 - 1) / 2
