"""Domain-decomposed evaluation (so3lr_b200_dd_* through so3lr_b200.domain) against the single-device evaluation.

The ranks run as threads on one GPU (ThreadWorld): the driver code, the halo plans and the three library phases are
exactly those of a multi-GPU run; only the transport differs (tensors are handed over in memory instead of NCCL).
Tolerances: energy 1e-5 relative, forces 1e-4 eV/A.
"""
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_threads(world, fn):
    from so3lr_b200 import domain as D
    from so3lr_b200.engine import Model
    Model.default(0)
    tw = D.ThreadWorld(world)
    out, err = [None] * world, []

    def body(rank):
        try:
            torch.cuda.set_device(0)
            out[rank] = fn(tw.comm(rank), rank)
        except Exception as e:  # pragma: no cover - surfaced below
            err.append(e)
            tw.barrier.abort()

    ts = [threading.Thread(target=body, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    if err:
        raise err[0]
    return out


@pytest.mark.parametrize("world", [1, 2, 3])
def test_decomposed_water_matches_single_device(reference_goldens, world):
    from so3lr_b200 import domain as D
    from so3lr_b200.engine import System
    g = reference_goldens
    Z, R, cell = g["water_Z"], np.asarray(g["water_R"], dtype=np.float32), g["water_cell"]
    skin = 0.5
    single = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=skin)
    ref = single.compute(torch.tensor(R, device="cuda"))
    E_ref, F_ref = float(ref["energy"].sum()), ref["forces"].cpu().numpy()
    q_ref = ref["partial_charges"].cpu().numpy()

    def fn(comm, rank):
        be = D.CudaBackend(cutoff_lr=12.0, damping=2.0, skin=skin, device=0)
        dom = D.DomainSystem(comm, be, Z, R, cell, skin=skin, cutoff_lr=12.0, device="cuda:0")
        E, _ = dom.compute(check_rebuild=False)
        F = dom.global_forces().cpu().numpy()
        q = dom.gather_global(dom.q).cpu().numpy()
        return float(E), F, q, dom.n0, dom.n_local

    res = _run_threads(world, fn)
    assert sum(r[3] for r in res) == len(Z)
    for E, F, q, n0, nl in res:
        assert abs(E - E_ref) <= 1e-5 * abs(E_ref), (E, E_ref)
        assert np.abs(F - F_ref).max() <= 1e-4, np.abs(F - F_ref).max()
        np.testing.assert_allclose(q, q_ref, atol=1e-5)
    # against the reference's golden vector as well (tests/test_jaxmd.py:246 allows 5e-4)
    np.testing.assert_allclose(res[0][1], g["water_forces_jaxmd"], atol=5e-4)


@pytest.mark.parametrize("world,method", [(2, "pme"), (3, "pme"), (2, "ewald")])
def test_decomposed_water_with_the_reciprocal_sum_matches_single_device(reference_goldens, world, method):
    """The charge mesh (or the structure factors) is summed over the ranks; everything else is per rank."""
    from so3lr_b200 import domain as D
    from so3lr_b200.engine import System
    g = reference_goldens
    Z, R, cell = g["water_Z"], np.asarray(g["water_R"], dtype=np.float32), g["water_cell"]
    skin, shape, smearing = 0.5, ((32, 30, 36) if method == "pme" else (21, 20, 19)), 2.4
    single = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=skin)
    single.enable_virial(True)
    single.set_kspace(shape, smearing, method)
    ref = single.compute(torch.tensor(R, device="cuda"))
    E_ref, F_ref, W_ref = float(ref["energy"].sum()), ref["forces"].cpu().numpy(), ref["virial"].cpu().numpy()

    def fn(comm, rank):
        be = D.CudaBackend(cutoff_lr=12.0, damping=2.0, skin=skin, device=0)
        be.enable_virial(True)
        dom = D.DomainSystem(comm, be, Z, R, cell, skin=skin, cutoff_lr=12.0, device="cuda:0")
        dom.set_kspace(shape, smearing, method)
        E, _ = dom.compute(check_rebuild=False)
        W = dom.virial().cpu().numpy()
        F = dom.global_forces().cpu().numpy()
        dom.set_kspace(None)
        E_plain, _ = dom.compute(check_rebuild=False)
        return float(E), F, W, float(E_plain)

    res = _run_threads(world, fn)
    single.set_kspace(None)
    E_plain_ref = float(single.compute(torch.tensor(R, device="cuda"))["energy"].sum())
    for E, F, W, E_plain in res:
        assert abs(E - E_ref) <= 1e-5 * abs(E_ref), (E, E_ref)
        assert np.abs(F - F_ref).max() <= 1e-4, np.abs(F - F_ref).max()
        assert np.abs(W - W_ref).max() <= 2e-3 + 1e-5 * np.abs(W_ref).max(), np.abs(W - W_ref).max()
        assert abs(E_plain - E_plain_ref) <= 1e-5 * abs(E_plain_ref)


def test_decomposed_nve_tracks_single_device_and_migrates(reference_goldens):
    from so3lr_b200 import domain as D
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    Z, R, cell = W.water_box(512, 24.9, 11, jitter=0.02)
    R = np.asarray(R, dtype=np.float32)
    V, m = W.maxwell_boltzmann(Z, 300.0, 12)
    V = (V + np.array([0.02, 0.0, 0.0])).astype(np.float32)     # drift along x so that atoms cross slab boundaries
    skin, dt, steps = 0.5, 0.5, 30
    s = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=skin)
    Rd, Vd = torch.tensor(R, device="cuda"), torch.tensor(V, device="cuda")
    md = torch.tensor(m, dtype=torch.float32, device="cuda")
    Fd = s.compute(Rd)["forces"].clone()
    s.nve(steps, dt, md, Rd, Vd, Fd)
    R_ref = Rd.cpu().numpy()

    def fn(comm, rank):
        be = D.CudaBackend(cutoff_lr=12.0, damping=2.0, skin=skin, device=0)
        dom = D.DomainSystem(comm, be, Z, R, cell, skin=skin, cutoff_lr=12.0, velocities=V, masses=m, device="cuda:0")
        dom.compute(check_rebuild=False)
        dom.nve(steps, dt)
        return dom.gather_global(dom.R[: dom.n0]).cpu().numpy(), dom.n_rebuilds, dom.global_forces().cpu().numpy(), float(dom.E)

    res = _run_threads(2, fn)
    Rdd, rebuilds, Fdd, Edd = res[0]
    assert rebuilds >= 2                       # the skin test fired: atoms were re-partitioned on the way
    # the decomposed state after migration is self-consistent: a fresh single-device evaluation of the same positions
    # gives the same energy and forces
    chk = System(Z, cell, cutoff_lr=12.0, damping=2.0, skin=0.0).compute(torch.tensor(Rdd, device="cuda"))
    assert abs(Edd - float(chk["energy"].sum())) <= 1e-5 * abs(Edd)
    assert np.abs(Fdd - chk["forces"].cpu().numpy()).max() <= 1e-4
    # and the trajectory stays on the single-device one (unequilibrated start: roundoff differences grow quickly)
    d = Rdd - R_ref
    d -= np.round(d / 24.9) * 24.9
    assert np.abs(d).max() < 5e-2 and np.median(np.abs(d)) < 1e-4, (np.abs(d).max(), np.median(np.abs(d)))


def test_sharded_molecule_batch_matches_unsharded(oracle_params):
    """Independent structures split over two ranks (evaluated one after the other on this GPU): same numbers as one batch."""
    from so3lr_b200 import batch as B
    from so3lr_b200 import workloads as W
    from so3lr_b200.engine import System
    Z, R, gs = W.molecule_batch(9, seed=1001)
    R = np.asarray(R, dtype=np.float32)
    whole = System(Z, None, cutoff_lr=1000.0, damping=2.0, lr_format="sparse", graph_start=gs).compute_host(R)
    parts = [B.ShardedBatch(Z, gs, 2, r).compute_host(R) for r in range(2)]
    np.testing.assert_allclose(np.concatenate([p["energy"] for p in parts]), whole["energy"], rtol=1e-6)
    np.testing.assert_allclose(np.concatenate([p["forces"] for p in parts]), whole["forces"], atol=2e-5)
    np.testing.assert_allclose(np.concatenate([p["dipole_vec"] for p in parts]), whole["dipole_vec"], atol=2e-5)


def test_halo_pack_and_unpack_rows_match_indexing():
    """The fused gather / scatter of the halo messages against plain tensor indexing: three arrays of different widths,
    repeated and unsorted row indices on the way out, distinct rows on the way back, and the empty message."""
    from so3lr_b200.domain import CudaBackend
    be = CudaBackend.__new__(CudaBackend)          # the packing calls need the device only, no model
    be.device = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(11)
    n = 1000
    tensors = [torch.randn(n, w, generator=g).cuda() for w in (128, 24, 2)]
    idx = torch.randint(0, n, (313,), generator=g).cuda()
    buf = be.pack_rows(tensors, idx)
    assert torch.equal(buf, torch.cat([t[idx] for t in tensors], 1))
    dst = [torch.zeros_like(t) for t in tensors]
    rows = torch.randperm(n, generator=g)[:313].cuda()
    be.unpack_rows(dst, rows, buf)
    o = 0
    for t, d in zip(tensors, dst):
        want = torch.zeros_like(t)
        want[rows] = buf[:, o:o + t.shape[1]]
        assert torch.equal(d, want)
        o += t.shape[1]
    empty = torch.empty(0, dtype=torch.int64, device="cuda")
    assert be.pack_rows(tensors, empty).shape == (0, 154)
    be.unpack_rows(dst, empty, be.pack_rows(tensors, empty))
