"""The allocation-free pair-list entry point against the allocating one (so3lr_b200_system_export_list) and against the
CPU oracle's pair sets.

Collected last on purpose: a run that stops at the first failure has then already run every other test.  The entry
point keeps its scratch in a fixed array inside the library, so the second of two back-to-back calls starts from the
first call's leftovers; both must give the same pair set as the allocating path, bit for bit after sorting.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _pairs(idx, count):
    p = np.stack([idx[0, :count], idx[1, :count]], 1)
    return p[np.lexsort((p[:, 1], p[:, 0]))]


@pytest.mark.parametrize("ordered", [False, True])
def test_no_alloc_list_matches_allocating_list_twice(reference_goldens, ordered):
    from so3lr_b200.engine import System, neighbor_list_noalloc
    g = reference_goldens
    Z, R, cell = g["water_Z"], np.asarray(g["water_R"], dtype=np.float32), g["water_cell"]
    n = len(Z)
    rc = 4.5
    Rt = torch.tensor(R, device="cuda")
    s = System(Z, cell, cutoff_lr=rc, damping=None, lr_format="ordered_sparse" if ordered else "sparse")
    _, want_count, _ = s.neighbor_list(Rt, 1, 1)
    cap = want_count + 37
    want_idx, want_count, ovf = s.neighbor_list(Rt, 1, cap)
    assert not ovf
    want = _pairs(want_idx.cpu().numpy(), want_count)

    idx = torch.full((2, cap), -7, dtype=torch.int32, device="cuda")
    count = torch.zeros(1, dtype=torch.int64, device="cuda")
    overflow = torch.full((1,), 5, dtype=torch.int32, device="cuda")
    # a different, smaller problem first, so the scratch holds stale rows of another shape when the real calls run
    small = torch.tensor(R[:300], device="cuda")
    neighbor_list_noalloc(small, cell, 6.0, ordered, idx, count, overflow)
    for _ in range(2):
        idx.fill_(-7)
        neighbor_list_noalloc(Rt, cell, rc, ordered, idx, count, overflow)
        torch.cuda.synchronize()
        assert int(count.item()) == want_count and int(overflow.item()) == 0
        got_idx = idx.cpu().numpy()
        assert (got_idx[:, want_count:] == n).all()                  # padding carries N
        assert (np.diff(got_idx[0, :want_count]) >= 0).all()         # grouped by centre
        assert np.array_equal(_pairs(got_idx, want_count), want)

    # too small a capacity: flag set, count still the true number, stored pairs are a subset
    cap2 = want_count // 2
    idx2 = torch.empty((2, cap2), dtype=torch.int32, device="cuda")
    neighbor_list_noalloc(Rt, cell, rc, ordered, idx2, count, overflow)
    torch.cuda.synchronize()
    assert int(count.item()) == want_count and int(overflow.item()) == 1
    sub = idx2.cpu().numpy()
    assert ((sub >= 0) & (sub < n)).all()


def test_no_alloc_free_space_and_size_limit(reference_goldens):
    from so3lr_b200._lib import So3lrB200Error
    from so3lr_b200.engine import NOALLOC_MAX_ATOMS, System, neighbor_list_noalloc
    g = reference_goldens
    Z, R = g["bb_Z"], np.asarray(g["bb_R"], dtype=np.float32)
    Rt = torch.tensor(R, device="cuda")
    s = System(Z, None, cutoff_lr=12.0, damping=None, lr_format="ordered_sparse")
    _, want_count, _ = s.neighbor_list(Rt, 1, 1)
    want_idx, want_count, _ = s.neighbor_list(Rt, 1, want_count)
    idx = torch.empty((2, want_count), dtype=torch.int32, device="cuda")
    count = torch.zeros(1, dtype=torch.int64, device="cuda")
    overflow = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):
        neighbor_list_noalloc(Rt, None, 12.0, True, idx, count, overflow)
        torch.cuda.synchronize()
        assert int(count.item()) == want_count and int(overflow.item()) == 0
        assert np.array_equal(_pairs(idx.cpu().numpy(), want_count), _pairs(want_idx.cpu().numpy(), want_count))
    big = torch.zeros(NOALLOC_MAX_ATOMS + 1, 3, device="cuda")
    with pytest.raises(So3lrB200Error) as e:
        neighbor_list_noalloc(big, None, 4.5, False, idx, count, overflow)
    assert e.value.status == 5


@pytest.mark.parametrize("ordered", [False, True])
def test_no_alloc_list_matches_oracle_in_a_triclinic_cell(ordered):
    """Directly against the oracle's pair set, in a sheared cell, two calls in a row; and the documented precondition (every
    perpendicular cell width at least twice the cutoff) is enforced instead of silently returning a minimum-image list."""
    from oracle import so3lr_oracle as O
    from so3lr_b200 import workloads as W
    from so3lr_b200._lib import So3lrB200Error
    from so3lr_b200.engine import neighbor_list_noalloc
    Z, R, _ = W.water_box(216, 18.7, 5)
    cell = np.array([[18.7, 0, 0], [3.1, 18.7, 0], [-2.0, 4.0, 18.7]])
    R = np.asarray(R, dtype=np.float32)
    rc = 5.5
    ii, jj = O.neighbor_list(R, cell, rc, ordered=ordered)
    want = np.stack([ii, jj], 1)
    want = want[np.lexsort((want[:, 1], want[:, 0]))]
    cap = len(ii) + 11
    Rt = torch.tensor(R, device="cuda")
    idx = torch.empty((2, cap), dtype=torch.int32, device="cuda")
    count = torch.zeros(1, dtype=torch.int64, device="cuda")
    overflow = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(2):
        idx.fill_(-3)
        neighbor_list_noalloc(Rt, cell, rc, ordered, idx, count, overflow)
        torch.cuda.synchronize()
        assert int(count.item()) == len(ii) and int(overflow.item()) == 0
        assert np.array_equal(_pairs(idx.cpu().numpy(), len(ii)), want)
    with pytest.raises(So3lrB200Error) as e:          # 18.7 A wide cell, 9.5 A cutoff: a second image would be inside
        neighbor_list_noalloc(Rt, cell, 9.5, ordered, idx, count, overflow)
    assert e.value.status == 1
