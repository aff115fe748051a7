"""Restart files of the MD loop (so3lr_b200.md.save_state / load_state; the reference's are so3lr/cli/so3lr_md.py:2286-2440)."""
import numpy as np
import pytest
import torch

from so3lr_b200 import md


def _state(n=11, chain=True, seed=0):
    g = torch.Generator().manual_seed(seed)
    R, V, F = (torch.randn(n, 3, generator=g) for _ in range(3))
    m = torch.rand(n, generator=g) * 15 + 1
    c = torch.randn(18, generator=g, dtype=torch.float64) if chain else None
    return md.MDState(R, V, F, m, c)


@pytest.mark.parametrize("ensemble", ["nve", "nvt", "npt"])
def test_restart_round_trip(tmp_path, ensemble):
    st = _state(chain=ensemble != "nve")
    box = np.diag([12.0, 13.0, 14.0]) if ensemble == "npt" else np.array([12.0, 13.0, 14.0])
    if ensemble == "npt":
        st.reference_box = np.diag([12.5, 12.5, 12.5])
    p = tmp_path / "restart.npz"
    md.save_state(st, box, 37, p, ensemble)
    back, box2, cycle = md.load_state(p, ensemble, device="cpu")
    assert cycle == 37
    np.testing.assert_allclose(box2, box)
    for a, b in ((back.position, st.position), (back.force, st.force), (back.mass, st.mass)):
        assert torch.equal(a, b)
    np.testing.assert_allclose(back.velocity.numpy(), st.velocity.numpy(), rtol=2e-7)      # stored as momentum, as in the reference
    if ensemble == "nve":
        assert back.chain is None
    else:
        assert torch.equal(back.chain, st.chain)
    if ensemble == "npt":
        np.testing.assert_allclose(back.reference_box, st.reference_box)
        np.testing.assert_allclose(back.box, box)


def test_restart_in_another_ensemble_is_refused(tmp_path):
    p = tmp_path / "r.npz"
    md.save_state(_state(), None, 1, p, "nvt")
    with pytest.raises(md.RestartInNewEnsembleError):
        md.load_state(p, "npt", device="cpu")
    with pytest.raises(ValueError):
        md.save_state(_state(chain=False), None, 1, p, "nvt")
    with pytest.raises(ValueError):
        md.save_state(_state(), None, 1, p, "nph")
