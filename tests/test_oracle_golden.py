"""The CPU oracle against every golden vector the reference's test-suite holds for the energy+force path
(tests/test_jaxmd.py:26-256 and tests/test_ase.py:9-142 of the reference)."""
import numpy as np
import pytest

from oracle import so3lr_oracle as O


def _run(P, g, name):
    cell = g[f"{name}_cell"] if f"{name}_cell" in g.files else None
    return O.energy_forces(P, g[f"{name}_R"], g[f"{name}_Z"], cell, cutoff_lr=12.0, damping=2.0)


@pytest.mark.parametrize("name", ["atat", "dha", "bb"])
def test_molecules_match_reference_goldens(oracle_params, reference_goldens, name):
    g = reference_goldens
    out = _run(oracle_params, g, name)
    # jax-md path, float64: the reference asserts E atol 1e-6, F atol 1e-4 (tests/test_jaxmd.py:89-99)
    assert abs(out["energy"] - float(g[f"{name}_energy_jaxmd"])) < 1e-6
    np.testing.assert_allclose(out["forces"], g[f"{name}_forces_jaxmd"], atol=2e-6)
    # ASE path goldens look float32-rounded: E atol 1e-5 + rtol 1e-6, F atol 1e-4 (tests/test_ase.py:34-45)
    np.testing.assert_allclose(out["energy"], float(g[f"{name}_energy_ase"]), atol=1e-5, rtol=1e-6)
    np.testing.assert_allclose(out["forces"], g[f"{name}_forces_ase"], atol=1e-4)
    # negative control as in the reference tests
    assert np.abs(out["forces"]).max() > 0.1


def test_periodic_water_matches_reference_goldens(oracle_params, reference_goldens):
    g = reference_goldens
    out = _run(oracle_params, g, "water")
    assert out["num_edges"] == 59280 and out["num_pairs"] == 557360
    # forces: reference asserts atol 5e-4 (tests/test_jaxmd.py:246-250); we hold 2e-6
    np.testing.assert_allclose(out["forces"], g["water_forces_jaxmd"], atol=2e-6)
    # energy: 2e-8 relative (4.4e-5 eV on -2681 eV)
    assert abs(out["energy"] - float(g["water_energy_jaxmd"])) < 1e-4
    np.testing.assert_allclose(out["energy"], float(g["water_energy_ase"]), rtol=1e-6)
    np.testing.assert_allclose(out["forces"], g["water_forces_ase"], atol=5e-4)


def test_ethanol_dipole_and_hirshfeld_match_the_reference_notebook(oracle_params, reference_goldens):
    """The reference's one published vector for the dipole and the Hirshfeld ratios: ethanol frame 49 evaluated in float32 by
    So3lr(calculate_forces=True, lr_cutoff=100) (examples/evaluate_so3lr_on_dataset.ipynb, output of `pprint(output)`)."""
    g = reference_goldens
    out = O.energy_forces(oracle_params, g["ethanol_R"], g["ethanol_Z"], None, cutoff_lr=100.0, damping=2.0, lr_format="sparse")
    assert abs(out["energy"] - float(g["ethanol_energy"])) < 1e-5 * abs(float(g["ethanol_energy"]))
    np.testing.assert_allclose(out["forces"], g["ethanol_forces"], atol=1e-5)
    np.testing.assert_allclose(out["dipole_vec"][0], g["ethanol_dipole_vec"], atol=1e-5)
    np.testing.assert_allclose(out["hirshfeld_ratios"], g["ethanol_hirshfeld_ratios"], atol=1e-5)
