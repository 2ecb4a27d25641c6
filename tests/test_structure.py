"""Structure derivation (couplings, monomials), model generator and host-side logic (CPU)."""
import json
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_coupling_tensors_are_orthonormal_and_equivariant(pkg):
    st = pkg.structure
    rng = np.random.default_rng(0)
    rot = st._random_rotation(rng)
    for l1, l2, l in [(1, 1, 0), (1, 1, 2), (2, 1, 3), (3, 1, 2), (2, 2, 2), (3, 2, 1)]:
        c = st.coupling_tensor(l1, l2, l)
        assert np.allclose(np.einsum("abm,abn->mn", c, c), np.eye(2 * l + 1), atol=1e-10)
        d1, d2, d = st.wigner_matrix(l1, rot), st.wigner_matrix(l2, rot), st.wigner_matrix(l, rot)
        assert np.allclose(np.einsum("ai,bj,ck,ijk->abc", d1, d2, d, c), c, atol=1e-9)
    assert st.coupling_tensor(1, 1, 3) is None


def test_harmonics_conventions(pkg):
    st = pkg.structure
    pts = np.random.default_rng(1).normal(size=(20, 3))
    y = st.real_harmonics(3, pts)
    u = pts / np.linalg.norm(pts, axis=1, keepdims=True)
    assert np.allclose(y[:, 1:4], np.sqrt(3.0) * u)          # l = 1 is sqrt(3) (x, y, z)
    for l in range(4):
        assert np.allclose(st._general_harmonics(l, pts), y[:, l * l:(l + 1) ** 2])


@pytest.mark.parametrize("shape,l_max,L_max", [("S0", 3, 0), ("S1", 3, 1), ("S2", 3, 2)])
def test_layer1_structure_matches_reference_contracts(pkg, shape, l_max, L_max):
    ref = json.loads((GOLDEN / "structure_reference.json").read_text())[shape]
    s = pkg.structure.r1_structure(l_max, L_max)
    assert [[a, b, c] for a, b, c in zip(s["Phi1_l"], s["Phi1_l1"], s["Phi1_l2"])] == ref["paths"]
    assert s["Phi1_lelm1lm2"] == ref["rows"] and s["Phi1_lme"] == ref["lme"]
    assert np.allclose(np.abs(s["Phi1_clebsch_gordan"]), ref["abs_cg"], atol=1e-10)


def test_contraction_monomials_match_reference_table(pkg):
    """Derived sets equal the reference's standard medium table except for 12 cubic terms whose
    coefficient vanishes for an equivariant model; model_tables() carries those as well."""
    ref = json.loads((GOLDEN / "structure_reference.json").read_text())["M0_medium"]
    derived = pkg.structure.model_structure(3, 1)["M0_monomials"]
    full = pkg.modelgen.model_tables(3, 1)["M0_monomials"]
    assert [len(full[str(k)]) for k in range(4)] == [94, 118, 92, 118]
    for k in range(4):
        assert full[str(k)] == ref[str(k)]
        assert {tuple(t) for t in derived[str(k)]} <= {tuple(t) for t in ref[str(k)]}
    assert derived["0"] == ref["0"] and derived["2"] == ref["2"]


def test_generated_model_is_rotation_invariant(pkg, model_path):
    from oracle import mace_numpy, neighbor

    path = model_path("small", 2)
    o = mace_numpy.NumpyMACE(str(path))
    rng = np.random.default_rng(4)
    pos = rng.random((12, 3)) * 6.0
    types = rng.integers(0, 3, size=12)
    cell = np.eye(3) * 30.0
    first, src, shifts = neighbor.build_neighbor_graph(pos, cell, 5.0)
    e0, _, f0, _ = o.energy_forces_stress(types, pos, cell, first, src, shifts)
    rot = pkg.structure._random_rotation(rng)
    pos2 = (pos - pos.mean(0)) @ rot.T + 15.0
    first2, src2, shifts2 = neighbor.build_neighbor_graph(pos2, cell, 5.0)
    e1, _, f1, s1 = o.energy_forces_stress(types, pos2, cell, first2, src2, shifts2)
    assert abs(e0 - e1) < 1e-9
    assert np.abs(f0 @ rot.T - f1).max() < 1e-9
    assert np.abs(s1 - s1.T).max() < 1e-12


def test_model_generator_is_deterministic(pkg):
    a = pkg.modelgen.make_model("small", seed=3)
    b = pkg.modelgen.make_model("small", seed=3)
    c = pkg.modelgen.make_model("small", seed=4)
    assert a == b and a["H0_weights"] != c["H0_weights"]
    assert a["num_channels"] == 32 and a["L_max"] == 0 and a["r_cut"] == 5.0
    m = pkg.modelgen.make_model("medium", seed=0)
    assert m["num_channels"] == 128 and len(m["Phi1_l"]) == 10 and len(m["Phi1_lme"]) == 86
    assert m["compact_radial"]["networks"]["R1"]["shape"] == [8, 64, 64, 64, 1280]


def test_srtio3_builder(pkg):
    pos, cell, types = pkg.modelgen.srtio3(3, 0.0, 0)
    assert pos.shape == (135, 3) and np.allclose(np.diag(cell), 3 * 3.905)
    assert sorted(np.bincount(types).tolist()) == [27, 27, 81]
    p2, _, _ = pkg.modelgen.srtio3((2, 1, 1), 0.05, 1)
    assert p2.shape == (10, 3)
