"""CPU tests of the oracles: the NumPy restatement against golden vectors produced by the
reference's own code (tests/golden/make_golden.py), and the neighbor-graph restatement against
a brute-force search and the reference's published edge counts."""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import mace_numpy, neighbor, ref

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("arch,scaled,zbl,agnesi", [("small", False, False, False), ("medium", False, False, False),
                                                    ("medium", True, False, False), ("large", False, False, False),
                                                    ("small", False, True, False), ("small", True, True, True)])
def test_numpy_restatement_matches_reference_evaluator_golden(pkg, model_dir, arch, scaled, zbl, agnesi):
    name = f"reference_evaluator_{arch}{'_scaled' if scaled else ''}{'_zbl' if zbl else ''}{'_agnesi' if agnesi else ''}.npz"
    g = np.load(GOLDEN / name)
    path = model_dir / f"golden_{arch}_{int(scaled)}_{int(zbl)}_{int(agnesi)}.json"
    pkg.modelgen.write_model(path, arch, seed=101, a0_scaled=scaled, a1_scaled=scaled, zbl=zbl, agnesi=agnesi)
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 202)
    assert np.array_equal(pos, g["positions"]) and np.array_equal(types, g["types"])
    xyz = neighbor.edge_vectors(pos, cell, g["first"], g["sources"], g["shifts"])
    o = mace_numpy.NumpyMACE(str(path))
    e, f = o.compute(types, g["first"], g["sources"], xyz)
    assert np.abs(e - g["node_energies"]).max() < 1e-11
    assert np.abs(f.reshape(-1) - g["edge_forces"]).max() < 1e-11
    for name in ("A0", "M0", "H1", "Phi1", "A1", "M1", "H2", "H1_adj", "A0_adj"):
        v = o.stage[name]
        got = np.array([v.sum(), np.abs(v).sum(), (v * v).sum()])
        assert np.allclose(got, g["sum_" + name], rtol=1e-10, atol=1e-10), name


VARIANTS = {k: v for k, v in json.loads((GOLDEN / "variants.json").read_text()).items() if not k.startswith("_")}


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_numpy_restatement_matches_reference_golden_of_model_variants(pkg, model_dir, name):
    """Stored pair splines, one interaction, the old basis of formats 1 / 2 and the pre_linear_up basis with a
    first-interaction residual: the restatement against vectors of the reference's MACECPU<double>."""
    arch, kwargs = VARIANTS[name]
    g = np.load(GOLDEN / f"reference_evaluator_variant_{name}.npz")
    path = model_dir / f"golden_variant_{name}.json"
    pkg.modelgen.write_model(path, arch, seed=101, **kwargs)
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 202)
    assert np.array_equal(pos, g["positions"]) and np.array_equal(types, g["types"])
    xyz = neighbor.edge_vectors(pos, cell, g["first"], g["sources"], g["shifts"])
    o = mace_numpy.NumpyMACE(str(path))
    e, f = o.compute(types, g["first"], g["sources"], xyz)
    assert np.abs(e - g["node_energies"]).max() < 1e-11
    assert np.abs(f.reshape(-1) - g["edge_forces"]).max() < 1e-11
    for stage in ("A0", "M0", "H1", "M1", "H2"):
        v = o.stage[stage]
        got = np.array([v.sum(), np.abs(v).sum(), (v * v).sum()])
        assert np.allclose(got, g["sum_" + stage], rtol=1e-10, atol=1e-10), stage


@pytest.mark.parametrize("name", sorted(VARIANTS))
def test_numpy_restatement_matches_live_reference_on_model_variants(pkg, model_path, name):
    """The same variants against oracle/_ref itself on another model seed and cell, when it is built."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    arch, kwargs = VARIANTS[name]
    path = model_path(arch, seed=71, **kwargs)
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 43)
    first, src, shifts = neighbor.build_neighbor_graph(pos, cell, pkg.modelgen.ARCHITECTURES[arch]["r_cut"])
    xyz = neighbor.edge_vectors(pos, cell, first, src, shifts)
    m = ref.ReferenceMACE(str(path), double=True)
    m.compute(types, np.diff(first), src, xyz)
    e, f = mace_numpy.NumpyMACE(str(path)).compute(types, first, src, xyz)
    assert np.abs(e - m.get("node_energies")).max() < 1e-11
    assert np.abs(f.reshape(-1) - m.get("node_forces")).max() < 1e-11


def test_numpy_restatement_matches_live_reference_evaluator(pkg, model_path):
    """Same check against oracle/_ref itself, float64 and float32, when it is built."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path("small", 5)
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 9)
    first, src, shifts = neighbor.build_neighbor_graph(pos, cell, 5.0)
    xyz = neighbor.edge_vectors(pos, cell, first, src, shifts)
    m = ref.ReferenceMACE(str(path), double=True)
    m.compute(types, np.diff(first), src, xyz)
    o = mace_numpy.NumpyMACE(str(path))
    e, f = o.compute(types, first, src, xyz)
    assert np.abs(e - m.get("node_energies")).max() < 1e-11
    assert np.abs(f.reshape(-1) - m.get("node_forces")).max() < 1e-11
    mf = ref.ReferenceMACE(str(path), double=False)
    mf.compute(types, np.diff(first), src, xyz)
    assert np.abs(e - mf.get("node_energies")).max() < 1e-4


def test_harmonics_match_reference_closed_forms():
    """Gradients of Y_lm against the reference's first-party l <= 3 closed forms
    (golden produced from symmetrix/source/symmetrix/jit_codegen.py:2851-2977)."""
    g = np.load(GOLDEN / "harmonics_reference.npz")
    Y, Yg = mace_numpy.harmonics(3, g["vectors"])
    assert np.abs(Yg - g["gradients"]).max() < 1e-12
    # closed-form properties of the values: Y_00 = 1, sum_m Y_lm^2 = 2l+1
    assert np.allclose(Y[:, 0], 1.0)
    for l in range(4):
        assert np.allclose((Y[:, l * l:(l + 1) ** 2] ** 2).sum(axis=1), 2 * l + 1)
    # gradient is tangential and matches finite differences
    v = g["vectors"]
    assert np.abs(np.einsum("ndl,nd->nl", Yg, v)).max() < 1e-12
    h = 1e-6
    for d in range(3):
        step = np.zeros(3)
        step[d] = h
        fd = (mace_numpy.harmonics(3, v + step)[0] - mace_numpy.harmonics(3, v - step)[0]) / (2 * h)
        assert np.abs(fd - Yg[:, d]).max() < 1e-7


def test_spline_tables_interpolate_network(pkg, model_path):
    import json

    model = json.loads(Path(model_path("small", 1)).read_text())
    t = mace_numpy.RadialTables(model["compact_radial"], model["r_cut"])
    c = t.coefficients("R0")
    nodes = t.x0 + np.arange(t.points) * t.h
    values = t.mlp("R0", t.features())
    got, _ = mace_numpy.spline_eval(c, t.x0, t.h, nodes[:-1] + 1e-13)
    assert np.abs(got - values[:-1]).max() < 1e-9
    # value and derivative vanish at the cutoff (edges at r >= r_cut contribute nothing)
    v, d = mace_numpy.spline_eval(c, t.x0, t.h, np.array([model["r_cut"]]))
    assert np.abs(v).max() < 1e-12 and np.abs(d).max() < 1e-9


def test_neighbor_graph_against_brute_force():
    rng = np.random.default_rng(5)
    for cell in (np.eye(3) * 9.0, np.array([[8.0, 0, 0], [2.0, 7.5, 0], [1.0, -1.5, 9.0]])):
        pos = rng.random((40, 3)) @ cell + rng.integers(-1, 2, size=(40, 3)) @ cell
        for cutoff in (3.0, 5.0):
            first, src, shifts = neighbor.build_neighbor_graph(pos, cell, cutoff)
            recv = np.repeat(np.arange(40), np.diff(first))
            mine = set(zip(recv.tolist(), src.tolist(), *shifts.T.tolist()))
            assert len(mine) == len(src)   # no duplicates
            assert mine == neighbor.brute_force_edges(pos, cell, cutoff, max_image=4)


def test_neighbor_graph_small_cell_multiple_images():
    """Cutoff larger than the cell: the same source appears under several images."""
    cell = np.eye(3) * 3.0
    pos = np.array([[0.1, 0.2, 0.3], [1.6, 1.4, 1.7]])
    first, src, shifts = neighbor.build_neighbor_graph(pos, cell, 4.0)
    recv = np.repeat(np.arange(2), np.diff(first))
    mine = set(zip(recv.tolist(), src.tolist(), *shifts.T.tolist()))
    assert mine == neighbor.brute_force_edges(pos, cell, 4.0, max_image=3)
    assert (src == recv).any()   # self images


def test_published_edge_counts_of_the_reference_case(pkg):
    """5,000-atom SrTiO3, sigma = 0.01 A, seed 17: 370,000 directed edges at 6.0 A
    (README.md:86-88 of the reference), i.e. the perfect lattice's neighbor shells: 74 per atom on
    average, the same count for every atom of one species."""
    pos, cell, types = pkg.modelgen.srtio3(10, 0.01, 17)
    first, src, shifts = neighbor.build_neighbor_graph(pos, cell, 6.0)
    assert len(src) == 370000
    counts = np.diff(first)
    for t in range(3):
        assert len(set(counts[types == t].tolist())) == 1
    # 496k-512k edges with the 0.5 A skin (511,962 published for the reference's random stream)
    first65, src65, _ = neighbor.build_neighbor_graph(pos, cell, 6.5)
    assert 500000 < len(src65) < 520000
