"""GPU parity tests: the CUDA path through the C ABI against the oracles on identical inputs.

Tolerances of the force path: |dE| <= 1e-5 eV/atom, |dF| <= 1e-4 eV/A per component,
|dsigma| <= 1e-6 eV/A^3; the neighbor list must be bit-exact.
"""
import json
from pathlib import Path

import numpy as np
import pytest

from conftest import csr_from_positions
from oracle import mace_numpy, neighbor, ref

pytestmark = pytest.mark.gpu

TOL_E, TOL_F, TOL_S = 1e-5, 1e-4, 1e-6

STAGES = ["A0", "M0", "H1", "Phi1", "A1", "M1", "H2", "H2_adj", "A1_adj", "dPhi1", "H1_adj", "M0_adj", "A0_adj"]


def _edge_set(first, src, shifts):
    recv = np.repeat(np.arange(len(first) - 1), np.diff(first))
    return np.stack([recv, src, shifts[:, 0], shifts[:, 1], shifts[:, 2]], axis=1)


@pytest.mark.parametrize("n,sigma,cutoff,seed", [(3, 0.05, 5.5, 0), (4, 0.05, 5.5, 1), (4, 0.3, 6.5, 2), (2, 0.05, 6.5, 3)])
def test_neighbor_graph_bit_exact(pkg, model_path, n, sigma, cutoff, seed):
    pos, cell, types = pkg.modelgen.srtio3(n, sigma, seed)
    ev = pkg.MACEB200(model_path("small"))
    res = ev._prepare_periodic_factorized_graph(types, pos, cell, np.linalg.inv(cell), cutoff)
    first, src, shifts = ev.graph(res["generation"])
    ofirst, osrc, oshifts = neighbor.build_neighbor_graph(pos, cell, cutoff)
    assert res["num_edges"] == len(osrc)
    # identical order, not only identical sets
    assert np.array_equal(first, ofirst)
    assert np.array_equal(src, osrc)
    assert np.array_equal(shifts, oshifts)


def test_neighbor_graph_triclinic_and_wrapped(pkg, model_path):
    rng = np.random.default_rng(7)
    cell = np.array([[9.0, 0.0, 0.0], [2.5, 8.0, 0.0], [-1.0, 1.5, 10.0]])
    pos = rng.random((60, 3)) @ cell + rng.integers(-2, 3, size=(60, 3)) @ cell  # atoms outside the home cell
    types = rng.integers(0, 3, size=60).astype(np.int32)
    ev = pkg.MACEB200(model_path("small"))
    res = ev._prepare_periodic_factorized_graph(types, pos, cell, np.linalg.inv(cell), 4.0)
    first, src, shifts = ev.graph(res["generation"])
    ofirst, osrc, oshifts = neighbor.build_neighbor_graph(pos, cell, 4.0)
    assert np.array_equal(first, ofirst) and np.array_equal(src, osrc) and np.array_equal(shifts, oshifts)
    brute = neighbor.brute_force_edges(pos, cell, 4.0, max_image=6)
    mine = set(map(tuple, _edge_set(first, src, shifts).tolist()))
    assert mine == brute


# with density scaling the device keeps Phi1 already divided by 1 + rho and A1_adj / dPhi1 / A0_adj
# not yet divided (the division is folded into the next kernel's load), so those stages differ by
# design from the serial evaluator's intermediates and are left to the energy / force comparison
SCALED_STAGES = ["A0", "M0", "H1", "A1", "M1", "H2", "H2_adj", "H1_adj", "M0_adj"]


@pytest.mark.parametrize("arch,n,scaled", [("small", 3, False), ("medium", 2, False), ("medium", 2, True), ("small", 3, True), ("large", 2, False), ("large", 2, True)])
def test_stage_tensors_match_oracle(pkg, model_path, arch, n, scaled):
    path = model_path(arch, a0_scaled=scaled, a1_scaled=scaled)
    pos, cell, types = pkg.modelgen.srtio3(n, 0.05, 11)
    cutoff = pkg.modelgen.ARCHITECTURES[arch]["r_cut"]
    first, src, shifts, xyz = csr_from_positions(pos, cell, cutoff)
    ev = pkg.MACEB200(path)
    ev.compute_node_energies_forces(len(pos), types, np.diff(first), src, types[src], xyz)
    oracle = mace_numpy.NumpyMACE(str(path))
    oracle.compute(types, first, src, xyz)
    for name in (SCALED_STAGES if scaled else STAGES):
        got = ev.stage(name)
        want = oracle.stage[name].reshape(-1)
        scale = max(1.0, np.abs(want).max())
        assert np.abs(got - want).max() <= 2e-5 * scale, name
    de = np.abs(ev.node_energies - oracle.stage["node_energies"]).max()
    df = np.abs(ev.node_forces.reshape(-1, 3) - oracle.stage["node_forces"]).max()
    assert de <= TOL_E and df <= TOL_F


@pytest.mark.parametrize("arch,n,seed,scaled,zbl,agnesi", [("small", 4, 0, False, False, False), ("medium", 3, 1, False, False, False),
                                                           ("medium", 3, 2, True, False, False), ("large", 2, 3, False, False, False),
                                                           ("small", 3, 4, False, True, False), ("medium", 2, 5, True, True, False),
                                                           ("small", 3, 6, False, False, True), ("medium", 2, 7, True, True, True),
                                                           ("large", 2, 8, False, False, True)])
def test_energy_forces_stress_vs_reference_evaluator(pkg, model_path, arch, n, seed, scaled, zbl, agnesi):
    """Against the reference's own serial evaluator (MACECPU<double> and <float>)."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path(arch, a0_scaled=scaled, a1_scaled=scaled, zbl=zbl, agnesi=agnesi)
    pos, cell, types = pkg.modelgen.srtio3(n, 0.05, seed)
    calc = pkg.Calculator(path, skin=0.5)
    out = calc.calculate(pos, cell, types)
    r_cut = calc.evaluator.r_cut
    # exact-cutoff graph for the reference (skin edges contribute exactly zero on the device path)
    first, src, shifts, xyz = csr_from_positions(pos, cell, r_cut)
    volume = abs(np.linalg.det(cell))
    for double in (True, False):
        m = ref.ReferenceMACE(str(path), double=double)
        m.compute(types, np.diff(first), src, xyz)
        F, S = ref.reduce_forces_stress(len(pos), np.diff(first), src, m.get("node_forces"), xyz, volume)
        e = m.get("node_energies")
        assert abs(out["energy"] - e.sum()) / len(pos) <= TOL_E
        assert np.abs(out["energies"] - e).max() <= TOL_E
        assert np.abs(out["forces"] - F).max() <= TOL_F
        assert np.abs(out["stress"] - S).max() <= TOL_S


def _reference_efs(path, pos, cell, types, r_cut, double=False):
    """Energy per node, atom forces and stress of the reference's serial evaluator on the exact-cutoff graph."""
    first, src, shifts, xyz = csr_from_positions(pos, cell, r_cut)
    m = ref.ReferenceMACE(str(path), double=double)
    m.compute(types, np.diff(first), src, xyz)
    F, S = ref.reduce_forces_stress(len(pos), np.diff(first), src, m.get("node_forces"), xyz, abs(np.linalg.det(cell)))
    return m.get("node_energies"), F, S


def _assert_matches_reference(out, e, F, S, natoms, node_tol=TOL_E):
    assert abs(out["energy"] - e.sum()) / natoms <= TOL_E
    assert np.abs(out["energies"] - e).max() <= node_tol
    assert np.abs(out["forces"] - F).max() <= TOL_F
    assert np.abs(out["stress"] - S).max() <= TOL_S


@pytest.mark.parametrize("arch,n,scaled,zbl", [("small", 3, False, False), ("small", 2, True, True), ("medium", 2, False, False)])
def test_pair_spline_models_vs_reference_evaluator(pkg, model_path, arch, n, scaled, zbl):
    """The stored pair-spline radial representation (nodal values and derivatives per unordered element
    pair instead of radial networks), with and without density splines and the pair repulsion."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path(arch, seed=23, radial="pair-splines", num_spline_points=96, a0_scaled=scaled, a1_scaled=scaled, zbl=zbl)
    pos, cell, types = pkg.modelgen.srtio3(n, 0.05, 29)
    calc = pkg.Calculator(path, skin=0.5)
    out = calc.calculate(pos, cell, types)
    for double in (True, False):
        e, F, S = _reference_efs(path, pos, cell, types, calc.evaluator.r_cut, double=double)
        _assert_matches_reference(out, e, F, S, len(pos))


@pytest.mark.parametrize("arch,n,kwargs", [("small", 3, {}), ("medium", 2, {"a0_scaled": True}), ("large", 2, {"zbl": True}),
                                           ("small", 2, {"radial": "pair-splines", "num_spline_points": 96})])
def test_single_layer_models_vs_reference_evaluator(pkg, model_path, arch, n, kwargs):
    """Models with one interaction (single_layer_readout): the readout polynomial acts on H1 and there is no second
    message step (libsymmetrix/source/mace.cpp:265-283), for hidden irreps up to l = 0, 1 and 2; untiled and tiled."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path(arch, seed=41, single_layer=True, **kwargs)
    pos, cell, types = pkg.modelgen.srtio3(n, 0.05, 43)
    calc = pkg.Calculator(path, skin=0.5)
    assert calc.evaluator.single_layer_readout
    out = calc.calculate(pos, cell, types)
    for double in (True, False):
        e, F, S = _reference_efs(path, pos, cell, types, calc.evaluator.r_cut, double=double)
        _assert_matches_reference(out, e, F, S, len(pos))
    tiled = pkg.Calculator(path, skin=0.5)
    tiled.evaluator.set_tile_size(16)
    out_tiled = tiled.calculate(pos, cell, types)
    _assert_matches_reference(out_tiled, e, F, S, len(pos))
    with pytest.raises(ValueError):
        rep = pkg.MACEB200(path)
        rep.set_deterministic(True)
        rep._prepare_periodic_factorized_graph(types, pos, cell, np.linalg.inv(cell), rep.r_cut + 0.5)


@pytest.mark.parametrize("arch,n,kwargs", [("small", 3, {}), ("medium", 2, {"a0_scaled": True, "a1_scaled": True}),
                                           ("medium", 2, {"radial": "pair-splines", "num_spline_points": 64}),
                                           ("small", 2, {"single_layer": True})])
def test_old_basis_models_vs_reference_evaluator(pkg, model_path, arch, n, kwargs):
    """Format version 2 (and 1): the first readout and the H1 -> H2 skip act on the scalar block of H1, after the linear
    (libsymmetrix/source/h1_affine_schema.hpp:5-30, mace.cpp:2516-2557); untiled and tiled.  The reference's own float and
    double evaluators differ by up to 8e-6 eV in single node energies on these models, hence the wider per-node bound."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path(arch, seed=71, format_version=2, **kwargs)
    pos, cell, types = pkg.modelgen.srtio3(n, 0.05, 29 if n == 3 else 43)
    calc = pkg.Calculator(path, skin=0.5)
    assert calc.evaluator.h1_affine_mode == "legacy"
    out = calc.calculate(pos, cell, types)
    e, F, S = _reference_efs(path, pos, cell, types, calc.evaluator.r_cut, double=True)
    _assert_matches_reference(out, e, F, S, len(pos), node_tol=3e-5)
    tiled = pkg.Calculator(path, skin=0.5)
    tiled.evaluator.set_tile_size(16)
    _assert_matches_reference(tiled.calculate(pos, cell, types), e, F, S, len(pos), node_tol=3e-5)


@pytest.mark.parametrize("arch,n,kwargs", [("small", 3, {}), ("medium", 2, {"first_residual": True}),
                                           ("large", 2, {"first_residual": True, "a0_scaled": True, "a1_scaled": True})])
def test_pre_linear_up_models_vs_reference_evaluator(pkg, model_path, arch, n, kwargs):
    """Format 4 in the pre_linear_up basis: the first readout and the skip act on x = M0[l=0] P0 (+ the scalar block of the
    first-interaction residual), and an element-dependent constant R U joins H1 (libsymmetrix/source/mace.cpp:1759-1888);
    untiled and tiled."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path(arch, seed=61, pre_linear_up=True, **kwargs)
    pos, cell, types = pkg.modelgen.srtio3(n, 0.05, 63)
    calc = pkg.Calculator(path, skin=0.5)
    assert calc.evaluator.h1_affine_mode == "pre_linear_up"
    out = calc.calculate(pos, cell, types)
    e, F, S = _reference_efs(path, pos, cell, types, calc.evaluator.r_cut, double=True)
    _assert_matches_reference(out, e, F, S, len(pos), node_tol=3e-5)
    tiled = pkg.Calculator(path, skin=0.5)
    tiled.evaluator.set_tile_size(16)
    _assert_matches_reference(tiled.calculate(pos, cell, types), e, F, S, len(pos), node_tol=3e-5)


GOLDEN = Path(__file__).resolve().parent / "golden"
GOLDEN_CASES = {"small": ("small", {}), "medium": ("medium", {}), "medium_scaled": ("medium", {"a0_scaled": True, "a1_scaled": True}),
                "large": ("large", {}), "small_zbl": ("small", {"zbl": True}),
                "small_scaled_zbl_agnesi": ("small", {"a0_scaled": True, "a1_scaled": True, "zbl": True, "agnesi": True})}
GOLDEN_CASES.update({"variant_" + k: tuple(v) for k, v in json.loads((GOLDEN / "variants.json").read_text()).items()
                     if not k.startswith("_")})


@pytest.mark.parametrize("name", sorted(GOLDEN_CASES))
def test_committed_golden_vectors_of_the_reference_evaluator(pkg, model_path, name):
    """Energies, forces and stress against the committed vectors of the reference's MACECPU<double> (tests/golden/,
    written by make_golden.py): the standard models and every model-file variant; needs no reference build."""
    arch, kwargs = GOLDEN_CASES[name]
    g = np.load(GOLDEN / f"reference_evaluator_{name}.npz")
    path = model_path(arch, seed=101, **kwargs)
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 202)
    assert np.array_equal(pos, g["positions"])
    out = pkg.Calculator(path, skin=0.5).calculate(pos, cell, types)
    xyz = neighbor.edge_vectors(pos, cell, g["first"], g["sources"], g["shifts"])
    F, S = ref.reduce_forces_stress(len(pos), np.diff(g["first"]), g["sources"], g["edge_forces"], xyz, abs(np.linalg.det(cell)))
    # bounds: the tolerances of the force path, or eight times the deviation of the reference's own float evaluator
    # from these double vectors on the same input (stored beside them), whichever is larger: on a 40-atom cell the
    # FP32 resolution of the model itself can come close to the stress tolerance
    floor = 8.0 * g["float_deviation"]
    assert abs(out["energy"] - g["node_energies"].sum()) / len(pos) <= TOL_E
    assert np.abs(out["energies"] - g["node_energies"]).max() <= max(TOL_E, floor[0])
    assert np.abs(out["forces"] - F).max() <= max(TOL_F, floor[1])
    assert np.abs(out["stress"] - S).max() <= max(TOL_S, floor[2])


def test_headline_configuration_vs_reference_evaluator(pkg, model_path):
    """The configuration the throughput is quoted on, at full size: OMAT-0-medium architecture,
    10x10x10 SrTiO3 (5,000 atoms, sigma 0.05 A), 0.5 A skin, against MACECPU<float>."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path("medium", seed=17)
    pos, cell, types = pkg.modelgen.srtio3(10, 0.05, 17)
    calc = pkg.Calculator(path, skin=0.5)
    out = calc.calculate(pos, cell, types)
    e, F, S = _reference_efs(path, pos, cell, types, calc.evaluator.r_cut)
    _assert_matches_reference(out, e, F, S, len(pos))


DISORDERED_ELEMENTS = (1, 6, 8, 13, 14, 22, 26, 38, 56, 79)


def test_disordered_ten_element_solid_vs_reference_evaluator(pkg, model_path):
    """Hidden irreps 0e+1o+2e, ten elements, a 2,000-atom cut of the seeded Poisson-disk solid
    (0.085 atoms/A^3, 1.8 A minimum separation: irregular neighbor counts) against MACECPU<float>."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path("large", seed=17, atomic_numbers=DISORDERED_ELEMENTS)
    pos, cell, types = pkg.modelgen.random_solid(2000, 0.085, 1.8, len(DISORDERED_ELEMENTS), 17)
    calc = pkg.Calculator(path, skin=0.5)
    out = calc.calculate(pos, cell, types)
    assert len(np.unique(types)) == len(DISORDERED_ELEMENTS)
    e, F, S = _reference_efs(path, pos, cell, types, calc.evaluator.r_cut)
    _assert_matches_reference(out, e, F, S, len(pos))


@pytest.mark.parametrize("arch,options", [("medium", {}), ("small", dict(a0_scaled=True, a1_scaled=True, zbl=True, agnesi=True))])
def test_inactive_element_slots(pkg, model_path, arch, options):
    """A model with ten element slots of which three non-adjacent ones (1, 4, 8) occur in the
    structure: the active-type tables must skip the unused slots."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path(arch, seed=5, atomic_numbers=DISORDERED_ELEMENTS, **options)
    pos, cell, base_types = pkg.modelgen.srtio3(3, 0.05, 9)
    types = np.array([1, 4, 8], dtype=np.int32)[base_types]
    calc = pkg.Calculator(path, skin=0.5)
    out = calc.calculate(pos, cell, types)
    for double in (True, False):
        e, F, S = _reference_efs(path, pos, cell, types, calc.evaluator.r_cut, double=double)
        _assert_matches_reference(out, e, F, S, len(pos))
    # a second structure that uses other slots on the same evaluator: the tables are rebuilt
    types2 = np.array([0, 9, 4], dtype=np.int32)[base_types]
    out2 = calc.calculate(pos, cell, types2)
    e, F, S = _reference_efs(path, pos, cell, types2, calc.evaluator.r_cut)
    _assert_matches_reference(out2, e, F, S, len(pos))


def test_multi_head_model_uses_the_selected_head(pkg, model_path, tmp_path):
    """Two prediction heads: the default head against the reference's evaluator (which applies the
    same selection), and the other head gives a different energy."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path("small", seed=8, heads=("pbe", "omat"), zbl=True)
    pos, cell, types = pkg.modelgen.srtio3(3, 0.05, 2)
    calc = pkg.Calculator(path, skin=0.5)
    assert calc.evaluator.head == "omat" and calc.evaluator.selected_head == "omat"
    assert calc.evaluator.available_heads == ["pbe", "omat"] and calc.evaluator.supports_factorized
    out = calc.calculate(pos, cell, types)
    e, F, S = _reference_efs(path, pos, cell, types, calc.evaluator.r_cut)
    _assert_matches_reference(out, e, F, S, len(pos))
    other = pkg.Calculator(path, skin=0.5, head="pbe").calculate(pos, cell, types)
    assert abs(other["energy"] - out["energy"]) > 1e-3


def test_tiny_systems_and_isolated_atoms(pkg, model_path):
    """3..9 atoms (tile-boundary sizes of the reference's tests) and an atom with no neighbors."""
    path = model_path("small")
    oracle = mace_numpy.NumpyMACE(str(path))
    rng = np.random.default_rng(3)
    for natoms in (3, 4, 5, 8, 9):
        cell = np.eye(3) * 14.0
        pos = rng.random((natoms, 3)) * 5.0 + 1.0
        pos[0] = [12.0, 12.0, 12.0] if natoms > 3 else pos[0]   # far from the others: empty neighbor list
        # keep a sane minimum distance
        for i in range(1, natoms):
            while i > 0 and np.min(np.linalg.norm(pos[:i] - pos[i], axis=1)) < 1.5:
                pos[i] = rng.random(3) * 5.0 + 1.0
        types = rng.integers(0, 3, size=natoms).astype(np.int32)
        calc = pkg.Calculator(path, skin=0.5)
        out = calc.calculate(pos, cell, types)
        first, src, shifts = neighbor.build_neighbor_graph(pos, cell, calc.evaluator.r_cut + 0.5)
        e, energies, F, S = oracle.energy_forces_stress(types, pos, cell, first, src, shifts)
        assert abs(out["energy"] - e) / natoms <= TOL_E
        assert np.abs(out["forces"] - F).max() <= TOL_F
        assert np.abs(out["stress"] - S).max() <= TOL_S


def test_skin_graph_matches_exact_graph_and_is_reused(pkg, model_path):
    """Skin 0.5 vs exact graph, and no rebuild after a 0.1 A move
    (reference: symmetrix/test/test_mace_streamed_edges.py:4592-4676)."""
    path = model_path("small")
    pos, cell, types = pkg.modelgen.srtio3(3, 0.05, 2)
    skin = pkg.Calculator(path, skin=0.5)
    exact = pkg.Calculator(path, skin=0.0)
    a, b = skin.calculate(pos, cell, types), exact.calculate(pos, cell, types)
    assert abs(a["energy"] - b["energy"]) / len(pos) <= 1e-6
    assert np.abs(a["forces"] - b["forces"]).max() <= 1e-5
    moved = pos + np.random.default_rng(0).normal(scale=0.03, size=pos.shape)
    a2 = skin.calculate(moved, cell, types)
    assert skin.rebuilds == 1
    b2 = pkg.Calculator(path, skin=0.0).calculate(moved, cell, types)
    assert abs(a2["energy"] - b2["energy"]) / len(pos) <= 1e-6
    assert np.abs(a2["forces"] - b2["forces"]).max() <= 1e-5


def test_stale_generation_and_bad_inputs_raise(pkg, model_path):
    ev = pkg.MACEB200(model_path("small"))
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 0)
    with pytest.raises(ValueError):
        ev._compute_prepared_factorized_positions(1, pos)            # nothing prepared
    res = ev._prepare_periodic_factorized_graph(types, pos, cell, np.linalg.inv(cell), 5.5)
    ev._compute_prepared_factorized_positions(res["generation"], pos)
    res2 = ev._prepare_periodic_factorized_graph(types, pos, cell, np.linalg.inv(cell), 5.5)
    assert res2["generation"] > res["generation"]
    with pytest.raises(ValueError):
        ev._compute_prepared_factorized_positions(res["generation"], pos)   # stale token
    with pytest.raises(ValueError):
        ev._prepare_periodic_factorized_graph(types, pos, cell, np.linalg.inv(cell) * 2.0, 5.5)  # inconsistent inverse
    with pytest.raises(ValueError):
        ev._prepare_periodic_factorized_graph(types + 7, pos, cell, np.linalg.inv(cell), 5.5)     # type out of range
    bad = pos.copy()
    bad[1] = bad[0]                                                     # zero-length edge
    res3 = ev._prepare_periodic_factorized_graph(types, pos, cell, np.linalg.inv(cell), 5.5)
    with pytest.raises(ValueError):
        ev._compute_prepared_factorized_positions(res3["generation"], bad)


@pytest.mark.parametrize("scaled,zbl,agnesi", [(False, False, False), (True, False, False), (False, True, False), (True, False, True)])
def test_forces_are_energy_gradient(pkg, model_path, scaled, zbl, agnesi):
    """Finite-difference check (reference: symmetrix/test/test_mace.py:74-85)."""
    path = model_path("small", a0_scaled=scaled, a1_scaled=scaled, zbl=zbl, agnesi=agnesi)
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 4)
    calc = pkg.Calculator(path, skin=0.5)
    base = calc.calculate(pos, cell, types)
    h = 2e-3
    for atom, axis in ((0, 0), (7, 1), (13, 2)):
        p, m = pos.copy(), pos.copy()
        p[atom, axis] += h
        m[atom, axis] -= h
        ep = calc.calculate(p, cell, types)["energy"]
        em = calc.calculate(m, cell, types)["energy"]
        fd = -(ep - em) / (2 * h)
        assert abs(fd - base["forces"][atom, axis]) <= 5e-3 * max(1.0, abs(fd))


def test_graphless_force_and_stress_reduction(pkg, model_path):
    """Directed forces reduced from explicit edge lists (reference: _reduce_atom_forces /
    _reduce_stress with execution_graph_generation = 0) agree with the fused reduction."""
    path = model_path("small")
    pos, cell, types = pkg.modelgen.srtio3(3, 0.05, 6)
    first, src, shifts, xyz = csr_from_positions(pos, cell, 5.0)
    ev = pkg.MACEB200(path)
    gen = ev.compute_node_energies_forces(len(pos), types, np.diff(first), src, types[src], xyz)
    volume = abs(np.linalg.det(cell))
    fused_f = ev._reduce_atom_forces(len(pos), execution_graph_generation=gen)
    fused_s = ev._reduce_stress(volume, execution_graph_generation=gen)
    recv = np.repeat(np.arange(len(pos)), np.diff(first))
    f, s = pkg.reduce_edge_forces(len(pos), recv, src, ev.node_forces, xyz, volume)
    want_f, want_s = ref.reduce_forces_stress(len(pos), np.diff(first), src, ev.node_forces, xyz, volume)
    assert np.abs(f - want_f).max() < 1e-12 and np.abs(s - want_s).max() < 1e-14
    assert np.abs(f - fused_f).max() < 1e-6 and np.abs(s - fused_s).max() < 1e-8
    with pytest.raises(ValueError):
        pkg.reduce_edge_forces(len(pos), recv, src + 1000, ev.node_forces, xyz, volume)


@pytest.mark.parametrize("arch,cells,tile,scaled", [("small", (2, 2, 2), 4, False), ("small", (3, 2, 2), 7, False),
                                                    ("medium", (2, 2, 2), 16, False), ("medium", (3, 2, 2), 32, False),
                                                    ("medium", (2, 2, 2), 16, True), ("large", (2, 2, 2), 16, False)])
def test_tiled_streaming_matches_untiled(pkg, model_path, arch, cells, tile, scaled):
    """Tiled streaming with a reusable workspace against the one-tile evaluation
    (reference: symmetrix/test/test_dual_layer_fixed_workspace.py:104-146, rtol 2e-4 / atol 2e-5)."""
    path = model_path(arch, a0_scaled=scaled, a1_scaled=scaled)
    pos, cell, types = pkg.modelgen.srtio3(cells, 0.05, 12)
    plain = pkg.Calculator(path, skin=0.5)
    a = plain.calculate(pos, cell, types)
    h1_adj = plain.evaluator.stage("H1_adj")
    tiled = pkg.Calculator(path, skin=0.5)
    tiled.evaluator.set_tile_size(tile)
    b = tiled.calculate(pos, cell, types)
    b = tiled.calculate(pos, cell, types)         # the workspace is reused across evaluations
    assert abs(a["energy"] - b["energy"]) / len(pos) <= 1e-7
    assert np.abs(a["energies"] - b["energies"]).max() <= 1e-6
    assert np.abs(a["forces"] - b["forces"]).max() <= 1e-5
    assert np.abs(a["stress"] - b["stress"]).max() <= 1e-8
    got = tiled.evaluator.stage("H1_adj")
    assert np.abs(got - h1_adj).max() <= 2e-5 * max(1.0, np.abs(h1_adj).max())
    with pytest.raises(ValueError):
        tiled.evaluator.stage("Phi1")
    if ref.available():      # and directly against the reference's evaluator
        e, F, S = _reference_efs(path, pos, cell, types, tiled.evaluator.r_cut)
        _assert_matches_reference(b, e, F, S, len(pos))


def test_tile_boundary_sizes(pkg, model_path):
    """3, 4, 5, 8 and 9 atoms with a tile capacity of 4 (the reference's tile-boundary cases)."""
    path = model_path("small")
    rng = np.random.default_rng(5)
    for natoms in (3, 4, 5, 8, 9):
        cell = np.eye(3) * 9.0
        pos = rng.random((natoms, 3)) * 9.0
        for i in range(1, natoms):
            while np.min(np.linalg.norm(pos[:i] - pos[i], axis=1)) < 1.6:
                pos[i] = rng.random(3) * 9.0
        types = rng.integers(0, 3, size=natoms).astype(np.int32)
        a = pkg.Calculator(path, skin=0.5).calculate(pos, cell, types)
        calc = pkg.Calculator(path, skin=0.5)
        calc.evaluator.set_tile_size(4)
        b = calc.calculate(pos, cell, types)
        assert abs(a["energy"] - b["energy"]) <= 1e-6
        assert np.abs(a["forces"] - b["forces"]).max() <= 1e-5


@pytest.mark.parametrize("arch,zbl", [("medium", False), ("small", True)])
def test_reproducible_mode_gives_identical_bits(pkg, model_path, arch, zbl):
    """Fixed-order accumulation over the source schedule (the reference's source-sorted schedule,
    libsymmetrix/source/mace_kokkos_factorized_lifecycle.cpp:2133-2195): repeated evaluations, and a second
    evaluator, give bit-identical energies, forces, stress and source adjoints; the values agree with the
    default (atomic) mode and with the reference's evaluator within the tolerances."""
    path = model_path(arch, seed=12, zbl=zbl)
    pos, cell, types = pkg.modelgen.srtio3(3, 0.05, 31)
    runs = []
    for instance in range(2):
        calc = pkg.Calculator(path, skin=0.5)
        calc.evaluator.set_deterministic(True)
        for repeat in range(2):
            out = calc.calculate(pos, cell, types)
            runs.append((out["energy"], out["energies"].copy(), out["forces"].copy(), out["stress"].copy(),
                         calc.evaluator.stage("H1_adj")))
    for other in runs[1:]:
        assert other[0] == runs[0][0]
        for a, b in zip(other[1:], runs[0][1:]):
            assert np.array_equal(a, b)
    plain = pkg.Calculator(path, skin=0.5).calculate(pos, cell, types)
    assert abs(plain["energy"] - runs[0][0]) / len(pos) <= 1e-7
    assert np.abs(plain["forces"] - runs[0][2]).max() <= 1e-5
    assert np.abs(plain["stress"] - runs[0][3]).max() <= 1e-8
    if ref.available():
        e, F, S = _reference_efs(path, pos, cell, types, calc.evaluator.r_cut)
        _assert_matches_reference({"energy": runs[0][0], "energies": runs[0][1], "forces": runs[0][2], "stress": runs[0][3]}, e, F, S,
                                  len(pos))
    scaled = pkg.Calculator(model_path("small", a0_scaled=True, a1_scaled=True), skin=0.5)
    scaled.evaluator.set_deterministic(True)
    with pytest.raises(ValueError):
        scaled.calculate(pos, cell, types)


def test_nve_energy_conservation(pkg, model_path):
    """20 velocity-Verlet steps of 1 fs at 300 K: total energy is conserved to integrator accuracy."""
    path = model_path("small")
    pos, cell, types = pkg.modelgen.srtio3(3, 0.05, 3)
    z = np.array([8, 22, 38])[types]
    masses = np.array([pkg.md.MASSES[int(v)] for v in z])
    vel = pkg.md.maxwell_boltzmann(masses, 300.0, 3)
    ev = pkg.MACEB200(path)
    md = pkg.md.NVEIntegrator(ev, pos, cell, types, masses, vel, dt_fs=1.0, skin=0.5)
    e = md.run(20)
    drift = np.abs(e - e[0]).max() / len(pos)
    assert drift < 2e-4, drift          # eV/atom over 20 fs
    assert md.kinetic() > 0
