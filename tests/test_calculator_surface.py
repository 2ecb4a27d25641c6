"""The evaluator surface the reference's ASE calculator drives (symmetrix/source/symmetrix/calculator.py:3162-3403),
replayed call by call: host-graph branch with a Cartesian or fractional reference geometry, cell updates,
non-periodic and mixed-periodic systems, and the attributes the calculator reads."""
import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu

TOL_E, TOL_F, TOL_S = 1e-5, 1e-4, 1e-6


def _reference(path, types, num_neigh, neigh, xyz):
    m = ref.ReferenceMACE(str(path), double=False)
    m.compute(types, num_neigh, neigh, xyz)
    forces = np.zeros((len(types), 3))
    recv = np.repeat(np.arange(len(types)), num_neigh)
    f = m.get("node_forces").reshape(-1, 3)
    np.add.at(forces, neigh, f)
    np.add.at(forces, recv, -f)
    return m.get("node_energies"), forces


def test_attribute_surface(pkg, model_path):
    ev = pkg.MACEB200(model_path("small"))
    assert ev.supports_streamed_edges() and ev.streamed_edges_mode == "direct"
    ev.set_streamed_edges("direct")
    with pytest.raises(ValueError):
        ev.set_streamed_edges("materialized")
    assert len(ev.atomic_energies) == len(ev.atomic_numbers) == 3 and ev.r_cut == 5.0
    assert ev.l_max == 3 and ev.L_max == 0 and not ev.single_layer_readout and ev.h1_affine_mode == "m0_composite"
    report = ev.execution_plan_report
    assert report["state"] == "pending" and report["candidates"][0]["qualified"]
    ev._validate_graph_cardinality(10, 12, 100)
    with pytest.raises(ValueError):
        ev._validate_graph_cardinality(10, 5, 100)
    with pytest.raises(ValueError):
        ev._validate_graph_cardinality(10, 12, 2 ** 31)
    # the calculator hands over the kernel plugin it built for its direct mode: a real plugin is accepted and recorded
    # (the compiled-in kernels keep serving the stage), anything else is refused
    with pytest.raises(RuntimeError):
        ev._load_jit_cuda_plugin("plugin.so")
    assert not ev.jit_cuda_plugin_ready
    ev._load_jit_cuda_plugin(pkg.LIBRARY_PATH, 4)       # this library exports the plugin query itself
    assert ev.jit_cuda_plugin_ready and ev.jit_cuda_plugin_artifact_id == "symmetrix-xl-b200-r1-32-l3-L0"
    environment = ev.device_cuda_environment
    assert environment["available"] and environment["backend"] == "cuda" and environment["compute_capability_code"] == 100
    assert environment["multiprocessor_count"] > 0 and environment["warp_width"] == 32
    wide = ev.execution_device_execution_environment
    assert wide["execution_space"] == "Cuda" and wide["device_memory"] > 0 and wide["architecture"] == "sm_100"
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 1)
    ev._prepare_periodic_factorized_graph(types, pos, cell, np.linalg.inv(cell), 5.5)
    report = ev.execution_plan_report
    assert report["state"] == "resolved" and report["candidates"][0]["estimated_bytes"] > 0 and report["available_bytes"] > 0


@pytest.mark.parametrize("pbc", [(False, False, False), (True, True, False), (True, False, False)])
def test_open_and_mixed_periodic_systems_through_the_host_graph(pkg, model_path, pbc):
    """Clusters, slabs and wires: list and reference edge vectors from the host, then evaluations from
    moved positions; against the reference's evaluator on the moved structure's own list."""
    if not ref.available():
        pytest.skip("oracle/_ref was not built")
    path = model_path("medium", seed=9)
    pos, cell, types = pkg.modelgen.srtio3((3, 3, 2), 0.05, 21)
    calc = pkg.Calculator(path, skin=0.5)
    first = calc.calculate(pos, cell, types, pbc=pbc)
    assert "stress" not in first
    moved = pos + np.random.default_rng(1).normal(scale=0.04, size=pos.shape)
    moved[3] += cell[0] * (1 if pbc[0] else 0)            # an atom that crossed the periodic boundary keeps its edges
    out = calc.calculate(moved, cell, types, pbc=pbc)
    assert calc.rebuilds == 1
    work_cell = cell.copy()
    for a in range(3):
        if not pbc[a]:
            work_cell[a] = 0.0
            work_cell[a, a] = 200.0
    num_neigh, neigh, xyz = pkg.evaluator.host_neighbor_list(moved, work_cell, pbc, calc.evaluator.r_cut)
    energies, forces = _reference(path, types, num_neigh, neigh, xyz)
    assert abs(out["energy"] - energies.sum()) / len(pos) <= TOL_E
    assert np.abs(out["energies"] - energies).max() <= TOL_E
    assert np.abs(out["forces"] - forces).max() <= TOL_F


def test_fractional_reference_geometry_and_cell_update(pkg, model_path):
    """The host-graph branch with fractional geometry (calculator.py:3283-3318): one list, then an affine
    change of the cell through _update_factorized_cell; against a fresh periodic evaluation."""
    path = model_path("small", seed=2)
    pos, cell, types = pkg.modelgen.srtio3(3, 0.05, 5)
    ev = pkg.MACEB200(path)
    pbc = (True, True, True)
    num_neigh, neigh, xyz = pkg.evaluator.host_neighbor_list(pos, cell, pbc, ev.r_cut + 0.5)
    ev._validate_graph_cardinality(len(pos), len(pos), len(neigh))
    gen = ev._prepare_factorized_graph(len(pos), types, num_neigh, neigh, types[neigh])
    inv = np.linalg.inv(cell)
    ev._prepare_factorized_fractional_geometry(gen, pos @ inv, xyz @ inv, cell, inv, np.array(pbc, dtype=np.int32))
    ev._compute_prepared_factorized_positions(gen, pos)
    want = pkg.Calculator(path, skin=0.5).calculate(pos, cell, types)
    assert abs(ev.node_energies.sum() - want["energy"]) / len(pos) <= 1e-6
    assert np.abs(ev._reduce_atom_forces(len(pos), execution_graph_generation=gen) - want["forces"]).max() <= 1e-5
    strain = np.eye(3) + np.array([[0.004, 0.002, 0.0], [0.0, -0.003, 0.001], [0.0, 0.0, 0.002]])
    new_cell, new_pos = cell @ strain, pos @ strain
    ev._update_factorized_cell(gen, new_cell, np.linalg.inv(new_cell))
    ev._compute_prepared_factorized_positions(gen, new_pos)
    want = pkg.Calculator(path, skin=0.5).calculate(new_pos, new_cell, types)
    assert abs(ev.node_energies.sum() - want["energy"]) / len(pos) <= 1e-6
    assert np.abs(ev._reduce_atom_forces(len(pos), execution_graph_generation=gen) - want["forces"]).max() <= 1e-5
    stress = ev._reduce_stress(abs(np.linalg.det(new_cell)), execution_graph_generation=gen)
    assert np.abs(stress - want["stress"]).max() <= 1e-7
    with pytest.raises(ValueError):
        ev._update_factorized_cell(gen + 1, new_cell, np.linalg.inv(new_cell))          # stale token
    with pytest.raises(ValueError):
        ev._update_factorized_cell(gen, new_cell, np.linalg.inv(cell) * 2.0)            # not the inverse


def test_affine_cell_change_reuses_the_neighbor_list(pkg, model_path):
    """A small homogeneous strain of a periodic cell keeps the device graph (calculator.py:2857-2888)."""
    path = model_path("small", seed=2)
    pos, cell, types = pkg.modelgen.srtio3(3, 0.05, 6)
    calc = pkg.Calculator(path, skin=0.5)
    calc.calculate(pos, cell, types)
    strain = np.eye(3) * 1.003
    got = calc.calculate(pos @ strain, cell @ strain, types)
    assert calc.rebuilds == 1 and calc.cell_updates == 1
    want = pkg.Calculator(path, skin=0.5).calculate(pos @ strain, cell @ strain, types)
    assert abs(got["energy"] - want["energy"]) / len(pos) <= 1e-6
    assert np.abs(got["forces"] - want["forces"]).max() <= 1e-5
    assert np.abs(got["stress"] - want["stress"]).max() <= 1e-7
    big = np.eye(3) * 1.08
    calc.calculate(pos @ big, cell @ big, types)
    assert calc.rebuilds == 2                      # a large strain rebuilds


def test_ensemble_returns_mean_committee_and_variance(pkg, model_path):
    """Committee of models evaluated in one process (symmetrix/source/symmetrix/ensemble.py:166-212)."""
    paths = [model_path("small", seed=s) for s in (31, 32, 33)]
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 8)
    ensemble = pkg.EnsembleCalculator(paths, skin=0.5)
    out = ensemble.calculate(pos, cell, types)
    singles = [pkg.Calculator(p, skin=0.5).calculate(pos, cell, types) for p in paths]
    assert ensemble.num_models == 3 and out["forces_comm"].shape == (3, len(pos), 3) and out["stress_comm"].shape == (3, 3, 3)
    for name in ("energy", "energies", "forces", "stress"):
        stack = np.stack([np.asarray(s[name]) for s in singles])
        assert np.abs(out[name + "_comm"] - stack).max() <= 1e-4
        assert np.allclose(out[name], out[name + "_comm"].mean(axis=0))
        assert np.allclose(out[name + "_var"], out[name + "_comm"].var(axis=0))
    assert isinstance(out["energy"], float) and out["energy_var"] > 0.0
    with pytest.raises(ValueError):
        pkg.EnsembleCalculator(paths, calculators=ensemble.calculators)
    with pytest.raises(ValueError):
        pkg.EnsembleCalculator(calculators=ensemble.calculators, skin=0.5)
    with pytest.raises(ValueError):
        pkg.EnsembleCalculator(calculators=[ensemble.calculators[0], pkg.Calculator(paths[1], skin=0.3)])
    with pytest.raises(ValueError):
        pkg.EnsembleCalculator(calculators=[ensemble.calculators[0], pkg.Calculator(model_path("medium", seed=31), skin=0.5)])
    with pytest.raises(TypeError):
        pkg.EnsembleCalculator(calculators=[ensemble.calculators[0], object()])
