"""CPU tests of host-side helpers that need no device: the host neighbor list for open and mixed boundaries, the
velocity initialisation of the MD driver and the model generator's file variants."""
import itertools

import numpy as np
import pytest


def _brute_force(positions, cell, pbc, cutoff, reach=3):
    """All (receiver, source, image) triples with |r_j + image - r_i| <= cutoff, excluding the atom itself."""
    n = len(positions)
    ranges = [range(-reach, reach + 1) if p else range(0, 1) for p in pbc]
    out = {}
    for i in range(n):
        found = []
        for j in range(n):
            for s in itertools.product(*ranges):
                if i == j and s == (0, 0, 0):
                    continue
                d = positions[j] + np.array(s, dtype=np.float64) @ cell - positions[i]
                if np.sqrt((d * d).sum()) <= cutoff:
                    found.append((j, tuple(np.round(d, 9))))
        out[i] = sorted(found)
    return out


@pytest.mark.parametrize("pbc", [(False, False, False), (True, True, False), (True, False, False), (True, True, True)])
def test_host_neighbor_list_against_brute_force(pkg, pbc):
    rng = np.random.default_rng(11)
    cell = np.array([[7.0, 0.0, 0.0], [1.5, 6.5, 0.0], [-0.8, 0.9, 8.0]])
    positions = rng.random((18, 3)) @ cell          # inside the cell: wrapping along periodic axes changes nothing
    cutoff = 4.2
    num_neigh, neigh, xyz = pkg.evaluator.host_neighbor_list(positions, cell, pbc, cutoff)
    assert num_neigh.dtype == np.int32 and neigh.dtype == np.int32 and xyz.shape == (num_neigh.sum(), 3)
    want = _brute_force(positions, cell, pbc, cutoff)
    first = np.concatenate([[0], np.cumsum(num_neigh)])
    for i in range(len(positions)):
        got = sorted((int(j), tuple(np.round(v, 9))) for j, v in zip(neigh[first[i]:first[i + 1]], xyz[first[i]:first[i + 1]]))
        assert got == want[i], i
    # every edge has its twin
    lengths = np.sort(np.round(np.sqrt((xyz * xyz).sum(axis=1)), 9))
    assert len(lengths) % 2 == 0 and np.array_equal(lengths[0::2], lengths[1::2])


def test_host_neighbor_list_wraps_atoms_along_periodic_axes_only(pkg):
    cell = np.diag([6.0, 6.0, 6.0])
    positions = np.array([[0.5, 0.5, 0.5], [5.8, 0.5, 0.5], [0.5, 0.5, 13.0]])        # the third sits far out along z
    num_neigh, neigh, xyz = pkg.evaluator.host_neighbor_list(positions, cell, (True, True, False), 1.0)
    assert num_neigh.tolist() == [1, 1, 0] and neigh.tolist() == [1, 0]               # 0 and 1 meet across the x boundary
    assert np.allclose(xyz[0], [-0.7, 0.0, 0.0]) and np.allclose(xyz[1], [0.7, 0.0, 0.0])
    shifted = positions + np.array([12.0, -6.0, 0.0])                                  # lattice vectors along periodic axes
    again = pkg.evaluator.host_neighbor_list(shifted, cell, (True, True, False), 1.0)
    assert again[0].tolist() == [1, 1, 0] and np.allclose(again[2], xyz)


def test_maxwell_boltzmann_velocities(pkg):
    masses = np.tile([15.999, 47.867, 87.62], 4000)
    v = pkg.md.maxwell_boltzmann(masses, 300.0, 5)
    assert np.abs((masses[:, None] * v).sum(axis=0)).max() < 1e-9                      # no net momentum
    kinetic = 0.5 * pkg.md.KINETIC * (masses[:, None] * v * v).sum()
    temperature = 2.0 * kinetic / (3.0 * len(masses) * pkg.md.KB)
    assert abs(temperature - 300.0) < 6.0
    assert np.array_equal(v, pkg.md.maxwell_boltzmann(masses, 300.0, 5))               # seeded


def test_model_generator_variants_are_well_formed(pkg):
    """Keys each file variant must and must not carry (the reference loader's expectations:
    libsymmetrix/source/mace.cpp:2676-2737, h1_affine_schema.hpp:179-240)."""
    make = pkg.modelgen.make_model
    single = make("medium", 3, single_layer=True)
    assert single["num_interactions"] == 1 and single["single_layer_readout"] and "Phi1_l" not in single
    assert "R1" not in single["compact_radial"]["networks"] and "A1_weights" not in single
    assert max(max(t) for t in single["M1_monomials"]) < 4
    stored = make("small", 3, radial="pair-splines", num_spline_points=16, a0_scaled=True)
    assert "compact_radial" not in stored and len(stored["radial_spline_values_0"]) == 6
    assert len(stored["radial_spline_values_0"][0]) == 4 * 32 and len(stored["radial_spline_values_0"][0][0]) == 16
    assert all(abs(f[-1]) < 1e-12 for pair in stored["radial_spline_values_1"] for f in pair)      # ends at zero
    assert stored["A0_spline_h"] == stored["radial_spline_h"] and "A1_spline_values" not in stored
    old = make("small", 3, format_version=2)
    assert old["symmetrix_format_version"] == 2 and "h1_affine_mode" not in old and "readout_1_weights" in old
    split = make("small", 3, pre_linear_up=True, first_residual=True)
    C = split["num_channels"]
    P = np.asarray(split["H1_product_weights"]).reshape(-1, C, C)
    U = np.asarray(split["H1_linear_up_weights"]).reshape(-1, C, C)
    assert np.allclose(np.asarray(split["H1_weights"]).reshape(-1, C, C), P @ U)
    assert split["first_interaction_residual"] and len(split["H1_first_residual_weights"]) == 3 * 1 * C
    for bad in (dict(first_residual=True), dict(pre_linear_up=True, single_layer=True), dict(radial="pair-splines", agnesi=True),
                dict(format_version=3), dict(single_layer=True, a1_scaled=True)):
        with pytest.raises(ValueError):
            make("small", 3, **bad)
