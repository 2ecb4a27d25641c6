"""Seeded synthetic compact-MACE models and benchmark structures.

The reference's converter needs mace-torch/e3nn checkpoints, so models here are
written directly in its format-v4 "compact" JSON layout (keys as read by
libsymmetrix/source/mace.cpp:2660-2959 and compact_radial.cpp:110-215; the test
fixture symmetrix/test/compact_r1_model.py shows the same layout) with random
weights from ``numpy.random.default_rng(seed)``.  Weights are scaled so that every
stage tensor stays O(1) and the energy per atom is O(1) eV, which keeps the
FP32 parity tolerances meaningful.

Structures: cubic SrTiO3 perovskite supercells with Gaussian perturbation, and a
seeded Poisson-disk random solid with irregular neighbour counts.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

from . import structure as _structure

# Cubic index triples that the reference's standard medium contraction table lists
# (libsymmetrix/source/standard_m0.hpp:56-484: 118 terms for LM=1 and LM=3) although
# their coefficient vanishes identically for a rotation-equivariant model; kept so
# that a generated model has the same 422-term table as an exported checkpoint.
_EXTRA_M0_TERMS_L3_L1 = {
    "1": [[3, 4, 8], [3, 9, 15], [3, 10, 14], [4, 8, 13], [9, 13, 15], [10, 13, 14]],
    "3": [[1, 4, 8], [1, 9, 15], [1, 10, 14], [4, 8, 11], [9, 11, 15], [10, 11, 14]],
}

ARCHITECTURES = {
    # name: channels, edge l_max, hidden L_max, r_cut
    "small": dict(channels=32, l_max=3, L_max=0, r_cut=5.0),
    "medium": dict(channels=128, l_max=3, L_max=1, r_cut=6.0),
    "large": dict(channels=128, l_max=3, L_max=2, r_cut=6.0),
}


def model_tables(l_max: int, L_max: int) -> dict:
    """Structural tables (paths, couplings, monomials) for the given harmonics."""
    s = dict(_structure.model_structure(l_max, L_max))
    m0 = {k: [list(t) for t in v] for k, v in s["M0_monomials"].items()}
    if (l_max, L_max) == (3, 1):
        for key, extra in _EXTRA_M0_TERMS_L3_L1.items():
            merged = {tuple(t) for t in m0[key]} | {tuple(t) for t in extra}
            m0[key] = [list(t) for t in sorted(merged, key=lambda t: (len(t), t))]
    s["M0_monomials"] = m0
    s["M1_monomials"] = [list(t) for t in s["M1_monomials"]]
    return s


def make_model(arch: str = "medium", seed: int = 0, atomic_numbers=(8, 22, 38), *,
               channels: int | None = None, num_spline_points: int = 256,
               radial_hidden=(64, 64, 64), num_bessel: int = 8, cutoff_p: int = 5,
               a0_scaled: bool = False, a1_scaled: bool = False, zbl: bool = False,
               agnesi: bool = False, heads=(), radial: str = "compact", single_layer: bool = False,
               format_version: int = 4, pre_linear_up: bool = False, first_residual: bool = False) -> dict:
    """Random-weight model of architecture ``arch`` as a JSON-serialisable dict.  ``radial`` selects the
    radial representation: "compact" (radial networks) or "pair-splines" (stored nodal values and
    derivatives per unordered element pair, the exporter's older form)."""
    if radial not in ("compact", "pair-splines"):
        raise ValueError("radial must be 'compact' or 'pair-splines'")
    if radial == "pair-splines" and agnesi:
        raise ValueError("the distance transform belongs to the compact representation")
    if format_version not in (2, 4):
        raise ValueError("format_version must be 4 or 2 (the old basis: first readout and skip stored on H1)")
    if format_version == 2 and heads:
        raise ValueError("prediction heads need format version 4")
    if first_residual and not pre_linear_up:
        raise ValueError("a first-interaction residual needs the pre_linear_up basis")
    if pre_linear_up and (format_version != 4 or single_layer or heads):
        raise ValueError("the pre_linear_up basis is a format-4, two-interaction, single-head form")
    if single_layer and a1_scaled:
        raise ValueError("a single-layer model has no second message step to scale")
    cfg = dict(ARCHITECTURES[arch])
    C = int(channels or cfg["channels"])
    l_max, L_max, r_cut = cfg["l_max"], cfg["L_max"], float(cfg["r_cut"])
    tables = model_tables(l_max, L_max)
    rng = np.random.default_rng(seed)
    A = len(atomic_numbers)
    num_lm, num_LM = (l_max + 1) ** 2, (L_max + 1) ** 2
    paths = len(tables["Phi1_l"])
    eta = tables["eta"]

    def normal(*shape, scale=1.0):
        return rng.normal(size=shape) * scale

    def network(out_width, out_scale, postprocess=None):
        shape = [num_bessel, *radial_hidden, out_width]
        weights = []
        for layer in range(len(shape) - 1):
            fan_in, fan_out = shape[layer], shape[layer + 1]
            w = normal(fan_out, fan_in, scale=1.0 / np.sqrt(fan_in))
            if layer == 0:
                w *= 0.2 if agnesi else 2.0  # Bessel features are O(0.3); O(3) in the transformed distance
            if layer == len(shape) - 2:
                w *= out_scale
            weights.append(w.reshape(-1).tolist())
        net = {"shape": shape, "weights": weights, "activation": "silu",
               "activation_scale": 1.679177}
        if postprocess:
            net["postprocess"] = postprocess
        return net

    # the transformed distance makes the channels more coherent: a smaller output scale keeps every stage O(1)
    radial_scale = 0.25 if agnesi else 0.4
    networks = {"R0": network((l_max + 1) * C, radial_scale), "R1": network(paths * C, radial_scale)}
    if a0_scaled:
        networks["A0"] = network(1, 0.3, "tanh-square")
    if a1_scaled:
        networks["A1"] = network(1, 0.3, "tanh-square")

    m0_monomials = tables["M0_monomials"]
    m1_monomials = tables["M1_monomials"]

    def poly_weights(L, count):
        """Equivariant contraction weights of output irrep L for ``count`` (element, channel)
        slots: one random weight per coupling chain, shared by all components M, expanded
        onto the monomial table (terms outside the derived set keep weight zero)."""
        derived, chains = _structure.contraction_basis(l_max, L)
        degree = np.array([d for d, _ in chains])
        scale = np.where(degree == 1, 0.7, np.where(degree == 2, 0.35, 0.25))
        w = rng.normal(size=(count, len(chains))) * scale
        per_m = []
        for M in range(2 * L + 1):
            table = m0_monomials[str(L * L + M)]
            basis = np.zeros((len(chains), len(table)))
            position = {tuple(t): i for i, t in enumerate(table)}
            cols = [position[t] for t in derived[M]]
            for c, (_, coeff) in enumerate(chains):
                basis[c, cols] = coeff[M]
            per_m.append(w @ basis)
        return per_m

    M0_weights = {str(a): {} for a in range(A)}
    for L in range(L_max + 1):
        per_m = poly_weights(L, A * C)
        for M in range(2 * L + 1):
            vals = per_m[M].reshape(A, C, -1)
            for a in range(A):
                M0_weights[str(a)][str(L * L + M)] = {str(k): vals[a, k].tolist() for k in range(C)}
    if single_layer:
        # one interaction: the readout polynomial acts on H1, its monomials index the (L_max+1)^2 hidden components
        derived, chains = _structure.contraction_basis(L_max, 0)
        m1_monomials = [list(t) for t in derived[0]]
        degree = np.array([d for d, _ in chains])
        w = rng.normal(size=(A * C, len(chains))) * np.where(degree == 1, 0.7, np.where(degree == 2, 0.35, 0.25))
        m1_vals = (w @ np.stack([coeff[0] for _, coeff in chains])).reshape(A, C, -1)
    else:
        m1_vals = poly_weights(0, A * C)[0].reshape(A, C, -1)
    M1_weights = {str(a): {str(k): m1_vals[a, k].tolist() for k in range(C)} for a in range(A)}

    model = {
        "symmetrix_format_version": 4,
        "h1_affine_mode": "m0_composite",
        "h1_affine_version": 1,
        "radial_representation": "compact",
        "model_type": "MACE",
        "num_elements": A,
        "num_channels": C,
        "num_interactions": 2,
        "r_cut": r_cut,
        "l_max": l_max,
        "L_max": L_max,
        "atomic_numbers": [int(z) for z in atomic_numbers],
        "atomic_energies": (-1.0 - 0.5 * rng.random(A)).tolist(),
        "has_zbl": bool(zbl),
        **({"zbl_a_exp": 0.3, "zbl_a_prefactor": 0.4543, "zbl_c": [0.1818, 0.5099, 0.2802, 0.02817], "zbl_p": 6,
            # synthetic covalent radii indexed by atomic number (a smooth stand-in, not a literature table)
            "zbl_covalent_radii": [0.0] + [round(0.6 + 0.45 * np.log1p(z) / np.log(10.0), 4) for z in range(1, 119)]}
           if zbl else {}),
        "H0_weights": normal(A * C).tolist(),
        "A0_weights": [[normal(C * C, scale=1.0 / np.sqrt(C)).tolist() for _ in range(l_max + 1)]
                       for _ in range(A)],
        "A0_scaled": bool(a0_scaled),
        "compact_radial": {
            "spline_grid_min": 1e-12,
            "num_spline_points": int(num_spline_points),
            "basis": {
                "type": "bessel",
                "weights": [float((n + 1) * np.pi / r_cut) for n in range(num_bessel)],
                "prefactor": float(np.sqrt(2.0 / r_cut)),
            },
            "cutoff": {"type": "polynomial", "r_max": r_cut, "p": int(cutoff_p)},
            # synthetic covalent radii per element slot (a smooth stand-in, not a literature table)
            "distance_transform": ({"type": "agnesi", "a": 1.0805, "q": 0.9183, "p": 4.5791,
                                    "covalent_radii": [round(0.6 + 0.45 * float(np.log1p(z)) / float(np.log(10.0)), 4)
                                                       for z in atomic_numbers]}
                                   if agnesi else {"type": "none"}),
            "networks": networks,
        },
        "M0_monomials": m0_monomials,
        "M0_weights": M0_weights,
        "H1_weights": normal((L_max + 1) * C * C, scale=1.0 / np.sqrt(C)).tolist(),
        "has_field_coupling": False,
        "field_couplings": [],
        "Phi1_l": tables["Phi1_l"],
        "Phi1_l1": tables["Phi1_l1"],
        "Phi1_l2": tables["Phi1_l2"],
        "Phi1_lme": tables["Phi1_lme"],
        "Phi1_lelm1lm2": tables["Phi1_lelm1lm2"],
        "Phi1_clebsch_gordan": tables["Phi1_clebsch_gordan"],
        "A1_weights": [normal(eta[l] * C * C, scale=1.0 / np.sqrt(eta[l] * C)).tolist()
                       for l in range(l_max + 1)],
        "A1_scaled": bool(a1_scaled),
        "M1_monomials": m1_monomials,
        "M1_weights": M1_weights,
        "H2_weights_for_M0": [normal(C * C, scale=1.0 / np.sqrt(C)).tolist() for _ in range(A)],
        "H2_weights_for_M1": normal(C * C, scale=1.0 / np.sqrt(C)).tolist(),
        "readout_1_weights_for_M0": normal(C, scale=1.0 / np.sqrt(C)).tolist(),
        "readout_2_weights_1": normal(16 * C, scale=1.0 / np.sqrt(C)).tolist(),
        "readout_2_weights_2": normal(16, scale=0.25).tolist(),
        "readout_2_hidden_size": 16,
        "readout_2_scale_factor": 1.679177,
    }
    if pre_linear_up:
        # the file keeps the product map P and linear_up U apart (H1_weights = P U still feeds the second interaction);
        # the first readout and the skip act on x = M0[l=0] P0 (+ the residual's scalar block)
        P = normal(L_max + 1, C, C, scale=1.0 / np.sqrt(C))
        U = normal(L_max + 1, C, C, scale=1.0 / np.sqrt(C)) + np.eye(C)[None] * 0.5
        model["h1_affine_mode"] = "pre_linear_up"
        model["H1_product_weights"] = P.reshape(-1).tolist()
        model["H1_linear_up_weights"] = U.reshape(-1).tolist()
        model["H1_weights"] = np.einsum("lij,ljk->lik", P, U).reshape(-1).tolist()
        model["readout_1_weights_for_H1_pre_linear_up"] = model.pop("readout_1_weights_for_M0")
        model["H2_weights_for_H1_pre_linear_up"] = model.pop("H2_weights_for_M0")
        if first_residual:
            model["first_interaction_residual"] = True
            residual = np.zeros((A, num_LM, C))
            residual[:, 0, :] = normal(A, C, scale=0.3)      # an element-dependent constant on the scalar block
            model["H1_first_residual_weights"] = residual.reshape(-1).tolist()
    if format_version == 2:
        # old basis (format versions 1 / 2): the first readout and the H1 -> H2 skip act on the scalar block of H1
        model["symmetrix_format_version"] = 2
        del model["h1_affine_mode"], model["h1_affine_version"]
        model["readout_1_weights"] = model.pop("readout_1_weights_for_M0")
        model["H2_weights_for_H1"] = model.pop("H2_weights_for_M0")
        if single_layer:
            # exported single-layer models carry a zero first readout; the reference's serial evaluator relies on it (it
            # clears the readout's adjoint on its single-layer path, libsymmetrix/source/mace.cpp:265-271)
            model["readout_1_weights"] = [0.0] * C
    if single_layer:
        # H1 feeds a cubic polynomial directly: keep it O(1) so that the readout stays well conditioned in FP32
        model["H1_weights"] = (0.3 * np.asarray(model["H1_weights"])).tolist()
        model["num_interactions"] = 1
        model["single_layer_readout"] = True
        for key in ("Phi1_l", "Phi1_l1", "Phi1_l2", "Phi1_lme", "Phi1_lelm1lm2", "Phi1_clebsch_gordan", "A1_weights"):
            del model[key]
        del model["compact_radial"]["networks"]["R1"]
    if radial == "pair-splines":
        # Stored pair splines on the exporter's grid linspace(1e-12, r_cut, points): smooth random
        # functions sum_b c_b sin(b pi r / r_cut) under the polynomial cutoff envelope, with their exact
        # derivatives; every unordered element pair (a <= b, row by row) gets coefficients of its own.
        del model["compact_radial"]
        model["radial_representation"] = "pair-splines"
        r, h = np.linspace(1e-12, r_cut, int(num_spline_points), retstep=True)
        u = r / r_cut
        p = float(cutoff_p)
        envelope = 1.0 - (p + 1) * (p + 2) / 2 * u ** p + p * (p + 2) * u ** (p + 1) - p * (p + 1) / 2 * u ** (p + 2)
        d_envelope = (-(p + 1) * (p + 2) / 2 * p * u ** (p - 1) + p * (p + 2) * (p + 1) * u ** p
                      - p * (p + 1) / 2 * (p + 2) * u ** (p + 1)) / r_cut
        envelope[-1] = d_envelope[-1] = 0.0
        k = np.arange(1, num_bessel + 1) * np.pi / r_cut
        waves = np.sin(np.outer(k, r))                      # [b][node]
        d_waves = k[:, None] * np.cos(np.outer(k, r))

        # amplitudes chosen so that the sums over ~50 neighbours keep every stage O(1), as the compact models do
        def functions(count, scale):
            c = rng.normal(size=(count, num_bessel)) * scale / np.sqrt(num_bessel)
            g, dg = c @ waves, c @ d_waves
            return g * envelope, dg * envelope + g * d_envelope

        tables = {key: [] for key in ("radial_spline_values_0", "radial_spline_derivs_0", "radial_spline_values_1",
                                      "radial_spline_derivs_1", "A0_spline_values", "A0_spline_derivs",
                                      "A1_spline_values", "A1_spline_derivs")}
        for a in range(A):
            for b in range(a, A):
                v, d = functions((l_max + 1) * C, 0.08)
                tables["radial_spline_values_0"].append(v.tolist())
                tables["radial_spline_derivs_0"].append(d.tolist())
                if not single_layer:
                    v, d = functions(paths * C, 0.08)
                    tables["radial_spline_values_1"].append(v.tolist())
                    tables["radial_spline_derivs_1"].append(d.tolist())
                for name, on in (("A0", a0_scaled), ("A1", a1_scaled)):
                    if on:   # tanh(g^2), as the exporter stores the density functions
                        g, dg = functions(1, 0.8)
                        tables[name + "_spline_values"].append(np.tanh(g[0] ** 2).tolist())
                        tables[name + "_spline_derivs"].append((2.0 * g[0] * dg[0] / np.cosh(g[0] ** 2) ** 2).tolist())
        model["radial_spline_h"] = float(h)
        model["radial_spline_min"] = float(r[0])
        for key in ("radial_spline_values_0", "radial_spline_derivs_0", "radial_spline_values_1", "radial_spline_derivs_1"):
            if tables[key]:
                model[key] = tables[key]
        for name, on in (("A0", a0_scaled), ("A1", a1_scaled)):
            if on:
                model[name + "_spline_h"] = float(h)
                model[name + "_spline_min"] = float(r[0])
                model[name + "_spline_values"] = tables[name + "_spline_values"]
                model[name + "_spline_derivs"] = tables[name + "_spline_derivs"]
    if heads:
        # multi-head file (schema of libsymmetrix/source/prediction_heads.hpp:10-90): every head carries its own
        # atomic energies, readouts and ZBL coefficients; the last head is the default, the top level holds the first
        fields = ["atomic_energies", "readout_1_weights_for_M0", "readout_2_weights_1", "readout_2_weights_2"]
        if zbl:
            fields.append("zbl_c")
        parameters = {}
        for index, name in enumerate(heads):
            payload = {key: model[key] for key in fields}
            if index > 0:
                payload = {"atomic_energies": (-1.0 - 0.5 * rng.random(A)).tolist(),
                           "readout_1_weights_for_M0": normal(C, scale=1.0 / np.sqrt(C)).tolist(),
                           "readout_2_weights_1": normal(16 * C, scale=1.0 / np.sqrt(C)).tolist(),
                           "readout_2_weights_2": normal(16, scale=0.25).tolist(),
                           **({"zbl_c": [0.2, 0.5, 0.25, 0.05]} if zbl else {})}
            parameters[name] = payload
        model["prediction_heads"] = {"schema_version": 1, "names": list(heads), "default": heads[-1],
                                     "parameters": parameters}
    return model


def write_model(path, arch: str = "medium", seed: int = 0, **kwargs) -> Path:
    path = Path(path)
    path.write_text(json.dumps(make_model(arch, seed, **kwargs), separators=(",", ":")))
    return path


# ----------------------------------------------------------------------------- structures
SRTIO3_A = 3.905
# type indices into atomic_numbers (8, 22, 38) = (O, Ti, Sr)
_SRTIO3_BASIS = [((0.0, 0.0, 0.0), 2), ((0.5, 0.5, 0.5), 1),
                 ((0.5, 0.5, 0.0), 0), ((0.5, 0.0, 0.5), 0), ((0.0, 0.5, 0.5), 0)]


def srtio3(n, sigma: float = 0.05, seed: int = 17, a: float = SRTIO3_A):
    """n x n x n (or (nx,ny,nz)) cubic SrTiO3 supercell, every coordinate + N(0, sigma^2).

    Returns (positions f64 [N,3], cell f64 [3,3], types i32 [N]); types index the
    default ``atomic_numbers`` (8, 22, 38)."""
    nx, ny, nz = (n, n, n) if np.isscalar(n) else n
    gx, gy, gz = np.meshgrid(np.arange(nx), np.arange(ny), np.arange(nz), indexing="ij")
    cells = np.stack([gx.ravel(), gy.ravel(), gz.ravel()], axis=1).astype(np.float64)
    basis = np.array([b[0] for b in _SRTIO3_BASIS])
    types = np.array([b[1] for b in _SRTIO3_BASIS], dtype=np.int32)
    pos = (cells[:, None, :] + basis[None, :, :]).reshape(-1, 3) * a
    typ = np.tile(types, cells.shape[0])
    rng = np.random.default_rng(seed)
    pos = pos + rng.normal(scale=sigma, size=pos.shape)
    cell = np.diag([nx * a, ny * a, nz * a]).astype(np.float64)
    return pos, cell, typ.astype(np.int32)


def random_solid(num_atoms: int = 20000, density: float = 0.085, min_dist: float = 1.8,
                 num_types: int = 10, seed: int = 0):
    """Seeded Poisson-disk (dart throwing on a cell grid) disordered solid in a periodic cube."""
    rng = np.random.default_rng(seed)
    L = (num_atoms / density) ** (1.0 / 3.0)
    ncell = max(1, int(L / min_dist))
    h = L / ncell
    grid: dict = {}
    pts = []
    while len(pts) < num_atoms:
        cand = rng.random((4 * num_atoms, 3)) * L
        for p in cand:
            c = tuple((p // h).astype(int) % ncell)
            ok = True
            for dx in (-1, 0, 1):
                for dy in (-1, 0, 1):
                    for dz in (-1, 0, 1):
                        for q in grid.get(((c[0] + dx) % ncell, (c[1] + dy) % ncell, (c[2] + dz) % ncell), ()):
                            d = p - q
                            d -= L * np.round(d / L)
                            if d @ d < min_dist * min_dist:
                                ok = False
                                break
                        if not ok:
                            break
                    if not ok:
                        break
                if not ok:
                    break
            if ok:
                grid.setdefault(c, []).append(p)
                pts.append(p)
                if len(pts) == num_atoms:
                    break
    pos = np.array(pts)
    types = rng.integers(0, num_types, size=num_atoms).astype(np.int32)
    return pos, np.eye(3) * L, types
