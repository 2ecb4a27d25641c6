"""Generates the golden fixtures of tests/golden/ from the reference's own code.

Run where the reference checkout is present, naming it as the first argument or in REFERENCE_ROOT
(the same variable oracle/Makefile reads):

    python tests/golden/make_golden.py <reference checkout> [evaluator] [variants] [harmonics] [structure]

1. reference_evaluator_<arch>.npz -- energies, directed edge forces and stage-tensor checksums of
   the reference's serial evaluator MACECPU<double> (built into oracle/_ref from the checkout's
   sources) on a small seeded SrTiO3 cell with a seeded synthetic model of each architecture.
   reference_evaluator_variant_<name>.npz -- the same for the model-file variants of variants.json.
2. harmonics_reference.npz -- Y_lm and their Cartesian gradients from the reference's first-party
   closed forms for l <= 3: the C text its generator emits for the device force kernels
   (symmetrix/source/symmetrix/jit_codegen.py, _render_direct_harmonic_gradient_helper, and the
   value table in the same file) is rendered, compiled with g++ and evaluated on seeded directions.
3. structure_reference.json -- path list, sparse coupling (row, lme, |coefficient|) and monomial tables
   read from the reference's execution-contract fixtures, to pin the first-principles derivation in
   symmetrix-xl_b200/structure.py.
The fixtures are outputs (numbers), not reference source.
"""
from __future__ import annotations

import ctypes
import importlib
import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
_reference_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
if not _reference_root:
    raise SystemExit("usage: make_golden.py <reference checkout>   (or set REFERENCE_ROOT)")
REFERENCE = Path(_reference_root)
OUT = Path(__file__).resolve().parent

import __graft_entry__ as graft  # noqa: E402


def float_deviation(ref, path, types, first, src, xyz, cell, reference_double):
    """[max |dE_node|, max |dF_atom|, max |dsigma|] between the reference's own float and double evaluators on this
    input: the FP32 resolution of the model itself, which a parity bound cannot undercut."""
    n = len(types)
    volume = abs(np.linalg.det(cell))
    m = ref.ReferenceMACE(str(path), double=False)
    m.compute(types, np.diff(first), src, xyz)
    Ff, Sf = ref.reduce_forces_stress(n, np.diff(first), src, m.get("node_forces"), xyz, volume)
    Fd, Sd = ref.reduce_forces_stress(n, np.diff(first), src, reference_double.get("node_forces"), xyz, volume)
    return np.array([np.abs(m.get("node_energies") - reference_double.get("node_energies")).max(), np.abs(Ff - Fd).max(),
                     np.abs(Sf - Sd).max()])


def evaluator_goldens():
    from oracle import neighbor, ref

    pkg = graft.load_package()
    # the third case is a density-scaled model (A0_scaled and A1_scaled, mace.cpp:1562-1636, 2381-2458)
    # and the fourth has hidden irreps up to l = 2 (17 paths, 243 rows)
    # the fifth adds the screened-Coulomb (ZBL) pair term (zbl.cpp), the sixth the Agnesi distance
    # transform (species-pair dependent radial tables, compact_radial.cpp:227-267) with density scaling and ZBL
    for arch, cells, cutoff, scaled, zbl, agnesi in (("small", 2, 5.0, False, False, False), ("medium", 2, 6.0, False, False, False),
                                                     ("medium", 2, 6.0, True, False, False), ("large", 2, 6.0, False, False, False),
                                                     ("small", 2, 5.0, False, True, False), ("small", 2, 5.0, True, True, True)):
        with tempfile.TemporaryDirectory() as tmp:
            path = Path(tmp) / "model.json"
            pkg.modelgen.write_model(path, arch, seed=101, a0_scaled=scaled, a1_scaled=scaled, zbl=zbl, agnesi=agnesi)
            pos, cell, types = pkg.modelgen.srtio3(cells, 0.05, 202)
            first, src, shifts = neighbor.build_neighbor_graph(pos, cell, cutoff)
            xyz = neighbor.edge_vectors(pos, cell, first, src, shifts)
            m = ref.ReferenceMACE(str(path), double=True)
            m.compute(types, np.diff(first), src, xyz)
            data = {"positions": pos, "cell": cell, "types": types, "first": first, "sources": src, "shifts": shifts,
                    "node_energies": m.get("node_energies"), "edge_forces": m.get("node_forces"),
                    "float_deviation": float_deviation(ref, path, types, first, src, xyz, cell, m)}
            for name in ("A0", "M0", "H1", "Phi1", "A1", "M1", "H2", "H1_adj", "A0_adj"):
                v = m.get(name)
                data["sum_" + name] = np.array([v.sum(), np.abs(v).sum(), (v * v).sum()])
            np.savez_compressed(OUT / f"reference_evaluator_{arch}{'_scaled' if scaled else ''}{'_zbl' if zbl else ''}{'_agnesi' if agnesi else ''}.npz", **data)
            print("wrote", arch, len(pos), "atoms", len(src), "edges")


def variant_goldens():
    """reference_evaluator_variant_<name>.npz: the model-file variants of tests/golden/variants.json (stored pair splines,
    one interaction, the old basis of formats 1 / 2, the pre_linear_up basis with a first-interaction residual), each
    evaluated by MACECPU<double> on the 40-atom cell."""
    from oracle import neighbor, ref

    pkg = graft.load_package()
    variants = json.loads((OUT / "variants.json").read_text())
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 202)
    for name, entry in variants.items():
        if name.startswith("_"):
            continue
        arch, kwargs = entry
        cutoff = pkg.modelgen.ARCHITECTURES[arch]["r_cut"]
        first, src, shifts = neighbor.build_neighbor_graph(pos, cell, cutoff)
        xyz = neighbor.edge_vectors(pos, cell, first, src, shifts)
        with tempfile.TemporaryDirectory() as tmp:
            path = Path(tmp) / "model.json"
            pkg.modelgen.write_model(path, arch, seed=101, **kwargs)
            m = ref.ReferenceMACE(str(path), double=True)
            m.compute(types, np.diff(first), src, xyz)
            data = {"positions": pos, "cell": cell, "types": types, "first": first, "sources": src, "shifts": shifts,
                    "node_energies": m.get("node_energies"), "edge_forces": m.get("node_forces"),
                    "float_deviation": float_deviation(ref, path, types, first, src, xyz, cell, m)}
            for stage in ("A0", "M0", "H1", "M1", "H2"):
                v = m.get(stage)
                data["sum_" + stage] = np.array([v.sum(), np.abs(v).sum(), (v * v).sum()])
            np.savez_compressed(OUT / f"reference_evaluator_variant_{name}.npz", **data)
            print("wrote variant", name)


def harmonics_goldens():
    sys.path.insert(0, str(REFERENCE / "symmetrix" / "source"))
    codegen = importlib.import_module("symmetrix.jit_codegen")
    helper = codegen._render_direct_harmonic_gradient_helper("static", 16)
    source = f"""
#include <cmath>
#include <cstddef>
#include <cstdint>
using Scalar = double;
{helper}
extern "C" void golden_gradients(const double* xyz, double radius, double* out) {{
    direct_harmonic_gradients(xyz, sizeof(double), 0u, 0, radius, out);
}}
"""
    rng = np.random.default_rng(77)
    vectors = rng.normal(size=(40, 3)) * rng.uniform(0.8, 5.5, size=(40, 1))
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "h.cpp"
        lib = Path(tmp) / "h.so"
        src.write_text(source)
        subprocess.run(["g++", "-O2", "-shared", "-fPIC", "-o", str(lib), str(src)], check=True)
        dll = ctypes.CDLL(str(lib))
        grads = np.zeros((len(vectors), 3, 16))
        for i, v in enumerate(vectors):
            v = np.ascontiguousarray(v)
            out = np.zeros(48)
            dll.golden_gradients(v.ctypes.data_as(ctypes.c_void_p), ctypes.c_double(float(np.linalg.norm(v))),
                                 out.ctypes.data_as(ctypes.c_void_p))
            grads[i] = out.reshape(3, 16)
    np.savez_compressed(OUT / "harmonics_reference.npz", vectors=vectors, gradients=grads)
    print("wrote harmonics goldens")


def structure_goldens():
    base = REFERENCE / "symmetrix" / "test" / "data" / "execution_contracts"
    out = {}
    for key, name in (("S0", "jit_r1_mace_omat0_small_contract.json"), ("S1", "jit_r1_mace_mpa0_medium_contract.json"),
                      ("S2", "jit_r1_mace_mp0b2_large_contract.json")):
        c = json.loads((base / name).read_text())
        terms = c["sparse_coupling"]["terms"]
        out[key] = {"paths": [[p["output_l"], p["edge_l"], p["source_l"]] for p in c["paths"]],
                    "rows": [t["row"] for t in terms], "lme": [t["lme"] for t in terms],
                    "abs_cg": [round(abs(t["coefficient"]), 12) for t in terms]}
    m0 = json.loads((base / "standard_m0_contract.json").read_text())
    out["M0_medium"] = {str(g["output_component"]): g["terms"] for g in m0["monomial_groups"]}
    (OUT / "structure_reference.json").write_text(json.dumps(out, separators=(",", ":")))
    print("wrote structure goldens")


if __name__ == "__main__":
    graft.build()
    which = sys.argv[2:] or ["evaluator", "variants", "harmonics", "structure"]
    if "evaluator" in which:
        evaluator_goldens()
    if "variants" in which:
        variant_goldens()
    if "harmonics" in which:
        harmonics_goldens()
    if "structure" in which:
        structure_goldens()
