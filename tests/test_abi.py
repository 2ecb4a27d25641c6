"""The C-ABI library loads and exports every symbol include/symmetrix_b200.h declares (CPU; no
compute call is made, a missing device must surface as a clean error)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        names.update(re.findall(r"\b(sxb_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.load_library()
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(pkg.SIGNATURES), "Python signature table and header disagree"
    assert hasattr(lib, "symmetrix_jit_cuda_plugin_query_v2")       # the reference's kernel-plugin query symbol


def test_errors_are_reported_without_a_device_or_model(pkg, tmp_path):
    lib = pkg.load_library()
    handle = ctypes.c_void_p()
    status = lib.sxb_create(str(tmp_path / "missing.json").encode(), 0, ctypes.byref(handle))
    assert status != 0 and not handle.value
    assert len(lib.sxb_last_error()) > 0
    with pytest.raises((RuntimeError, ValueError)):
        pkg.MACEB200(tmp_path / "missing.json")


def test_product_does_not_import_the_oracle():
    """The oracle is test infrastructure: no file of the package may reference it."""
    for path in (ROOT / "symmetrix-xl_b200").rglob("*"):
        if path.suffix in {".py", ".cu", ".cuh", ".cpp", ".hpp", ".h"}:
            text = path.read_text()
            assert "oracle" not in text.replace("oracles", ""), path


def test_model_loader_selects_prediction_heads_on_the_host(pkg, tmp_path):
    """Multi-head files: the default head's parameters replace the top-level ones, a named head can be
    asked for, and malformed sections are refused (reference: select_prediction_head,
    libsymmetrix/source/prediction_heads.hpp:10-90).  Parsed on the host; no device is needed."""
    import json

    import numpy as np

    model = pkg.modelgen.make_model("small", seed=3, heads=("pbe", "omat"))
    path = tmp_path / "two_heads.json"
    path.write_text(json.dumps(model))
    heads = model["prediction_heads"]["parameters"]
    info = pkg.model_file_info(path)
    assert info["head"] == "omat" and info["num_channels"] == 32 and info["shape_id"] == 0
    assert np.allclose(info["atomic_energies"], heads["omat"]["atomic_energies"])
    assert not np.allclose(info["atomic_energies"], heads["pbe"]["atomic_energies"])
    info = pkg.model_file_info(path, head="pbe")
    assert info["head"] == "pbe" and np.allclose(info["atomic_energies"], heads["pbe"]["atomic_energies"])
    with pytest.raises(ValueError):
        pkg.model_file_info(path, head="missing")
    broken = json.loads(path.read_text())
    del broken["prediction_heads"]["parameters"]["pbe"]["readout_2_weights_2"]
    (tmp_path / "broken.json").write_text(json.dumps(broken))
    with pytest.raises(ValueError):
        pkg.model_file_info(tmp_path / "broken.json")
    broken = json.loads(path.read_text())
    broken["prediction_heads"]["default"] = "nobody"
    (tmp_path / "broken2.json").write_text(json.dumps(broken))
    with pytest.raises(ValueError):
        pkg.model_file_info(tmp_path / "broken2.json")
    # a single-head file names no head; asking for one is an error
    single = tmp_path / "single.json"
    pkg.modelgen.write_model(single, "small", seed=3)
    assert pkg.model_file_info(single)["head"] == ""
    with pytest.raises(ValueError):
        pkg.model_file_info(single, head="pbe")


def test_model_loader_reads_and_validates_pair_splines_on_the_host(pkg, tmp_path):
    """Stored pair splines (libsymmetrix/source/mace.cpp:2714-2737): accepted when every table is complete and ends
    at zero with zero slope at the cutoff (edges at or beyond the cutoff are skipped on the device), refused otherwise."""
    import json

    model = pkg.modelgen.make_model("small", seed=3, radial="pair-splines", num_spline_points=32, a0_scaled=True)
    path = tmp_path / "pairs.json"
    path.write_text(json.dumps(model))
    info = pkg.model_file_info(path)
    assert info["num_channels"] == 32 and info["shape_id"] == 0 and info["r_cut"] == 5.0

    def refused(change, error=ValueError):
        broken = json.loads(path.read_text())
        change(broken)
        (tmp_path / "broken.json").write_text(json.dumps(broken))
        with pytest.raises(error):
            pkg.model_file_info(tmp_path / "broken.json")

    refused(lambda m: m["radial_spline_values_0"][2][5].__setitem__(-1, 0.3))      # does not vanish at the cutoff
    refused(lambda m: m["radial_spline_derivs_1"][0][0].__setitem__(-1, 0.5))      # slope at the cutoff
    refused(lambda m: m["radial_spline_values_1"].pop())                           # a pair is missing
    refused(lambda m: m["radial_spline_values_0"][1].pop())                        # a function is missing
    refused(lambda m: m.__setitem__("radial_spline_h", m["radial_spline_h"] * 0.5))  # grid does not reach the cutoff
    refused(lambda m: m.__setitem__("A0_spline_h", m["A0_spline_h"] * 2.0))        # density grid differs
    refused(lambda m: m.__delitem__("A0_spline_values"), RuntimeError)              # a missing key is the parser's error


def test_model_loader_reads_single_layer_models_on_the_host(pkg, tmp_path):
    """single_layer_readout files carry one interaction, no Phi1 tables, no R1 network and a readout polynomial over the
    hidden components (libsymmetrix/source/mace.cpp:2676-2679, 2768-2771, 2902-2914)."""
    import json

    for arch, hidden in (("small", 0), ("medium", 1), ("large", 2)):
        model = pkg.modelgen.make_model(arch, seed=5, single_layer=True)
        path = tmp_path / f"single_{arch}.json"
        path.write_text(json.dumps(model))
        info = pkg.model_file_info(path)
        assert info["single_layer"] and info["L_max"] == hidden and info["shape_id"] == hidden
        assert max(max(t) for t in model["M1_monomials"]) < (hidden + 1) ** 2
    assert not pkg.model_file_info(pkg.modelgen.write_model(tmp_path / "two.json", "small", seed=5))["single_layer"]

    def refused(change):
        broken = json.loads((tmp_path / "single_small.json").read_text())
        change(broken)
        (tmp_path / "broken.json").write_text(json.dumps(broken))
        with pytest.raises(ValueError):
            pkg.model_file_info(tmp_path / "broken.json")

    refused(lambda m: m.__setitem__("num_interactions", 2))                     # metadata disagree
    refused(lambda m: m.__setitem__("Phi1_l", [0]))                             # a second message step in a single-layer file
    refused(lambda m: m["M1_monomials"].__setitem__(0, [7]))                    # component outside H1
    refused(lambda m: m.__setitem__("A1_scaled", True))


def test_model_loader_tells_the_h1_affine_basis_on_the_host(pkg, tmp_path):
    """Format 4 (`m0_composite`) and the old basis of formats 1 / 2 are told apart by the version; mixed or partial
    declarations are refused (libsymmetrix/source/h1_affine_schema.hpp:179-240)."""
    import json

    new = pkg.modelgen.make_model("small", seed=7)
    old = pkg.modelgen.make_model("small", seed=7, format_version=2)
    assert "readout_1_weights" in old and "readout_1_weights_for_M0" not in old and "h1_affine_mode" not in old

    def info(model):
        (tmp_path / "m.json").write_text(json.dumps(model))
        return pkg.model_file_info(tmp_path / "m.json")

    assert info(new)["h1_affine_mode"] == "m0_composite" and info(old)["h1_affine_mode"] == "legacy"
    split = pkg.modelgen.make_model("small", seed=7, pre_linear_up=True, first_residual=True)
    assert info(split)["h1_affine_mode"] == "pre_linear_up"
    for change in (lambda m: m.__delitem__("H1_product_weights"),                       # the split basis needs P
                   lambda m: m.__setitem__("readout_1_weights_for_M0", [0.0] * 32),     # a field of the other basis
                   lambda m: m.__setitem__("H1_first_residual_weights", [0.0] * 5),     # wrong residual extent
                   lambda m: m.__setitem__("single_layer_readout", True)):
        broken = json.loads(json.dumps(split))
        change(broken)
        with pytest.raises(ValueError):
            info(broken)
    residual_in_m0 = json.loads(json.dumps(new))
    residual_in_m0["first_interaction_residual"] = True                                  # needs the pre_linear_up basis
    with pytest.raises(ValueError):
        info(residual_in_m0)
    for change in (lambda m: m.__setitem__("h1_affine_mode", "m0_composite"),          # a format-4 field in a format-2 file
                   lambda m: m.__setitem__("symmetrix_format_version", 3),
                   lambda m: m.__setitem__("prediction_heads", {})):
        broken = json.loads(json.dumps(old))
        change(broken)
        with pytest.raises(ValueError):
            info(broken)
    for change in (lambda m: m.__setitem__("h1_affine_mode", "pre_linear_up"),          # without the fields of that basis
                   lambda m: m.__setitem__("h1_affine_version", 2),
                   lambda m: m.__setitem__("readout_1_weights", m["readout_1_weights_for_M0"])):   # old-basis field in format 4
        broken = json.loads(json.dumps(new))
        change(broken)
        with pytest.raises(ValueError):
            info(broken)


def test_lammps_pair_style_compiles_against_the_header_shim():
    """LAMMPS is not installed here: the pair style is checked for syntax and for agreement with the C ABI
    against minimal stand-ins of the LAMMPS headers it includes."""
    import subprocess

    lammps = ROOT / "symmetrix-xl_b200" / "lammps"
    result = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-Werror", "-I", str(lammps / "shim"),
                             "-I", str(ROOT / "include"), str(lammps / "pair_symmetrix_mace_b200.cpp")],
                            capture_output=True, text=True)
    assert result.returncode == 0, result.stderr
