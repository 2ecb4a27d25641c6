"""The C-ABI library loads and exports every symbol include/symmetrix_b200.h declares (CPU; no
compute call is made, a missing device must surface as a clean error)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "symmetrix_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sxb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.load_library()
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(pkg.SIGNATURES), "Python signature table and header disagree"


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
