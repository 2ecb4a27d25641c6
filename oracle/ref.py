"""ctypes access to the reference's own serial evaluator built into oracle/_ref/.

TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline).  The library is
compiled by ``make -C oracle`` from the reference checkout's sources
(libsymmetrix/source/mace.cpp and friends); this module only marshals arrays.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

_LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libsymmetrix_ref.so"
_lib = None


def available() -> bool:
    return _LIB_PATH.exists()


def _load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(str(_LIB_PATH))
        lib.symref_create.restype = ctypes.c_void_p
        lib.symref_create.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
        lib.symref_destroy.argtypes = [ctypes.c_void_p]
        lib.symref_last_error.restype = ctypes.c_char_p
        lib.symref_last_error.argtypes = [ctypes.c_void_p]
        lib.symref_compute.restype = ctypes.c_int
        lib.symref_compute.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_long] + [ctypes.c_void_p] * 6 + [ctypes.c_char_p]
        lib.symref_get.restype = ctypes.c_long
        lib.symref_get.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_long]
        lib.symref_info.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        _lib = lib
    return _lib


class ReferenceMACE:
    """MACECPU<float> (default) or MACECPU<double> of the reference, behind a C wrapper."""

    def __init__(self, json_path, double: bool = False):
        lib = _load()
        err = ctypes.create_string_buffer(512)
        self._h = lib.symref_create(str(json_path).encode(), int(double), err, 512)
        if not self._h:
            raise RuntimeError("reference evaluator: " + err.value.decode())
        info = (ctypes.c_int * 8)()
        rc = ctypes.c_double()
        lib.symref_info(self._h, info, ctypes.byref(rc))
        (self.num_elements, self.num_channels, self.l_max, self.L_max,
         self.num_lme, self.num_rows, self.num_paths, self.has_zbl) = list(info)
        self.r_cut = rc.value

    def __del__(self):
        if getattr(self, "_h", None):
            _load().symref_destroy(self._h)
            self._h = None

    def compute(self, node_types, num_neigh, neigh_indices, xyz, r=None, mode: str = ""):
        """Runs compute_node_energies_forces (mace.cpp:232-319) on a receiver-major CSR graph."""
        node_types = np.ascontiguousarray(node_types, dtype=np.int32)
        num_neigh = np.ascontiguousarray(num_neigh, dtype=np.int32)
        neigh_indices = np.ascontiguousarray(neigh_indices, dtype=np.int32)
        neigh_types = np.ascontiguousarray(node_types[neigh_indices], dtype=np.int32)
        xyz = np.ascontiguousarray(xyz, dtype=np.float64).reshape(-1, 3)
        if r is None:
            r = np.sqrt((xyz * xyz).sum(axis=1))
        r = np.ascontiguousarray(r, dtype=np.float64)
        lib = _load()
        rc = lib.symref_compute(self._h, len(node_types), len(neigh_indices),
                                node_types.ctypes.data, num_neigh.ctypes.data, neigh_indices.ctypes.data,
                                neigh_types.ctypes.data, xyz.ctypes.data, r.ctypes.data, mode.encode())
        if rc != 0:
            raise RuntimeError("reference evaluator: " + lib.symref_last_error(self._h).decode())

    def get(self, name: str) -> np.ndarray:
        lib = _load()
        n = lib.symref_get(self._h, name.encode(), None, 0)
        if n < 0:
            raise KeyError(name)
        out = np.empty(n, dtype=np.float64)
        lib.symref_get(self._h, name.encode(), out.ctypes.data, n)
        return out


def reduce_forces_stress(num_nodes, num_neigh, neigh_indices, edge_forces, xyz, volume):
    """F_j += f_ij, F_i -= f_ij; sigma = -(1/V) sum f_ij (x) xyz_ij
    (libsymmetrix/source/mace_kokkos_evaluate.cpp:92-106, 157-186)."""
    f = np.asarray(edge_forces, dtype=np.float64).reshape(-1, 3)
    xyz = np.asarray(xyz, dtype=np.float64).reshape(-1, 3)
    recv = np.repeat(np.arange(num_nodes), num_neigh)
    forces = np.zeros((num_nodes, 3))
    np.add.at(forces, np.asarray(neigh_indices), f)
    np.add.at(forces, recv, -f)
    stress = -(f[:, :, None] * xyz[:, None, :]).sum(axis=0) / volume
    return forces, stress
