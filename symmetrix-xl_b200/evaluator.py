"""Host-side mirror of the reference evaluator class over the C-ABI library.

``MACEB200`` keeps the method names, argument meaning and error behaviour of the
pybind class ``MACEKokkosFloat`` that the reference's ASE calculator drives
(symmetrix/source/cpp/mace_kokkos.cpp:262+; call order in
symmetrix/source/symmetrix/calculator.py:2953-2971, 3253-3273, 3821-3894), so the
parity tests read like the reference's own.  Arrays are copied in; results are
fresh float64 NumPy arrays.  There is no CPU fallback: if the CUDA library is
missing or no device is usable, construction raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

_PKG_DIR = Path(__file__).resolve().parent
LIBRARY_PATH = _PKG_DIR / "libsymmetrix_b200.so"

SXB_ERR_INVALID_ARGUMENT = -1
SXB_ERR_RUNTIME = -2
SXB_ERR_STALE_GRAPH = -3
SXB_ERR_CAPACITY = -4

_lib = None


class ModelInfo(ctypes.Structure):
    _fields_ = [("num_elements", ctypes.c_int32), ("num_channels", ctypes.c_int32), ("l_max", ctypes.c_int32),
                ("hidden_l_max", ctypes.c_int32), ("num_paths", ctypes.c_int32), ("num_lme", ctypes.c_int32),
                ("shape_id", ctypes.c_int32), ("single_layer", ctypes.c_int32), ("h1_basis", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("r_cut", ctypes.c_double)]


H1_BASIS_NAMES = ("m0_composite", "legacy", "pre_linear_up")     # sxb_model_info.h1_basis


# name -> (restype, argtypes); every symbol include/symmetrix_b200.h declares
_P = ctypes.c_void_p
SIGNATURES = {
    "sxb_create": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(_P)]),
    "sxb_create_with_head": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int, ctypes.c_char_p, ctypes.POINTER(_P)]),
    "sxb_selected_head": (ctypes.c_int, [_P, ctypes.c_char_p, ctypes.c_int32]),
    "sxb_available_heads": (ctypes.c_int, [_P, ctypes.c_char_p, ctypes.c_int32]),
    "sxb_model_file_info": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_char_p, ctypes.POINTER(ModelInfo), ctypes.c_char_p,
                                           ctypes.c_int32, _P, ctypes.c_int32]),
    "sxb_measure_device_peaks": (ctypes.c_int, [ctypes.c_int32, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]),
    "sxb_jit_plugin_coupling": (ctypes.c_int, [_P, ctypes.c_int32, _P, _P]),
    "sxb_destroy": (None, [_P]),
    "sxb_last_error": (ctypes.c_char_p, []),
    "sxb_device_count": (ctypes.c_int, []),
    "sxb_device_properties": (ctypes.c_int, [ctypes.c_int32, ctypes.c_char_p, ctypes.c_int32, _P]),
    "sxb_model_info_get": (ctypes.c_int, [_P, ctypes.POINTER(ModelInfo)]),
    "sxb_atomic_numbers": (ctypes.c_int, [_P, _P, ctypes.c_int32]),
    "sxb_atomic_energies": (ctypes.c_int, [_P, _P, ctypes.c_int32]),
    "sxb_memory_report": (ctypes.c_int, [_P, ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]),
    "sxb_prepare_reference_geometry": (ctypes.c_int, [_P, ctypes.c_uint64, ctypes.c_int32, _P, _P, _P, _P, _P]),
    "sxb_update_cell": (ctypes.c_int, [_P, ctypes.c_uint64, _P, _P]),
    "sxb_prepare_periodic_graph": (ctypes.c_int, [_P, ctypes.c_int32, _P, _P, _P, _P, ctypes.c_double,
                                                  ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_int64)]),
    "sxb_prepare_graph": (ctypes.c_int, [_P, ctypes.c_int32, _P, _P, _P, _P, _P, ctypes.POINTER(ctypes.c_uint64)]),
    "sxb_get_graph": (ctypes.c_int, [_P, ctypes.c_uint64, _P, _P, _P]),
    "sxb_compute_positions": (ctypes.c_int, [_P, ctypes.c_uint64, _P]),
    "sxb_compute_positions_device": (ctypes.c_int, [_P, ctypes.c_uint64, _P]),
    "sxb_compute_edge_vectors": (ctypes.c_int, [_P, ctypes.c_uint64, _P]),
    "sxb_synchronize": (ctypes.c_int, [_P]),
    "sxb_get_node_energies": (ctypes.c_int, [_P, _P, ctypes.c_int64]),
    "sxb_set_keep_edge_forces": (ctypes.c_int, [_P, ctypes.c_int32]),
    "sxb_get_edge_forces": (ctypes.c_int, [_P, _P, ctypes.c_int64]),
    "sxb_reduce_atom_forces": (ctypes.c_int, [_P, ctypes.c_uint64, _P, ctypes.c_int64]),
    "sxb_reduce_stress": (ctypes.c_int, [_P, ctypes.c_uint64, ctypes.c_double, _P]),
    "sxb_get_energy": (ctypes.c_int, [_P, ctypes.POINTER(ctypes.c_double)]),
    "sxb_reduce_edge_forces": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int64, _P, _P, _P, _P, ctypes.c_double, _P, _P]),
    "sxb_reduce_edge_forces_static": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int64, _P, _P, _P, _P, ctypes.c_double, _P, _P,
                                                     _P, _P]),
    "sxb_device_results": (ctypes.c_int, [_P, ctypes.POINTER(_P), ctypes.POINTER(_P), ctypes.POINTER(_P)]),
    "sxb_get_stage": (ctypes.c_int, [_P, ctypes.c_char_p, _P, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64)]),
    "sxb_launch_count": (ctypes.c_int, [_P, ctypes.POINTER(ctypes.c_int64)]),
    "sxb_last_compute_ms": (ctypes.c_int, [_P, ctypes.POINTER(ctypes.c_float)]),
    "sxb_prepare_local_graph": (ctypes.c_int, [_P, ctypes.c_int32, ctypes.c_int32, _P, _P, ctypes.c_double,
                                               ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_int64)]),
    "sxb_distributed_begin": (ctypes.c_int, [_P, ctypes.c_uint64, _P]),
    "sxb_prepare_local_graph_csr": (ctypes.c_int, [_P, ctypes.c_int32, ctypes.c_int32, _P, _P, _P, ctypes.c_int32,
                                                   ctypes.POINTER(ctypes.c_uint64)]),
    "sxb_distributed_begin_edge_vectors": (ctypes.c_int, [_P, ctypes.c_uint64, _P]),
    "sxb_distributed_begin_host": (ctypes.c_int, [_P, ctypes.c_uint64, _P]),
    "sxb_halo_rows_get": (ctypes.c_int, [_P, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, _P]),
    "sxb_halo_rows_put": (ctypes.c_int, [_P, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, _P, ctypes.c_int32]),
    "sxb_distributed_continue": (ctypes.c_int, [_P]),
    "sxb_distributed_finish": (ctypes.c_int, [_P]),
    "sxb_halo_pack": (ctypes.c_int, [_P, ctypes.c_int32, _P, ctypes.c_int64, _P]),
    "sxb_halo_unpack": (ctypes.c_int, [_P, ctypes.c_int32, _P, ctypes.c_int64, _P, ctypes.c_int32]),
    "sxb_add_force_rows": (ctypes.c_int, [_P, _P, ctypes.c_int64, _P]),
    "sxb_halo_tensor": (ctypes.c_int, [_P, ctypes.c_int32, ctypes.POINTER(_P), ctypes.POINTER(ctypes.c_int64),
                                       ctypes.POINTER(ctypes.c_int64)]),
    "sxb_gather_position_rows": (ctypes.c_int, [_P, _P, _P, ctypes.c_int64, _P, _P]),
    "sxb_pack_ghost_forces": (ctypes.c_int, [_P, ctypes.c_int32, _P, ctypes.c_int64, _P]),
    "sxb_unpack_ghost_forces": (ctypes.c_int, [_P, ctypes.c_int32, _P, _P, ctypes.c_int64, _P, _P]),
    "sxb_set_halo_plan": (ctypes.c_int, [_P, _P, ctypes.c_int64, _P, _P, ctypes.c_int32, _P, _P]),
    "sxb_distributed_replayed": (ctypes.c_int, [_P, ctypes.c_uint64, ctypes.c_int64]),
    "sxb_distributed_abort": (ctypes.c_int, [_P]),
    "sxb_set_stream": (ctypes.c_int, [_P, _P]),
    "sxb_device_alloc": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int64, ctypes.POINTER(_P)]),
    "sxb_device_free": (ctypes.c_int, [_P]),
    "sxb_ipc_export": (ctypes.c_int, [_P, ctypes.c_char_p]),
    "sxb_peer_create": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(_P)]),
    "sxb_peer_flags": (ctypes.c_int, [_P, ctypes.POINTER(_P)]),
    "sxb_peer_status": (ctypes.c_int, [_P, ctypes.POINTER(ctypes.c_int32)]),
    "sxb_peer_open": (ctypes.c_int, [_P, ctypes.c_char_p, ctypes.POINTER(_P)]),
    "sxb_peer_plan": (ctypes.c_int, [_P, ctypes.c_int32, _P, _P, ctypes.c_int32, _P, _P, _P, _P, ctypes.c_int32]),
    "sxb_internal_rows": (ctypes.c_int, [_P, _P, ctypes.c_int64, _P]),
    "sxb_peer_advance": (ctypes.c_int, [_P, _P]),
    "sxb_peer_exchange": (ctypes.c_int, [_P, ctypes.c_int32, _P]),
    "sxb_peer_destroy": (ctypes.c_int, [_P]),
    "sxb_peer_set_wait_limit": (ctypes.c_int, [_P, ctypes.c_double]),
    "sxb_set_tile_size": (ctypes.c_int, [_P, ctypes.c_int32]),
    "sxb_set_deterministic": (ctypes.c_int, [_P, ctypes.c_int32]),
    "sxb_set_profiling": (ctypes.c_int, [_P, ctypes.c_int32]),
    "sxb_profile_entry": (ctypes.c_int, [_P, ctypes.c_int32, ctypes.c_char_p, ctypes.c_int32, ctypes.POINTER(ctypes.c_float),
                                         ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]),
}


def load_library():
    """Loads the in-tree CUDA library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIBRARY_PATH.exists():
            raise RuntimeError(f"{LIBRARY_PATH} is missing: build it with __graft_entry__.build(); "
                               "this package has no CPU fallback")
        lib = ctypes.CDLL(str(LIBRARY_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def _check(status):
    if status == 0:
        return
    message = load_library().sxb_last_error().decode()
    if status in (SXB_ERR_INVALID_ARGUMENT, SXB_ERR_STALE_GRAPH, SXB_ERR_CAPACITY):
        raise ValueError(message)
    raise RuntimeError(message)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _f64(a):
    return np.ascontiguousarray(a, dtype=np.float64)


def model_file_info(filename, head: str = ""):
    """Host-only inspection of a model file: structure, selected prediction head and its atomic energies."""
    lib = load_library()
    info = ModelInfo()
    name = ctypes.create_string_buffer(256)
    energies = np.zeros(512, dtype=np.float64)
    _check(lib.sxb_model_file_info(str(filename).encode(), (head or "").encode(), ctypes.byref(info), name, 256,
                                   energies.ctypes.data, energies.size))
    return {"num_elements": info.num_elements, "num_channels": info.num_channels, "l_max": info.l_max,
            "L_max": info.hidden_l_max, "num_paths": info.num_paths, "num_lme": info.num_lme, "shape_id": info.shape_id,
            "r_cut": info.r_cut, "single_layer": bool(info.single_layer),
            "h1_affine_mode": H1_BASIS_NAMES[info.h1_basis], "head": name.value.decode(), "atomic_energies": energies[:info.num_elements].copy()}


def measure_device_peaks(device: int = 0):
    """Measured FP32 FMA rate (TFLOP/s) and L2-to-SM read bandwidth (GB/s) of a device."""
    lib = load_library()
    fma, l2 = ctypes.c_double(), ctypes.c_double()
    _check(lib.sxb_measure_device_peaks(int(device), ctypes.byref(fma), ctypes.byref(l2)))
    return {"fp32_fma_tflops": fma.value, "l2_read_gbs": l2.value}


class MACEB200:
    """FP32 evaluator of a compact two-layer MACE model on one B200."""

    def __init__(self, filename, device: int = 0, head: str = ""):
        lib = load_library()
        handle = _P()
        _check(lib.sxb_create_with_head(str(filename).encode(), int(device), (head or "").encode(), ctypes.byref(handle)))
        self._h = handle
        self._lib = lib
        self.device = int(device)
        self.jit_cuda_plugin_ready = False
        self.jit_cuda_plugin_path = ""
        name = ctypes.create_string_buffer(256)
        _check(lib.sxb_selected_head(self._h, name, 256))
        self.head = name.value.decode()
        self.selected_head = self.head
        names = ctypes.create_string_buffer(4096)
        _check(lib.sxb_available_heads(self._h, names, 4096))
        self.available_heads = [n for n in names.value.decode().split("\n") if n]
        self.supports_factorized = True      # the calculator's "auto" then selects its direct mode
        info = ModelInfo()
        _check(lib.sxb_model_info_get(self._h, ctypes.byref(info)))
        self.num_elements = info.num_elements
        self.num_channels = info.num_channels
        self.l_max = info.l_max
        self.L_max = info.hidden_l_max
        self.num_lme = info.num_lme
        self.num_paths = info.num_paths
        self.r_cut = info.r_cut
        z = np.zeros(info.num_elements, dtype=np.int32)
        _check(lib.sxb_atomic_numbers(self._h, z.ctypes.data, len(z)))
        self.atomic_numbers = z.tolist()
        e0 = np.zeros(info.num_elements, dtype=np.float64)
        _check(lib.sxb_atomic_energies(self._h, e0.ctypes.data, len(e0)))
        self.atomic_energies = e0.tolist()
        self.single_layer_readout = bool(info.single_layer)
        self.h1_affine_mode = H1_BASIS_NAMES[info.h1_basis]
        self._num_nodes = 0
        self._num_edges = 0
        self._tile_size = 0

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.sxb_destroy(self._h)
            self._h = None

    # -- graph -----------------------------------------------------------------------------
    def _prepare_periodic_factorized_graph(self, node_types, positions, cell, inverse_cell, neighbor_cutoff):
        node_types, positions = _i32(node_types), _f64(positions).reshape(-1)
        cell, inverse_cell = _f64(cell).reshape(-1), _f64(inverse_cell).reshape(-1)
        if positions.size != 3 * node_types.size or cell.size != 9 or inverse_cell.size != 9:
            raise ValueError("Neighbor graph input extents are inconsistent.")
        gen, edges = ctypes.c_uint64(), ctypes.c_int64()
        _check(self._lib.sxb_prepare_periodic_graph(self._h, node_types.size, node_types.ctypes.data, positions.ctypes.data,
                                                    cell.ctypes.data, inverse_cell.ctypes.data, float(neighbor_cutoff),
                                                    ctypes.byref(gen), ctypes.byref(edges)))
        self._num_nodes, self._num_edges, self._num_receivers = int(node_types.size), int(edges.value), int(node_types.size)
        return {"generation": int(gen.value), "num_edges": int(edges.value)}

    def _prepare_factorized_graph(self, num_nodes, node_types, num_neigh, neigh_indices, neigh_types=None,
                                  shifts=None, cell=None):
        node_types, num_neigh, neigh_indices = _i32(node_types), _i32(num_neigh), _i32(neigh_indices)
        if node_types.size != num_nodes or num_neigh.size != num_nodes or neigh_indices.size != int(num_neigh.sum()):
            raise ValueError("Graph input extents are inconsistent.")
        if neigh_types is not None and not np.array_equal(_i32(neigh_types), node_types[neigh_indices]):
            raise ValueError("neigh_types disagree with node_types[neigh_indices].")
        sp = cp = None
        if shifts is not None:
            shifts = _i32(shifts).reshape(-1)
            cell = _f64(cell).reshape(-1)
            if shifts.size != 3 * neigh_indices.size or cell.size != 9:
                raise ValueError("Graph shift extents are inconsistent.")
            sp, cp = shifts.ctypes.data, cell.ctypes.data
        gen = ctypes.c_uint64()
        _check(self._lib.sxb_prepare_graph(self._h, int(num_nodes), node_types.ctypes.data, num_neigh.ctypes.data,
                                           neigh_indices.ctypes.data, sp, cp, ctypes.byref(gen)))
        self._num_nodes, self._num_edges, self._num_receivers = int(num_nodes), int(neigh_indices.size), int(num_nodes)
        return int(gen.value)

    # -- what else the reference's calculator reads from its evaluator (calculator.py:1956-2640, 3162-3403) ------
    def supports_streamed_edges(self):
        return True

    @property
    def streamed_edges_mode(self):
        """Edge state is always regenerated inside the kernels and never stored graph-wide: the reference's
        ``direct`` streamed mode."""
        return "direct"

    def set_streamed_edges(self, mode):
        if str(mode) not in ("direct", "generic", "auto", "True", "true"):
            raise ValueError("this evaluator only runs streamed edges (mode 'direct'); got %r" % (mode,))

    def _validate_graph_cardinality(self, num_receivers, num_feature_nodes, num_edges):
        limit = 2 ** 31 - 1
        if num_receivers < 0 or num_feature_nodes < num_receivers:
            raise ValueError("Graph receivers must not outnumber the feature nodes.")
        if num_feature_nodes > limit or num_edges > limit:
            raise ValueError("Graph exceeds 32-bit node or edge indexing.")

    def _load_jit_cuda_plugin(self, path, persistent_blocks_per_compute_unit=4):
        """The reference calculator builds a model-specific kernel plugin for its ``direct`` mode and hands it to the
        evaluator (calculator.py:2549-2563).  This library's layer-1 kernels are specialised at compile time, so the
        plugin is checked -- it must be a loadable library that exports ``symmetrix_jit_cuda_plugin_query_v2`` -- and
        recorded, and the compiled-in kernels keep serving the stage.  A file that is no such plugin raises, as the
        reference's loader does."""
        if int(persistent_blocks_per_compute_unit) <= 0:
            raise ValueError("persistent_blocks_per_compute_unit must be positive")
        try:
            plugin = ctypes.CDLL(str(path))
            getattr(plugin, "symmetrix_jit_cuda_plugin_query_v2")
        except (OSError, AttributeError) as error:
            raise RuntimeError(f"{path} is not a loadable Symmetrix CUDA kernel plugin: {error}") from error
        self.jit_cuda_plugin_path = str(path)
        self.jit_cuda_plugin_ready = True

    @property
    def jit_cuda_plugin_artifact_id(self):
        """Identity of the layer-1 kernels in use: the compiled-in ones."""
        return f"symmetrix-xl-b200-r1-{self.num_channels}-l{self.l_max}-L{self.L_max}"

    @property
    def device_cuda_environment(self):
        """The dictionary the calculator reads to choose a compile target (symmetrix/source/cpp/mace_kokkos.cpp:807-828)."""
        name = ctypes.create_string_buffer(256)
        values = (ctypes.c_int64 * 6)()
        _check(load_library().sxb_device_properties(self.device, name, 256, values))
        code = int(values[0])
        return {"available": True, "backend": "cuda", "device_name": name.value.decode(), "device_ordinal": self.device,
                "compute_capability": f"{code // 10}.{code % 10}", "compute_capability_code": code,
                "multiprocessor_count": int(values[1]), "warp_width": int(values[2]), "runtime_version": int(values[3]),
                "driver_version": int(values[4])}

    @property
    def execution_device_execution_environment(self):
        """Wider form of the same report (symmetrix/source/cpp/device_environment.hpp:7-37)."""
        base = self.device_cuda_environment
        memory_mib = (ctypes.c_int64 * 6)()
        name = ctypes.create_string_buffer(256)
        _check(load_library().sxb_device_properties(self.device, name, 256, memory_mib))
        base.update({"execution_space": "Cuda", "memory_space": "CudaSpace", "device_memory": int(memory_mib[5]) << 20,
                     "architecture": f"sm_{base['compute_capability_code']}", "native_subgroup_width": base["warp_width"],
                     "compute_unit_count": base["multiprocessor_count"], "aot_available": True, "jit_available": False,
                     "batched_blas_available": False})
        return base

    @property
    def execution_plan_report(self):
        """Shape of the reference's plan report (libsymmetrix/source/execution_plan.hpp:32-50) for the one plan this
        library has per setting: whole-graph work buffers, or tiled streaming with a reusable tile workspace."""
        work, free, total = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        _check(self._lib.sxb_memory_report(self._h, ctypes.byref(work), ctypes.byref(free), ctypes.byref(total)))
        plan = "tiled-streaming(%d)" % self._tile_size if self._tile_size else "streamed-edges"
        return {"requested_algorithm": "direct", "requested_profile": "capacity" if self._tile_size else "speed",
                "selection_source": "request", "state": "resolved" if self._num_nodes else "pending", "selected_id": plan,
                "selection_reason": "the only plan of this evaluator for the current tile setting",
                "available_bytes": int(free.value), "reserve_bytes": 0, "boundary_attempt": False,
                "candidates": [{"id": plan, "qualified": True, "estimated_bytes": int(work.value), "reason": "in use"}]}

    def _prepare_factorized_geometry(self, execution_graph_generation, reference_positions, reference_xyz, cell, inverse_cell, pbc):
        self._reference_geometry(execution_graph_generation, False, reference_positions, reference_xyz, cell, inverse_cell, pbc)

    def _prepare_factorized_fractional_geometry(self, execution_graph_generation, fractional_positions, fractional_xyz, cell,
                                                inverse_cell, pbc):
        self._reference_geometry(execution_graph_generation, True, fractional_positions, fractional_xyz, cell, inverse_cell, pbc)

    def _reference_geometry(self, generation, fractional, positions, xyz, cell, inverse_cell, pbc):
        positions, xyz = _f64(positions).reshape(-1), _f64(xyz).reshape(-1)
        cell, inverse_cell, pbc = _f64(cell).reshape(-1), _f64(inverse_cell).reshape(-1), _i32(pbc).reshape(-1)
        if positions.size != 3 * self._num_nodes or xyz.size != 3 * self._num_edges or cell.size != 9 or inverse_cell.size != 9 or pbc.size != 3:
            raise ValueError("Reference geometry extents do not match the prepared graph.")
        _check(self._lib.sxb_prepare_reference_geometry(self._h, int(generation), int(fractional), positions.ctypes.data, xyz.ctypes.data,
                                                        cell.ctypes.data, inverse_cell.ctypes.data, pbc.ctypes.data))

    def _update_factorized_cell(self, execution_graph_generation, cell, inverse_cell):
        cell, inverse_cell = _f64(cell).reshape(-1), _f64(inverse_cell).reshape(-1)
        if cell.size != 9 or inverse_cell.size != 9:
            raise ValueError("Cell extents are inconsistent.")
        _check(self._lib.sxb_update_cell(self._h, int(execution_graph_generation), cell.ctypes.data, inverse_cell.ctypes.data))

    def prepare_local_graph(self, num_receivers, node_types, positions, neighbor_cutoff):
        """Graph of an open node set whose first ``num_receivers`` nodes are receivers (owned atoms) and
        whose other nodes are ghosts (reference: prepare_factorized_graph_device with num_receivers <
        num_feature_nodes, libsymmetrix/source/mace_kokkos.hpp:672-697)."""
        node_types, positions = _i32(node_types), _f64(positions).reshape(-1)
        if positions.size != 3 * node_types.size:
            raise ValueError("Neighbor graph input extents are inconsistent.")
        gen, edges = ctypes.c_uint64(), ctypes.c_int64()
        _check(self._lib.sxb_prepare_local_graph(self._h, int(num_receivers), node_types.size, node_types.ctypes.data,
                                                 positions.ctypes.data, float(neighbor_cutoff), ctypes.byref(gen),
                                                 ctypes.byref(edges)))
        self._num_nodes, self._num_edges, self._num_receivers = int(node_types.size), int(edges.value), int(num_receivers)
        return {"generation": int(gen.value), "num_edges": int(edges.value)}

    def prepare_local_graph_csr(self, num_receivers, node_types, num_neigh, neigh_indices):
        """Caller-built CSR over owned atoms (first ``num_receivers`` nodes) and ghosts, host arrays
        (reference: prepare_factorized_graph_device, libsymmetrix/source/mace_kokkos.hpp:399-413)."""
        node_types, num_neigh, neigh_indices = _i32(node_types), _i32(num_neigh), _i32(neigh_indices)
        if num_neigh.size != int(num_receivers) or neigh_indices.size != int(num_neigh.sum()):
            raise ValueError("Graph input extents are inconsistent.")
        gen = ctypes.c_uint64()
        _check(self._lib.sxb_prepare_local_graph_csr(self._h, int(num_receivers), node_types.size, node_types.ctypes.data,
                                                     num_neigh.ctypes.data, neigh_indices.ctypes.data, 0, ctypes.byref(gen)))
        self._num_nodes, self._num_edges, self._num_receivers = int(node_types.size), int(neigh_indices.size), int(num_receivers)
        return int(gen.value)

    def prepare_local_graph_csr_device(self, num_receivers, num_nodes, num_edges, node_types_ptr, num_neigh_ptr, neigh_indices_ptr):
        """The same from device arrays (int32) on the evaluator's device."""
        gen = ctypes.c_uint64()
        _check(self._lib.sxb_prepare_local_graph_csr(self._h, int(num_receivers), int(num_nodes), ctypes.c_void_p(node_types_ptr),
                                                     ctypes.c_void_p(num_neigh_ptr), ctypes.c_void_p(neigh_indices_ptr), 1,
                                                     ctypes.byref(gen)))
        self._num_nodes, self._num_edges, self._num_receivers = int(num_nodes), int(num_edges), int(num_receivers)
        return int(gen.value)

    def distributed_begin_host(self, generation, positions):
        positions = _f64(positions).reshape(-1)
        if positions.size != 3 * self._num_nodes:
            raise ValueError("positions extent does not match the prepared graph.")
        _check(self._lib.sxb_distributed_begin_host(self._h, int(generation), positions.ctypes.data))

    def halo_rows_get(self, which, first_row, count):
        """Caller-order rows [first_row, first_row + count) of H1 (0) / H1_adj (1) as a float32 host array."""
        out = np.empty((int(count), (self.L_max + 1) ** 2 * self.num_channels), dtype=np.float32)
        _check(self._lib.sxb_halo_rows_get(self._h, int(which), int(first_row), int(count), out.ctypes.data))
        return out

    def halo_rows_put(self, which, first_row, rows, accumulate=False):
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        _check(self._lib.sxb_halo_rows_put(self._h, int(which), int(first_row), rows.shape[0], rows.ctypes.data, int(bool(accumulate))))

    def distributed_begin_edge_vectors(self, generation, device_xyz_ptr):
        _check(self._lib.sxb_distributed_begin_edge_vectors(self._h, int(generation), ctypes.c_void_p(device_xyz_ptr)))

    # three-phase evaluation and halo rows (device pointers as integers)
    def distributed_begin(self, generation, device_positions_ptr):
        _check(self._lib.sxb_distributed_begin(self._h, int(generation), ctypes.c_void_p(device_positions_ptr)))

    def distributed_continue(self):
        _check(self._lib.sxb_distributed_continue(self._h))

    def distributed_finish(self):
        _check(self._lib.sxb_distributed_finish(self._h))

    def halo_pack(self, which, indices_ptr, count, out_ptr):
        _check(self._lib.sxb_halo_pack(self._h, int(which), ctypes.c_void_p(indices_ptr), int(count), ctypes.c_void_p(out_ptr)))

    def halo_unpack(self, which, indices_ptr, count, in_ptr, accumulate):
        _check(self._lib.sxb_halo_unpack(self._h, int(which), ctypes.c_void_p(indices_ptr), int(count), ctypes.c_void_p(in_ptr),
                                         int(bool(accumulate))))

    def add_force_rows(self, indices_ptr, count, in_ptr):
        _check(self._lib.sxb_add_force_rows(self._h, ctypes.c_void_p(indices_ptr), int(count), ctypes.c_void_p(in_ptr)))

    def halo_tensor(self, which):
        """(device address, floats per row, first ghost row) of H1 (0) or H1_adj (1)."""
        ptr, row, first = _P(), ctypes.c_int64(), ctypes.c_int64()
        _check(self._lib.sxb_halo_tensor(self._h, int(which), ctypes.byref(ptr), ctypes.byref(row), ctypes.byref(first)))
        return ptr.value, row.value, first.value

    def gather_position_rows(self, rows_ptr, indices_ptr, count, offsets_ptr, out_ptr):
        _check(self._lib.sxb_gather_position_rows(self._h, ctypes.c_void_p(rows_ptr), ctypes.c_void_p(indices_ptr), int(count),
                                                  ctypes.c_void_p(offsets_ptr), ctypes.c_void_p(out_ptr)))

    def pack_ghost_forces(self, world, ghost_begin_ptr, num_ghosts, out_ptr):
        _check(self._lib.sxb_pack_ghost_forces(self._h, int(world), ctypes.c_void_p(ghost_begin_ptr), int(num_ghosts),
                                               ctypes.c_void_p(out_ptr)))

    def unpack_ghost_forces(self, world, send_begin_ptr, indices_ptr, num_rows, in_ptr, totals_ptr):
        _check(self._lib.sxb_unpack_ghost_forces(self._h, int(world), ctypes.c_void_p(send_begin_ptr), ctypes.c_void_p(indices_ptr),
                                                 int(num_rows), ctypes.c_void_p(in_ptr), ctypes.c_void_p(totals_ptr)))

    def set_halo_plan(self, send_indices_ptr, num_send, send_rows_ptr, received_rows_ptr, world, ghost_begin_ptr, force_send_ptr):
        _check(self._lib.sxb_set_halo_plan(self._h, ctypes.c_void_p(send_indices_ptr), int(num_send), ctypes.c_void_p(send_rows_ptr),
                                           ctypes.c_void_p(received_rows_ptr), int(world), ctypes.c_void_p(ghost_begin_ptr),
                                           ctypes.c_void_p(force_send_ptr)))

    def distributed_abort(self):
        _check(self._lib.sxb_distributed_abort(self._h))

    def distributed_replayed(self, generation, launches):
        _check(self._lib.sxb_distributed_replayed(self._h, int(generation), int(launches)))

    def internal_rows(self, indices_ptr, count, out_ptr):
        _check(self._lib.sxb_internal_rows(self._h, ctypes.c_void_p(indices_ptr), int(count), ctypes.c_void_p(out_ptr)))

    def set_deterministic(self, enabled: bool):
        """Reproducible mode: fixed-order accumulation, bit-identical results from run to run (prepare the
        graph again afterwards)."""
        _check(self._lib.sxb_set_deterministic(self._h, int(bool(enabled))))

    def set_tile_size(self, receivers_per_tile: int):
        """Tiled streaming with a reusable workspace (0 = off); prepare the graph again afterwards."""
        _check(self._lib.sxb_set_tile_size(self._h, int(receivers_per_tile)))
        self._tile_size = int(receivers_per_tile)

    def set_stream(self, stream_ptr):
        _check(self._lib.sxb_set_stream(self._h, ctypes.c_void_p(stream_ptr)))

    def graph(self, generation, with_shifts=True):
        """(first_neigh, sources, shifts) of the prepared graph in caller node order."""
        first = np.zeros(getattr(self, "_num_receivers", None) or self._num_nodes, dtype=np.int32)
        first = np.zeros(len(first) + 1, dtype=np.int32)
        sources = np.zeros(self._num_edges, dtype=np.int32)
        shifts = np.zeros((self._num_edges, 3), dtype=np.int32) if with_shifts else None
        _check(self._lib.sxb_get_graph(self._h, int(generation), first.ctypes.data, sources.ctypes.data,
                                       shifts.ctypes.data if with_shifts else None))
        return first, sources, shifts

    # -- evaluation ------------------------------------------------------------------------
    def _compute_prepared_factorized_positions(self, graph_generation, positions):
        positions = _f64(positions).reshape(-1)
        if positions.size != 3 * self._num_nodes:
            raise ValueError("positions extent does not match the prepared graph.")
        _check(self._lib.sxb_compute_positions(self._h, int(graph_generation), positions.ctypes.data))

    def compute_positions_device(self, graph_generation, device_pointer: int):
        """Evaluation from float64 positions already resident on the evaluator's device."""
        _check(self._lib.sxb_compute_positions_device(self._h, int(graph_generation), ctypes.c_void_p(device_pointer)))

    def _compute_prepared_factorized(self, execution_graph_generation, xyz, r=None):
        xyz = _f64(xyz).reshape(-1)
        if xyz.size != 3 * self._num_edges:
            raise ValueError("xyz extent does not match the prepared graph.")
        _check(self._lib.sxb_compute_edge_vectors(self._h, int(execution_graph_generation), xyz.ctypes.data))

    def compute_node_energies_forces(self, num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r=None,
                                     execution_graph_generation=0):
        """One-shot evaluation from a CSR graph and edge vectors; keeps the directed forces."""
        if execution_graph_generation == 0:
            execution_graph_generation = self._prepare_factorized_graph(num_nodes, node_types, num_neigh,
                                                                       neigh_indices, neigh_types)
        self.set_keep_edge_forces(True)
        self._compute_prepared_factorized(execution_graph_generation, xyz, r)
        return execution_graph_generation

    def set_keep_edge_forces(self, enabled: bool):
        _check(self._lib.sxb_set_keep_edge_forces(self._h, int(bool(enabled))))

    @property
    def node_energies(self):
        out = np.empty(getattr(self, "_num_receivers", self._num_nodes), dtype=np.float64)
        _check(self._lib.sxb_get_node_energies(self._h, out.ctypes.data, out.size))
        return out

    @property
    def node_forces(self):
        """Directed forces dE/d(xyz_ij), [3*num_edges], caller edge order."""
        out = np.zeros(3 * self._num_edges, dtype=np.float64)
        _check(self._lib.sxb_get_edge_forces(self._h, out.ctypes.data, out.size))
        return out

    def _reduce_atom_forces(self, num_nodes, edge_receivers=None, edge_sources=None, execution_graph_generation=0):
        if execution_graph_generation == 0:
            raise ValueError("Atom-force reduction needs the generation of the prepared graph.")
        out = (np.empty if int(num_nodes) == self._num_nodes else np.zeros)((int(num_nodes), 3), dtype=np.float64)
        _check(self._lib.sxb_reduce_atom_forces(self._h, int(execution_graph_generation), out.ctypes.data, out.size))
        return out

    def _reduce_stress(self, volume, xyz=None, execution_graph_generation=0):
        if execution_graph_generation == 0:
            raise ValueError("Stress reduction needs the generation of the prepared graph.")
        out = np.zeros((3, 3), dtype=np.float64)
        _check(self._lib.sxb_reduce_stress(self._h, int(execution_graph_generation), float(volume), out.ctypes.data))
        return out

    @property
    def energy(self):
        value = ctypes.c_double()
        _check(self._lib.sxb_get_energy(self._h, ctypes.byref(value)))
        return value.value

    def stage(self, name):
        """A stage tensor of the last evaluation as float64, caller node order (parity tests)."""
        count = ctypes.c_int64()
        _check(self._lib.sxb_get_stage(self._h, name.encode(), None, 0, ctypes.byref(count)))
        out = np.zeros(count.value, dtype=np.float64)
        _check(self._lib.sxb_get_stage(self._h, name.encode(), out.ctypes.data, out.size, ctypes.byref(count)))
        return out

    def device_results(self):
        e, f, v = _P(), _P(), _P()
        _check(self._lib.sxb_device_results(self._h, ctypes.byref(e), ctypes.byref(f), ctypes.byref(v)))
        return e.value, f.value, v.value

    def synchronize(self):
        _check(self._lib.sxb_synchronize(self._h))

    def set_profiling(self, enabled: bool):
        _check(self._lib.sxb_set_profiling(self._h, int(bool(enabled))))

    def profile(self):
        """[(stage name, device ms, kernel launches)] of the last evaluation (profiling must be on)."""
        count = ctypes.c_int32()
        _check(self._lib.sxb_profile_entry(self._h, -1, None, 0, None, None, ctypes.byref(count)))
        out = []
        for i in range(count.value):
            name = ctypes.create_string_buffer(64)
            ms, launches = ctypes.c_float(), ctypes.c_int32()
            _check(self._lib.sxb_profile_entry(self._h, i, name, 64, ctypes.byref(ms), ctypes.byref(launches), None))
            out.append((name.value.decode(), ms.value, launches.value))
        return out

    @property
    def launch_count(self):
        value = ctypes.c_int64()
        _check(self._lib.sxb_launch_count(self._h, ctypes.byref(value)))
        return value.value

    @property
    def last_compute_ms(self):
        value = ctypes.c_float()
        _check(self._lib.sxb_last_compute_ms(self._h, ctypes.byref(value)))
        return value.value


def reduce_edge_forces(num_nodes, edge_receivers, edge_sources, edge_forces, xyz, volume):
    """Atom forces [N,3] and stress [3,3] from directed edge forces and explicit edge lists (the
    graph-less mode of the reference's _reduce_atom_forces / _reduce_stress)."""
    lib = load_library()
    recv, src = _i32(edge_receivers), _i32(edge_sources)
    f, r = _f64(edge_forces).reshape(-1), _f64(xyz).reshape(-1)
    if recv.size != src.size or f.size != 3 * recv.size or r.size != 3 * recv.size:
        raise ValueError("Atom-force reduction edge extents are inconsistent.")
    forces = np.zeros((int(num_nodes), 3), dtype=np.float64)
    stress = np.zeros((3, 3), dtype=np.float64)
    _check(lib.sxb_reduce_edge_forces(int(num_nodes), recv.size, recv.ctypes.data, src.ctypes.data, f.ctypes.data,
                                      r.ctypes.data, float(volume), forces.ctypes.data, stress.ctypes.data))
    return forces, stress


def host_neighbor_list(positions, cell, pbc, cutoff):
    """Receiver-major neighbor list of a system with any mix of periodic axes, built on the host the way
    the reference's calculator does for non-periodic and mixed-periodic systems (its host-graph branch,
    symmetrix/source/symmetrix/calculator.py:2973-2996): images of the atoms along the periodic axes out
    to the cutoff, then a k-d tree.  Returns (num_neigh int32[N], neigh_indices int32[E], xyz f64[E,3])."""
    from scipy.spatial import cKDTree

    positions = _f64(positions).reshape(-1, 3)
    cell = _f64(cell).reshape(3, 3)
    pbc = [bool(p) for p in pbc]
    n = len(positions)
    if any(pbc):
        inv = np.linalg.inv(cell)
        spacing = 1.0 / np.sqrt((inv ** 2).sum(axis=0))
        reach = [int(np.ceil(cutoff / spacing[a])) if pbc[a] else 0 for a in range(3)]
        frac = positions @ inv
        for a in range(3):
            if pbc[a]:
                frac[:, a] -= np.floor(frac[:, a])
        home = frac @ cell
    else:
        reach, home = [0, 0, 0], positions
    images, owners = [], []
    for sx in range(-reach[0], reach[0] + 1):
        for sy in range(-reach[1], reach[1] + 1):
            for sz in range(-reach[2], reach[2] + 1):
                images.append(home + np.array([sx, sy, sz], dtype=np.float64) @ cell)
                owners.append(np.arange(n))
    images, owners = np.concatenate(images), np.concatenate(owners)
    zero_image = (len(images) // n) // 2          # the (0, 0, 0) image sits in the middle of the loop order
    tree = cKDTree(images)
    lists = tree.query_ball_point(home, cutoff)
    num_neigh = np.zeros(n, dtype=np.int32)
    neigh, xyz = [], []
    for i, row in enumerate(lists):
        row = np.array(sorted(row), dtype=np.int64)
        row = row[row != zero_image * n + i]
        num_neigh[i] = len(row)
        neigh.append(owners[row])
        xyz.append(images[row] - home[i])
    neigh = np.concatenate(neigh).astype(np.int32) if n else np.zeros(0, dtype=np.int32)
    xyz = np.concatenate(xyz) if n else np.zeros((0, 3))
    return num_neigh, neigh, xyz


class Calculator:
    """Minimal stand-in for the reference's ASE calculator hot path (``Symmetrix.calculate``,
    symmetrix/source/symmetrix/calculator.py:3934-4021): Verlet-skin neighbor cache (rebuild when
    the largest displacement exceeds skin/2, :2894-2899), reuse of the list under an affine change of a
    fully periodic cell (:2857-2888), device graph builder for fully periodic systems, host graph with a
    reference geometry for non-periodic and mixed-periodic ones (:2973-2996, 3274-3359), evaluation from
    positions, and result assembly (:3821-3894)."""

    def __init__(self, model_path, skin: float = 0.5, device: int = 0, head: str = ""):
        self.evaluator = MACEB200(model_path, device, head)
        self.skin = float(skin)
        self._generation = 0
        self._reference_positions = None
        self._reference_cell = None
        self._reference_fractional = None
        self._types = None
        self._pbc = None
        self.rebuilds = 0
        self.cell_updates = 0

    def _can_reuse(self, positions, cell, node_types, pbc):
        if self._generation == 0 or self._reference_positions.shape != positions.shape:
            return False, False
        if not np.array_equal(self._types, node_types) or self._pbc != pbc:
            return False, False
        if np.array_equal(self._reference_cell, cell):
            delta = positions - self._reference_positions
            if any(pbc) and not all(pbc):
                # the reference geometry of the host graph follows an atom across a periodic boundary: measure the
                # displacement to the nearest image (the device graph of a fully periodic cell does not, it stores shifts)
                frac = delta @ self._work_inverse
                for a in range(3):
                    if pbc[a]:
                        frac[:, a] -= np.round(frac[:, a])
                delta = frac @ self._work_cell
            moved = np.sqrt((delta ** 2).sum(axis=1).max())
            return moved <= 0.5 * self.skin, False
        if not all(pbc):
            return False, False
        # affine change of a periodic cell: the list stays valid while no pair distance can have changed by more
        # than the skin -- largest fractional displacement and the strain of the cell, both measured against the cutoff
        frac = positions @ np.linalg.inv(cell)
        dfrac = frac - self._reference_fractional
        dfrac -= np.round(dfrac)
        moved = np.sqrt((((dfrac @ cell)) ** 2).sum(axis=1).max())
        strain = np.linalg.norm(np.linalg.inv(self._reference_cell) @ cell - np.eye(3), ord=2)
        reach = self.evaluator.r_cut + self.skin
        return moved + strain * reach <= 0.5 * self.skin, True

    def calculate(self, positions, cell, node_types, pbc=(True, True, True)):
        positions = _f64(positions).reshape(-1, 3)
        cell = _f64(cell).reshape(3, 3)
        node_types = _i32(node_types)
        pbc = tuple(bool(p) for p in pbc)
        ev = self.evaluator
        reuse, new_cell = self._can_reuse(positions, cell, node_types, pbc)
        if reuse and new_cell:
            ev._update_factorized_cell(self._generation, cell, np.linalg.inv(cell))
            self.cell_updates += 1
        elif not reuse:
            cutoff = ev.r_cut + self.skin
            if all(pbc):
                result = ev._prepare_periodic_factorized_graph(node_types, positions, cell, np.linalg.inv(cell), cutoff)
                self._generation = result["generation"]
            else:
                # axes that are not periodic get a stand-in cell vector long enough that nothing wraps
                work_cell = cell.copy()
                span = np.ptp(positions, axis=0).max() + 4.0 * cutoff + 1.0
                for a in range(3):
                    if not pbc[a]:
                        work_cell[a] = 0.0
                        work_cell[a, a] = span
                self._work_cell, self._work_inverse = work_cell, np.linalg.inv(work_cell)
                num_neigh, neigh, xyz = host_neighbor_list(positions, work_cell, pbc, cutoff)
                ev._validate_graph_cardinality(len(positions), len(positions), len(neigh))
                self._generation = ev._prepare_factorized_graph(len(positions), node_types, num_neigh, neigh, node_types[neigh])
                ev._prepare_factorized_geometry(self._generation, positions, xyz, work_cell, np.linalg.inv(work_cell),
                                                np.array(pbc, dtype=np.int32))
            self._reference_positions = positions.copy()
            self._reference_cell = cell.copy()
            self._reference_fractional = positions @ np.linalg.inv(cell) if all(pbc) else None
            self._types = node_types.copy()
            self._pbc = pbc
            self.rebuilds += 1
        ev._compute_prepared_factorized_positions(self._generation, positions)
        n = len(node_types)
        energies = ev.node_energies
        out = {"energy": float(energies.sum()), "energies": energies,
               "forces": ev._reduce_atom_forces(n, execution_graph_generation=self._generation)}
        if all(pbc):
            out["stress"] = ev._reduce_stress(abs(np.linalg.det(cell)), execution_graph_generation=self._generation)
        return out


class EnsembleCalculator:
    """Same-process committee of calculators, after the reference's ``SymmetrixEnsemble``
    (symmetrix/source/symmetrix/ensemble.py:65-212): members are evaluated one after the other on the same
    input; every property ``x`` is returned as the member mean under ``x``, the stacked member values under
    ``x_comm`` and the population variance under ``x_var``.  Members must agree on cutoff, element list and
    skin (the reference's compatibility check, :133-144).  Exactly one of ``model_files`` / ``calculators``."""

    def __init__(self, model_files=None, *, calculators=None, **calculator_kwargs):
        if (model_files is None) == (calculators is None):
            raise ValueError("Provide exactly one of model_files or calculators.")
        if model_files is not None:
            if isinstance(model_files, (str, bytes)) or hasattr(model_files, "__fspath__"):
                model_files = (model_files,)
            members = tuple(Calculator(path, **calculator_kwargs) for path in model_files)
        else:
            if calculator_kwargs:
                raise ValueError("Calculator construction options cannot be used with calculators: "
                                 + ", ".join(sorted(calculator_kwargs)) + ".")
            members = (calculators,) if isinstance(calculators, Calculator) else tuple(calculators)
        if not members:
            raise ValueError("An ensemble must contain at least one member.")
        for index, member in enumerate(members):
            if not isinstance(member, Calculator):
                raise TypeError(f"Ensemble members must be calculators; member {index} is {type(member).__name__}.")
        first = members[0]
        for index, member in enumerate(members[1:], start=1):
            for name, expected, actual in (("cutoff", first.evaluator.r_cut, member.evaluator.r_cut),
                                           ("atomic-number mapping", tuple(first.evaluator.atomic_numbers),
                                            tuple(member.evaluator.atomic_numbers)),
                                           ("neighbor skin", first.skin, member.skin)):
                if expected != actual:
                    raise ValueError(f"Ensemble member {index} has incompatible {name}: expected {expected!r}, got {actual!r}.")
        self.calculators = members
        self.num_models = len(members)

    def calculate(self, positions, cell, node_types, pbc=(True, True, True)):
        outputs = [member.calculate(positions, cell, node_types, pbc) for member in self.calculators]
        results = {}
        for name in outputs[0]:
            committee = np.stack([np.asarray(out[name], dtype=np.float64) for out in outputs], axis=0)
            mean, variance = committee.mean(axis=0), committee.var(axis=0)
            results[name] = float(mean) if mean.ndim == 0 else mean
            results[name + "_var"] = float(variance) if variance.ndim == 0 else variance
            results[name + "_comm"] = committee
        return results
