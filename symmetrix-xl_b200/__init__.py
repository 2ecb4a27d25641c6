"""B200-native force path for compact two-layer MACE models.

Host-side mirror of the reference evaluator interface (pybind class ``MACEKokkos``,
symmetrix/source/cpp/mace_kokkos.cpp:262+) over a C-ABI shared library of
hand-written sm_100a CUDA kernels (``csrc/``).  The directory name carries a
hyphen, so the package is loaded under the importable name ``symmetrix_xl_b200``
(``__graft_entry__.load_package``).
"""
from . import structure, modelgen, distributed, md, evaluator  # noqa: F401
from .evaluator import MACEB200, Calculator, EnsembleCalculator, load_library, measure_device_peaks, model_file_info, reduce_edge_forces, LIBRARY_PATH, SIGNATURES  # noqa: F401

__all__ = ["structure", "modelgen", "distributed", "md", "MACEB200", "Calculator", "EnsembleCalculator", "load_library", "measure_device_peaks", "model_file_info", "reduce_edge_forces", "LIBRARY_PATH", "SIGNATURES"]
