"""Layer-1 kernels on one GPU, side by side: the reference's own generated CUDA plugin and this library.

TEST INFRASTRUCTURE ONLY.  Both shared libraries export the reference's kernel-plugin query symbol
(symmetrix/source/symmetrix/jit_cuda_plugin_abi.h:354-385): oracle/_ref/libsymmetrix_ref_r1_cuda.so is
the plugin the reference's generator renders for the OMAT-0 / MPA-0 medium structure (built by
oracle/build_reference_r1_plugin.py), symmetrix-xl_b200/libsymmetrix_b200.so serves the same interface
from its own kernels.  This script fills the interface's argument blocks once, from the benchmark's
5,000-atom SrTiO3 case (medium model, list cutoff 6.5 A), launches the forward tensor product and the
fused coordinate reverse of either plugin on the same device buffers, times every launch with CUDA
events (L2 flushed in between), and compares the outputs.

    python oracle/kernel_ab.py [--cells 10] [--repeats 10] [--out report.json]
"""
from __future__ import annotations

import argparse
import ctypes
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

P = ctypes.c_void_p


class Radial(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("edge_types", ctypes.c_uint32), ("intervals", ctypes.c_uint32),
                ("functions", ctypes.c_uint32), ("h", ctypes.c_double), ("x0", ctypes.c_double), ("coefficients", P)]


class ForwardArgs(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("active_type_count", ctypes.c_uint32), ("num_nodes", ctypes.c_int64),
                ("num_edges", ctypes.c_int64), ("node_types", P), ("num_neigh", P), ("first_neigh", P), ("neigh_indices", P),
                ("neigh_types", P), ("type_to_active", P), ("radius", P), ("radial", Radial), ("harmonics_values", P),
                ("neighbor_features", P), ("output", P), ("cutoff", ctypes.c_double)]


class SourceArgs(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("active_type_count", ctypes.c_uint32), ("num_nodes", ctypes.c_int64),
                ("num_edges", ctypes.c_int64), ("node_types", P), ("neigh_types", P), ("source_offsets", P), ("source_edges", P),
                ("edge_receivers", P), ("type_to_active", P), ("radius", P), ("radial", Radial), ("harmonics_values", P),
                ("output_adjoint", P), ("source_adjoint", P), ("cutoff", ctypes.c_double)]


class EdgeArgs(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("active_type_count", ctypes.c_uint32), ("coordinate_scalar_size", ctypes.c_uint32),
                ("coordinates_are_unit", ctypes.c_uint32), ("num_nodes", ctypes.c_int64), ("num_edges", ctypes.c_int64),
                ("node_types", P), ("neigh_indices", P), ("neigh_types", P), ("edge_receivers", P), ("type_to_active", P), ("xyz", P),
                ("radius", P), ("radial", Radial), ("harmonics_values", P), ("harmonics_gradients", P), ("neighbor_features", P),
                ("output_adjoint", P), ("directed_forces", P), ("cutoff", ctypes.c_double)]


FORWARD = ctypes.CFUNCTYPE(ctypes.c_int32, ctypes.POINTER(ForwardArgs), P, ctypes.c_int32)
REVERSE = ctypes.CFUNCTYPE(ctypes.c_int32, ctypes.POINTER(SourceArgs), ctypes.POINTER(EdgeArgs), P, ctypes.c_int32)


class Plugin(ctypes.Structure):
    _fields_ = [("abi_version", ctypes.c_uint32), ("struct_size", ctypes.c_uint32), ("pointer_size", ctypes.c_uint32),
                ("byte_order", ctypes.c_uint32), ("capabilities", ctypes.c_uint32), ("scalar_kind", ctypes.c_uint32),
                ("scalar_size", ctypes.c_uint32), ("reserved", ctypes.c_uint32), ("abi_tag", ctypes.c_char_p),
                ("artifact_id", ctypes.c_char_p), ("contract_fingerprint", ctypes.c_char_p), ("semantic_fingerprint", ctypes.c_char_p),
                ("structure_fingerprint", ctypes.c_char_p), ("channels", ctypes.c_int32), ("embedding", ctypes.c_int32),
                ("edge_l_max", ctypes.c_int32), ("source_l_max", ctypes.c_int32), ("target_compute_capability", ctypes.c_int32),
                ("forward_threads_per_block", ctypes.c_int32), ("source_threads_per_block", ctypes.c_int32),
                ("edge_threads_per_block", ctypes.c_int32), ("r1_forward_launch", FORWARD), ("r1_coordinate_reverse_launch", REVERSE)]


def load_plugin(path):
    lib = ctypes.CDLL(str(path))
    lib.symmetrix_jit_cuda_plugin_query_v2.restype = ctypes.POINTER(Plugin)
    plugin = lib.symmetrix_jit_cuda_plugin_query_v2().contents
    assert plugin.abi_version == 2 and plugin.struct_size == ctypes.sizeof(Plugin) and plugin.channels == 128
    return lib, plugin


def main(argv=None):
    parser = argparse.ArgumentParser()
    parser.add_argument("--cells", type=int, default=10)
    parser.add_argument("--repeats", type=int, default=10)
    parser.add_argument("--out", default=None, help="also write the report to this file")
    args = parser.parse_args(argv)

    import torch

    import __graft_entry__ as graft
    from oracle import mace_numpy, neighbor

    pkg = graft.load_package()
    reference_path = ROOT / "oracle" / "_ref" / "libsymmetrix_ref_r1_cuda.so"
    coupling_path = ROOT / "oracle" / "_ref" / "r1_medium_coupling.json"
    if not reference_path.exists():
        print(json.dumps({"unavailable": "oracle/_ref/libsymmetrix_ref_r1_cuda.so was not built in this snapshot"}))
        return None
    torch.cuda.set_device(0)
    rng = np.random.default_rng(17)
    model = pkg.modelgen.make_model("medium", seed=17)
    pos, cell, types = pkg.modelgen.srtio3(args.cells, 0.05, 17)
    r_cut = float(model["r_cut"])
    first, src, shifts = neighbor.build_neighbor_graph(pos, cell, r_cut + 0.5)
    xyz = neighbor.edge_vectors(pos, cell, first, src, shifts)
    radius = np.sqrt((xyz * xyz).sum(axis=1))
    n, e = len(pos), len(src)
    tables = mace_numpy.RadialTables(model["compact_radial"], r_cut)
    # The interface indexes the table by the unordered pair of active species, whether or not the radial functions
    # depend on it (radial_index / pair_type of the generated kernels; the reference's own table is
    # [A(A+1)/2][intervals][4][paths*C], mace_kokkos_factorized_lifecycle.cpp:4126-4436): one copy per pair.
    active_types = 3
    pairs = active_types * (active_types + 1) // 2
    coeff = np.ascontiguousarray(np.tile(tables.coefficients("R1")[None], (pairs, 1, 1, 1)), dtype=np.float32)
    y = np.ascontiguousarray(mace_numpy.harmonics(3, xyz)[0], dtype=np.float32)
    num_neigh = np.diff(first).astype(np.int32)
    receivers = np.repeat(np.arange(n, dtype=np.int32), num_neigh)
    order = np.argsort(src, kind="stable").astype(np.int32)
    source_offsets = np.concatenate([[0], np.cumsum(np.bincount(src, minlength=n))]).astype(np.int32)
    h1 = rng.normal(size=(n, 4, 128)).astype(np.float32)
    dphi = rng.normal(size=(n, 40, 128)).astype(np.float32)

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    d = {"node_types": dev(types.astype(np.int32)), "num_neigh": dev(num_neigh), "first": dev(first[:-1].astype(np.int32)),
         "src": dev(src.astype(np.int32)), "neigh_types": dev(types[src].astype(np.int32)),
         "type_to_active": dev(np.arange(3, dtype=np.int32)), "radius": dev(radius), "coeff": dev(coeff), "y": dev(y),
         "unit": dev((xyz / radius[:, None]).astype(np.float32)), "h1": dev(h1), "dphi": dev(dphi), "receivers": dev(receivers),
         "source_offsets": dev(source_offsets), "source_edges": dev(order)}
    phi = torch.zeros((n, 40, 128), dtype=torch.float32, device="cuda")
    h1_adj = torch.zeros((n, 4, 128), dtype=torch.float32, device="cuda")
    forces = torch.zeros((e, 3), dtype=torch.float64, device="cuda")
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")

    radial = Radial(ctypes.sizeof(Radial), pairs, coeff.shape[1], coeff.shape[3], tables.h, tables.x0, d["coeff"].data_ptr())
    fwd = ForwardArgs(ctypes.sizeof(ForwardArgs), 3, n, e, d["node_types"].data_ptr(), d["num_neigh"].data_ptr(), d["first"].data_ptr(),
                      d["src"].data_ptr(), d["neigh_types"].data_ptr(), d["type_to_active"].data_ptr(), d["radius"].data_ptr(), radial,
                      d["y"].data_ptr(), d["h1"].data_ptr(), phi.data_ptr(), r_cut)
    sargs = SourceArgs(ctypes.sizeof(SourceArgs), 3, n, e, d["node_types"].data_ptr(), d["neigh_types"].data_ptr(),
                       d["source_offsets"].data_ptr(), d["source_edges"].data_ptr(), d["receivers"].data_ptr(),
                       d["type_to_active"].data_ptr(), d["radius"].data_ptr(), radial, d["y"].data_ptr(), d["dphi"].data_ptr(),
                       h1_adj.data_ptr(), r_cut)
    eargs = EdgeArgs(ctypes.sizeof(EdgeArgs), 3, 4, 1, n, e, d["node_types"].data_ptr(), d["src"].data_ptr(), d["neigh_types"].data_ptr(),
                     d["receivers"].data_ptr(), d["type_to_active"].data_ptr(), d["unit"].data_ptr(), d["radius"].data_ptr(), radial,
                     d["y"].data_ptr(), None, d["h1"].data_ptr(), d["dphi"].data_ptr(), forces.data_ptr(), r_cut)

    ours_lib, ours = load_plugin(pkg.LIBRARY_PATH)
    # install the contract's coupling coefficients (path signs are the convention of whoever derived them)
    rows, outs = (ctypes.c_int32 * 86)(), (ctypes.c_int32 * 86)()
    ours_lib.sxb_jit_plugin_coupling.argtypes = [P, ctypes.c_int32, P, P]
    assert ours_lib.sxb_jit_plugin_coupling(None, 0, rows, outs) == 86
    contract = {(t["row"], t["output"]): t["coefficient"] for t in json.loads(coupling_path.read_text())["terms"]}
    cg = (ctypes.c_float * 86)(*[contract[(rows[t], outs[t])] for t in range(86)])
    assert ours_lib.sxb_jit_plugin_coupling(cg, 86, None, None) == 86
    _ref_lib, reference = load_plugin(reference_path)

    sms = torch.cuda.get_device_properties(0).multi_processor_count
    stream = torch.cuda.current_stream()
    results = {}

    def run(name, plugin, persistent):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        times = {"forward": [], "reverse": []}
        for it in range(3 + args.repeats):
            phi.zero_()
            h1_adj.zero_()
            forces.zero_()
            flush.fill_(1)
            torch.cuda.synchronize()
            start.record()
            rc = plugin.r1_forward_launch(ctypes.byref(fwd), P(stream.cuda_stream), persistent)
            stop.record()
            stop.synchronize()
            assert rc == 0, f"{name}: forward launch returned {rc}"
            if it >= 3:
                times["forward"].append(start.elapsed_time(stop))
            flush.fill_(1)
            torch.cuda.synchronize()
            start.record()
            rc = plugin.r1_coordinate_reverse_launch(ctypes.byref(sargs), ctypes.byref(eargs), P(stream.cuda_stream), persistent)
            stop.record()
            stop.synchronize()
            assert rc == 0, f"{name}: reverse launch returned {rc}"
            if it >= 3:
                times["reverse"].append(start.elapsed_time(stop))
        results[name] = {"forward_ms": float(np.median(times["forward"])), "reverse_ms": float(np.median(times["reverse"])),
                         "phi": phi.cpu().numpy().copy(), "h1_adj": h1_adj.cpu().numpy().copy(), "forces": forces.cpu().numpy().copy()}

    run("reference", reference, 8 * sms)
    run("ours", ours, 8 * sms)
    a, b = results["reference"], results["ours"]
    active = int((radius < r_cut).sum())
    report = {"workload": f"medium structure, {n}-atom SrTiO3, {e} edges ({active} inside the model cutoff), 128 channels",
              "gpu": torch.cuda.get_device_name(0), "repeats": args.repeats, "l2": "flushed before every launch (256 MiB write)",
              "reference_plugin": {"artifact": reference.artifact_id.decode(), "forward_ms": a["forward_ms"], "reverse_ms": a["reverse_ms"],
                                   "persistent_blocks": 8 * sms},
              "this_library": {"artifact": ours.artifact_id.decode(), "forward_ms": b["forward_ms"], "reverse_ms": b["reverse_ms"]},
              "speedup": {"forward": a["forward_ms"] / b["forward_ms"], "reverse": a["reverse_ms"] / b["reverse_ms"]},
              "max_abs_difference": {k: float(np.abs(a[k] - b[k]).max()) for k in ("phi", "h1_adj", "forces")},
              "max_abs_value": {k: float(np.abs(a[k]).max()) for k in ("phi", "h1_adj", "forces")}}
    for k in ("phi", "h1_adj", "forces"):
        assert report["max_abs_difference"][k] <= 2e-4 * max(1.0, report["max_abs_value"][k]), (k, report["max_abs_difference"][k])
    if args.out:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(json.dumps(report, indent=1))
    print(json.dumps(report))
    return report


if __name__ == "__main__":
    main()
