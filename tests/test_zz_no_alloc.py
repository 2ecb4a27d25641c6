"""The allocation-free force/stress reduction (sxb_reduce_edge_forces_static) against the
allocating entry point (sxb_reduce_edge_forces), through the C ABI.

Some hosts of this library cannot allocate device memory when they need forces: an MD engine that
has handed the whole GPU to its own memory pool, or a force callback in the middle of a time step
where cudaMalloc would stall the device.  The static variant keeps its scratch inside the library;
this test drives it with device buffers the test owns, twice in a row with different inputs (the
scratch keeps the previous call's contents), and checks the limit on the edge count.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(pkg, seed, cells):
    rng = np.random.default_rng(seed)
    pos, cell, types = pkg.modelgen.srtio3(cells, 0.05, seed)
    from oracle import neighbor

    first, src, shifts = neighbor.build_neighbor_graph(pos, cell, 5.0)
    xyz = neighbor.edge_vectors(pos, cell, first, src, shifts)
    recv = np.repeat(np.arange(len(pos)), np.diff(first)).astype(np.int32)
    forces = rng.normal(size=(len(src), 3))
    return len(pos), recv, src.astype(np.int32), forces, xyz, abs(np.linalg.det(cell))


def test_static_reduction_matches_allocating_entry_point_twice(pkg):
    import torch

    lib = pkg.load_library()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream()
    for call, (seed, cells) in enumerate([(11, 3), (12, 2)]):       # second call: smaller, other data
        n, recv, src, forces, xyz, volume = _case(pkg, seed, cells)
        want_f, want_s = pkg.reduce_edge_forces(n, recv, src, forces, xyz, volume)
        d_recv, d_src = torch.from_numpy(recv).cuda(), torch.from_numpy(src).cuda()
        d_f, d_x = torch.from_numpy(forces.reshape(-1)).cuda(), torch.from_numpy(xyz.reshape(-1)).cuda()
        d_out = torch.full((3 * n,), 7.0, dtype=torch.float64, device="cuda")      # garbage: must be overwritten
        d_stress = torch.full((9,), 7.0, dtype=torch.float64, device="cuda")
        d_status = torch.full((1,), 5, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.sxb_reduce_edge_forces_static(n, len(src), d_recv.data_ptr(), d_src.data_ptr(), d_f.data_ptr(), d_x.data_ptr(),
                                               ctypes.c_double(volume), d_out.data_ptr(), d_stress.data_ptr(),
                                               d_status.data_ptr(), ctypes.c_void_p(stream.cuda_stream))
        assert rc == 0, lib.sxb_last_error()
        stream.synchronize()
        if call > 0:
            # once the first call has looked up the scratch address, a call takes no device memory
            assert torch.cuda.mem_get_info()[0] == free_before
        got_f = d_out.cpu().numpy().reshape(n, 3)
        got_s = d_stress.cpu().numpy().reshape(3, 3)
        assert int(d_status.cpu()[0]) == 0
        # FP64 atomics add in a different order in the two entry points: rounding-level agreement
        assert np.abs(got_f - want_f).max() <= 1e-11 * max(1.0, np.abs(want_f).max()), f"call {call}"
        assert np.abs(got_s - want_s).max() <= 1e-13 * max(1.0, np.abs(want_s).max()), f"call {call}"


def test_static_reduction_rejects_oversized_and_flags_bad_edges(pkg):
    import torch

    lib = pkg.load_library()
    torch.cuda.set_device(0)
    n, recv, src, forces, xyz, volume = _case(pkg, 13, 2)
    d_recv, d_src = torch.from_numpy(recv).cuda(), torch.from_numpy(src).cuda()
    d_f, d_x = torch.from_numpy(forces.reshape(-1)).cuda(), torch.from_numpy(xyz.reshape(-1)).cuda()
    d_out = torch.zeros(3 * n, dtype=torch.float64, device="cuda")
    d_stress = torch.zeros(9, dtype=torch.float64, device="cuda")
    too_many = 4194304 + 1
    rc = lib.sxb_reduce_edge_forces_static(n, too_many, d_recv.data_ptr(), d_src.data_ptr(), d_f.data_ptr(), d_x.data_ptr(),
                                           ctypes.c_double(volume), d_out.data_ptr(), d_stress.data_ptr(), None, None)
    assert rc != 0 and b"4,194,304" in lib.sxb_last_error()
    bad = src.copy()
    bad[5] = n + 3
    d_bad = torch.from_numpy(bad).cuda()
    d_status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.sxb_reduce_edge_forces_static(n, len(src), d_recv.data_ptr(), d_bad.data_ptr(), d_f.data_ptr(), d_x.data_ptr(),
                                           ctypes.c_double(volume), d_out.data_ptr(), d_stress.data_ptr(), d_status.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(d_status.cpu()[0]) == 1
    # the status word is optional; a volume that is not finite and positive is refused
    rc = lib.sxb_reduce_edge_forces_static(n, len(src), d_recv.data_ptr(), d_src.data_ptr(), d_f.data_ptr(), d_x.data_ptr(),
                                           ctypes.c_double(volume), d_out.data_ptr(), d_stress.data_ptr(), None, None)
    assert rc == 0
    torch.cuda.synchronize()
    for bad_volume in (float("inf"), float("nan"), 0.0):
        rc = lib.sxb_reduce_edge_forces_static(n, len(src), d_recv.data_ptr(), d_src.data_ptr(), d_f.data_ptr(), d_x.data_ptr(),
                                               ctypes.c_double(bad_volume), d_out.data_ptr(), d_stress.data_ptr(), None, None)
        assert rc != 0
    # an empty edge list gives zero forces and zero stress
    d_out.fill_(3.0)
    d_stress.fill_(3.0)
    rc = lib.sxb_reduce_edge_forces_static(n, 0, d_recv.data_ptr(), d_src.data_ptr(), d_f.data_ptr(), d_x.data_ptr(),
                                           ctypes.c_double(volume), d_out.data_ptr(), d_stress.data_ptr(), None, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert float(d_out.abs().max()) == 0.0 and float(d_stress.abs().max()) == 0.0
