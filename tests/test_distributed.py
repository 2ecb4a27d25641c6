"""Domain decomposition: brick selection and the exchange plan on CPU (gloo, 2 / 4 / 8 ranks), decomposed evaluation and
the peer exchange on the GPU."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _brute_ghosts(dec, positions, rank):
    wf, wrap = dec.wrapped_fractional(positions)
    owner = dec.owner(positions)
    b = dec.brick_of_rank(rank)
    lo = np.array([b[a] / dec.grid[a] for a in range(3)]) - dec.halo_frac
    hi = np.array([(b[a] + 1) / dec.grid[a] for a in range(3)]) + dec.halo_frac
    out = set()
    for i in range(len(positions)):
        for sx in range(-2, 3):
            for sy in range(-2, 3):
                for sz in range(-2, 3):
                    f = wf[i] + np.array([sx, sy, sz])
                    if ((f >= lo) & (f < hi)).all() and not (owner[i] == rank and (sx, sy, sz) == (0, 0, 0)):
                        out.add((i, sx - wrap[i, 0], sy - wrap[i, 1], sz - wrap[i, 2]))
    return out


@pytest.mark.parametrize("grid", [(1, 1, 1), (2, 1, 1), (2, 2, 1), (2, 2, 2)])
def test_brick_selection_covers_every_atom_and_image(pkg, grid):
    pos, cell, types = pkg.modelgen.srtio3((4, 3, 3), 0.05, 3)
    pos = pos + np.array([0.3, -0.2, 40.0])          # atoms outside the home cell
    dec = pkg.distributed.BrickDecomposition(cell, grid, 6.5)
    owned_all = []
    for rank in range(dec.world):
        owned, gidx, gshift, oshift, owner = dec.select(pos, rank)
        owned_all.append(owned)
        got = set(zip(gidx.tolist(), *gshift.T.tolist()))
        assert len(got) == len(gidx)
        assert got == _brute_ghosts(dec, pos, rank)
        assert (np.diff(owner[gidx]) >= 0).all()      # ordered by owner rank
        # every neighbor within the halo of an owned atom is owned or a ghost
        local = np.concatenate([pos[owned] + oshift @ cell, pos[gidx] + gshift @ cell])
        from oracle import neighbor

        first, src, shifts = neighbor.build_neighbor_graph(pos, cell, 6.5)
        for i in owned[:5]:
            li = np.flatnonzero(owned == i)[0]
            d = np.linalg.norm(local - local[li], axis=1)
            assert (d <= 6.5).sum() - 1 == first[i + 1] - first[i]
    allowned = np.concatenate(owned_all)
    assert sorted(allowned.tolist()) == list(range(len(pos)))


def _plan_worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as graft

    pkg = graft.load_package()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    pos, cell, types = pkg.modelgen.srtio3((4, 2, 2), 0.05, 5)
    dec = pkg.distributed.BrickDecomposition(cell, pkg.distributed.GRIDS[world], 6.5)
    comm = pkg.distributed.make_comm()
    plan = pkg.distributed.ExchangePlan(dec, pos, comm, "cpu")
    # forward exchange of positions reproduces the ghost positions
    owned_pos = torch.from_numpy(pos[plan.owned] + plan.owned_shift @ cell)
    got = comm.all_to_all(owned_pos[torch.from_numpy(plan.send_local).long()], plan.send_counts, plan.recv_counts).numpy()
    wrap = dec.wrapped_fractional(pos)[1]
    want = pos[plan.ghost_idx] - wrap[plan.ghost_idx] @ cell
    ok_forward = np.abs(got - want).max() < 1e-12
    # reverse exchange: every ghost returns 1.0 to its owner; owners sum how often they are ghosts elsewhere
    back = comm.all_to_all(torch.ones(plan.num_ghost, 1, dtype=torch.float64), plan.recv_counts, plan.send_counts).numpy()
    tally = np.zeros(len(pos))
    np.add.at(tally, plan.owned[plan.send_local], back[:, 0])
    total = torch.from_numpy(tally)
    comm.all_reduce_sum(total)
    ghosts = torch.tensor([float(plan.num_ghost)], dtype=torch.float64)
    comm.all_reduce_sum(ghosts)
    ok_reverse = abs(total.sum().item() - ghosts.item()) < 1e-9
    np.save(Path(out_dir) / f"r{rank}.npy", np.array([ok_forward, ok_reverse, plan.num_owned, plan.num_ghost]))
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_exchange_plan_over_gloo_ranks(tmp_path, world):
    """The exchange plan on 2, 4 and 8 CPU ranks (brick grids 2x1x1, 2x2x1, 2x2x2): the forward exchange reproduces every
    ghost position and the reverse exchange returns every ghost's contribution to its owner."""
    import torch.multiprocessing as mp

    port = 29500 + (os.getpid() + 17 * world) % 2000
    mp.spawn(_plan_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    results = [np.load(tmp_path / f"r{rank}.npy") for rank in range(world)]
    assert all(r[0] and r[1] for r in results)
    assert sum(int(r[2]) for r in results) == 4 * 2 * 2 * 5
    assert all(r[2] > 0 and r[3] > 0 for r in results)


@pytest.mark.gpu
@pytest.mark.parametrize("arch,cells,options", [("small", (3, 3, 3), {}), ("medium", (3, 2, 2), {}),
                                                ("medium", (3, 2, 2), dict(a0_scaled=True, a1_scaled=True, zbl=True, agnesi=True)),
                                                ("large", (3, 2, 2), {})])
def test_single_rank_decomposition_matches_periodic_evaluation(pkg, model_path, arch, cells, options):
    """One rank whose ghosts are the periodic images of its own atoms: the three-phase path with
    halo pack/unpack must reproduce the periodic single-GPU result (also with density scaling, ZBL
    and species-pair tables, and for hidden irreps up to l = 2)."""
    path = model_path(arch, **options)
    pos, cell, types = pkg.modelgen.srtio3(cells, 0.05, 8)
    ref_out = pkg.Calculator(path, skin=0.5).calculate(pos, cell, types)
    calc = pkg.distributed.DistributedCalculator(path, pkg.MACEB200, skin=0.5, device=0)
    plan = calc.prepare(pos, cell, types)
    assert plan.num_owned == len(pos) and plan.num_ghost > 0
    for _ in range(2):                                    # twice: state must reset between evaluations
        out = calc.calculate()
        forces = out["forces"].cpu().numpy()
        assert abs(out["energy"] - ref_out["energy"]) / len(pos) <= 1e-6
        assert np.abs(forces - ref_out["forces"][out["owned"]]).max() <= 1e-5
        assert np.abs(out["stress"] - ref_out["stress"]).max() <= 1e-7
    from conftest import csr_from_positions
    from oracle import ref

    if ref.available():      # and directly against the reference's serial evaluator
        first, src, shifts, xyz = csr_from_positions(pos, cell, calc.ev.r_cut)
        m = ref.ReferenceMACE(str(path), double=False)
        m.compute(types, np.diff(first), src, xyz)
        F, S = ref.reduce_forces_stress(len(pos), np.diff(first), src, m.get("node_forces"), xyz, abs(np.linalg.det(cell)))
        assert abs(out["energy"] - m.get("node_energies").sum()) / len(pos) <= 1e-5
        assert np.abs(forces - F[out["owned"]]).max() <= 1e-4
        assert np.abs(out["stress"] - S).max() <= 1e-6


@pytest.mark.gpu
def test_distributed_phase_order_is_enforced(pkg, model_path):
    import torch

    ev = pkg.MACEB200(model_path("small"))
    pos, cell, types = pkg.modelgen.srtio3(2, 0.05, 1)
    res = ev.prepare_local_graph(len(pos), types, pos, 5.5)
    with pytest.raises(ValueError):
        ev.distributed_continue()
    d = torch.from_numpy(pos.reshape(-1).copy()).cuda()
    ev.distributed_begin(res["generation"], d.data_ptr())
    with pytest.raises(ValueError):
        ev.distributed_finish()                        # continue was skipped: phase resets
    with pytest.raises(ValueError):
        ev.distributed_continue()


@pytest.mark.gpu
def test_two_rank_decomposition_matches_single_gpu(pkg, tmp_path):
    """Two processes on two GPUs (NCCL) against the periodic single-GPU evaluation."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = tmp_path / "dd.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29611", str(ROOT / "tests" / "dd_worker.py"), str(out)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    subprocess.run(cmd, check=True, cwd=str(ROOT), env=env, timeout=600)
    import json

    r = json.loads(out.read_text())
    assert r["dE_per_atom"] <= 1e-6 and r["dF"] <= 1e-5 and r["dS"] <= 1e-7


@pytest.mark.gpu
@pytest.mark.parametrize("arch,on_device", [("small", False), ("medium", True)])
def test_caller_built_list_and_edge_vectors_drive_the_three_phases(pkg, model_path, arch, on_device):
    """The way the reference's LAMMPS pair style drives the evaluator: its own full neighbor list over
    owned atoms first and ghosts after (pair_symmetrix/pair_symmetrix_mace_kokkos.cpp:1380-1462), built
    at cutoff + skin, and per-step edge vectors with list-skin edges clamped to the cutoff (:1532-1560).
    One rank; the ghosts are the periodic images of its own atoms, so the forward / reverse halo is a
    row copy / row sum.  Energy and forces against the reference's serial evaluator."""
    import torch
    from scipy.spatial import cKDTree

    from conftest import csr_from_positions
    from oracle import ref

    path = model_path(arch, seed=4)
    pos, cell, types = pkg.modelgen.srtio3(3, 0.05, 14)
    ev = pkg.MACEB200(path)
    skin = 0.5
    halo = ev.r_cut + skin
    dec = pkg.distributed.BrickDecomposition(cell, (1, 1, 1), halo)
    owned, ghost_idx, ghost_shift, owned_shift, _owner = dec.select(pos, 0)
    n_own, n_ghost = len(owned), len(ghost_idx)
    local = np.concatenate([pos[owned] + owned_shift @ cell, pos[ghost_idx] + ghost_shift @ cell])
    local_types = np.concatenate([types[owned], types[ghost_idx]]).astype(np.int32)
    tree = cKDTree(local)
    lists = tree.query_ball_point(local[:n_own], halo)
    num_neigh = np.array([len(row) - 1 for row in lists], dtype=np.int32)
    neigh = np.concatenate([[j for j in sorted(row) if j != i] for i, row in enumerate(lists)]).astype(np.int32)
    recv = np.repeat(np.arange(n_own), num_neigh)
    xyz = local[neigh] - local[recv]
    r = np.linalg.norm(xyz, axis=1)
    clamp = r >= ev.r_cut
    xyz[clamp] *= (ev.r_cut / r[clamp])[:, None]                      # the pair style's clamp of skin edges
    d_xyz = torch.from_numpy(xyz.reshape(-1).copy()).cuda()
    if on_device:
        d_types, d_num, d_neigh = (torch.from_numpy(a).cuda() for a in (local_types, num_neigh, neigh))
        gen = ev.prepare_local_graph_csr_device(n_own, len(local), len(neigh), d_types.data_ptr(), d_num.data_ptr(), d_neigh.data_ptr())
    else:
        gen = ev.prepare_local_graph_csr(n_own, local_types, num_neigh, neigh)
    row = (ev.L_max + 1) ** 2 * ev.num_channels
    ghost_nodes = torch.arange(n_own, n_own + n_ghost, dtype=torch.int32, device="cuda")
    owner_local = torch.from_numpy(np.searchsorted(owned, ghost_idx).astype(np.int32)).cuda()
    buf = torch.empty((n_ghost, row), dtype=torch.float32, device="cuda")
    for _ in range(2):
        ev.distributed_begin_edge_vectors(gen, d_xyz.data_ptr())
        ev.halo_pack(0, owner_local.data_ptr(), n_ghost, buf.data_ptr())           # forward: ghosts get their owners' H1
        ev.halo_unpack(0, ghost_nodes.data_ptr(), n_ghost, buf.data_ptr(), False)
        ev.distributed_continue()
        ev.halo_pack(1, ghost_nodes.data_ptr(), n_ghost, buf.data_ptr())           # reverse: owners sum their ghosts' H1_adj
        ev.halo_unpack(1, owner_local.data_ptr(), n_ghost, buf.data_ptr(), True)
        ev.distributed_finish()
        ev.synchronize()
        forces = ev._reduce_atom_forces(n_own + n_ghost, execution_graph_generation=gen)
        total = forces[:n_own].copy()
        np.add.at(total, np.searchsorted(owned, ghost_idx), forces[n_own:])       # ghost forces back to the owners
        energies = ev.node_energies
        if ref.available():
            first, src, shifts, exact = csr_from_positions(pos, cell, ev.r_cut)
            m = ref.ReferenceMACE(str(path), double=False)
            m.compute(types, np.diff(first), src, exact)
            F, _S = ref.reduce_forces_stress(len(pos), np.diff(first), src, m.get("node_forces"), exact, abs(np.linalg.det(cell)))
            assert np.abs(energies - m.get("node_energies")[owned]).max() <= 1e-5
            assert np.abs(total - F[owned]).max() <= 1e-4
    with pytest.raises(ValueError):
        ev.prepare_local_graph_csr(n_own, local_types, num_neigh, neigh + len(local))    # index out of range
    with pytest.raises(ValueError):
        ev.prepare_local_graph_csr(n_own, local_types, -num_neigh, neigh)                # negative count


@pytest.mark.gpu
def test_host_buffer_halo_as_a_plain_lammps_pair_style_drives_it(pkg, model_path):
    """The call sequence of symmetrix-xl_b200/lammps/pair_symmetrix_mace_b200.cpp: list from the host, positions
    from the host, H1 / H1_adj rows through host buffers (what LAMMPS' forward / reverse communication
    callbacks pack and unpack), against the periodic evaluation of the same system."""
    from scipy.spatial import cKDTree

    path = model_path("medium", seed=6)
    pos, cell, types = pkg.modelgen.srtio3((3, 2, 2), 0.05, 15)
    want = pkg.Calculator(path, skin=0.5).calculate(pos, cell, types)
    ev = pkg.MACEB200(path)
    halo = ev.r_cut + 0.5
    dec = pkg.distributed.BrickDecomposition(cell, (1, 1, 1), halo)
    owned, ghost_idx, ghost_shift, owned_shift, _owner = dec.select(pos, 0)
    n_own, n_ghost = len(owned), len(ghost_idx)
    local = np.concatenate([pos[owned] + owned_shift @ cell, pos[ghost_idx] + ghost_shift @ cell])
    local_types = np.concatenate([types[owned], types[ghost_idx]]).astype(np.int32)
    lists = cKDTree(local).query_ball_point(local[:n_own], halo)
    num_neigh = np.array([len(row) - 1 for row in lists], dtype=np.int32)
    neigh = np.concatenate([[j for j in sorted(row) if j != i] for i, row in enumerate(lists)]).astype(np.int32)
    gen = ev.prepare_local_graph_csr(n_own, local_types, num_neigh, neigh)
    owner_local = np.searchsorted(owned, ghost_idx)
    for _ in range(2):
        ev.distributed_begin_host(gen, local)
        h1 = ev.halo_rows_get(0, 0, n_own)
        ev.halo_rows_put(0, n_own, h1[owner_local])                       # forward communication
        ev.distributed_continue()
        back = ev.halo_rows_get(1, n_own, n_ghost)
        summed = np.zeros_like(h1)
        np.add.at(summed, owner_local, back)                              # reverse communication
        ev.halo_rows_put(1, 0, summed, accumulate=True)
        ev.distributed_finish()
        ev.synchronize()
        forces = ev._reduce_atom_forces(n_own + n_ghost, execution_graph_generation=gen)
        total = forces[:n_own].copy()
        np.add.at(total, owner_local, forces[n_own:])
        assert abs(ev.node_energies.sum() - want["energy"]) / len(pos) <= 1e-6
        assert np.abs(total - want["forces"][owned]).max() <= 1e-5
        stress = ev._reduce_stress(abs(np.linalg.det(cell)), execution_graph_generation=gen)
        assert np.abs(stress - want["stress"]).max() <= 1e-7


@pytest.mark.gpu
def test_arrival_wait_runs_out_and_reports_instead_of_hanging(pkg):
    """A peer that never raises its flag: the exchange kernel gives up after the wait limit, the status word shows
    it, and the CUDA context stays usable.  One process stands for rank 0 of two; the absent rank 1's flag table and
    receive buffer are plain local buffers that nothing ever writes."""
    import torch

    lib = pkg.load_library()
    peer = pkg.distributed.PeerTransport(lib, 0, 0, 2)
    try:
        peer.set_wait_limit(0.05)
        with pytest.raises(RuntimeError):
            peer.set_wait_limit(0.0)
        rows = 64
        send = torch.arange(rows * 4, dtype=torch.float32, device="cuda").reshape(rows, 4)       # 16-byte rows
        mine = peer.alloc(rows * 16)                 # where "my own" segment lands (rank 0 -> rank 0)
        absent = peer.alloc(rows * 16)               # stands for rank 1's receive buffer
        absent_flags = peer.alloc(8 * 16 * 4)        # stands for rank 1's flag table: rank 0 may raise its flag there
        peer.plan(peer.PHASE_H1, send.data_ptr(), [0, rows // 2, rows], 16, [mine, absent], [peer.flags, absent_flags])
        stream = torch.cuda.current_stream().cuda_stream
        peer.advance(stream)
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        peer.exchange(peer.PHASE_H1, stream)
        stop.record()
        torch.cuda.synchronize()
        assert peer.status() == 32                   # rank 1 never delivered
        assert 20.0 <= start.elapsed_time(stop) <= 2000.0      # it waited about the limit, not the default ten seconds
        assert peer.status() == 0                    # reading clears the word
        # my own half arrived, and the context still runs kernels
        landed = torch.empty(rows // 2 * 4, dtype=torch.float32, device="cuda")
        view = torch.as_tensor(_DeviceArray(mine, rows // 2 * 4), device="cuda")
        landed.copy_(view)
        assert torch.equal(landed.reshape(rows // 2, 4), send[: rows // 2])
        assert float((send + 1).sum()) > 0.0
    finally:
        peer.close()


class _DeviceArray:
    """Zero-copy view of device memory for torch (float32)."""

    def __init__(self, pointer, count):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (int(pointer), False), "version": 2}
