"""Spatial domain decomposition of one evaluation over the GPUs of a node, one process per GPU.

The periodic cell is cut into a px x py x pz grid of bricks in fractional coordinates.  A rank owns
the atoms inside its brick and keeps ghost copies of every atom image within the halo (model cutoff
+ skin) of the brick.  Owned atoms are the receivers of the rank's graph; ghosts only supply
``H1`` rows and collect ``H1_adj`` rows and forces.  A two-layer model therefore needs exactly one
forward exchange of ghost features and one reverse exchange of ghost adjoints per evaluation, plus
ghost positions in and ghost forces out -- the protocol of the reference's LAMMPS pair style
(pair_symmetrix/pair_symmetrix_mace_kokkos.cpp:1285-1938; phases
libsymmetrix/source/mace_kokkos_evaluate.cpp:1658-2101), carried here, instead of LAMMPS' MPI brick
swaps, by pushes into the peers' memory over NVLink (``PeerTransport``: every rank writes its rows into
the receiving rank's buffers and raises a flag there) or, where peer mapping is unavailable, by
``torch.distributed`` all-to-all exchanges (NCCL between GPUs, gloo in the CPU tests of the exchange
plan).  Remote rows always land in the receiving rank's own memory before any kernel reads them; no
kernel of this package reads another GPU's memory.
"""
from __future__ import annotations

import os

import numpy as np

GRIDS = {1: (1, 1, 1), 2: (2, 1, 1), 4: (2, 2, 1), 8: (2, 2, 2)}


class BrickDecomposition:
    """Ownership and ghost selection for a brick grid over a periodic cell."""

    def __init__(self, cell, grid, halo):
        self.cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        self.inv = np.linalg.inv(self.cell)
        self.grid = tuple(int(g) for g in grid)
        self.halo = float(halo)
        # distance between the lattice planes of axis a is 1/|column a of the inverse cell|
        self.halo_frac = self.halo * np.sqrt((self.inv ** 2).sum(axis=0))

    @property
    def world(self):
        return self.grid[0] * self.grid[1] * self.grid[2]

    def brick_of_rank(self, rank):
        px, py, pz = self.grid
        return rank // (py * pz), (rank // pz) % py, rank % pz

    def wrapped_fractional(self, positions):
        frac = np.asarray(positions, dtype=np.float64).reshape(-1, 3) @ self.inv
        return frac - np.floor(frac), np.floor(frac).astype(np.int64)

    def owner(self, positions):
        """Rank owning each atom: the brick its wrapped fractional position falls in."""
        wf, _ = self.wrapped_fractional(positions)
        idx = [np.minimum(self.grid[a] - 1, (wf[:, a] * self.grid[a]).astype(np.int64)) for a in range(3)]
        return (idx[0] * self.grid[1] + idx[1]) * self.grid[2] + idx[2]

    def select(self, positions, rank):
        """Owned atoms and ghost images of ``rank``.

        Returns (owned global indices ascending, ghost global indices, ghost image shifts int[G,3]
        relative to the atoms' given (unwrapped) positions), ghosts ordered by (owner rank, atom, image).
        A ghost is any atom image whose fractional coordinates lie in the brick widened by the halo on
        every side, except the home image of an owned atom."""
        positions = np.asarray(positions, dtype=np.float64).reshape(-1, 3)
        wf, wrap = self.wrapped_fractional(positions)
        owner = self.owner(positions)
        owned = np.flatnonzero(owner == rank)
        b = self.brick_of_rank(rank)
        lo = np.array([b[a] / self.grid[a] for a in range(3)]) - self.halo_frac
        hi = np.array([(b[a] + 1) / self.grid[a] for a in range(3)]) + self.halo_frac
        reach = [int(np.ceil(self.halo_frac[a])) for a in range(3)]
        ghost_idx, ghost_shift = [], []
        for sx in range(-reach[0], reach[0] + 1):
            for sy in range(-reach[1], reach[1] + 1):
                for sz in range(-reach[2], reach[2] + 1):
                    s = np.array([sx, sy, sz])
                    f = wf + s
                    inside = ((f >= lo) & (f < hi)).all(axis=1)
                    if sx == 0 and sy == 0 and sz == 0:
                        inside &= owner != rank
                    hit = np.flatnonzero(inside)
                    ghost_idx.append(hit)
                    # shift relative to the unwrapped input position: image minus the wrap of the atom
                    ghost_shift.append(s[None, :] - wrap[hit])
        ghost_idx = np.concatenate(ghost_idx)
        ghost_shift = np.concatenate(ghost_shift)
        # owned atoms are wrapped into the home cell too: their shift is minus their wrap
        order = np.lexsort((ghost_shift[:, 2], ghost_shift[:, 1], ghost_shift[:, 0], ghost_idx, owner[ghost_idx]))
        return owned, ghost_idx[order], ghost_shift[order], -wrap[owned], owner


class _SoloComm:
    """Stand-in for a one-process world: the all-to-all of a single rank is a copy."""

    rank, world = 0, 1

    def all_to_all(self, send, send_counts, recv_counts, out=None):
        if out is None:
            return send.clone()
        out.copy_(send)
        return out

    def all_reduce_sum(self, tensor):
        return tensor


class _TorchComm:
    def __init__(self):
        import torch.distributed as dist

        self.dist = dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()

    def all_to_all(self, send, send_counts, recv_counts, out=None):
        import torch

        if out is None:
            row = send.shape[1:] if send.dim() > 1 else ()
            out = torch.empty((int(sum(recv_counts)), *row), dtype=send.dtype, device=send.device)
        self.dist.all_to_all_single(out, send if send.is_contiguous() else send.contiguous(),
                                    output_split_sizes=recv_counts if isinstance(recv_counts, list) else [int(c) for c in recv_counts],
                                    input_split_sizes=send_counts if isinstance(send_counts, list) else [int(c) for c in send_counts])
        return out

    def all_reduce_sum(self, tensor):
        self.dist.all_reduce(tensor, op=self.dist.ReduceOp.SUM)
        return tensor


def make_comm():
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return _TorchComm()
    except ImportError:
        pass
    return _SoloComm()


class ExchangePlan:
    """Who sends which owned rows to whom.  Built once per neighbor-list rebuild."""

    def __init__(self, decomposition, positions, comm, device="cpu"):
        import torch

        self.comm = comm
        self.device = device
        rank, world = comm.rank, comm.world
        owned, ghost_idx, ghost_shift, owned_shift, owner = decomposition.select(positions, rank)
        self.owned = owned
        self.owned_shift = owned_shift
        self.ghost_idx, self.ghost_shift = ghost_idx, ghost_shift
        ghost_owner = owner[ghost_idx]
        self.recv_counts = np.bincount(ghost_owner, minlength=world).astype(np.int64)     # ghosts I receive, per owner
        # tell every owner which of its atoms I need
        counts = torch.from_numpy(self.recv_counts).to(device)
        self.send_counts = comm.all_to_all(counts, [1] * world, [1] * world).cpu().numpy().astype(np.int64)
        wanted = comm.all_to_all(torch.from_numpy(ghost_idx.astype(np.int64)).to(device), self.recv_counts, self.send_counts)
        wanted = wanted.cpu().numpy()
        local = np.searchsorted(owned, wanted)
        if len(wanted) and (local >= len(owned)).any() or (len(wanted) and (owned[np.minimum(local, len(owned) - 1)] != wanted).any()):
            raise RuntimeError("exchange plan: a rank asked for an atom its owner does not hold")
        self.send_local = local.astype(np.int32)          # my owned rows to send, ordered by destination rank
        self.num_owned, self.num_ghost = len(owned), len(ghost_idx)


class PeerTransport:
    """The four exchanges of a step over NVLink peer memory (csrc/peer_exchange.cu): every rank maps the
    receive buffers of its peers through CUDA IPC; an exchange is one kernel on the calculator's stream that pushes
    the rows, raises this rank's flag at every peer and waits, with a time limit, for the peers' flags.  Receive buffers: the ghost tail of the position array, the ghost tail of
    the evaluator's H1 tensor, the returned-adjoint rows and the returned-force rows."""

    PHASE_POSITIONS, PHASE_H1, PHASE_H1_ADJ, PHASE_FORCES = 0, 1, 2, 3

    def __init__(self, lib, device_index, rank, world):
        import ctypes

        self.lib, self.ctypes = lib, ctypes
        self.device_index, self.rank, self.world = device_index, rank, world
        self.handle = ctypes.c_void_p()
        self._check(lib.sxb_peer_create(device_index, rank, world, ctypes.byref(self.handle)))
        flags = ctypes.c_void_p()
        self._check(lib.sxb_peer_flags(self.handle, ctypes.byref(flags)))
        self.flags = flags.value
        self.owned_buffers = []

    def _check(self, status):
        if status != 0:
            raise RuntimeError(self.lib.sxb_last_error().decode())

    def alloc(self, nbytes):
        ptr = self.ctypes.c_void_p()
        self._check(self.lib.sxb_device_alloc(self.device_index, max(int(nbytes), 256), self.ctypes.byref(ptr)))
        self.owned_buffers.append(ptr.value)
        return ptr.value

    def export(self, ptr):
        buf = self.ctypes.create_string_buffer(64)
        self._check(self.lib.sxb_ipc_export(self.ctypes.c_void_p(ptr), buf))
        return bytes(buf.raw)

    def open(self, handle):
        out = self.ctypes.c_void_p()
        self._check(self.lib.sxb_peer_open(self.handle, handle, self.ctypes.byref(out)))
        return out.value

    def plan(self, phase, send_ptr, send_begin, row_bytes, remote_ptrs, remote_flags, row_source=None, row_dest=None, accumulate=False):
        c = self.ctypes
        begin = (c.c_int64 * (self.world + 1))(*[int(v) for v in send_begin])
        remotes = (c.c_void_p * self.world)(*[c.c_void_p(int(v)) for v in remote_ptrs])
        flags = (c.c_void_p * self.world)(*[c.c_void_p(int(v)) for v in remote_flags])
        self._check(self.lib.sxb_peer_plan(self.handle, int(phase), c.c_void_p(send_ptr), begin, int(row_bytes), remotes, flags,
                                           c.c_void_p(row_source), c.c_void_p(row_dest), int(bool(accumulate))))

    def advance(self, stream_ptr):
        self._check(self.lib.sxb_peer_advance(self.handle, self.ctypes.c_void_p(stream_ptr)))

    def exchange(self, phase, stream_ptr):
        self._check(self.lib.sxb_peer_exchange(self.handle, int(phase), self.ctypes.c_void_p(stream_ptr)))

    def set_wait_limit(self, seconds):
        """Limit of every arrival wait from now on (ten seconds by default)."""
        self._check(self.lib.sxb_peer_set_wait_limit(self.handle, float(seconds)))

    def status(self):
        out = self.ctypes.c_int32()
        self._check(self.lib.sxb_peer_status(self.handle, self.ctypes.byref(out)))
        return out.value

    def close(self):
        if self.handle:
            self.lib.sxb_peer_destroy(self.handle)
            self.handle = None
            for ptr in self.owned_buffers:
                self.lib.sxb_device_free(self.ctypes.c_void_p(ptr))
            self.owned_buffers = []


class DistributedCalculator:
    """Energy, forces and stress of a periodic system decomposed over the ranks of the process group.

    Per evaluation a rank issues four exchanges and no other collective: ghost positions in, ``H1`` rows
    forward (received straight into the tail of the feature tensor), ``H1_adj`` rows back (sent
    straight from the tail of the adjoint tensor, summed at the owner), ghost forces back together with
    every rank's energy and virial.  All of it is enqueued on one stream with a single host
    synchronisation at the end."""

    TOTALS_ROWS = 4     # energy + 9 virial components travel as four rows of three doubles

    def __init__(self, model_path, evaluator_cls, skin=0.5, device=0):
        import torch

        self.torch = torch
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.ev = evaluator_cls(model_path, device=device)
        # the evaluator's kernels and the exchanges share one stream of their own (a stream that can be
        # captured into CUDA graphs, which the legacy default stream cannot)
        self.stream = torch.cuda.Stream(self.device)
        self.ev.set_stream(self.stream.cuda_stream)
        self.skin = float(skin)
        self.comm = make_comm()
        self.transport = "NCCL" if self.comm.world > 1 else "local-copy"
        self.peer = None
        self.generation = 0

    def prepare(self, positions, cell, types, grid=None):
        """Decomposes the global system (every rank passes the same arrays) and builds the local graph."""
        torch = self.torch
        positions = np.asarray(positions, dtype=np.float64).reshape(-1, 3)
        types = np.asarray(types, dtype=np.int32)
        self.cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        self.volume = abs(np.linalg.det(self.cell))
        grid = grid or GRIDS[self.comm.world]
        halo = self.ev.r_cut + self.skin
        self.decomposition = BrickDecomposition(self.cell, grid, halo)
        if self.decomposition.world != self.comm.world:
            raise ValueError("brick grid does not match the number of ranks")
        # every rank must own atoms: decided together, so that no rank leaves the others waiting in an exchange
        owner = self.decomposition.owner(positions)
        if np.bincount(owner, minlength=self.comm.world).min() == 0:
            raise ValueError("domain decomposition: a brick of the grid owns no atom; use fewer ranks or another grid")
        # mappings of the peers' buffers are closed on every rank before any rank may re-allocate what it exported
        self._release_peer()
        self.comm.all_reduce_sum(torch.zeros(1, dtype=torch.float64, device=self.device))
        plan = ExchangePlan(self.decomposition, positions, self.comm, self.device)
        self.plan = plan
        n_own, n_ghost = plan.num_owned, plan.num_ghost
        owned_pos = positions[plan.owned] + plan.owned_shift @ self.cell
        ghost_pos = positions[plan.ghost_idx] + plan.ghost_shift @ self.cell
        local_pos = np.concatenate([owned_pos, ghost_pos], axis=0)
        local_types = np.concatenate([types[plan.owned], types[plan.ghost_idx]])
        result = self.ev.prepare_local_graph(n_own, local_types, local_pos, halo)
        self.generation = result["generation"]
        self.num_edges = result["num_edges"]
        dev = self.device
        world = self.comm.world
        self.send_local = torch.from_numpy(plan.send_local).to(dev)
        n_send = len(self.send_local)
        self.send_counts = [int(c) for c in plan.send_counts]
        self.recv_counts = [int(c) for c in plan.recv_counts]
        # a ghost sits at its owner's current (wrapped-at-prepare) position plus a fixed image offset; the
        # owners learn the offsets of their rows once, so the per-step gather already yields ghost positions
        owner_shift_of_ghost = -self.decomposition.wrapped_fractional(positions)[1][plan.ghost_idx]
        ghost_offset = torch.from_numpy((plan.ghost_shift - owner_shift_of_ghost) @ self.cell).to(dev)
        self.send_offset = self.comm.all_to_all(ghost_offset, self.recv_counts, self.send_counts,
                                                out=torch.empty((n_send, 3), dtype=torch.float64, device=dev))
        self.row = (self.ev.L_max + 1) ** 2 * self.ev.num_channels
        # per-step buffers, allocated once per graph: the step issues no allocation and few host operations
        extra = self.TOTALS_ROWS
        n_local = n_own + n_ghost
        self.peer = self._make_peer_transport()
        if self.peer is not None:
            # receive buffers that peers write into must be plain device allocations (they are shared by IPC handle)
            self.local_positions = _as_tensor(torch, self.peer.alloc(24 * n_local), (n_local, 3), torch.float64, dev)
            self.local_positions.copy_(torch.from_numpy(local_pos))
            self._got_rows = None          # the peers add their H1_adj rows straight into this rank's tensor
            self._force_recv = _as_tensor(torch, self.peer.alloc(24 * (n_send + extra * world)), (n_send + extra * world, 3),
                                          torch.float64, dev)
        else:
            self.local_positions = torch.from_numpy(local_pos).to(dev)       # [owned | ghosts], the step's input buffer
            self._got_rows = torch.empty((n_send, self.row), dtype=torch.float32, device=dev)
            self._force_recv = torch.empty((n_send + extra * world, 3), dtype=torch.float64, device=dev)
        self.owned_positions = self.local_positions[:n_own]
        self._send_pos = torch.empty((n_send, 3), dtype=torch.float64, device=dev)
        self._send_rows = torch.empty((n_send, self.row), dtype=torch.float32, device=dev)
        self._force_send = torch.empty((n_ghost + extra * world, 3), dtype=torch.float64, device=dev)
        self._force_send_counts = [c + extra for c in self.recv_counts]
        self._force_recv_counts = [c + extra for c in self.send_counts]
        self._ghost_begin = torch.tensor(np.concatenate([[0], np.cumsum(self.recv_counts)]), dtype=torch.int32, device=dev)
        self._send_begin = torch.tensor(np.concatenate([[0], np.cumsum(self.send_counts)]), dtype=torch.int32, device=dev)
        self._totals = torch.zeros(10, dtype=torch.float64, device=dev)
        self._totals_host = torch.empty(10, dtype=torch.float64).pin_memory()
        # ghost rows of H1 / H1_adj: the tail of the evaluator's own tensors
        h1_ptr, row, first = self.ev.halo_tensor(0)
        adj_ptr, _, _ = self.ev.halo_tensor(1)
        assert row == self.row and first == n_own
        self._h1_tail = _as_tensor(torch, h1_ptr, (n_local, self.row), torch.float32, dev)[n_own:]
        self._h1_adj_tail = _as_tensor(torch, adj_ptr, (n_local, self.row), torch.float32, dev)[n_own:]
        # packing and unpacking run inside the evaluator's phases (and their captured graphs)
        if self.peer is None:
            self.ev.set_halo_plan(self.send_local.data_ptr(), n_send, self._send_rows.data_ptr(), self._got_rows.data_ptr(), world,
                                  self._ghost_begin.data_ptr(), self._force_send.data_ptr())
        self._step_graph, self._step_graph_launches, self._eager_steps = None, 0, 0
        self._capture_allowed = os.environ.get("SXB_STEP_GRAPH", "1") != "0"
        if self.peer is not None:
            self._plan_peer_exchanges(h1_ptr, adj_ptr)
            self.transport = "NVLink peer-memory"
            # collectives captured in a graph tie the communicator to it; the peer kernels have no such tie
        elif world > 1:
            self.transport = "NCCL"
            self._capture_allowed = self._capture_allowed and os.environ.get("SXB_STEP_GRAPH_NCCL", "0") == "1"
        return plan

    def _make_peer_transport(self):
        """A PeerTransport when every rank can create one (and SXB_HALO_TRANSPORT does not say ``nccl``), else None."""
        if self.comm.world == 1 or os.environ.get("SXB_HALO_TRANSPORT", "peer") == "nccl":
            return None
        from .evaluator import load_library

        torch = self.torch
        peer = None
        try:
            peer = PeerTransport(load_library(), self.device.index, self.comm.rank, self.comm.world)
            peer.export(peer.flags)        # fails where CUDA IPC is not available
            ok = 1.0
        except Exception:
            ok = 0.0
        agreed = self.comm.all_reduce_sum(torch.tensor([ok], dtype=torch.float64, device=self.device))
        if float(agreed[0]) < self.comm.world:
            if peer is not None:
                peer.close()
            return None
        return peer

    def _release_peer(self):
        if getattr(self, "peer", None) is not None:
            self.torch.cuda.synchronize(self.device)
            self._step_graph = None
            self.peer.close()
            self.peer = None

    def _plan_peer_exchanges(self, h1_ptr, adj_ptr):
        """Exchanges handles and row offsets with every rank and registers the four push plans."""
        import torch.distributed as dist

        peer, plan, world, me = self.peer, self.plan, self.comm.world, self.comm.rank
        n_own, extra, row_bytes = plan.num_owned, self.TOTALS_ROWS, 4 * self.row
        ghost_begin = np.concatenate([[0], np.cumsum(self.recv_counts)]).astype(np.int64)
        send_begin = np.concatenate([[0], np.cumsum(self.send_counts)]).astype(np.int64)
        torch, dev = self.torch, self.device
        n_send = len(self.send_local)
        # rows of the evaluator's tensors that hold my send list: H1 rows are gathered straight out of the tensor
        # while they are pushed, and the peers add their H1_adj rows straight into mine
        self._send_rows_internal = torch.zeros(max(n_send, 1), dtype=torch.int32, device=dev)
        self.ev.internal_rows(self.send_local.data_ptr(), n_send, self._send_rows_internal.data_ptr())
        mine = {"n_own": n_own, "ghost_begin": ghost_begin.tolist(), "send_begin": send_begin.tolist(),
                "send_rows_internal": self._send_rows_internal[:n_send].cpu().numpy(),
                "positions": peer.export(self.local_positions.data_ptr()), "h1": peer.export(h1_ptr), "h1_adj": peer.export(adj_ptr),
                "force_recv": peer.export(self._force_recv.data_ptr()), "flags": peer.export(peer.flags)}
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        local = {"positions": self.local_positions.data_ptr(), "h1": h1_ptr, "h1_adj": adj_ptr,
                 "force_recv": self._force_recv.data_ptr(), "flags": peer.flags}
        base = [{k: (local[k] if p == me else peer.open(everyone[p][k])) for k in local} for p in range(world)]
        flags = [base[p]["flags"] for p in range(world)]
        # where my segment starts in peer p's receive buffers
        ghost_slot = [everyone[p]["n_own"] + everyone[p]["ghost_begin"][me] for p in range(world)]     # rows behind p's owned atoms
        sent_slot = [everyone[p]["send_begin"][me] for p in range(world)]                              # position in p's send list
        peer.plan(peer.PHASE_POSITIONS, self._send_pos.data_ptr(), send_begin, 24,
                  [base[p]["positions"] + 24 * ghost_slot[p] for p in range(world)], flags)
        peer.plan(peer.PHASE_H1, h1_ptr, send_begin, row_bytes,
                  [base[p]["h1"] + row_bytes * ghost_slot[p] for p in range(world)], flags,
                  row_source=self._send_rows_internal.data_ptr())
        # my ghost g, owned by p, is entry (sent_slot[p] + k) of p's send list: its adjoint goes to that row of p's H1_adj
        owner_rows = [np.asarray(everyone[p]["send_rows_internal"][sent_slot[p]:sent_slot[p] + self.recv_counts[p]], dtype=np.int32)
                      for p in range(world)]
        self._ghost_owner_rows = torch.from_numpy(np.concatenate(owner_rows + [np.zeros(1, dtype=np.int32)])).to(dev)
        peer.plan(peer.PHASE_H1_ADJ, adj_ptr + row_bytes * n_own, ghost_begin, row_bytes,
                  [base[p]["h1_adj"] for p in range(world)], flags, row_dest=self._ghost_owner_rows.data_ptr(), accumulate=True)
        force_begin = ghost_begin + extra * np.arange(world + 1)
        peer.plan(peer.PHASE_FORCES, self._force_send.data_ptr(), force_begin, 24,
                  [base[p]["force_recv"] + 24 * (sent_slot[p] + extra * me) for p in range(world)], flags)
        # the evaluator then neither packs H1 rows nor unpacks H1_adj rows itself
        self.ev.set_halo_plan(self.send_local.data_ptr(), n_send, 0, 0, world, self._ghost_begin.data_ptr(), self._force_send.data_ptr())
        dist.barrier()        # nobody pushes before every rank has mapped and planned

    def calculate(self, owned_positions=None):
        """One evaluation.  ``owned_positions``: device tensor f64 [num_owned, 3]; by default the head of
        ``local_positions`` is used as it stands (a caller may write the new positions there directly).
        Returns energy and stress of the whole system and the forces on this rank's owned atoms
        (device tensor).

        After two eager evaluations of a prepared graph the whole step -- the gather, the three phases
        and the four exchanges -- is captured into one CUDA graph and replayed from then on (every
        buffer of the step is fixed per graph); ``SXB_STEP_GRAPH=0`` keeps it eager."""
        torch = self.torch
        n_own = self.plan.num_owned
        caller_stream = torch.cuda.current_stream(self.device)
        self.stream.wait_stream(caller_stream)
        with torch.cuda.stream(self.stream):
            if owned_positions is not None and owned_positions.data_ptr() != self.local_positions.data_ptr():
                self.local_positions[:n_own].copy_(owned_positions)
            if self._step_graph is not None and not getattr(self, "_profiling", False):
                self._step_graph.replay()
                self.ev.distributed_replayed(self.generation, self._step_graph_launches)
            elif self._capture_allowed and self._eager_steps >= 2 and self._step_graph is None:
                self._capture_step()
            else:
                self._enqueue_step()
                self._eager_steps += 1
            self.ev.synchronize()        # one host synchronisation; fetches the status word (raises on a device-side error)
            if self.peer is not None and self.peer.status() != 0:
                raise RuntimeError("halo exchange: a peer did not deliver its rows within the time limit; this step is invalid")
        caller_stream.wait_stream(self.stream)
        host = self._totals_host.numpy()
        _e, f_ptr, _v = self.ev.device_results()
        forces = _as_tensor(torch, f_ptr, (n_own + self.plan.num_ghost, 3), torch.float64, self.device)
        return {"energy": float(host[0]), "stress": -host[1:].reshape(3, 3).copy() / self.volume,
                "forces": forces[:n_own], "owned": self.plan.owned}

    def close(self):
        """Releases the captured step.  Call it before the process group is destroyed: a communicator whose
        collectives sit in a live CUDA graph cannot be torn down."""
        if getattr(self, "_step_graph", None) is not None:
            self.torch.cuda.synchronize(self.device)
            self._step_graph = None
            self._capture_allowed = False
        self._release_peer()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _capture_step(self):
        """Captures one step into a CUDA graph on the calculator's stream (it also runs once, by replay)."""
        torch = self.torch
        before = self.ev.launch_count
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream, capture_error_mode="thread_local"):
                self._enqueue_step()
            self._step_graph_launches = self.ev.launch_count - before
            self._step_graph = graph
            graph.replay()
            self.ev.distributed_replayed(self.generation, 0)
        except Exception:       # capture is an optimisation: any refusal falls back to eager launches for good
            self._capture_allowed = False
            self._step_graph = None
            torch.cuda.synchronize(self.device)
            self.ev.distributed_abort()
            self._enqueue_step()

    def set_profiling(self, enabled: bool):
        """Per-stage event timing of the evaluator's kernels (``ev.profile()``); steps then run as eager launches,
        because the replayed graph of a normal step has no stage boundaries."""
        self._profiling = bool(enabled)
        self.ev.set_profiling(enabled)

    def timeline(self, repeats=5):
        """Device time of the seven segments of a step -- the four exchanges and the three phases -- from CUDA events
        between eager launches on the calculator's stream (ms, mean over ``repeats`` steps).  A diagnostic: the
        replayed graph of a normal step has no such boundaries.  Collective: every rank must call it."""
        torch = self.torch
        names = ["positions", "phase_1", "h1", "phase_2", "h1_adj", "phase_3", "forces"]
        total = dict.fromkeys(names, 0.0)
        with torch.cuda.stream(self.stream):
            for _ in range(repeats):
                marks = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
                self._marks = iter(marks)
                next(self._marks).record(self.stream)
                self._enqueue_step()
                self._marks = None
                self.ev.synchronize()
                for name, a, b in zip(names, marks[:-1], marks[1:]):
                    total[name] += a.elapsed_time(b) / repeats
        return total

    def _mark(self):
        marks = getattr(self, "_marks", None)
        if marks is not None:
            next(marks).record(self.stream)

    def _enqueue_step(self):
        ev, plan, comm = self.ev, self.plan, self.comm
        n_own, n_ghost = plan.num_owned, plan.num_ghost
        sc, rc = self.send_counts, self.recv_counts
        n_send = len(self.send_local)
        world = comm.world
        local_pos = self.local_positions
        # ghost positions: owners gather their rows, displaced to the images, straight into the peers' tails
        peer, stream = self.peer, self.stream.cuda_stream
        if peer is not None:
            peer.advance(stream)
        ev.gather_position_rows(local_pos.data_ptr(), self.send_local.data_ptr(), n_send, self.send_offset.data_ptr(),
                                self._send_pos.data_ptr())
        if peer is not None:
            peer.exchange(peer.PHASE_POSITIONS, stream)
        else:
            comm.all_to_all(self._send_pos, sc, rc, out=local_pos[n_own:])
        self._mark()
        ev.distributed_begin(self.generation, local_pos.data_ptr())       # ends by packing my H1 rows into _send_rows
        self._mark()
        # forward halo: into the tail of the feature tensor of the ranks that hold my atoms as ghosts
        if peer is not None:
            peer.exchange(peer.PHASE_H1, stream)
        else:
            comm.all_to_all(self._send_rows, sc, rc, out=self._h1_tail)
        self._mark()
        ev.distributed_continue()
        self._mark()
        # reverse halo: H1_adj rows of my ghosts leave from the tail of the adjoint tensor and are summed at their owners
        if peer is not None:
            peer.exchange(peer.PHASE_H1_ADJ, stream)
        else:
            comm.all_to_all(self._h1_adj_tail, rc, sc, out=self._got_rows)
        self._mark()
        ev.distributed_finish()       # starts by adding _got_rows, ends by packing ghost forces + totals into _force_send
        self._mark()
        # ghost forces back to the owners, with every rank's energy and virial riding along
        if peer is not None:
            peer.exchange(peer.PHASE_FORCES, stream)
        else:
            comm.all_to_all(self._force_send, self._force_send_counts, self._force_recv_counts, out=self._force_recv)
        ev.unpack_ghost_forces(world, self._send_begin.data_ptr(), self.send_local.data_ptr(), n_send, self._force_recv.data_ptr(),
                               self._totals.data_ptr())
        self._totals_host.copy_(self._totals, non_blocking=True)
        self._mark()


def _as_tensor(torch, ptr, shape, dtype, device):
    """Zero-copy torch view of device memory owned by the evaluator."""
    count = int(np.prod(shape))

    class _Array:
        __cuda_array_interface__ = {"shape": (count,), "typestr": "<f8" if dtype == torch.float64 else "<f4",
                                    "data": (int(ptr), False), "version": 2}

    return torch.as_tensor(_Array(), device=device).view(*shape)
