"""Benchmark of the force path: us/atom/step for one complete energy + forces + stress evaluation.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload at every N: the MACE-OMAT-0-medium architecture (random-init weights from a seed) on a
10x10x10 cubic SrTiO3 supercell (5,000 atoms, a = 3.905 A, sigma = 0.05 A perturbation, 0.5 A
neighbor skin), FP32 -- per GPU.  For N > 1 the ranks share one periodic system of N x 5,000 atoms,
decomposed in space (weak scaling: 5,000 owned atoms per GPU; ghost features, adjoints and forces
cross NVLink), and the line carries the difference to a single-GPU evaluation of the same system.
`value` is timed with the positions already resident in HBM; `e2e` goes through the host-facing
call with pinned host buffers (positions H2D, energies / forces / stress D2H inside the timed
region).  The reference arm (`--impl reference`) times the reference's own serial CPU evaluator
(oracle/_ref) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "us/atom/step (E+F+stress, FP32)"
UNIT = "us/atom"
SUPERCELL = 10
SIGMA = 0.05
SKIN = 0.5
PARITY_ATOM_LIMIT = 1_500_000   # largest system the N > 1 runs re-evaluate on one GPU for the parity entry
SEED = 17
# algorithmic work of the reference's formulation per (edge, channel)
FLOP_PER_EDGE_CHANNEL = {"l0_forward": 56, "l0_reverse": 284, "l1_forward": 408, "l1_reverse": 850}


def _peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "reasons": sorted(reasons), "samples": len(sm)}


RANDOM_SOLID_ELEMENTS = (1, 6, 8, 13, 14, 22, 26, 38, 56, 79)


def build_workload(tmpdir, cells=SUPERCELL, workload="srtio3", atoms=20000):
    """srtio3: medium model (128x0e+128x1o) on a perturbed SrTiO3 supercell.
    random: higher-order model (128x0e+128x1o+128x2e, 10 elements) on a seeded Poisson-disk
    disordered solid at 0.085 atoms/A^3 with 1.8 A minimum separation."""
    import __graft_entry__ as graft

    pkg = graft.load_package()
    if workload == "random":
        model = Path(tmpdir) / "large.json"
        pkg.modelgen.write_model(model, "large", seed=SEED, atomic_numbers=RANDOM_SOLID_ELEMENTS)
        pos, cell, types = pkg.modelgen.random_solid(atoms, 0.085, 1.8, len(RANDOM_SOLID_ELEMENTS), SEED)
        return pkg, model, pos, cell, types
    model = Path(tmpdir) / "medium.json"
    pkg.modelgen.write_model(model, "medium", seed=SEED)
    pos, cell, types = pkg.modelgen.srtio3(cells, SIGMA, SEED)
    return pkg, model, pos, cell, types


def edge_kernel_roofline(ev, stage_ms, num_edges, active_edges, n, measured, hbm_peak, peak_kind, traffic_key=None):
    """The `roofline` object of the bench line from the per-stage times of one rank: for every edge kernel the FP32,
    L2 and HBM fractions against measured denominators; the dominant kernel's larger fraction is `frac`.
    n = receivers of the rank, num_edges / active_edges = its edges in the list / inside the model cutoff."""
    C = ev.num_channels
    dominant = max((k for k in stage_ms if k in FLOP_PER_EDGE_CHANNEL), key=lambda k: stage_ms[k])
    num_lme, num_hidden = ev.num_lme, (ev.L_max + 1) ** 2
    # compulsory HBM bytes of one launch of each edge kernel: geometry record + source
    # index per edge, plus the node rows the kernel must read / write once
    node_rows = {"l0_forward": 16, "l0_reverse": 16, "l1_forward": num_lme + num_hidden,
                 "l1_reverse": num_lme + 3 * num_hidden}
    # spline coefficients the formulation pulls from L2 per active edge: 16 B per radial function
    # (+ the source feature rows in layer 1)
    l2_bytes_per_edge = {"l0_forward": 16 * 4 * C, "l0_reverse": 16 * 4 * C,
                         "l1_forward": 16 * ev.num_paths * C + 4 * num_hidden * C,
                         "l1_reverse": 16 * ev.num_paths * C + 8 * num_hidden * C}
    kernels = {}
    for name in FLOP_PER_EDGE_CHANNEL:
        if name not in stage_ms:
            continue
        seconds = stage_ms[name] * 1e-3
        flops = FLOP_PER_EDGE_CHANNEL[name] * active_edges * C
        hbm_bytes = num_edges * 20 + n * node_rows[name] * C * 4
        l2_bytes = l2_bytes_per_edge[name] * active_edges
        kernels[name] = {"ms": stage_ms[name], "fp32_tflops": flops / seconds / 1e12,
                         "fp32_frac": flops / seconds / 1e12 / measured["fp32_fma_tflops"],
                         "hbm_gbs": hbm_bytes / seconds / 1e9, "hbm_frac": hbm_bytes / seconds / 1e9 / hbm_peak,
                         "l2_gbs": l2_bytes / seconds / 1e9, "l2_frac": l2_bytes / seconds / 1e9 / measured["l2_read_gbs"]}
    dom = kernels[dominant]
    alg_bytes = num_edges * 20 + n * node_rows[dominant] * C * 4
    alg_flops = FLOP_PER_EDGE_CHANNEL[dominant] * active_edges * C
    # DRAM bytes of one launch (dram__bytes_read.sum + dram__bytes_write.sum) from the tracked ncu
    # summary of this kernel and workload, when one exists
    traffic = None
    captured = ROOT / "profiles" / "dram_traffic.json"
    if captured.exists() and traffic_key is not None:
        traffic = json.loads(captured.read_text()).get(traffic_key, {}).get(dominant)
    # the edge kernels move their compulsory HBM bytes at a few per cent of the copy bandwidth; what
    # bounds them is FP32 issue (gradient kernels) or L2-to-SM delivery (forward kernels), so the
    # fraction reported is the larger of the FP32 and the HBM fraction, each against a measured peak
    if dom["fp32_frac"] >= dom["hbm_frac"]:
        roofline = {"bound": "fp32", "kernel": dominant, "achieved": dom["fp32_tflops"], "peak": measured["fp32_fma_tflops"],
                    "unit": "TFLOP/s", "frac": dom["fp32_frac"], "peak_source": "measured FMA probe (sxb_measure_device_peaks)"}
    else:
        roofline = {"bound": "hbm", "kernel": dominant, "achieved": dom["hbm_gbs"], "peak": hbm_peak, "unit": "GB/s",
                    "frac": dom["hbm_frac"], "peak_source": f"{peak_kind} copy bandwidth"}
    roofline.update({"traffic": traffic, "kernel_ms": stage_ms[dominant], "algorithmic_bytes": alg_bytes,
                     "algorithmic_gflop": alg_flops / 1e9, "hbm_gbs": dom["hbm_gbs"], "hbm_peak_gbs": hbm_peak,
                     "hbm_frac": dom["hbm_frac"], "l2_read_gbs": dom["l2_gbs"], "l2_peak_gbs": measured["l2_read_gbs"],
                     "l2_frac": dom["l2_frac"], "fp32_peak_tflops": measured["fp32_fma_tflops"],
                     "edge_kernels": {k: {q: round(v, 4) for q, v in d.items()} for k, d in kernels.items()}})
    return roofline


def run_distributed(args):
    """N > 1: one periodic SrTiO3 system of 5,000 atoms per GPU (10x10x10 cells per brick), decomposed
    in space over the ranks; ghost positions, features, adjoints and forces cross NVLink as pushes into peer memory
    (NCCL all-to-alls where peer mapping is unavailable)."""
    # NCCL only carries the set-up collectives and the barriers here: in-switch reduction buys nothing, and a rank that
    # dies while bound to an NVLink multicast object can disturb its peers' GPUs
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def all_reduce(tensor, op=None):
        if world > 1:
            dist.all_reduce(tensor, op=op if op is not None else dist.ReduceOp.SUM)

    import __graft_entry__ as graft

    pkg = graft.load_package()
    with tempfile.TemporaryDirectory() as tmp:
        grid = pkg.distributed.GRIDS[world]
        if args.workload == "random":
            # the 20,000-atom disordered solid as one system split over the ranks (strong scaling)
            model = Path(tmp) / f"large_{rank}.json"
            pkg.modelgen.write_model(model, "large", seed=SEED, atomic_numbers=RANDOM_SOLID_ELEMENTS)
            pos, cell, types = pkg.modelgen.random_solid(args.atoms, 0.085, 1.8, len(RANDOM_SOLID_ELEMENTS), SEED)
        else:
            model = Path(tmp) / f"medium_{rank}.json"
            pkg.modelgen.write_model(model, "medium", seed=SEED)
            pos, cell, types = pkg.modelgen.srtio3(tuple(args.cells * g for g in grid), SIGMA, SEED)
        total_atoms = len(pos)
        calc = pkg.distributed.DistributedCalculator(model, pkg.MACEB200, skin=SKIN, device=local_rank)
        if args.tile > 0:
            calc.ev.set_tile_size(args.tile)
        plan = calc.prepare(pos, cell, types, grid)
        n_own = plan.num_owned
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
        owned_dev = calc.owned_positions
        pinned = owned_dev.cpu().pin_memory()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def step_device():
            start.record()
            calc.calculate(owned_dev)
            stop.record()
            stop.synchronize()
            return start.elapsed_time(stop)

        def step_e2e():
            t0 = time.perf_counter()
            calc.owned_positions.copy_(pinned, non_blocking=True)      # H2D straight into the step's input buffer
            out = calc.calculate()
            forces = out["forces"].cpu()
            return (time.perf_counter() - t0) * 1e3, out, forces

        sampler = ClockSampler(local_rank)
        sampler.start()
        for _ in range(max(args.warmup, 3)):
            flush.fill_(1)
            step_device()
        t_busy = time.perf_counter()
        while time.perf_counter() - t_busy < 0.4:
            step_device()
        barrier()
        launches_before = calc.ev.launch_count
        # K steps between two barriers; every step is timed with CUDA events on this rank's stream after an L2
        # flush of its own.  No barrier inside the loop: the ranks meet at the exchanges of the step itself, as they
        # do in a running simulation, so a late exit from a barrier is not billed to every step.
        device_ms = []
        wall0 = time.perf_counter()
        for _ in range(args.steps):
            flush.fill_(1)
            device_ms.append(step_device())
        barrier()
        wall_ms = (time.perf_counter() - wall0) * 1e3
        launches = calc.ev.launch_count - launches_before
        for _ in range(3):
            step_e2e()
        barrier()
        e2e_ms = []
        for _ in range(args.steps):
            flush.fill_(1)
            torch.cuda.synchronize()
            ms, last_out, _forces = step_e2e()
            e2e_ms.append(ms)
        barrier()
        clocks = sampler.stop()
        # per-stage device times of this rank's kernels (separate passes with event pairs around each stage)
        calc.set_profiling(True)
        stage_ms = {}
        for _ in range(3):
            flush.fill_(1)
            barrier()
            step_device()
            for name, ms, _l in calc.ev.profile():
                stage_ms[name] = stage_ms.get(name, 0.0) + ms / 3
        calc.set_profiling(False)
        # roofline of this rank's edge kernels from those stage times (rank 0 reports); edges inside the model cutoff are
        # counted from the local graph while it is small enough to fetch
        roofline = None
        if rank == 0 and stage_ms:
            local_edges = int(calc.num_edges)
            if n_own + plan.num_ghost <= 200000:
                first, sources, _shifts = calc.ev.graph(calc.generation, with_shifts=False)
                local = calc.local_positions.cpu().numpy()
                recv = np.repeat(np.arange(n_own), np.diff(first))
                d = local[sources] - local[recv]
                active_local = int((np.sqrt((d * d).sum(1)) < calc.ev.r_cut).sum())
            else:
                active_local = int(round(local_edges * 0.7441))     # ratio measured on the 5,000-atom case
            hbm_peak, peak_kind = _peaks()
            roofline = edge_kernel_roofline(calc.ev, stage_ms, local_edges, active_local, n_own,
                                            pkg.measure_device_peaks(local_rank), hbm_peak, peak_kind)
            roofline["scope"] = "rank 0's kernels"
        # where a step spends its time: the four exchanges and the three phases, from eager launches (outside the timed region)
        barrier()
        timeline = calc.timeline(5)
        barrier()
        t = torch.tensor([float(np.mean(device_ms)), float(np.mean(e2e_ms))], device="cuda", dtype=torch.float64)
        if world > 1:
            all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms, e2e_step_ms = float(t[0]), float(t[1])
        counts = torch.tensor([float(n_own), float(plan.num_ghost), float(calc.num_edges), float(launches)], device="cuda",
                              dtype=torch.float64)
        all_reduce(counts)
        # outside the timed region: the same global system evaluated by rank 0's GPU alone
        gathered = torch.zeros((total_atoms, 3), dtype=torch.float64, device="cuda")
        gathered[torch.from_numpy(last_out["owned"]).cuda()] = last_out["forces"]
        all_reduce(gathered)
        parity = None
        # the whole system on one GPU beside the decomposed state: only while it fits comfortably
        if rank == 0 and total_atoms <= PARITY_ATOM_LIMIT:
            single_calc = pkg.Calculator(model, skin=SKIN, device=local_rank)
            if args.tile > 0:
                single_calc.evaluator.set_tile_size(args.tile)
            single = single_calc.calculate(pos, cell, types)
            parity = {"dE_eV_per_atom": abs(last_out["energy"] - single["energy"]) / total_atoms,
                      "max_dF_eV_per_A": float(np.abs(gathered.cpu().numpy() - single["forces"]).max()),
                      "max_dstress_eV_per_A3": float(np.abs(last_out["stress"] - single["stress"]).max())}
            del single_calc
        if rank == 0:
            row_bytes = calc.row * 4
            ghosts = int(counts[1].item())
            print(json.dumps({
                "metric": METRIC, "value": step_ms * 1e3 / total_atoms, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": False,
                "scaling": "strong" if args.workload == "random" else "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": (f"large-{total_atoms}-random-solid split over {world} GPUs" if args.workload == "random"
                                        else f"medium-{total_atoms // world}-SrTiO3 per GPU"),
                           "atoms_per_gpu": total_atoms // world,
                           "tile": args.tile if args.tile > 0 else None,
                           "total_atoms": total_atoms, "edges_total": int(counts[2].item()), "ghosts_total": ghosts, "skin": SKIN,
                           "parallelism": f"domain decomposition {grid[0]}x{grid[1]}x{grid[2]}, {calc.transport} halo exchange",
                           "halo_bytes_per_step": ghosts * (2 * row_bytes + 24 + 24), "elements": int(types.max()) + 1,
                           "l2": "flushed between timed steps (256 MiB write)"},
                "atoms_per_s": total_atoms / (step_ms * 1e-3),
                "us_per_atom_per_gpu": step_ms * 1e3 / (total_atoms / world),
                "e2e": {"value": e2e_step_ms * 1e3 / total_atoms, "unit": UNIT, "h2d_bytes_per_step": 24 * total_atoms,
                        "d2h_bytes_per_step": 24 * total_atoms + 80 * world, "ms_per_step": e2e_step_ms},
                "gpu_launches": int(counts[3].item()),
                "clocks": clocks,
                "roofline": roofline,
                "parity_vs_single_gpu": parity,
                "stage_ms_rank0": {k: round(v, 4) for k, v in stage_ms.items()},
                "step_timeline_ms_rank0": {k: round(v, 4) for k, v in timeline.items()},
                "step_ms_rank0": {"min": float(np.min(device_ms)), "median": float(np.median(device_ms)), "max": float(np.max(device_ms))},
                "energy_eV_per_atom": last_out["energy"] / total_atoms,
                "wall_ms_timed_region": wall_ms,
            }))
        calc.close()          # the captured step holds the communicator's kernels: release it before the group goes
        del calc
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            dist.destroy_process_group()


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.decomposed:
        return run_distributed(args)
    torch.cuda.set_device(local_rank)
    with tempfile.TemporaryDirectory() as tmp:
        pkg, model, pos, cell, types = build_workload(tmp, args.cells, args.workload, args.atoms)
        ev = pkg.MACEB200(model, device=local_rank)
        if args.tile > 0:
            ev.set_tile_size(args.tile)
        n = len(pos)
        volume = abs(np.linalg.det(cell))
        res = ev._prepare_periodic_factorized_graph(types, pos, cell, np.linalg.inv(cell), ev.r_cut + SKIN)
        gen, num_edges = res["generation"], res["num_edges"]
        if n <= 100000:
            first, sources, shifts = ev.graph(gen)
            recv = np.repeat(np.arange(n), np.diff(first))
            xyz = pos[sources] - pos[recv] + shifts @ cell
            active_edges = int((np.sqrt((xyz * xyz).sum(1)) < ev.r_cut).sum())
        else:
            active_edges = int(round(num_edges * 0.7441))     # ratio measured on the 5,000-atom case

        d_pos = torch.from_numpy(pos.reshape(-1).copy()).cuda()
        flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
        pinned_pos = torch.from_numpy(pos.reshape(-1).copy()).pin_memory()
        host_pos = pinned_pos.numpy()

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def step_device():
            ev.compute_positions_device(gen, d_pos.data_ptr())
            return ev.last_compute_ms

        def step_e2e():
            t0 = time.perf_counter()
            ev._compute_prepared_factorized_positions(gen, host_pos)
            energies = ev.node_energies
            forces = ev._reduce_atom_forces(n, execution_graph_generation=gen)
            stress = ev._reduce_stress(volume, execution_graph_generation=gen)
            return (time.perf_counter() - t0) * 1e3, float(energies.sum()), forces, stress

        sampler = ClockSampler(local_rank)
        sampler.start()
        for _ in range(max(args.warmup, 3)):
            flush.fill_(1)
            step_device()
        # keep the GPU under the same load for ~0.4 s so that the 50 ms clock samples see it busy
        t_busy = time.perf_counter()
        while time.perf_counter() - t_busy < 0.4:
            step_device()
        barrier()
        launches_before = ev.launch_count
        wall0 = time.perf_counter()
        device_ms = []
        for _ in range(args.steps):
            flush.fill_(1)
            torch.cuda.synchronize()
            device_ms.append(step_device())
        barrier()
        wall_ms = (time.perf_counter() - wall0) * 1e3
        launches = ev.launch_count - launches_before
        # end to end through the host-facing call
        for _ in range(3):
            step_e2e()
        e2e_ms = []
        for _ in range(args.steps):
            flush.fill_(1)
            torch.cuda.synchronize()
            ms, last_energy, _f, _s = step_e2e()
            e2e_ms.append(ms)
        clocks = sampler.stop()
        # per-kernel device times (separate pass with event pairs around each stage)
        ev.set_profiling(True)
        stage_ms = {}
        reps = 5
        for _ in range(reps):
            flush.fill_(1)
            torch.cuda.synchronize()
            step_device()
            for name, ms, _l in ev.profile():
                stage_ms[name] = stage_ms.get(name, 0.0) + ms / reps
        ev.set_profiling(False)

        step_ms = float(np.mean(device_ms))
        e2e_step_ms = float(np.mean(e2e_ms))
        if world > 1:
            t = torch.tensor([step_ms, e2e_step_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            step_ms, e2e_step_ms = float(t[0]), float(t[1])
        total_atoms = n * world
        value = step_ms * 1e3 / n          # us/atom/step on each GPU's own replica; atoms/s scales with N
        e2e_value = e2e_step_ms * 1e3 / n

        hbm_peak, peak_kind = _peaks()
        measured = pkg.measure_device_peaks(local_rank)      # FP32 FMA rate and L2-to-SM bandwidth, probed now
        roofline = edge_kernel_roofline(ev, stage_ms, num_edges, active_edges, n, measured, hbm_peak, peak_kind,
                                        "medium-5000-SrTiO3" if args.workload == "srtio3" and n == 5000 and args.tile == 0 else None)

        md_report = None
        if args.md_steps > 0:
            # 20-step NVE sequence of the capacity case: velocities at 300 K from the seed, 1 fs steps
            z = np.array(ev.atomic_numbers)[types]
            masses = np.array([pkg.md.MASSES[int(v)] for v in z])
            vel = pkg.md.maxwell_boltzmann(masses, 300.0, SEED)
            integ = pkg.md.NVEIntegrator(ev, pos, cell, types, masses, vel, dt_fs=1.0, skin=SKIN)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            energies = integ.run(args.md_steps)
            torch.cuda.synchronize()
            md_ms = (time.perf_counter() - t0) * 1e3 / args.md_steps
            md_report = {"steps": args.md_steps, "dt_fs": 1.0, "temperature_K": 300.0, "ms_per_step": md_ms,
                         "us_per_atom_per_step": md_ms * 1e3 / n, "rebuilds": integ.rebuilds,
                         "max_energy_drift_eV_per_atom": float(np.abs(energies - energies[0]).max() / n)}
        # neighbor-graph rebuild (cell list, ordered CSR, permutation, tables), outside the timed region: the
        # host-facing call from host positions to a ready graph, wall clock including its synchronisation
        build_ms = []
        inverse_cell = np.linalg.inv(cell)
        for _ in range(3 if n <= 2_000_000 else 1):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ev._prepare_periodic_factorized_graph(types, pos, cell, inverse_cell, ev.r_cut + SKIN)
            build_ms.append((time.perf_counter() - t0) * 1e3)
        cpu = None
        if rank == 0 and world == 1 and args.cells == SUPERCELL and args.workload == "srtio3":
            cpu = cpu_baseline(pkg, model, sample_cells=3, calls=2)

        if world > 1:
            dist.barrier()
        if rank == 0:
            line = {
                "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": False, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"medium-{n}-SrTiO3" if args.workload == "srtio3" else f"large-{n}-random-solid",
                           "atoms_per_gpu": n, "total_atoms": total_atoms,
                           "tile": args.tile if args.tile > 0 else None,
                           "device_memory_gb": round(torch.cuda.mem_get_info()[1] / 1e9 - torch.cuda.mem_get_info()[0] / 1e9, 2),
                           "edges_per_gpu": num_edges, "active_edges_per_gpu": active_edges, "skin": SKIN,
                           "parallelism": "replicas" if world > 1 else "single", "elements": int(types.max()) + 1,
                           "l2": "flushed between timed steps (256 MiB write)"},
                "atoms_per_s": total_atoms / (step_ms * 1e-3),
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 24 * n,
                        "d2h_bytes_per_step": 8 * n + 24 * n + 72 + 80, "ms_per_step": e2e_step_ms},
                "gpu_launches": int(launches),
                "clocks": clocks,
                "roofline": roofline,
                "stage_ms": {k: round(v, 4) for k, v in stage_ms.items()},
                "graph_build_ms": round(float(np.median(build_ms)), 3),
                "energy_eV_per_atom": last_energy / n,
                "wall_ms_timed_region": wall_ms,
            }
            if md_report is not None:
                line["md"] = md_report
            if cpu is not None:
                line["cpu_baseline"] = cpu
            print(json.dumps(line))
        if world > 1:
            dist.destroy_process_group()


def _time_reference(pkg, model, cells, warm, steps, threads):
    """Throughput of the reference's serial evaluator MACECPU<float> (oracle/_ref) on the host cores:
    its source has no OpenMP, so the cores are used the only way it allows - `threads` independent
    evaluator instances, one per thread, each computing the same bounded sample `steps` times (the
    foreign call releases the interpreter lock).  Returns (us/atom aggregated over the threads,
    ms per call of one instance, atoms, edges)."""
    import threading

    from oracle import neighbor, ref

    pos, cell, types = pkg.modelgen.srtio3(cells, SIGMA, SEED)
    probe = ref.ReferenceMACE(str(model), double=False)
    first, src, shifts = neighbor.build_neighbor_graph(pos, cell, probe.r_cut)
    xyz = neighbor.edge_vectors(pos, cell, first, src, shifts)
    counts = np.diff(first)
    start = threading.Barrier(threads + 1)
    done = threading.Barrier(threads + 1)
    per_call = [0.0] * threads

    def worker(index):
        m = probe if index == 0 else ref.ReferenceMACE(str(model), double=False)
        for _ in range(warm):
            m.compute(types, counts, src, xyz)   # the first call also builds the radial cache
        start.wait()
        t0 = time.perf_counter()
        for _ in range(steps):
            m.compute(types, counts, src, xyz)
        per_call[index] = (time.perf_counter() - t0) / steps
        done.wait()

    pool = [threading.Thread(target=worker, args=(i,), daemon=True) for i in range(threads)]
    for t in pool:
        t.start()
    start.wait()
    t0 = time.perf_counter()
    done.wait()
    wall = time.perf_counter() - t0
    for t in pool:
        t.join()
    value = wall * 1e6 / (threads * steps * len(pos))
    return value, float(np.mean(per_call)) * 1e3, len(pos), len(src)


def _host_threads():
    """Host threads available to this process (capped: every thread holds its own evaluator instance)."""
    try:
        count = len(os.sched_getaffinity(0))
    except AttributeError:
        count = os.cpu_count() or 1
    return max(1, min(count, 128))


def cpu_baseline(pkg, model, sample_cells=3, calls=2):
    """Times the reference's evaluator (oracle/_ref, MACECPU<float>) on a bounded sample, all host cores."""
    from oracle import ref

    if not ref.available():
        return {"value": None, "unit": UNIT, "cores": 0, "kind": "reference", "sample": "oracle/_ref not built"}
    threads = _host_threads()
    value, call_ms, atoms, edges = _time_reference(pkg, model, sample_cells, 1, calls, threads)
    return {"value": value, "unit": UNIT, "cores": threads, "kind": "reference",
            "sample": f"{atoms}-atom SrTiO3 ({sample_cells}x{sample_cells}x{sample_cells}), same model, {edges} edges at the "
                      f"model cutoff; {threads} independent instances of the serial MACECPU<float>, one per host thread, "
                      f"{calls} calls each ({call_ms:.0f} ms per call); one instance alone: {call_ms * 1e3 / atoms:.0f} us/atom"}


def _available_memory_gb():
    try:
        for line in Path("/proc/meminfo").read_text().splitlines():
            if line.startswith("MemAvailable:"):
                return float(line.split()[1]) / 1e6
    except OSError:
        pass
    return 16.0


def run_reference(args):
    """The reference's own CPU implementation of the path (its serial evaluator MACECPU<float>, compiled
    from the reference's sources into oracle/_ref) on this arm's configuration: the full 5,000-atom
    SrTiO3 system with the medium model.  Its source has no OpenMP, so the host cores are used the only
    way it allows: independent evaluator instances, one per thread, each evaluating the whole system
    (about 3 GB of host memory and 15-30 s per call each; the instance count is capped by the memory)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    with tempfile.TemporaryDirectory() as tmp:
        pkg, model, pos, cell, types = build_workload(tmp)
        from oracle import ref

        if not ref.available():
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref was not built in this snapshot"}))
            return
        cells = SUPERCELL
        warm = 1                                   # the first call also builds the radial cache
        steps = max(1, min(args.steps, 2))
        threads = max(1, min(_host_threads(), int(_available_memory_gb() / 4.0)))
        value, call_ms, atoms, edges = _time_reference(pkg, model, cells, warm, steps, threads)
        ms = value * atoms / 1e3      # aggregated time per 5,000-atom evaluation
        sample = (f"the whole workload: {atoms}-atom SrTiO3 ({cells}x{cells}x{cells}), {edges} edges at the model cutoff; "
                  f"{threads} independent instances of the reference's serial evaluator MACECPU<float> (no OpenMP in its "
                  f"source), one per host thread, {steps} timed calls each after {warm} warm-up, {call_ms / 1e3:.1f} s per call")
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "medium-5000-SrTiO3", "atoms_per_gpu": atoms, "total_atoms": atoms, "skin": 0.0,
                       "elements": int(types.max()) + 1},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "reference", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--cells", type=int, default=SUPERCELL, help="SrTiO3 supercell edge (per GPU); default 10 = 5,000 atoms")
    parser.add_argument("--md-steps", type=int, default=0, help="also run this many NVE steps (1 fs, 300 K) and report the drift")
    parser.add_argument("--tile", type=int, default=0, help="receivers per tile for tiled streaming (0 = off)")
    parser.add_argument("--workload", default="srtio3", choices=["srtio3", "random"],
                        help="srtio3: medium model on SrTiO3 (default); random: 0e+1o+2e model on a disordered 10-element solid")
    parser.add_argument("--atoms", type=int, default=20000, help="atoms of the random workload")
    parser.add_argument("--decomposed", action="store_true",
                        help="with one GPU: run the domain-decomposed path on a single rank (ghosts = periodic images of "
                             "the rank's own atoms), to separate its bookkeeping from the inter-GPU exchange")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
