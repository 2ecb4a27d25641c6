"""Worker of the multi-GPU decomposition test: launched by torch.distributed.run, one rank per GPU.
Compares the decomposed evaluation with the periodic single-GPU evaluation of the same system."""
import json
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as graft  # noqa: E402


def main():
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = graft.load_package()
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / f"model_{rank}.json"
        pkg.modelgen.write_model(path, "medium", seed=21)
        grid = pkg.distributed.GRIDS[world]
        pos, cell, types = pkg.modelgen.srtio3(tuple(4 * g for g in grid), 0.05, 9)
        calc = pkg.distributed.DistributedCalculator(path, pkg.MACEB200, skin=0.5, device=local)
        calc.prepare(pos, cell, types)
        for _ in range(4):       # two eager evaluations, then the captured step and one replay
            out = calc.calculate()
        assert calc._step_graph is not None or os.environ.get("SXB_STEP_GRAPH") == "0", "the step was not captured"
        forces = torch.zeros((len(pos), 3), dtype=torch.float64, device="cuda")
        forces[torch.from_numpy(out["owned"]).cuda()] = out["forces"]
        dist.all_reduce(forces)
        if rank == 0:
            single = pkg.Calculator(path, skin=0.5, device=local).calculate(pos, cell, types)
            result = {"dE_per_atom": abs(out["energy"] - single["energy"]) / len(pos),
                      "dF": float(np.abs(forces.cpu().numpy() - single["forces"]).max()),
                      "dS": float(np.abs(out["stress"] - single["stress"]).max()), "world": world, "atoms": len(pos)}
            Path(sys.argv[1]).write_text(json.dumps(result))
            print(result)
        calc.close()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
