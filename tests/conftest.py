import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import __graft_entry__ as graft  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def pkg():
    return graft.load_package()


@pytest.fixture(scope="session")
def model_dir(tmp_path_factory):
    return tmp_path_factory.mktemp("models")


@pytest.fixture(scope="session")
def model_path(pkg, model_dir):
    """Returns a function (arch, seed) -> path of a generated model JSON (cached per session)."""
    cache = {}

    def get(arch="small", seed=1, **kwargs):
        key = (arch, seed, tuple(sorted(kwargs.items())))
        if key not in cache:
            path = model_dir / f"{arch}_{seed}_{len(cache)}.json"
            pkg.modelgen.write_model(path, arch, seed=seed, **kwargs)
            cache[key] = path
        return cache[key]

    return get


def csr_from_positions(positions, cell, cutoff):
    from oracle import neighbor

    first, src, shifts = neighbor.build_neighbor_graph(positions, cell, cutoff)
    xyz = neighbor.edge_vectors(positions, cell, first, src, shifts)
    return first, src, shifts, xyz
