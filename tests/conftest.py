"""Shared fixtures: tiny configurations, model folders in temporary directories,
and the `gpu` marker."""
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_configs():
    from helpers import tiny_configs as make
    return make()


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory, tiny_configs):
    """name -> (folder, page size) of every tiny configuration, weights stored in float32."""
    from helpers import write_tiny_model
    out = {}
    for name, (cfg, page) in tiny_configs.items():
        d = tmp_path_factory.mktemp(f"model_{name}")
        write_tiny_model(cfg, d, seed=11 + len(out), dtype=torch.float32)
        out[name] = (d, page)
    return out


@pytest.fixture(scope="session")
def cuda_kernels():
    from inferflux_b200.csrc import CudaKernels
    return CudaKernels("cuda:0")
