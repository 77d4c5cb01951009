import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (B200); run with -m gpu")


def _has_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import build, oracle as O
    build.build_oracle()
    return O


@pytest.fixture(scope="session")
def hq():
    """The product package with libhq.so loaded (built in-tree if missing)."""
    import hecbench_b200
    if not hecbench_b200.lib_path().exists():
        from hecbench_b200 import build
        build.build()
    hecbench_b200.load_library()
    return hecbench_b200


@pytest.fixture(scope="session")
def dev():
    import torch
    return torch.device("cuda:0")


def to_dev(a: np.ndarray, dev):
    import torch
    if a.dtype == np.uint32:
        a = a.view(np.int32)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)
