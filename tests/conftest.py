import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # GPU tests are selected with -m gpu; without a device they are skipped rather than failed
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def ref_cuda_ops():
    """torch.ops namespaces of the reference's own CUDA kernels (oracle/_ref/_C_ref.so),
    or None when that library was not built."""
    import torch
    so = ROOT / "oracle" / "_ref" / "_C_ref.so"
    if not so.exists():
        return None
    torch.ops.load_library(str(so))
    return torch.ops._C_ref, torch.ops._C_ref_cache_ops
