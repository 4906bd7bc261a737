import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def dev():
    import torch
    return torch.device("cuda:0")


def bf16_dev(x, device):
    """fp32 numpy array of bf16-exact values -> bf16 CUDA tensor."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(device=device, dtype=torch.bfloat16)


def f32_dev(x, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(device)


def i32_dev(x, device):
    import torch
    return torch.tensor(np.asarray(x, dtype=np.int32), dtype=torch.int32, device=device)


def host(t):
    """CUDA tensor -> fp32 / int numpy array."""
    import torch
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.float()
    return t.detach().cpu().numpy()
