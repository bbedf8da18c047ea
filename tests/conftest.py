import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no sm_100 GPU in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o

    o.lib()
    return o


def signed_decay(n, lam, seed, m=None):
    """Small seeded test matrix: +-exp(-lam*|i-j|) * (0.5 + u), independent of the library's generators."""
    m = n if m is None else m
    rng = np.random.default_rng(seed)
    i = np.arange(m)[:, None]
    j = np.arange(n)[None, :]
    mag = np.exp(-lam * np.abs(i - j)) * (0.5 + rng.random((m, n)))
    sign = rng.integers(0, 2, size=(m, n)) * 2 - 1
    return (mag * sign).astype(np.float32)


def rel_fro(x, ref):
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    d = np.linalg.norm(x - ref)
    n = np.linalg.norm(ref)
    return d / n if n > 0 else d
