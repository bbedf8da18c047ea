"""Row-block sharding over real GPUs: torchrun with one rank per GPU, NCCL broadcast of B, all-gather of B's norm
map, gather of the C slabs; rank 0 compares the gathered C and the total survivor count with the CPU checker."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _gpus():
    import torch

    return torch.cuda.device_count()


@pytest.mark.parametrize("exchange", ["push", "nccl"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_matches_checker(world, exchange):
    """exchange: how B's norm-map shares travel -- peer stores from inside the norm kernel, or an NCCL all-gather."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29700 + world + (10 if exchange == "nccl" else 0)), str(ROOT / "tests" / "_sharded_worker.py"),
           "1024", "1e-6", exchange]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600,
                       env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0, r.stdout[-3000:]
    assert "ok=True" in r.stdout
    assert f"push={exchange == 'push'}" in r.stdout
