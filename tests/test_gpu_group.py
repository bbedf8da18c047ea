"""Several GPUs driven by one process through the group entry points of the C ABI (the reference's DEVICEDIM form,
para.h:9, cuSpAMM.cu:404-451,470-537), against the CPU checker: on one device always, on two and four when the
machine has them.  Whole host matrices in and out; sizes that are not multiples of 32; shares of B of unequal size."""
import numpy as np
import pytest

from conftest import rel_fro, signed_decay

pytestmark = pytest.mark.gpu
C_TOL = 1e-3


def _gpus():
    import torch

    return torch.cuda.device_count()


@pytest.mark.parametrize("n_devices", [1, 2, 4])
@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (520, 330, 700)])
def test_group_matches_checker(oracle, n_devices, shape):
    from cuspamm_b200 import SpammGroup, pad_to_tiles

    if _gpus() < n_devices:
        pytest.skip(f"needs {n_devices} GPUs")
    M, K, N = shape
    A = np.ascontiguousarray(signed_decay(max(M, K), 0.02, seed=61)[:M, :K])
    B = np.ascontiguousarray(signed_decay(max(K, N), 0.03, seed=62)[:K, :N])
    Ap, Bp = pad_to_tiles(A), pad_to_tiles(B)
    tau = float(np.median(oracle.norm_map(Ap)[:, :, None] * oracle.norm_map(Bp)[None]))
    C_ref, S, nA, nB, counts = oracle.spamm(Ap, Bp, tau, want_maps=True)
    C_ref = C_ref[:M, :N]
    with SpammGroup(M, K, N, n_devices=n_devices) as g:
        assert len(g.plans) == n_devices
        assert sum(p.row_tile_count for p in g.plans) == -(-M // 32)
        g.upload(A, B)
        for _ in range(3):                       # several steps: the double-buffered maps and the flags are reused
            g.run(tau)
        g.sync()
        assert g.survivors() == S
        assert rel_fro(g.download_c(), C_ref) <= C_TOL
        for p in g.plans:                        # every device holds the whole map of B, bit for bit
            assert np.array_equal(p.norm_b().view(np.uint32), nB.view(np.uint32))
            assert np.array_equal(p.norm_a().view(np.uint32),
                                  nA[p.row_tile_begin:p.row_tile_begin + p.row_tile_count].view(np.uint32))
            got, _ = p.counts()
            assert np.array_equal(got, counts[p.row_tile_begin:p.row_tile_begin + p.row_tile_count])
        # host matrices in and out in one call, twice (buffers reused), then a step on the resident matrices again
        for _ in range(2):
            C, st = g.multiply(A, B, tau)
            assert st["survivors"] == S and rel_fro(C, C_ref) <= C_TOL
        g.run(0.0)
        g.sync()
        assert g.survivors() == (-(-M // 32)) * (-(-K // 32)) * (-(-N // 32))
