"""Generates tests/golden/spamm_small.npz: a small SpAMM case evaluated by a plain numpy restatement that shares
no code with the C checker or the CUDA path (float64 sums, explicit python loops over tiles).

    python tests/golden/make_golden.py

Contents: A, B (float32), tau, norm_a / norm_b (float64 tile norms), mask[i, k, j] (bool; float32 product of the
float32-rounded norms, >= float32(tau)), C (float64 sum over the surviving k of the half-rounded tile products, stored as float32).
The tile norms come from float64 sums, so a consumer compares norm maps with a tolerance and recomputes the mask
from its own norm map only where it wants bit equality; the committed mask has no product within 1e-4 relative of
tau (checked below), so any correctly rounded float norm gives the same mask.
"""
from pathlib import Path

import numpy as np

T = 32


def tile_norms(X):
    r, c = X.shape[0] // T, X.shape[1] // T
    X64 = X.astype(np.float64)
    return np.sqrt((X64 * X64).reshape(r, T, c, T).sum(axis=(1, 3)))


def make(seed=20240607, M=128, K=96, N=160, tau=None):
    rng = np.random.default_rng(seed)
    i = np.arange(M)[:, None]
    k = np.arange(K)[None, :]
    A = (rng.choice([-1.0, 1.0], size=(M, K)) * np.exp(-0.12 * np.abs(i - k)) * (0.25 + rng.random((M, K))))
    k2 = np.arange(K)[:, None]
    j = np.arange(N)[None, :]
    B = (rng.choice([-1.0, 1.0], size=(K, N)) * np.exp(-0.09 * np.abs(k2 - j * K / N)) * (0.25 + rng.random((K, N))))
    A, B = A.astype(np.float32), B.astype(np.float32)
    nA, nB = tile_norms(A), tile_norms(B)
    prod = nA.astype(np.float32)[:, :, None] * nB.astype(np.float32)[None, :, :]
    if tau is None:   # about half of the products survive
        tau = float(np.round(np.median(prod), 2))
    assert np.abs(prod.astype(np.float64) / tau - 1.0).min() > 1e-4, "a product sits too close to tau; change the seed"
    mask = prod >= np.float32(tau)
    Ah = A.astype(np.float16).astype(np.float64)
    Bh = B.astype(np.float16).astype(np.float64)
    C = np.zeros((M, N))
    for ti in range(M // T):
        for tj in range(N // T):
            for tk in range(K // T):
                if mask[ti, tk, tj]:
                    C[ti * T:(ti + 1) * T, tj * T:(tj + 1) * T] += (
                        Ah[ti * T:(ti + 1) * T, tk * T:(tk + 1) * T] @ Bh[tk * T:(tk + 1) * T, tj * T:(tj + 1) * T])
    return dict(A=A, B=B, tau=np.float64(tau), norm_a=nA, norm_b=nB, mask=mask, C=C.astype(np.float32))


if __name__ == "__main__":
    out = Path(__file__).resolve().parent / "spamm_small.npz"
    d = make()
    np.savez_compressed(out, **d)
    print(out, "survivors", int(d["mask"].sum()), "of", d["mask"].size)
