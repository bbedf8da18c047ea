"""The CPU checker against independent restatements: numpy, the committed golden fixture and known answers."""
from pathlib import Path

import numpy as np
import pytest

from conftest import rel_fro, signed_decay

GOLDEN = Path(__file__).resolve().parent / "golden" / "spamm_small.npz"


def np_mask(nA, nB, tau):
    return (nA.astype(np.float32)[:, :, None] * nB.astype(np.float32)[None, :, :]) >= np.float32(tau)


def lists_to_mask(counts, offsets, kidx, TK):
    TM, TN = counts.shape
    m = np.zeros((TM, TK, TN), dtype=bool)
    for t in range(TM * TN):
        for k in kidx[offsets[t]:offsets[t + 1]]:
            m[t // TN, k, t % TN] = True
    return m


def test_half_rounding_matches_ieee(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal(200000).astype(np.float32) * (10.0 ** rng.integers(-9, 5, 200000)).astype(np.float32)
    special = np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e6, -1e6, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                        2.0 ** -14, 2.0 ** -14 * 0.9999, 6.1e-5, 5.96e-8, np.inf, -np.inf], dtype=np.float32)
    x = np.concatenate([x, special])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(oracle.round_to_half(x).view(np.uint32), want.view(np.uint32))
    # exhaustive over all finite half values: conversion is the identity on them
    h = np.arange(0, 0x7c00, dtype=np.uint16).view(np.float16).astype(np.float32)
    assert np.array_equal(oracle.round_to_half(h), h)
    assert np.isnan(oracle.round_to_half(np.array([np.nan], dtype=np.float32))[0])


def test_norm_map_definition(oracle):
    rng = np.random.default_rng(1)
    X = (rng.standard_normal((96, 160)) * np.exp(rng.uniform(-8, 2, (96, 160)))).astype(np.float32)
    got = oracle.norm_map(X)
    want = np.sqrt((X.astype(np.float64) ** 2).reshape(3, 32, 5, 32).sum(axis=(1, 3)))
    assert got.shape == (3, 5) and got.dtype == np.float32
    np.testing.assert_allclose(got, want, rtol=3e-7)
    with pytest.raises(ValueError):
        oracle.norm_map(np.zeros((33, 32), dtype=np.float32))


def test_norm_map_known_values(oracle):
    ones = np.ones((64, 64), dtype=np.float32)          # getNormMatrix, tool.cu:370-406: every tile norm is 32
    assert np.array_equal(oracle.norm_map(ones), np.full((2, 2), 32.0, dtype=np.float32))
    eye = np.eye(96, dtype=np.float32)
    want = np.sqrt(np.float32(32)) * np.eye(3, dtype=np.float32)
    assert np.array_equal(oracle.norm_map(eye), want)
    assert not oracle.norm_map(np.zeros((32, 32), dtype=np.float32)).any()


def test_lists_match_numpy(oracle):
    A = signed_decay(256, 0.05, 7)
    B = signed_decay(256, 0.08, 8)
    nA, nB = oracle.norm_map(A), oracle.norm_map(B)
    for tau in [0.0, 1e-3, 0.5, 3.0, 1e9]:
        counts, offsets, kidx = oracle.lists(nA, nB, tau)
        m = np_mask(nA, nB, tau)
        assert np.array_equal(counts, m.sum(axis=1))
        assert np.array_equal(lists_to_mask(counts, offsets, kidx, 8), m)
        for t in range(counts.size):                      # ascending k inside a list (cuSpAMM.cu:315-326)
            seg = kidx[offsets[t]:offsets[t + 1]]
            assert np.all(np.diff(seg) > 0)
    # row block: the reference's main_row_offset
    counts_b, offs_b, kidx_b = oracle.lists(nA, nB, 0.5, row_begin=3, row_count=2)
    full, _, _ = oracle.lists(nA, nB, 0.5)
    assert np.array_equal(counts_b, full[3:5])


def test_threshold_is_inclusive(oracle):
    """`>=` as in cuSpAMM.cu:306 and tool.cu:513: a product equal to tau survives, and tau = 0 keeps 0*0."""
    nA = np.array([[2.0, 0.0]], dtype=np.float32)
    nB = np.array([[3.0], [5.0]], dtype=np.float32)
    counts, _, kidx = oracle.lists(nA, nB, 6.0)
    assert counts[0, 0] == 1 and kidx.tolist() == [0]
    counts, _, kidx = oracle.lists(nA, nB, np.nextafter(np.float32(6.0), np.float32(7.0)))
    assert counts[0, 0] == 0
    counts, _, kidx = oracle.lists(nA, nB, 0.0)
    assert counts[0, 0] == 2 and kidx.tolist() == [0, 1]


def test_spamm_known_answers(oracle):
    A = signed_decay(128, 0.1, 3)
    B = signed_decay(128, 0.15, 4)
    Ah = A.astype(np.float16).astype(np.float64)
    Bh = B.astype(np.float16).astype(np.float64)
    C0, S0 = oracle.spamm(A, B, 0.0)                       # tau = 0: the dense product of the half-rounded inputs
    assert S0 == 4 ** 3
    assert rel_fro(C0, Ah @ Bh) < 1e-6
    Cbig, Sbig = oracle.spamm(A, B, 1e12)                  # tau above every product: nothing survives
    assert Sbig == 0 and not Cbig.any()
    eye = np.eye(128, dtype=np.float32)                    # A = I: list of C(i,j) is {i} when sqrt(32)*nB(i,j) >= tau
    nB = oracle.norm_map(B)
    tau = float(np.sqrt(np.float32(32)) * np.median(nB))
    Ci, Si, _, _, counts = oracle.spamm(eye, B, tau, want_maps=True)
    keep = (np.sqrt(np.float32(32)) * nB) >= np.float32(tau)
    assert np.array_equal(counts, keep.astype(np.int32))
    want = Bh.reshape(4, 32, 4, 32) * keep[:, None, :, None]
    assert np.array_equal(Ci, want.reshape(128, 128).astype(np.float32))


def test_reference_default_configuration(oracle):
    """para.h:2,6-8,14 + cuSpAMM.cu:428-431: 2048^3, c/(|i-j|^v+1) with c=v=0.1 stored as half, Norm=1.548969.
    12850 of 262144 tile products survive; tile norms lie in [1.019, 1.522]."""
    A = oracle.round_to_half(oracle.gen_decay_alg(0.1, 0.1, 2048, 2048))
    nA = oracle.norm_map(A)
    assert 1.0190 < nA.min() < 1.0192 and 1.5219 < nA.max() < 1.5221
    counts, offsets, _ = oracle.lists(nA, nA, 1.548969)
    assert int(offsets[-1]) == 12850
    assert int(np_mask(nA, nA, 1.548969).sum()) == 12850


def test_golden_fixture(oracle):
    d = np.load(GOLDEN)
    A, B, tau = d["A"], d["B"], float(d["tau"])
    C, S, nA, nB, counts = oracle.spamm(A, B, tau, want_maps=True)
    np.testing.assert_allclose(nA, d["norm_a"], rtol=3e-7)
    np.testing.assert_allclose(nB, d["norm_b"], rtol=3e-7)
    assert S == int(d["mask"].sum())
    assert np.array_equal(counts, d["mask"].sum(axis=1))
    _, offsets, kidx = oracle.lists(nA, nB, tau)
    assert np.array_equal(lists_to_mask(counts, offsets, kidx, d["mask"].shape[1]), d["mask"])
    assert rel_fro(C, d["C"]) < 2e-6


def test_row_blocks_tile_the_result(oracle):
    A = signed_decay(256, 0.04, 21)
    B = signed_decay(256, 0.05, 22)
    C, S = oracle.spamm(A, B, 0.3)
    parts, total = [], 0
    for b, n in [(0, 3), (3, 1), (4, 4)]:
        Cb, Sb = oracle.spamm(A, B, 0.3, row_begin=b, row_count=n)
        parts.append(Cb)
        total += Sb
    assert total == S and np.array_equal(np.vstack(parts), C)


def test_generators_follow_the_reference_formulas(oracle):
    i = np.arange(64)[:, None]
    j = np.arange(96)[None, :]
    d = np.abs(i - j).astype(np.float64)
    e = oracle.gen_decay_exp(1.0, 0.1, 64, 96)             # cuSpAMM.cu:425-426 calls it with c=1, v=0.1
    np.testing.assert_allclose(e, (np.float32(0.1).astype(np.float64) ** d).astype(np.float32), rtol=1e-6)
    a = oracle.gen_decay_alg(0.1, 0.1, 64, 96)
    want = np.float32(0.1) / ((d ** np.float64(np.float32(0.1))).astype(np.float32) + np.float32(1))
    np.testing.assert_allclose(a, want, rtol=1e-6)


def test_tuner_reaches_the_expected_rate(oracle):
    A = oracle.gen_decay_alg(0.1, 0.1, 512, 512)
    nA = oracle.norm_map(A)
    tau, rate, iters = oracle.tune_valid_rate(nA, nA, 0.75, 20, 0.01)
    assert abs(rate - 0.75) < 0.01 and 0 < iters < 20
    assert abs(np_mask(nA, nA, tau).mean() - 0.75) < 0.011


def test_exact_product_is_the_double_precision_gated_sum(oracle):
    """The checker of the split-precision mode: same lists as the half-precision checker, product of the unrounded
    inputs accumulated in double and rounded once."""
    rng = np.random.default_rng(41)
    A = (rng.standard_normal((96, 128)) * np.exp(-rng.random((96, 128)) * 4)).astype(np.float32)
    B = (rng.standard_normal((128, 160)) * np.exp(-rng.random((128, 160)) * 4)).astype(np.float32)
    # tau = 0: the plain product
    C0, S0 = oracle.spamm_exact(A, B, 0.0)
    assert S0 == 3 * 4 * 5
    # (the order of the double additions may differ from numpy's: allow one float rounding)
    np.testing.assert_allclose(C0, (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32), rtol=2e-7, atol=1e-9)
    # a threshold that drops about half of the tile products: tile by tile against numpy on the surviving k
    nA, nB = oracle.norm_map(A), oracle.norm_map(B)
    tau = float(np.median(nA[:, :, None] * nB[None]))
    C, S = oracle.spamm_exact(A, B, tau)
    C_half, S_half = oracle.spamm(A, B, tau)
    assert S == S_half and 0 < S < S0
    keep = (nA[:, :, None] * nB[None]) >= np.float32(tau)
    ref = np.zeros((96, 160), dtype=np.float64)
    for i in range(3):
        for j in range(5):
            for k in range(4):
                if keep[i, k, j]:
                    ref[i * 32:(i + 1) * 32, j * 32:(j + 1) * 32] += (
                        A[i * 32:(i + 1) * 32, k * 32:(k + 1) * 32].astype(np.float64)
                        @ B[k * 32:(k + 1) * 32, j * 32:(j + 1) * 32].astype(np.float64))
    np.testing.assert_allclose(C, ref.astype(np.float32), rtol=2e-7, atol=1e-9)
    # and the half-precision checker is a few 1e-4 away from it, as half rounding predicts
    err = np.linalg.norm(C_half - C) / np.linalg.norm(C)
    assert 1e-5 < err < 2e-3
