"""Parity of the CUDA path (through the C ABI) with the CPU checker on the same seeded inputs.

Bars: norm maps bit-equal; skip lists (lengths and k indices) bit-equal; C within relative Frobenius error 1e-3
of the checker (the tolerance the target states for half inputs; observed values are ~1e-6, the difference being
only the order of the float accumulation inside the tensor cores).
"""
import numpy as np
import pytest

from conftest import rel_fro, signed_decay

pytestmark = pytest.mark.gpu

C_TOL = 1e-3


def run_plan(A, B, tau, row_begin=0, row_count=None):
    from cuspamm_b200 import SpammPlan

    M, K = A.shape
    N = B.shape[1]
    with SpammPlan(M, K, N, row_begin, row_count) as p:
        p.upload(np.ascontiguousarray(A[p.row_tile_begin * 32:(p.row_tile_begin + p.row_tile_count) * 32]), B)
        p.run(tau)
        p.sync()
        out = dict(C=p.download_c(), nA=p.norm_a(), nB=p.norm_b())
        out["counts"], out["S"] = p.counts()
        out["offsets"], out["kidx"] = p.lists()
    return out


def check_against_oracle(oracle, A, B, tau, row_begin=0, row_count=None):
    got = run_plan(A, B, tau, row_begin, row_count)
    Cref, S, nA, nB, counts = oracle.spamm(A, B, tau, row_begin, row_count, want_maps=True)
    assert np.array_equal(got["nA"].view(np.uint32), nA.view(np.uint32)), "norm map of A differs"
    assert np.array_equal(got["nB"].view(np.uint32), nB.view(np.uint32)), "norm map of B differs"
    assert got["S"] == S
    assert np.array_equal(got["counts"], counts)
    full_nA = oracle.norm_map(A)
    _, offs, kidx = oracle.lists(full_nA, nB, tau, row_begin, counts.shape[0])
    assert np.array_equal(got["offsets"], offs)
    assert np.array_equal(got["kidx"], kidx)
    err = rel_fro(got["C"], Cref)
    assert err <= C_TOL, f"C rel-Frobenius error {err}"
    # tiles whose list is empty are exact zeros
    empty = counts == 0
    if empty.any():
        Ct = got["C"].reshape(counts.shape[0], 32, counts.shape[1], 32)
        assert not Ct.transpose(0, 2, 1, 3)[empty].any()
    return got, err


@pytest.mark.parametrize("n", [32, 64, 96, 128])
def test_tiny_elementwise(oracle, n):
    A = signed_decay(n, 0.3, seed=n)
    B = signed_decay(n, 0.2, seed=n + 1)
    got, _ = check_against_oracle(oracle, A, B, 1e-3)
    Cref, _ = oracle.spamm(A, B, 1e-3)
    np.testing.assert_allclose(got["C"], Cref, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("tau", [0.0, 1e-6, 1e-2, 0.5, 5.0, 1e9])
def test_partial_masks_256(oracle, tau):
    A = signed_decay(256, 0.05, seed=7)
    B = signed_decay(256, 0.08, seed=8)
    check_against_oracle(oracle, A, B, tau)


def test_rectangular(oracle):
    rng = np.random.default_rng(3)
    A = (rng.standard_normal((160, 96)) * np.exp(-rng.random((160, 96)) * 6)).astype(np.float32)
    B = (rng.standard_normal((96, 416)) * np.exp(-rng.random((96, 416)) * 6)).astype(np.float32)
    check_against_oracle(oracle, A, B, 0.6)


@pytest.mark.parametrize("tau", [1e-6, 1e-4, 3e-3])
def test_ragged_steps_across_list_batches(oracle, tau):
    """Tile magnitudes spread over six decades, independently per tile: a k then has up to four steps (nested row
    sets) whose columns fall into several runs, a macro tile's list is several times 32 steps long (the multiply
    kernel reads it 32 steps at a time and a k's steps may straddle two reads), and the last macro tile row and
    column are cut (9 x 48 x 17 tiles)."""
    rng = np.random.default_rng(41)
    M, K, N = 288, 1536, 544

    def ragged(rows, cols):
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        scale = np.power(10.0, -6.0 * rng.random((rows // 32, cols // 32))).astype(np.float32)
        return (x.reshape(rows // 32, 32, cols // 32, 32) * scale[:, None, :, None]).reshape(rows, cols) / 32

    A, B = ragged(M, K), ragged(K, N)
    got, _ = check_against_oracle(oracle, A, B, tau)
    # the case is what it claims to be: lists longer than one read, and tiles with partly filled lists
    assert got["counts"].max() > 8
    assert 0 < got["S"] < (M // 32) * (K // 32) * (N // 32)


def test_random_shapes_and_magnitudes(oracle):
    """Two dozen seeded cases of random tile counts (1-13 x 1-259 x 1-39), spreads of the tile magnitudes (half a
    decade to eight) and thresholds: lists bit-equal, C within tolerance, whatever mix of full, partial and empty
    steps, runs of columns and list lengths comes out."""
    rng = np.random.default_rng(2024)

    def ragged(rows, cols, decades):
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        scale = np.power(10.0, -decades * rng.random((rows // 32, cols // 32))).astype(np.float32)
        return (x.reshape(rows // 32, 32, cols // 32, 32) * scale[:, None, :, None]).reshape(rows, cols) / 32

    survivors = []
    for _ in range(24):
        mt, kt, nt = int(rng.integers(1, 14)), int(rng.integers(1, 260)), int(rng.integers(1, 40))
        decades = float(rng.choice([0.5, 2, 4, 6, 8]))
        tau = float(10.0 ** rng.uniform(-7, -0.5))
        A, B = ragged(32 * mt, 32 * kt, decades), ragged(32 * kt, 32 * nt, decades)
        got, _ = check_against_oracle(oracle, A, B, tau)
        survivors.append(got["S"] / (mt * kt * nt))
    assert min(survivors) < 0.05 and max(survivors) > 0.5     # the cases span nearly empty to mostly full


def test_config1_n1024(oracle):
    """The smallest benchmark configuration: N=1024, A=B, a_ij = +-exp(-0.5|i-j|), tau=1e-6."""
    from cuspamm_b200 import gen_signed_exp

    A = gen_signed_exp(0.5, 1, 1024, 1024)
    got, err = check_against_oracle(oracle, A, A.copy(), 1e-6)
    assert 0 < got["S"] < 32 ** 3
    assert err < 1e-4


def test_row_block(oracle):
    A = signed_decay(512, 0.02, seed=11)
    B = signed_decay(512, 0.03, seed=12)
    full, _ = check_against_oracle(oracle, A, B, 0.05)
    part, _ = check_against_oracle(oracle, A, B, 0.05, row_begin=5, row_count=7)
    assert rel_fro(part["C"], full["C"][5 * 32:12 * 32]) < 1e-6
    assert np.array_equal(part["counts"], full["counts"][5:12])


def test_count_valid_and_tuner(oracle):
    """countValid / tuneValidRate of the reference (tool.cu:438-529) on the GPU against the CPU restatement."""
    from cuspamm_b200 import SpammPlan, gen_decay_alg

    n = 1024
    A = gen_decay_alg(0.1, 0.1, n, n)          # the reference's default generator (cuSpAMM.cu:428-431)
    B = gen_decay_alg(0.1, 0.1, n, n)
    nA, nB = oracle.norm_map(A), oracle.norm_map(B)
    with SpammPlan(n, n, n) as p:
        p.upload(A, B)
        p.norms()
        for tau in [0.0, 0.5, 1.548969, 2.0, 100.0]:
            cnt, s = p.count_valid(tau)
            prod = nA[:, :, None] * nB[None, :, :]
            assert cnt == int((prod >= np.float32(tau)).sum())
            assert abs(s - prod.astype(np.float64).sum()) <= 1e-9 * abs(s)
        tau_g, rate_g, it_g = p.tune_tau(0.75, 20, 0.01)
    tau_o, rate_o, it_o = oracle.tune_valid_rate(nA, nB, 0.75, 20, 0.01)
    assert it_g == it_o
    assert rate_g == rate_o
    assert abs(tau_g - tau_o) <= 1e-6 * abs(tau_o)


@pytest.mark.parametrize("chunk_tiles", [4, 8, 12])
def test_pipelined_host_to_host_multiply(oracle, chunk_tiles):
    """spamm_multiply with the rows of A processed in chunks (uploads, kernels and downloads overlapped): same
    result, same lists as the one-pass path; the last chunk is shorter than the others for 12."""
    from cuspamm_b200 import SpammPlan

    n = 640                                      # 20 tile rows
    A = signed_decay(n, 0.03, seed=41)
    B = signed_decay(n, 0.04, seed=42)
    tau = 0.2
    Cref, S, nA, nB, counts = oracle.spamm(A, B, tau, want_maps=True)
    with SpammPlan(n, n, n) as p:
        p.set_chunk_tiles(chunk_tiles)
        for _ in range(2):                       # twice: flags and lists of the first call must not leak
            C, st = p.multiply(A, B, tau)
            assert st["survivors"] == S
            assert rel_fro(C, Cref) <= C_TOL
        got_counts, got_s = p.counts()
        assert got_s == S and np.array_equal(got_counts, counts)
        assert np.array_equal(p.norm_a().view(np.uint32), nA.view(np.uint32))
        offs, kidx = p.lists()
        _, o2, k2 = oracle.lists(nA, nB, tau)
        assert np.array_equal(offs, o2) and np.array_equal(kidx, k2)
        assert st["packed_tiles_a"] == int((nA[:, :, None] * nB[None] >= np.float32(tau)).any(axis=2).sum())
        assert st["packed_tiles_b"] == int((nA[:, :, None] * nB[None] >= np.float32(tau)).any(axis=0).sum())


def test_bounded_device_wait_reports_and_leaves_the_plan_usable(oracle):
    """Failure detection without a GPU fault: a device-side wait on flags that nothing sets must give up after its
    limit, come back as SPAMM_ERR_DEVICE_WAIT, and the same plan must still compute correctly afterwards."""
    import time

    from cuspamm_b200 import SpammPlan, _lib

    lib = _lib.load()
    n = 256
    A = signed_decay(n, 0.05, seed=51)
    B = signed_decay(n, 0.06, seed=52)
    with SpammPlan(n, n, n) as p:
        t0 = time.perf_counter()
        st = lib.spamm_peer_wait_selftest(p._h, 4, 200)
        dt = time.perf_counter() - t0
        assert st == 4, "the wait did not run out"           # SPAMM_ERR_DEVICE_WAIT
        assert 0.15 < dt < 2.0
        C, stats = p.multiply(A, B, 0.3)
    C_ref, S = oracle.spamm(A, B, 0.3)
    assert stats["survivors"] == S and rel_fro(C, C_ref) <= C_TOL


def test_dense_macro_tiles_with_and_without_the_paired_kernel(oracle):
    """Dense macro tiles are multiplied by pairs of SMs when the previous lists of the plan were mostly dense, by the
    one-SM kernel otherwise; the switch is a speed hint and must never change the result."""
    from cuspamm_b200 import SpammPlan

    n = 768                                       # 6 macro-tile rows: three vertical pairs
    A = signed_decay(n, 0.002, seed=61)
    B = signed_decay(n, 0.002, seed=62)
    C_ref, S = oracle.spamm(A, B, 0.0)
    with SpammPlan(n, n, n) as p:
        p.upload(A, B)
        results = []
        for tau in (1e12, 0.0, 0.0, 1e12, 0.0):   # sparse -> dense (hint says sparse) -> dense (hint says dense) -> ...
            p.run(tau)
            p.sync()                              # reading the counters refreshes the hint
            results.append((tau, p.download_c(), p.counts()[1]))
    for tau, C, s in results:
        if tau == 0.0:
            assert s == S == (n // 32) ** 3
            assert rel_fro(C, C_ref) <= 2e-6
        else:
            assert s == 0 and not C.any()
    # a mixed case: upper half dense, lower half sparse -> pairs only where both neighbours are dense
    A2 = A.copy()
    A2[384:] *= np.float32(1e-6)
    tau = float(np.median(oracle.norm_map(A2)[:, :, None] * oracle.norm_map(B)[None]))
    C_ref2, S2 = oracle.spamm(A2, B, tau)
    with SpammPlan(n, n, n) as p:
        p.upload(A2, B)
        for _ in range(2):
            p.run(tau)
            p.sync()
            assert p.counts()[1] == S2
            assert rel_fro(p.download_c(), C_ref2) <= C_TOL


def test_half_conversion_modes_give_the_same_result(oracle):
    """Tiles are converted to half either one by one as the lists name them (its own kernel) or all of them inside
    the norm pass; "auto" switches on counters read back from the previous step.  The mode is a speed choice: maps,
    lists and C must not depend on it."""
    from cuspamm_b200 import SpammPlan

    rng = np.random.default_rng(17)
    # shapes that leave partial macro tiles (5 tile rows, 11 tile columns) and partial strips (7 tiles of K)
    M, K, N = 160, 224, 352
    A = (rng.standard_normal((M, K)) * np.exp(-rng.random((M, K)) * 5)).astype(np.float32)
    B = (rng.standard_normal((K, N)) * np.exp(-rng.random((K, N)) * 5)).astype(np.float32)
    nA, nB = oracle.norm_map(A), oracle.norm_map(B)
    for tau in (0.0, float(np.median(nA[:, :, None] * nB[None])), 1e9):
        C_ref, S = oracle.spamm(A, B, tau)
        out = {}
        for mode in ("listed", "all"):
            with SpammPlan(M, K, N) as p:
                p.set_pack_mode(mode)
                p.upload(A, B)
                st = p.run_timed(tau)
                assert st["survivors"] == S
                if mode == "all":
                    assert st["packed_tiles_a"] == nA.size and st["packed_tiles_b"] == nB.size
                assert np.array_equal(p.norm_a().view(np.uint32), nA.view(np.uint32))
                assert np.array_equal(p.norm_b().view(np.uint32), nB.view(np.uint32))
                out[mode] = p.download_c()
            assert rel_fro(out[mode], C_ref) <= C_TOL
        assert np.array_equal(out["listed"], out["all"]), "C depends on the conversion mode"

    # auto: dense lists turn the conversion-in-the-norm-pass on for the next step, sparse lists turn it off again
    n = 512
    A = signed_decay(n, 0.002, seed=71)
    B = signed_decay(n, 0.002, seed=72)
    C_dense, S_dense = oracle.spamm(A, B, 0.0)
    tau_mid = 0.4
    C_mid, S_mid = oracle.spamm(A, B, tau_mid)
    all_tiles = (n // 32) ** 2
    with SpammPlan(n, n, n) as p:
        p.upload(A, B)
        seen = []
        for tau, C_ref, S in ((0.0, C_dense, S_dense), (0.0, C_dense, S_dense), (tau_mid, C_mid, S_mid),
                              (1e12, None, 0), (1e12, None, 0), (0.0, C_dense, S_dense)):
            st = p.run_timed(tau)
            assert st["survivors"] == S
            C = p.download_c()
            if C_ref is None:
                assert not C.any()
            else:
                assert rel_fro(C, C_ref) <= C_TOL
            seen.append(st["packed_tiles_a"])
    # step 1 converts what the lists name (= everything at tau=0), step 2 and 3 everything in the norm pass,
    # step 4 still everything (the hint comes from step 3 only if that named most tiles), step 5 nothing
    assert seen[0] == all_tiles and seen[1] == all_tiles
    assert seen[4] == 0


def test_c_cleared_early_when_few_macro_tiles_have_steps(oracle):
    """When the counters of the previous step show that few macro tiles have steps, the next step clears C with a
    memset beside the list build and its multiply writes only the macro tiles that have steps.  Whatever C held
    before and whatever the hint said, the result must be the checker's, with exact zeros in the empty tiles."""
    from cuspamm_b200 import SpammPlan

    n = 2048
    A = signed_decay(n, 0.5, seed=81)             # narrow band: about a fifth of the macro tiles have steps
    B = signed_decay(n, 0.5, seed=82)
    refs = {tau: oracle.spamm(A, B, tau, want_maps=True) for tau in (1e-6, 0.0)}
    busy = (refs[1e-6][4].reshape(n // 128, 4, n // 256, 8) > 0).any(axis=(1, 3))
    assert 0 < busy.mean() <= 0.25, "the workload does not reach the early-clearing path"
    with SpammPlan(n, n, n) as p:
        p.upload(A, B)
        for tau in (0.0, 1e-6, 1e-6, 1e-6, 0.0, 0.0, 1e-6):
            p.run(tau)
            p.sync()                              # reading the counters refreshes the hint
            C = p.download_c()
            C_ref, S, _, _, counts = refs[tau]
            assert p.counts()[1] == S
            assert rel_fro(C, C_ref) <= C_TOL
            Ct = C.reshape(n // 32, 32, n // 32, 32).transpose(0, 2, 1, 3)
            assert not Ct[counts == 0].any(), "an empty tile is not zero"
        # the lists alone leave C alone, and a multiply repeated on the same lists writes all of C again
        p.run(1e-6)
        p.sync()
        C1 = p.download_c()
        p.build_lists(1e-6)
        assert np.array_equal(p.download_c(), C1)
        p.pack()
        p.gated_multiply()
        p.gated_multiply()
        p.sync()
        assert np.array_equal(p.download_c(), C1)


def test_c_cleared_early_with_cut_macro_tiles(oracle):
    """The same path where the last macro-tile row and column of C are cut (93 x 95 tiles) and have products."""
    from cuspamm_b200 import SpammPlan

    M, K, N = 2976, 3104, 3040
    A = np.ascontiguousarray(signed_decay(3104, 0.5, seed=83)[:M, :K])
    B = np.ascontiguousarray(signed_decay(3104, 0.5, seed=84)[:K, :N])
    C_ref, S, _, _, counts = oracle.spamm(A, B, 1e-6, want_maps=True)
    pad = np.zeros((96, 96), dtype=bool)
    pad[:93, :95] = counts > 0
    busy = pad.reshape(24, 4, 12, 8).any(axis=(1, 3))
    assert busy[-1].any() and busy[:, -1].any() and busy.mean() <= 0.25
    with SpammPlan(M, K, N) as p:
        p.upload(A, B)
        for _ in range(3):
            p.run(1e-6)
            p.sync()
            C = p.download_c()
            assert p.counts()[1] == S
            assert rel_fro(C, C_ref) <= C_TOL
            assert not C.reshape(93, 32, 95, 32).transpose(0, 2, 1, 3)[counts == 0].any()


def test_split_precision_reaches_float_accuracy(oracle):
    """The float-accuracy mode (operands as sums of two halves, three tensor-core passes; stands in for the
    reference's float build, cuSpAMM.cu:126-274): same norm maps and lists, C within 1e-5 relative Frobenius error of
    the product of the UNROUNDED inputs accumulated in double, where the half mode is at 1e-4 ... 1e-3."""
    from cuspamm_b200 import SpammPlan

    n = 512
    A = signed_decay(n, 0.02, seed=91)
    B = signed_decay(n, 0.03, seed=92)
    for tau in (0.0, 0.05, 1e9):
        C_exact, S = oracle.spamm_exact(A, B, tau)
        C_half_ref, S2 = oracle.spamm(A, B, tau)
        assert S == S2
        with SpammPlan(n, n, n) as p:
            p.upload(A, B)
            errs = {}
            for mode in ("half", "split", "split", "half"):       # twice: the second step runs with refreshed hints
                p.set_precision(mode)
                p.run(tau)
                p.sync()
                assert p.counts()[1] == S
                C = p.download_c()
                if S == 0:
                    assert not C.any()
                    continue
                errs.setdefault(mode, []).append(rel_fro(C, C_exact))
                if mode == "half":
                    assert rel_fro(C, C_half_ref) <= 2e-6
        if S:
            assert max(errs["split"]) <= 1e-5, errs
            assert min(errs["half"]) > 10 * max(errs["split"]), errs
    # the host-to-host call in chunks of rows, and a rectangular shape with cut macro tiles
    rng = np.random.default_rng(23)
    M, K, N = 160, 224, 352
    A = (rng.standard_normal((M, K)) * np.exp(-rng.random((M, K)) * 5)).astype(np.float32)
    B = (rng.standard_normal((K, N)) * np.exp(-rng.random((K, N)) * 5)).astype(np.float32)
    tau = float(np.median(oracle.norm_map(A)[:, :, None] * oracle.norm_map(B)[None]))
    C_exact, S = oracle.spamm_exact(A, B, tau)
    with SpammPlan(M, K, N) as p:
        p.set_precision("split")
        p.set_chunk_tiles(4)
        C, st = p.multiply(A, B, tau)
        assert st["survivors"] == S and rel_fro(C, C_exact) <= 1e-5
        p.set_chunk_tiles(64)
        C, st = p.multiply(A, B, tau)
        assert st["survivors"] == S and rel_fro(C, C_exact) <= 1e-5


def test_all_ones_known_answer():
    """The reference's all-ones input (getNormMatrix, tool.cu:370-406): every tile norm is exactly 32, every norm
    product exactly 1024, so the threshold 1024 keeps every product (the comparison is >=) and the next float above it
    keeps none; with all kept, every element of C is K."""
    from cuspamm_b200 import SpammPlan, gen_ones

    n = 256
    A, B = gen_ones(n, n), gen_ones(n, n)
    with SpammPlan(n, n, n) as p:
        p.upload(A, B)
        p.run(1024.0)
        p.sync()
        assert np.array_equal(p.norm_a(), np.full((8, 8), 32.0, dtype=np.float32))
        assert np.array_equal(p.norm_b(), np.full((8, 8), 32.0, dtype=np.float32))
        counts, S = p.counts()
        assert S == 8 ** 3 and np.array_equal(counts, np.full((8, 8), 8, dtype=np.int32))
        assert np.array_equal(p.download_c(), np.full((n, n), float(n), dtype=np.float32))
        p.run(float(np.nextafter(np.float32(1024.0), np.float32(2048.0))))
        p.sync()
        assert p.counts()[1] == 0 and not p.download_c().any()


def test_identity_known_answer(oracle):
    """A = I: tile norms sqrt(32) on the diagonal and 0 elsewhere, so the list of C(i,j) is {i} exactly where
    sqrt(32) * ||B(i,j)|| >= tau, and C equals the half-rounded B on those tiles and zero on the others."""
    from cuspamm_b200 import SpammPlan

    n = 256
    A = np.eye(n, dtype=np.float32)
    B = signed_decay(n, 0.2, seed=5)
    nB = oracle.norm_map(B)
    keep = (np.float32(np.sqrt(np.float32(32.0))) * nB) >= np.float32(0.5)
    assert keep.any() and not keep.all()
    with SpammPlan(n, n, n) as p:
        p.upload(A, B)
        p.run(0.5)
        p.sync()
        counts, S = p.counts()
        offsets, kidx = p.lists()
        C = p.download_c()
    assert np.array_equal(counts, keep.astype(np.int32)) and S == int(keep.sum())
    rows = np.repeat(np.arange(8), 8).reshape(8, 8)
    assert np.array_equal(kidx, rows[keep])
    want = oracle.round_to_half(B).reshape(8, 32, 8, 32) * keep[:, None, :, None]
    assert np.array_equal(C, want.reshape(n, n))


@pytest.mark.parametrize("precision", ["half", "split"])
def test_repeated_multiply_on_the_same_lists(oracle, precision):
    """spamm_gated_multiply may be called again on the same lists: every call must rebuild all of C, whichever of the
    two multiply kernels owns a macro tile.  A matrix whose upper rows are dense (those macro tiles go to pairs of
    SMs) and whose lower rows are gated; C is overwritten with garbage between the calls."""
    import torch

    from cuspamm_b200 import BUF_C, SpammPlan

    M, K, N = 768, 256, 768
    rng = np.random.default_rng(31)
    A = rng.uniform(0.5, 1.0, (M, K)).astype(np.float32)
    B = rng.uniform(0.5, 1.0, (K, N)).astype(np.float32)
    # lower third: every tile scaled by its own factor around 1, so that some of its products pass and some do not
    A[512:] *= np.repeat(np.repeat(rng.uniform(0.5, 1.2, (8, K // 32)), 32, axis=0), 32, axis=1).astype(np.float32)
    nA, nB = oracle.norm_map(A), oracle.norm_map(B)
    tau = float(np.min(nA[:16, :, None] * nB[None])) * 0.999              # every product of the upper rows survives
    C_ref, S = (oracle.spamm_exact if precision == "split" else oracle.spamm)(A, B, tau)
    counts, _, _ = oracle.lists(nA, nB, tau)
    low = counts[16:]
    assert (counts[:16] == K // 32).all() and (low < K // 32).any() and (low > 0).any() and S > 0
    with SpammPlan(M, K, N) as p:
        p.set_precision(precision)
        p.upload(A, B)
        p.run(tau)
        p.sync()                       # the hints now say "mostly dense": the next multiply launches the two-SM kernel
        p.run(tau)
        p.sync()
        first = p.download_c()
        assert rel_fro(first, C_ref) <= (1e-5 if precision == "split" else C_TOL)
        for _ in range(3):
            p.as_tensor(BUF_C).fill_(float("nan"))
            torch.cuda.synchronize()
            p.gated_multiply()
            p.sync()
            assert np.array_equal(p.download_c(), first)


def test_sizes_that_are_not_multiples_of_32(oracle):
    """The library pads on the GPU (main.h:54-56): host matrices keep their own sizes and leading dimensions on the way
    in and out, the result equals the checker's on zero-padded copies, also per row block and through the pipelined
    host-to-host call."""
    from cuspamm_b200 import SpammPlan, pad_to_tiles

    rng = np.random.default_rng(41)
    M, K, N = 203, 570, 333
    A = (rng.standard_normal((M, K)) * np.exp(-rng.random((M, K)) * 5)).astype(np.float32)
    B = (rng.standard_normal((K, N)) * np.exp(-rng.random((K, N)) * 5)).astype(np.float32)
    Ap, Bp = pad_to_tiles(A), pad_to_tiles(B)
    tau = float(np.median(oracle.norm_map(Ap)[:, :, None] * oracle.norm_map(Bp)[None]))
    C_ref, S, nA, nB, counts = oracle.spamm(Ap, Bp, tau, want_maps=True)
    with SpammPlan(M, K, N) as p:
        assert (p.row_tile_count, p.k_tiles, p.n_tiles, p.rows) == (7, 18, 11, M)
        p.upload(A, B)
        p.run(tau)
        p.sync()
        assert np.array_equal(p.norm_a().view(np.uint32), nA.view(np.uint32))
        assert np.array_equal(p.norm_b().view(np.uint32), nB.view(np.uint32))
        got_counts, got_s = p.counts()
        assert got_s == S and np.array_equal(got_counts, counts)
        C = p.download_c()
        assert C.shape == (M, N) and rel_fro(C, C_ref[:M, :N]) <= C_TOL
        for chunk in (4, 64):
            p.set_chunk_tiles(chunk)
            C2, st = p.multiply(A, B, tau)
            assert st["survivors"] == S and rel_fro(C2, C_ref[:M, :N]) <= C_TOL
    # the last row block ends inside the padding: it holds 203 - 4*32 = 75 rows of the caller's matrices
    with SpammPlan(M, K, N, 4, 3) as q:
        assert q.rows == 75
        q.upload(np.ascontiguousarray(A[128:]), B)
        q.run(tau)
        q.sync()
        assert q.counts()[1] == int(counts[4:].sum())
        assert rel_fro(q.download_c(), C_ref[128:M, :N]) <= C_TOL


def test_split_precision_on_small_magnitudes(oracle):
    """Inputs four orders of magnitude below 1: the low parts are stored scaled by 2^11, so they stay normal halves and
    the float-accuracy mode keeps its accuracy where unscaled residuals would fall into half's subnormal range."""
    from cuspamm_b200 import SpammPlan

    n = 256
    A = signed_decay(n, 0.02, seed=93) * np.float32(1e-4)
    B = signed_decay(n, 0.03, seed=94) * np.float32(1e-4)
    C_exact, S = oracle.spamm_exact(A, B, 0.0)
    with SpammPlan(n, n, n) as p:
        p.upload(A, B)
        p.set_precision("split")
        p.run(0.0)
        p.sync()
        assert p.counts()[1] == S
        assert rel_fro(p.download_c(), C_exact) <= 1e-5


def _lattice_like(M, K, N, seed):
    """Matrices whose lists are long and partly full: a smooth decay away from the diagonal times random magnitudes,
    so that neighbouring tiles keep similar but not identical sets of k."""
    rng = np.random.default_rng(seed)
    i = np.arange(M)[:, None] / M
    k = np.arange(K)[None, :] / K
    A = (np.exp(-6.0 * np.abs(i - k)) * rng.uniform(0.2, 1.0, (M, K)) * rng.choice([-1.0, 1.0], (M, K))).astype(np.float32)
    k2 = np.arange(K)[:, None] / K
    j = np.arange(N)[None, :] / N
    B = (np.exp(-6.0 * np.abs(k2 - j)) * rng.uniform(0.2, 1.0, (K, N)) * rng.choice([-1.0, 1.0], (K, N))).astype(np.float32)
    return A, B


@pytest.mark.parametrize("shape", [(256, 256, 256), (512, 768, 512), (384, 512, 800), (160, 96, 416), (1024, 2048, 1024)])
def test_gated_kernel_on_pairs_of_sms(oracle, shape):
    """The gated two-SM kernel (two vertically adjacent macro tiles share the tiles of B), forced for every pair of
    macro-tile rows: same norm maps and lists, C within tolerance, for full, partial and odd numbers of macro-tile rows
    and columns, at thresholds from 'everything' to 'nothing'; a repeat on the same lists; the float-accuracy mode."""
    from cuspamm_b200 import SpammPlan

    M, K, N = shape
    A, B = _lattice_like(M, K, N, seed=M + N)
    prods = oracle.norm_map(A)[:, :, None] * oracle.norm_map(B)[None]
    taus = [0.0, float(np.quantile(prods, 0.3)), float(np.quantile(prods, 0.7)), float(np.quantile(prods, 0.97)),
            float(prods.max()) * 2]
    with SpammPlan(M, K, N) as p:
        p.set_multiply_mode("gated_pairs")
        p.upload(A, B)
        for tau in taus:
            C_ref, S, _, _, counts = oracle.spamm(A, B, tau, want_maps=True)
            p.run(tau)
            p.sync()
            got_counts, got_s = p.counts()
            assert got_s == S and np.array_equal(got_counts, counts)
            C = p.download_c()
            assert rel_fro(C, C_ref) <= C_TOL, (tau, rel_fro(C, C_ref))
            empty = counts == 0
            if empty.any():
                assert not C.reshape(M // 32, 32, N // 32, 32).transpose(0, 2, 1, 3)[empty].any()
            p.gated_multiply()                       # again on the same lists
            p.sync()
            assert np.array_equal(p.download_c(), C)
        tau = taus[2]
        C_exact, S = oracle.spamm_exact(A, B, tau)
        p.set_precision("split")
        p.run(tau)
        p.sync()
        assert p.counts()[1] == S and rel_fro(p.download_c(), C_exact) <= 1e-5
        p.set_precision("half")
        p.set_multiply_mode("one_sm")
        C_ref, S = oracle.spamm(A, B, tau)
        p.run(tau)
        p.sync()
        assert rel_fro(p.download_c(), C_ref) <= C_TOL
