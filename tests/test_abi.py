"""The C-ABI library without a GPU: it loads, exports everything include/spamm.h declares, validates arguments
before touching CUDA, and its host-side generators follow their formulas."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from cuspamm_b200 import _lib

    return _lib.load()


def declared_symbols():
    text = (ROOT / "include" / "spamm.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(spamm_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from cuspamm_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in spamm.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures out of step with spamm.h"


def test_status_strings(lib):
    assert lib.spamm_status_string(0) == b"ok"
    assert b"invalid" in lib.spamm_status_string(1)
    assert lib.spamm_status_string(12345) == b"unknown status"


def test_argument_validation_needs_no_gpu(lib):
    h = C.c_void_p()
    assert lib.spamm_plan_create(None, 64, 64, 64, 0, 2, 0) == 1
    assert lib.spamm_plan_create(C.byref(h), 0, 64, 64, 0, 2, 0) == 1         # empty matrix
    assert lib.spamm_plan_create(C.byref(h), 64, 64, 64, 1, 2, 0) == 1        # row block outside the matrix
    assert lib.spamm_plan_create(C.byref(h), 65, 64, 64, 1, 3, 0) == 1        # 65 rows are 3 tile rows, not 4
    assert lib.spamm_plan_create(C.byref(h), 64, 32 * 70000, 64, 0, 2, 0) == 6  # k index does not fit 16 bits
    assert lib.spamm_plan_destroy(None) == 0
    assert lib.spamm_norms(None) == 1
    assert lib.spamm_norm_map_dev(None, 32, 32, 32, None, None) == 1
    assert lib.spamm_norm_map_dev(C.c_void_p(16), 33, 32, 32, C.c_void_p(16), None) == 1
    assert lib.spamm_gated_multiply_dev(None, None, None, None, None, None, None, 1, 1, 1, None, 32, None) == 1
    assert lib.spamm_count_valid_scratch_bytes(512, 512) == 512 * 2 * 16


def hash3(seed, i, j):
    def mix(z):
        z = (z + np.uint64(0x9E3779B97F4A7C15))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))

    with np.errstate(over="ignore"):
        return mix(mix(mix(np.uint64(seed)) + i.astype(np.uint64)) + j.astype(np.uint64))


def test_generators():
    import cuspamm_b200 as S

    rows, cols, rb = 48, 80, 16
    i = (np.arange(rows) + rb)[:, None] * np.ones((1, cols), dtype=np.int64)
    j = np.ones((rows, 1), dtype=np.int64) * np.arange(cols)[None, :]
    d = np.abs(i - j).astype(np.float64)
    np.testing.assert_allclose(S.gen_decay_exp(1.0, 0.1, rows, cols, rb),
                               (np.float64(np.float32(0.1)) ** d).astype(np.float32), rtol=1e-6)
    np.testing.assert_allclose(S.gen_decay_alg(0.1, 0.1, rows, cols, rb),
                               np.float32(0.1) / ((d ** np.float64(np.float32(0.1))).astype(np.float32) + 1), rtol=1e-6)
    h = hash3(5, i, j)
    sign = np.where((h >> np.uint64(63)) == 1, -1.0, 1.0)
    np.testing.assert_allclose(S.gen_signed_exp(0.5, 5, rows, cols, rb), (sign * np.exp(-0.5 * d)).astype(np.float32),
                               rtol=1e-6)
    u = (h >> np.uint64(11)).astype(np.float64) / 2.0 ** 53
    np.testing.assert_allclose(S.gen_uniform(5, rows, cols, rb), (2 * u - 1).astype(np.float32), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(S.gen_uniform_alg(5, rows, cols, rb), ((2 * u - 1) / (d * d + 1)).astype(np.float32),
                               rtol=1e-6, atol=1e-9)
    # a block of rows equals the same rows of the whole matrix
    whole = S.gen_signed_exp(0.1, 9, 64, 64)
    assert np.array_equal(S.gen_signed_exp(0.1, 9, 16, 64, 32), whole[32:48])
    L = 4
    lat = S.gen_lattice(L, 3)
    assert lat.shape == (64, 64) and np.array_equal(lat, lat.T)
    assert np.all(np.abs(np.diag(lat)) >= 0.5) and np.all(np.abs(np.diag(lat)) < 1.0)
    # |a_ij| = u * exp(-dist): nearest neighbours along z are at distance 1
    assert 0.5 * np.exp(-1) <= abs(lat[0, 1]) < np.exp(-1)
    assert np.array_equal(S.gen_lattice(L, 3, rows=8, row_begin=24), lat[24:32])


def test_row_blocks():
    from cuspamm_b200 import row_blocks

    for tiles, world in [(512, 1), (512, 2), (512, 8), (1024, 8), (36, 8), (5, 2), (3, 4), (0, 2), (100, 3)]:
        blocks = row_blocks(tiles, world)
        assert len(blocks) == world
        assert blocks[0][0] == 0 and sum(n for _, n in blocks) == tiles
        for (b0, n0), (b1, _) in zip(blocks, blocks[1:]):
            assert b0 + n0 == b1
        if tiles >= 4 * world:
            assert all(b % 4 == 0 for b, _ in blocks)
    assert row_blocks(512, 8) == [(64 * r, 64) for r in range(8)]     # the reference's T/G split


def test_macro_tile_order_is_a_permutation(lib):
    for row_tiles, n_tiles in [(512, 512), (64, 512), (5, 9), (1, 1), (130, 70)]:
        n = ((row_tiles + 3) // 4) * ((n_tiles + 7) // 8)
        order = np.full(n, -1, dtype=np.int32)
        assert lib.spamm_macro_tile_order(row_tiles, n_tiles, order.ctypes.data) == 0
        assert np.array_equal(np.sort(order), np.arange(n))


def test_group_argument_validation_needs_no_gpu(lib):
    g = C.c_void_p()
    ids = (C.c_int * 2)(0, 0)
    assert lib.spamm_group_create(None, 64, 64, 64, 1, None) == 1
    assert lib.spamm_group_create(C.byref(g), 64, 64, 64, 0, None) == 1       # no device
    assert lib.spamm_group_create(C.byref(g), 64, 64, 64, 9, None) == 1       # more than 8
    assert lib.spamm_group_create(C.byref(g), 64, 0, 64, 1, None) == 1        # empty matrix
    assert lib.spamm_group_create(C.byref(g), 64, 64, 64, 2, ids) == 1        # the same device twice
    assert lib.spamm_group_destroy(None) == 0
    assert lib.spamm_group_size(None) == 0
    assert lib.spamm_group_run(None, 0.0) == 1
    assert lib.spamm_group_multiply(None, None, None, None, 0.0, None) == 1
    assert lib.spamm_run_shared(None, 0.0, 0, 1) == 1
    assert lib.spamm_upload_b_rows(None, None, 0, 0) == 1
    assert lib.spamm_multiply_b_resident(None, None, None, 0.0, None, None) == 1
