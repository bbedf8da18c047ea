"""The allocation-free valid-product count (`spamm_count_valid_static`) against the version that takes caller
scratch (`spamm_count_valid_dev`), both called through the C ABI on device memory the test owns.

Some hosts of the library cannot allocate device memory where they need the count (their framework's pool owns all
of HBM, or they must avoid the device-wide stall of an allocation), so that entry point keeps its work space in a
fixed array inside the library.  Two calls in a row share that array: the second must not be disturbed by what the
first left there.  The count is an integer and both entry points run the same two kernels, so the results must be
equal exactly; the sum of products is a double accumulated in a fixed order and must be equal as well.

This file sorts last on purpose: a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    import torch

    from cuspamm_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cpu").manual_seed(1234)
    cases = [(96, 80, 300, 0.35), (40, 64, 33, 0.6)]     # (row_tiles, k_tiles, n_tiles, tau): second is smaller,
    for row_tiles, k_tiles, n_tiles, tau in cases:         # so stale partials of the first lie beyond its range
        nA = torch.rand(row_tiles, k_tiles, generator=g).to(dev)
        nB = torch.rand(k_tiles, n_tiles, generator=g).to(dev)
        need = lib.spamm_count_valid_scratch_bytes(row_tiles, n_tiles)
        scratch = torch.empty(need, dtype=torch.uint8, device=dev)
        out_ref = torch.zeros(2, dtype=torch.int64, device=dev)      # [count, bits of the double sum]
        out_new = torch.full((2,), -1, dtype=torch.int64, device=dev)
        st = lib.spamm_count_valid_dev(_ptr(nA), _ptr(nB), row_tiles, k_tiles, n_tiles, tau, _ptr(scratch), need,
                                       _ptr(out_ref), C.c_void_p(out_ref.data_ptr() + 8), None)
        assert st == 0
        st = lib.spamm_count_valid_static(_ptr(nA), _ptr(nB), row_tiles, k_tiles, n_tiles, tau, _ptr(out_new),
                                          C.c_void_p(out_new.data_ptr() + 8), None)
        assert st == 0, lib.spamm_last_cuda_error()
        torch.cuda.synchronize()
        ref, new = out_ref.cpu().numpy(), out_new.cpu().numpy()
        want = int(((nA.cpu().numpy()[:, :, None] * nB.cpu().numpy()[None, :, :]) >= np.float32(tau)).sum())
        assert int(ref[0]) == want
        assert int(new[0]) == int(ref[0])
        assert new[1:].view(np.float64)[0] == ref[1:].view(np.float64)[0]


def test_static_scratch_refuses_sizes_beyond_its_array():
    import torch

    from cuspamm_b200 import _lib

    lib = _lib.load()
    limit = lib.spamm_count_valid_static_max_blocks()
    assert limit == 8192
    dev = torch.device("cuda", 0)
    dummy = torch.zeros(16, dtype=torch.float32, device=dev)
    out = torch.zeros(2, dtype=torch.int64, device=dev)
    # limit+1 tile rows with one span of columns: refused before anything is launched or read
    st = lib.spamm_count_valid_static(_ptr(dummy), _ptr(dummy), limit + 1, 1, 1, 0.5, _ptr(out), None, None)
    assert st == 6
    assert b"built-in" in lib.spamm_last_cuda_error()
    torch.cuda.synchronize()
    assert int(out[0].item()) == 0
