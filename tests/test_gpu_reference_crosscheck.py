"""The CPU checker and the CUDA path against the reference's OWN kernels (buaa-hipo/cuSpAMM, cuSpAMM.cu), compiled
unmodified for sm_100a by oracle/build_ref.sh into oracle/_ref/libref_<N>.so (one library per size: the reference
fixes its sizes at compile time).  This is the pin of the checker on the reference itself; the reference ships no
tests or golden vectors of its own.  Skipped when the libraries were not built (no reference sources at build time).

What is compared
  * unroll_get_Fnorm_pri (float norms, cuSpAMM.cu:21-71) against the checker's norm map: same quantity, different
    summation order, so equal to a few ulp, not bit for bit;
  * get_C_FP16_B32 (cuSpAMM.cu:276-392) fed with the checker's norm maps and threshold against the checker's gated
    product and against this library's C: one wrong bit in a skip list changes a whole 32x32 tile by O(1);
  * the reference's default run (para.h: 2048^3, c/(|i-j|^v+1) with c=v=0.1 stored as half, Norm=1.548969) with its
    own half-precision norm kernel unroll_get_Fnorm_FP16.
"""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from conftest import rel_fro, signed_decay

pytestmark = pytest.mark.gpu
REF_DIR = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


def ref_lib(n):
    path = REF_DIR / f"libref_{n}.so"
    if not path.exists():
        pytest.skip(f"{path.name} not built (reference sources were absent at build time)")
    lib = C.CDLL(str(path))
    m, k, nn = C.c_int(), C.c_int(), C.c_int()
    lib.ref_dims(C.byref(m), C.byref(k), C.byref(nn))
    assert (m.value, k.value, nn.value) == (n, n, n)
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    lib.ref_norm_fp32.argtypes = [vp, vp, i, i]
    lib.ref_norm_fp16.argtypes = [vp, vp, i, i]
    lib.ref_get_c_fp16.argtypes = [vp, vp, vp, vp, vp, i, i, f]
    return lib


def dev(x):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def test_reference_float_norm_kernel(oracle):
    import torch

    n = 512
    lib = ref_lib(n)
    X = signed_decay(n, 0.02, seed=5) * np.float32(3.0)
    dX = dev(X)
    dmap = torch.zeros((n // 32, n // 32), dtype=torch.float32, device="cuda")
    assert lib.ref_norm_fp32(dX.data_ptr(), dmap.data_ptr(), n, n) == 0
    np.testing.assert_allclose(dmap.cpu().numpy(), oracle.norm_map(X), rtol=2e-6)


@pytest.mark.parametrize("tau", [0.0, 0.05, 0.4, 3.0])
def test_reference_gated_multiply_agrees_with_checker_and_library(oracle, tau):
    import torch

    from cuspamm_b200 import SpammPlan

    n = 512
    lib = ref_lib(n)
    A = signed_decay(n, 0.02, seed=11)
    B = signed_decay(n, 0.03, seed=12)
    C_chk, S, nA, nB, counts = oracle.spamm(A, B, tau, want_maps=True)
    dA, dB = dev(A).half(), dev(B).half()               # round to nearest even, as __float2half (tool.cu:418)
    dC = torch.full((n, n), float("nan"), dtype=torch.float32, device="cuda")
    assert lib.ref_get_c_fp16(dA.data_ptr(), dev(nA).data_ptr(), dB.data_ptr(), dev(nB).data_ptr(), dC.data_ptr(),
                              0, n // 32, tau) == 0
    C_ref = dC.cpu().numpy()
    assert np.isfinite(C_ref).all()
    assert rel_fro(C_chk, C_ref) < 2e-6, "checker disagrees with the reference kernel"
    empty = counts == 0
    if empty.any():
        assert not C_ref.reshape(16, 32, 16, 32).transpose(0, 2, 1, 3)[empty].any()
    with SpammPlan(n, n, n) as p:
        C_lib, st = p.multiply(A, B, tau)
    assert st["survivors"] == S
    assert rel_fro(C_lib, C_ref) < 2e-6, "library disagrees with the reference kernel"
    # a row block, the reference's main_row_offset (cuSpAMM.cu:291,530)
    dC2 = torch.zeros((n, n), dtype=torch.float32, device="cuda")
    assert lib.ref_get_c_fp16(dA.data_ptr(), dev(nA).data_ptr(), dB.data_ptr(), dev(nB).data_ptr(), dC2.data_ptr(),
                              4, 8, tau) == 0
    assert np.array_equal(dC2.cpu().numpy()[128:384], C_ref[128:384])


def test_reference_default_run(oracle):
    """para.h defaults: 2048^3, algebraic decay c=v=0.1 stored as half, Norm = 1.548969, half norm kernel."""
    import torch

    n, tau = 2048, 1.548969
    lib = ref_lib(n)
    A32 = oracle.gen_decay_alg(0.1, 0.1, n, n)          # getDecayMatrixAlg(h_A, 0.1, 0.1, M, K), cuSpAMM.cu:429
    dA = dev(A32).half()
    Ah = dA.float().cpu().numpy()                        # the values the reference holds
    assert np.array_equal(Ah, oracle.round_to_half(A32))
    dmap = torch.zeros((n // 32, n // 32), dtype=torch.float32, device="cuda")
    assert lib.ref_norm_fp16(dA.data_ptr(), dmap.data_ptr(), n, n) == 0
    n_ref = dmap.cpu().numpy()
    n_chk = oracle.norm_map(Ah)
    # the reference squares and sums columns in half precision (cuSpAMM.cu:98-102): close, not equal
    np.testing.assert_allclose(n_ref, n_chk, rtol=3e-3)
    S_chk = int(oracle.lists(n_chk, n_chk, tau)[1][-1])
    assert S_chk == 12850
    counts_r, offs_r, kidx_r = oracle.lists(n_ref, n_ref, tau)   # the checker's skip rule on the reference's own map
    S_ref = int(offs_r[-1])
    assert abs(S_ref - S_chk) <= 0.02 * S_chk
    dC = torch.zeros((n, n), dtype=torch.float32, device="cuda")
    assert lib.ref_get_c_fp16(dA.data_ptr(), dmap.data_ptr(), dA.data_ptr(), dmap.data_ptr(), dC.data_ptr(),
                              0, n // 32, tau) == 0
    C_ref = dC.cpu().numpy()
    C_chk = oracle.gated_multiply(Ah, Ah, offs_r, kidx_r)
    assert rel_fro(C_chk, C_ref) < 2e-6
    # and the library on the same half-valued inputs (float norms, so its own lists): close to the reference's C,
    # the difference being the handful of products whose half-precision norm falls on the other side of Norm
    from cuspamm_b200 import SpammPlan

    with SpammPlan(n, n, n) as p:
        C_lib, st = p.multiply(Ah, Ah, tau)
    assert st["survivors"] == S_chk
    C_chk32, _ = oracle.spamm(Ah, Ah, tau)
    assert rel_fro(C_lib, C_chk32) < 2e-6
