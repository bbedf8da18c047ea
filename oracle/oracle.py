"""ctypes wrapper of the CPU checker (oracle/spamm_oracle.c).  TEST INFRASTRUCTURE: only tests/, the smoke run
and the benchmark's CPU-baseline legs may import this module; the product package never does."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB = _DIR / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src = _DIR / "spamm_oracle.c"
    if force or not _LIB.exists() or _LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "-B", "liboracle.so"], check=True, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT)
    return _LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_LIB))
        vp, i, i64, f = C.c_void_p, C.c_int, C.c_int64, C.c_float
        L.oracle_f2h_bits.restype, L.oracle_f2h_bits.argtypes = C.c_uint16, [f]
        L.oracle_h2f.restype, L.oracle_h2f.argtypes = f, [C.c_uint16]
        L.oracle_round_to_half.restype, L.oracle_round_to_half.argtypes = None, [vp, vp, i64]
        L.oracle_norm_map.restype, L.oracle_norm_map.argtypes = i, [vp, i, i, i64, vp]
        L.oracle_count_lists.restype = i64
        L.oracle_count_lists.argtypes = [vp, vp, i, i, i, i, f, vp]
        L.oracle_fill_lists.restype, L.oracle_fill_lists.argtypes = None, [vp, vp, i, i, i, i, f, vp, vp]
        L.oracle_gated_multiply.restype = None
        L.oracle_gated_multiply.argtypes = [vp, vp, i, i, i, vp, vp, vp]
        L.oracle_gated_multiply_exact.restype = None
        L.oracle_gated_multiply_exact.argtypes = [vp, vp, i, i, i, vp, vp, vp]
        L.oracle_spamm.restype = i64
        L.oracle_spamm.argtypes = [vp, vp, vp, i, i, i, i, i, f, vp, vp, vp]
        L.oracle_gen_decay_exp.restype, L.oracle_gen_decay_exp.argtypes = None, [vp, f, f, i, i]
        L.oracle_gen_decay_alg.restype, L.oracle_gen_decay_alg.argtypes = None, [vp, f, f, i, i]
        L.oracle_tune_valid_rate.restype = f
        L.oracle_tune_valid_rate.argtypes = [vp, vp, i, i, i, C.c_double, i, C.c_double, C.POINTER(C.c_double),
                                             C.POINTER(i)]
        L.oracle_num_threads.restype, L.oracle_num_threads.argtypes = i, []
        L.oracle_set_num_threads.restype, L.oracle_set_num_threads.argtypes = None, [i]
        _lib = L
    return _lib


def _f32(x) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32)


def round_to_half(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().oracle_round_to_half(x.ctypes.data, out.ctypes.data, x.size)
    return out


def norm_map(x) -> np.ndarray:
    x = _f32(x)
    rows, cols = x.shape
    out = np.empty((rows // 32, cols // 32), dtype=np.float32)
    if lib().oracle_norm_map(x.ctypes.data, rows, cols, cols, out.ctypes.data):
        raise ValueError("dimensions must be multiples of 32")
    return out


def lists(nA, nB, tau: float, row_begin: int = 0, row_count=None):
    """(counts[row_count, TN], offsets, k_idx) for rows [row_begin, row_begin+row_count) of the A map."""
    nA, nB = _f32(nA), _f32(nB)
    TK, TN = nB.shape
    if row_count is None:
        row_count = nA.shape[0] - row_begin
    counts = np.zeros((row_count, TN), dtype=np.int32)
    S = lib().oracle_count_lists(nA.ctypes.data, nB.ctypes.data, TK, TN, row_begin, row_count, tau,
                                 counts.ctypes.data)
    offsets = np.zeros(row_count * TN + 1, dtype=np.int64)
    np.cumsum(counts.ravel(), out=offsets[1:])
    kidx = np.empty(max(int(S), 1), dtype=np.int32)
    lib().oracle_fill_lists(nA.ctypes.data, nB.ctypes.data, TK, TN, row_begin, row_count, tau,
                            offsets.ctypes.data, kidx.ctypes.data)
    return counts, offsets, kidx[: int(S)]


def gated_multiply(Ah_rows, Bh, offsets, kidx) -> np.ndarray:
    """Ah_rows: the half-rounded rows of one row block; offsets/kidx index that block's tiles."""
    Ah_rows, Bh = _f32(Ah_rows), _f32(Bh)
    rows, K = Ah_rows.shape
    N = Bh.shape[1]
    Cm = np.empty((rows, N), dtype=np.float32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int64)
    kidx = np.ascontiguousarray(kidx, dtype=np.int32)
    kp = kidx.ctypes.data if kidx.size else np.zeros(1, np.int32).ctypes.data
    lib().oracle_gated_multiply(Ah_rows.ctypes.data, Bh.ctypes.data, K, N, rows // 32, offsets.ctypes.data, kp,
                                Cm.ctypes.data)
    return Cm


def gated_multiply_exact(A_rows, B, offsets, kidx) -> np.ndarray:
    """The gated sum on the unrounded float inputs, double accumulation (checker of the split-precision mode)."""
    A_rows, B = _f32(A_rows), _f32(B)
    rows, K = A_rows.shape
    N = B.shape[1]
    Cm = np.empty((rows, N), dtype=np.float32)
    offsets = np.ascontiguousarray(offsets, dtype=np.int64)
    kidx = np.ascontiguousarray(kidx, dtype=np.int32)
    kp = kidx.ctypes.data if kidx.size else np.zeros(1, np.int32).ctypes.data
    lib().oracle_gated_multiply_exact(A_rows.ctypes.data, B.ctypes.data, K, N, rows // 32, offsets.ctypes.data, kp,
                                      Cm.ctypes.data)
    return Cm


def spamm_exact(A, B, tau: float):
    """(C, S): same norm maps and lists as `spamm`, product of the unrounded inputs in double."""
    A, B = _f32(A), _f32(B)
    nA, nB = norm_map(A), norm_map(B)
    counts, offsets, kidx = lists(nA, nB, tau)
    return gated_multiply_exact(A, B, offsets, kidx), int(counts.sum())


def spamm(A, B, tau: float, row_begin: int = 0, row_count=None, want_maps: bool = False):
    """The whole path.  Returns (C_rows, S) or (C_rows, S, nA_rows, nB, counts)."""
    A, B = _f32(A), _f32(B)
    M, K = A.shape
    N = B.shape[1]
    if row_count is None:
        row_count = M // 32 - row_begin
    Cm = np.empty((row_count * 32, N), dtype=np.float32)
    nA = np.empty((row_count, K // 32), dtype=np.float32)
    nB = np.empty((K // 32, N // 32), dtype=np.float32)
    counts = np.empty((row_count, N // 32), dtype=np.int32)
    S = lib().oracle_spamm(A.ctypes.data, B.ctypes.data, Cm.ctypes.data, M, K, N, row_begin, row_count, tau,
                           nA.ctypes.data, nB.ctypes.data, counts.ctypes.data)
    if S < 0:
        raise ValueError("oracle_spamm rejected the arguments")
    return (Cm, int(S), nA, nB, counts) if want_maps else (Cm, int(S))


def tune_valid_rate(nA, nB, expected: float = 0.75, max_iters: int = 20, tolerance: float = 0.01):
    """(tau, rate, iterations) of the reference's bisection tuner."""
    nA, nB = _f32(nA), _f32(nB)
    rate, it = C.c_double(), C.c_int()
    tau = lib().oracle_tune_valid_rate(nA.ctypes.data, nB.ctypes.data, nA.shape[0], nB.shape[0], nB.shape[1],
                                       expected, max_iters, tolerance, C.byref(rate), C.byref(it))
    return float(tau), float(rate.value), int(it.value)


def gen_decay_exp(c: float, v: float, m: int, n: int) -> np.ndarray:
    out = np.empty((m, n), dtype=np.float32)
    lib().oracle_gen_decay_exp(out.ctypes.data, c, v, m, n)
    return out


def gen_decay_alg(c: float, v: float, m: int, n: int) -> np.ndarray:
    out = np.empty((m, n), dtype=np.float32)
    lib().oracle_gen_decay_alg(out.ctypes.data, c, v, m, n)
    return out


def num_threads() -> int:
    return lib().oracle_num_threads()


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(n)
