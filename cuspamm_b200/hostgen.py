"""Host-side input generators (csrc/generators.cpp) from their own small library, libspamm_gen.so.

They are plain C++ on host arrays: the two deterministic generators of the reference (tool.cu:370-436) and the seeded
families of the benchmark configurations.  A process that only needs input matrices loads this library and never the
GPU library.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import build as _build

_i64, _f, _vp = C.c_int64, C.c_float, C.c_void_p
SIGNATURES = {
    "spamm_gen_decay_exp": [_vp, _f, _f, _i64, _i64, _i64],
    "spamm_gen_decay_alg": [_vp, _f, _f, _i64, _i64, _i64],
    "spamm_gen_ones": [_vp, _i64, _i64, _i64],
    "spamm_gen_signed_exp": [_vp, C.c_double, C.c_uint64, _i64, _i64, _i64],
    "spamm_gen_uniform_alg": [_vp, C.c_uint64, _i64, _i64, _i64],
    "spamm_gen_uniform": [_vp, C.c_uint64, _i64, _i64, _i64],
    "spamm_gen_lattice": [_vp, C.c_int, C.c_uint64, _i64, _i64],
}
_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        lib = C.CDLL(str(_build.build_generators()))
        for name, args in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = C.c_int, args
        _lib = lib
    return _lib


def fill(fn_name: str, out: np.ndarray, *args) -> np.ndarray:
    """Runs one generator into `out` (C-contiguous float32)."""
    if out.dtype != np.float32 or not out.flags["C_CONTIGUOUS"]:
        raise ValueError("generators write C-contiguous float32 arrays")
    st = getattr(load(), fn_name)(out.ctypes.data, *args)
    if st != 0:
        raise ValueError(f"{fn_name}: bad arguments (status {st})")
    return out


def _gen(fn_name: str, rows: int, cols: int, *args) -> np.ndarray:
    return fill(fn_name, np.empty((rows, cols), dtype=np.float32), *args)


def gen_decay_exp(c: float, v: float, rows: int, cols: int, row_begin: int = 0) -> np.ndarray:
    """a_ij = c * v^|i-j| (getDecayMatrixExp, tool.cu:409-422)."""
    return _gen("spamm_gen_decay_exp", rows, cols, c, v, row_begin, rows, cols)


def gen_decay_alg(c: float, v: float, rows: int, cols: int, row_begin: int = 0) -> np.ndarray:
    """a_ij = c / (|i-j|^v + 1) (getDecayMatrixAlg, tool.cu:426-436)."""
    return _gen("spamm_gen_decay_alg", rows, cols, c, v, row_begin, rows, cols)


def gen_ones(rows: int, cols: int) -> np.ndarray:
    """a_ij = 1 (getNormMatrix, tool.cu:370-406): every full tile has norm 32."""
    return _gen("spamm_gen_ones", rows, cols, 0, rows, cols)


def gen_signed_exp(lam: float, seed: int, rows: int, cols: int, row_begin: int = 0) -> np.ndarray:
    """a_ij = s_ij * exp(-lam*|i-j|), s_ij = +-1 from a hash of (seed, i, j)."""
    return _gen("spamm_gen_signed_exp", rows, cols, lam, seed, row_begin, rows, cols)


def gen_uniform_alg(seed: int, rows: int, cols: int, row_begin: int = 0) -> np.ndarray:
    """a_ij = u_ij / (|i-j|^2 + 1), u uniform in [-1, 1)."""
    return _gen("spamm_gen_uniform_alg", rows, cols, seed, row_begin, rows, cols)


def gen_uniform(seed: int, rows: int, cols: int, row_begin: int = 0) -> np.ndarray:
    """a_ij uniform in [-1, 1)."""
    return _gen("spamm_gen_uniform", rows, cols, seed, row_begin, rows, cols)


def gen_lattice(L: int, seed: int, rows: Optional[int] = None, row_begin: int = 0) -> np.ndarray:
    """Symmetric surrogate of a density matrix on an L^3 grid: a_ij = +-u * exp(-|r_i - r_j|), u in [0.5, 1)."""
    n = L ** 3
    rows = n - row_begin if rows is None else rows
    return _gen("spamm_gen_lattice", rows, n, L, seed, row_begin, rows)
