"""ctypes binding of libspamm.so (the C ABI declared in include/spamm.h).

There is no CPU fallback: if the library is missing it is built with nvcc, and if that fails the import of
this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

_PKG = Path(__file__).resolve().parent


class SpammStats(C.Structure):
    """Mirror of `spamm_stats` in include/spamm.h."""

    _fields_ = [
        ("ms_h2d", C.c_float),
        ("ms_norm", C.c_float),
        ("ms_lists", C.c_float),
        ("ms_pack", C.c_float),
        ("ms_multiply", C.c_float),
        ("ms_d2h", C.c_float),
        ("ms_device_total", C.c_float),
        ("survivors", C.c_int64),
        ("tile_products", C.c_int64),
        ("steps", C.c_int64),
        ("packed_tiles_a", C.c_int64),
        ("packed_tiles_b", C.c_int64),
        ("executed_flops", C.c_double),
    ]

    def as_dict(self) -> dict:
        return {n: getattr(self, n) for n, _ in self._fields_}


_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every symbol include/spamm.h declares
SIGNATURES = {
    "spamm_plan_create": (_i, [_pp, _i, _i, _i, _i, _i, _i]),
    "spamm_plan_destroy": (_i, [_vp]),
    "spamm_upload": (_i, [_vp, _vp, _vp]),
    "spamm_plan_set_chunk_tiles": (_i, [_vp, _i]),
    "spamm_plan_set_pack_mode": (_i, [_vp, _i]),
    "spamm_plan_set_multiply_mode": (_i, [_vp, _i]),
    "spamm_clear_c_early": (_i, [_vp]),
    "spamm_plan_set_precision": (_i, [_vp, _i]),
    "spamm_norms": (_i, [_vp]),
    "spamm_norms_share": (_i, [_vp, _i, _i]),
    "spamm_norm_b_share": (_i, [_vp, _i, _i]),
    "spamm_norm_a": (_i, [_vp]),
    "spamm_peer_handles": (_i, [_vp, _vp, _sz]),
    "spamm_peer_attach": (_i, [_vp, _i, _i, _vp]),
    "spamm_norm_b_share_push": (_i, [_vp, _i, _i]),
    "spamm_run_shared": (_i, [_vp, _f, _i, _i]),
    "spamm_norms_shared": (_i, [_vp, _i, _i]),
    "spamm_upload_b_rows": (_i, [_vp, _vp, _i, _i]),
    "spamm_multiply_b_resident": (_i, [_vp, _vp, _vp, _f, _vp, C.POINTER(SpammStats)]),
    "spamm_group_create": (_i, [_pp, _i, _i, _i, _i, C.POINTER(_i)]),
    "spamm_group_destroy": (_i, [_vp]),
    "spamm_group_size": (_i, [_vp]),
    "spamm_group_plan": (_i, [_vp, _i, _pp]),
    "spamm_group_upload": (_i, [_vp, _vp, _vp]),
    "spamm_group_run": (_i, [_vp, _f]),
    "spamm_group_sync": (_i, [_vp]),
    "spamm_group_download_c": (_i, [_vp, _vp]),
    "spamm_group_survivors": (_i, [_vp, C.POINTER(_i64)]),
    "spamm_group_multiply": (_i, [_vp, _vp, _vp, _vp, _f, C.POINTER(SpammStats)]),
    "spamm_peer_wait_selftest": (_i, [_vp, _i, C.c_uint]),
    "spamm_build_lists": (_i, [_vp, _f]),
    "spamm_pack": (_i, [_vp]),
    "spamm_gated_multiply": (_i, [_vp]),
    "spamm_run": (_i, [_vp, _f]),
    "spamm_finish": (_i, [_vp, _f]),
    "spamm_sync": (_i, [_vp]),
    "spamm_download_c": (_i, [_vp, _vp]),
    "spamm_multiply": (_i, [_vp, _vp, _vp, _vp, _f, C.POINTER(SpammStats)]),
    "spamm_run_timed": (_i, [_vp, _f, C.POINTER(SpammStats)]),
    "spamm_get_norm_a": (_i, [_vp, _vp]),
    "spamm_get_norm_b": (_i, [_vp, _vp]),
    "spamm_get_counts": (_i, [_vp, _vp, C.POINTER(_i64)]),
    "spamm_get_lists": (_i, [_vp, _vp, _vp]),
    "spamm_error_norms": (_i, [_vp, _vp, C.POINTER(C.c_double)]),
    "spamm_error_norms_scratch_bytes": (_sz, []),
    "spamm_error_norms_dev": (_i, [_vp, _vp, _sz, _vp, _sz, _vp, _vp]),
    "spamm_count_valid": (_i, [_vp, _f, C.POINTER(_i64), C.POINTER(C.c_double)]),
    "spamm_tune_tau": (_i, [_vp, C.c_double, _i, C.c_double, C.POINTER(_f), C.POINTER(C.c_double), C.POINTER(_i)]),
    "spamm_count_valid_scratch_bytes": (_sz, [_i, _i]),
    "spamm_count_valid_dev": (_i, [_vp, _vp, _i, _i, _i, _f, _vp, _sz, _vp, _vp, _vp]),
    "spamm_count_valid_static": (_i, [_vp, _vp, _i, _i, _i, _f, _vp, _vp, _vp]),
    "spamm_count_valid_static_max_blocks": (_i, []),
    "spamm_device_buffer": (_i, [_vp, _i, _pp, C.POINTER(_sz)]),
    "spamm_stream": (_i, [_vp, _pp]),
    "spamm_plan_dims": (_i, [_vp] + [C.POINTER(_i)] * 5),
    "spamm_norm_map_dev": (_i, [_vp, _i, _i, _i64, _vp, _vp]),
    "spamm_norm_map_pair_dev": (_i, [_vp, _i, _i, _i64, _vp, _vp, _i, _i, _i64, _vp, _vp]),
    "spamm_build_lists_scratch_bytes": (_sz, [_i, _i, _i]),
    "spamm_build_lists_dev": (_i, [_vp, _vp, _i, _i, _i, _f] + [_vp] * 10),
    "spamm_pack_half_dev": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "spamm_gated_multiply_dev": (_i, [_vp] * 7 + [_i, _i, _i, _vp, _i64, _vp]),
    "spamm_macro_tile_order": (_i, [_i, _i, _vp]),
    "spamm_gen_decay_exp": (_i, [_vp, _f, _f, _i64, _i64, _i64]),
    "spamm_gen_decay_alg": (_i, [_vp, _f, _f, _i64, _i64, _i64]),
    "spamm_gen_ones": (_i, [_vp, _i64, _i64, _i64]),
    "spamm_gen_signed_exp": (_i, [_vp, C.c_double, C.c_uint64, _i64, _i64, _i64]),
    "spamm_gen_uniform_alg": (_i, [_vp, C.c_uint64, _i64, _i64, _i64]),
    "spamm_gen_uniform": (_i, [_vp, C.c_uint64, _i64, _i64, _i64]),
    "spamm_gen_lattice": (_i, [_vp, _i, C.c_uint64, _i64, _i64]),
    "spamm_status_string": (C.c_char_p, [_i]),
    "spamm_last_cuda_error": (C.c_char_p, []),
    "spamm_kernel_launches": (_i64, [_vp]),
}

_lib = None


def load() -> C.CDLL:
    """Loads (building first if needed) libspamm.so and sets the argument types of every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    try:
        path = _build.build_library()      # returns at once when the library is newer than every source and header
    except _build.NvccMissing:
        if not path.exists():              # no compiler here: a library that travelled with the tree is used as it is
            raise
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class SpammError(RuntimeError):
    def __init__(self, status: int, where: str):
        lib = load()
        msg = lib.spamm_status_string(status).decode()
        detail = lib.spamm_last_cuda_error().decode()
        super().__init__(f"{where}: {msg} (status {status})" + (f": {detail}" if detail and status in (2, 3) else ""))
        self.status = status


def check(status: int, where: str) -> None:
    if status != 0:
        raise SpammError(status, where)
