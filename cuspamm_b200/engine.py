"""Host-side mirror of the reference driver (`main`, cuSpAMM.cu:395-556) on top of the C ABI.

`SpammPlan` is one GPU working on one block of C tile rows -- the reference's per-device plan (`TGPUplan`,
cuSpAMM.cu:6-12) with its row offset (cuSpAMM.cu:503,530).  `ShardedSpamm` is the multi-GPU split: one process
per GPU, C sharded by row blocks, B and its norm map moved between the GPUs with NCCL (torch.distributed is used
for the plumbing only), C slabs gathered on request.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import SpammStats, check

TILE = 32
MT_ROWS = 4
MT_COLS = 8

BUF_A, BUF_B, BUF_C, BUF_NORM_A, BUF_NORM_B, BUF_COUNTS, BUF_STEPS, BUF_STEP_COUNTS, BUF_HALF_A, BUF_HALF_B = range(10)


def _host_ptr(x, nbytes: Optional[int] = None) -> int:
    """Address of a contiguous float32 host array (numpy array or CPU torch tensor)."""
    if x is None:
        return 0
    if isinstance(x, np.ndarray):
        if x.dtype != np.float32 or not x.flags["C_CONTIGUOUS"]:
            raise ValueError("host matrices must be C-contiguous float32")
        if nbytes is not None and x.nbytes != nbytes:
            raise ValueError(f"host matrix has {x.nbytes} bytes, expected {nbytes}")
        return x.ctypes.data
    if hasattr(x, "data_ptr"):  # torch tensor
        import torch

        if x.device.type != "cpu" or x.dtype != torch.float32 or not x.is_contiguous():
            raise ValueError("host matrices must be contiguous float32 CPU tensors")
        if nbytes is not None and x.numel() * 4 != nbytes:
            raise ValueError(f"host matrix has {x.numel() * 4} bytes, expected {nbytes}")
        return x.data_ptr()
    raise TypeError("expected a numpy array or a CPU torch tensor")


def pad_to_tiles(x: np.ndarray) -> np.ndarray:
    """Zero-pads a float32 matrix to multiples of 32 in both dimensions, the reference's padded sizes
    (main.h:54-56; the reference leaves the padding uninitialised, zeros make it harmless).  The library pads by
    itself on the GPU; this helper only serves comparisons on the host."""
    r, c = x.shape
    R, Cc = -(-r // TILE) * TILE, -(-c // TILE) * TILE
    if (R, Cc) == (r, c) and x.dtype == np.float32 and x.flags["C_CONTIGUOUS"]:
        return x
    out = np.zeros((R, Cc), dtype=np.float32)
    out[:r, :c] = x
    return out


def row_blocks(row_tiles: int, world: int) -> list:
    """Contiguous blocks of C tile rows, one per GPU, as the reference splits them (cuSpAMM.cu:503,530:
    device d owns tile rows [d*T/G, (d+1)*T/G)).  Boundaries fall on multiples of 4 tile rows (one macro tile)
    when there are enough rows, so that no GPU works on a partly filled macro tile; the remainder goes to the
    first blocks.  Returns [(begin, count)] * world."""
    if world <= 0 or row_tiles < 0:
        raise ValueError("bad partition")
    unit = MT_ROWS if row_tiles >= MT_ROWS * world else 1
    units = row_tiles // unit
    base, extra = divmod(units, world)
    out, begin = [], 0
    for r in range(world):
        n = (base + (1 if r < extra else 0)) * unit
        if r == world - 1:
            n = row_tiles - begin
        out.append((begin, n))
        begin += n
    return out


def balanced_row_blocks(weights, world: int, unit: int = MT_ROWS) -> list:
    """Contiguous blocks of C tile rows, one per GPU, whose largest total weight is as small as a contiguous split
    on multiples of `unit` tile rows allows.  `weights[i]` is the cost of tile row i (for example its number of
    surviving products plus a constant for the row's share of the norm pass and of writing C).  The reference
    always splits evenly (cuSpAMM.cu:503,530), which leaves GPUs idle when the survivors are unevenly spread
    (a lattice, a matrix with a dense corner).  Returns [(begin, count)] * world; every block gets at least one
    unit when there are enough units."""
    w = np.asarray(weights, dtype=np.float64)
    row_tiles = int(w.shape[0])
    if world <= 0 or w.ndim != 1 or (w < 0).any():
        raise ValueError("bad partition")
    if not w.any():
        return row_blocks(row_tiles, world)
    if row_tiles < unit * world:
        unit = 1
    n_units = -(-row_tiles // unit)
    uw = np.array([w[u * unit:(u + 1) * unit].sum() for u in range(n_units)], dtype=np.float64)

    def cut(cap: float):
        """Greedy split: a block is closed when the next unit would exceed `cap`, or when the units left are just
        enough to give every remaining block one.  Returns the unit index where every block starts."""
        starts, load = [0], 0.0
        for u in range(n_units):
            must = n_units - u <= world - len(starts) and u > starts[-1]
            if u > starts[-1] and (load + uw[u] > cap or must) and len(starts) < world:
                starts.append(u)
                load = 0.0
            load += uw[u]
        return starts

    def worst(starts):
        ends = starts[1:] + [n_units]
        return max(uw[a:b].sum() for a, b in zip(starts, ends)) if n_units else 0.0

    lo, hi = (float(uw.max()) if n_units else 0.0), float(uw.sum())
    for _ in range(60):                       # bisection on the largest block weight
        mid = 0.5 * (lo + hi)
        if worst(cut(mid)) <= mid:
            hi = mid
        else:
            lo = mid
    starts = cut(hi)
    starts += [n_units] * (world - len(starts))          # more GPUs than units: empty blocks at the end
    out = []
    for r in range(world):
        b = min(starts[r] * unit, row_tiles)
        e = min((starts[r + 1] if r + 1 < world else n_units) * unit, row_tiles)
        out.append((b, e - b))
    return out


class _DeviceView:
    """Zero-copy view of plan-owned device memory for torch.as_tensor."""

    def __init__(self, ptr: int, shape: Tuple[int, ...], typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 2}


class SpammPlan:
    """One GPU, one block of C tile rows.  Method names follow the steps of the reference's timed loop."""

    def __init__(self, M: int, K: int, N: int, row_tile_begin: int = 0, row_tile_count: Optional[int] = None,
                 device: int = 0):
        self._lib = _lib.load()
        if row_tile_count is None:
            row_tile_count = -(-M // TILE) - row_tile_begin
        self.M, self.K, self.N = M, K, N                       # the caller's sizes; the library pads to 32 on the GPU
        self.Mp, self.Kp, self.Np = (-(-x // TILE) * TILE for x in (M, K, N))
        self.row_tile_begin, self.row_tile_count = row_tile_begin, row_tile_count
        self.device = device
        self._h = C.c_void_p()
        self._owned = True
        check(self._lib.spamm_plan_create(C.byref(self._h), M, K, N, row_tile_begin, row_tile_count, device),
              "spamm_plan_create")

    @classmethod
    def _borrowed(cls, handle: int, device: int) -> "SpammPlan":
        """A view of a plan that somebody else owns (a device of a `SpammGroup`): same methods, `close` does nothing."""
        self = cls.__new__(cls)
        self._lib = _lib.load()
        self._h = C.c_void_p(handle)
        self._owned = False
        dims = [C.c_int() for _ in range(5)]
        check(self._lib.spamm_plan_dims(self._h, *[C.byref(d) for d in dims]), "spamm_plan_dims")
        self.M, self.K, self.N, self.row_tile_begin, self.row_tile_count = (d.value for d in dims)
        self.Mp, self.Kp, self.Np = (-(-x // TILE) * TILE for x in (self.M, self.K, self.N))
        self.device = device
        return self

    # ---- lifetime
    def close(self) -> None:
        if getattr(self, "_h", None) and self._h.value:
            if self._owned:
                self._lib.spamm_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- shapes
    @property
    def rows(self) -> int:
        """Rows of the caller's A and C inside this plan's block (the last block may end inside the padding)."""
        return max(0, min(self.row_tile_count * TILE, self.M - self.row_tile_begin * TILE))

    @property
    def k_tiles(self) -> int:
        return self.Kp // TILE

    @property
    def n_tiles(self) -> int:
        return self.Np // TILE

    def set_chunk_tiles(self, tiles: int) -> None:
        """Tile rows per chunk of the pipelined `multiply` (multiple of 4)."""
        check(self._lib.spamm_plan_set_chunk_tiles(self._h, int(tiles)), "spamm_plan_set_chunk_tiles")

    def set_pack_mode(self, mode: str) -> None:
        """Which tiles are converted to half: "auto" (default), "listed" (only tiles a skip list names, by `pack`)
        or "all" (every tile, inside `norms`).  Results are the same in every mode."""
        modes = {"auto": 0, "listed": 1, "all": 2}
        if mode not in modes:
            raise ValueError(f"pack mode must be one of {sorted(modes)}")
        check(self._lib.spamm_plan_set_pack_mode(self._h, modes[mode]), "spamm_plan_set_pack_mode")

    def set_multiply_mode(self, mode: str) -> None:
        """Which multiply kernels may run: "auto" (default, by the counters of the previous step), "one_sm", or
        "gated_pairs" (the gated kernel on pairs of SMs for every pair of macro-tile rows).  Same results."""
        modes = {"auto": 0, "one_sm": 1, "gated_pairs": 2}
        if mode not in modes:
            raise ValueError(f"multiply mode must be one of {sorted(modes)}")
        check(self._lib.spamm_plan_set_multiply_mode(self._h, modes[mode]), "spamm_plan_set_multiply_mode")

    # ---- the driver steps
    def upload(self, a_rows=None, b=None) -> None:
        pa = _host_ptr(a_rows, self.rows * self.K * 4) if a_rows is not None else 0
        pb = _host_ptr(b, self.K * self.N * 4) if b is not None else 0
        check(self._lib.spamm_upload(self._h, pa, pb), "spamm_upload")

    def norms(self) -> None:
        check(self._lib.spamm_norms(self._h), "spamm_norms")

    def norms_share(self, b_tile_begin: int, b_tile_count: int) -> None:
        check(self._lib.spamm_norms_share(self._h, b_tile_begin, b_tile_count), "spamm_norms_share")

    def norm_b_share(self, b_tile_begin: int, b_tile_count: int) -> None:
        check(self._lib.spamm_norm_b_share(self._h, b_tile_begin, b_tile_count), "spamm_norm_b_share")

    def peer_handles(self) -> bytes:
        buf = C.create_string_buffer(192)
        check(self._lib.spamm_peer_handles(self._h, buf, 192), "spamm_peer_handles")
        return buf.raw

    def peer_attach(self, world: int, rank: int, all_handles: bytes) -> None:
        check(self._lib.spamm_peer_attach(self._h, world, rank, all_handles), "spamm_peer_attach")

    def norm_b_share_push(self, b_tile_begin: int, b_tile_count: int) -> None:
        check(self._lib.spamm_norm_b_share_push(self._h, b_tile_begin, b_tile_count), "spamm_norm_b_share_push")

    def run_shared(self, tau: float, b_tile_begin: int, b_tile_count: int) -> None:
        """One whole step of a plan that shares B's norm map with attached peers, in one call."""
        check(self._lib.spamm_run_shared(self._h, float(tau), b_tile_begin, b_tile_count), "spamm_run_shared")

    def norms_shared(self, b_tile_begin: int, b_tile_count: int) -> None:
        """The first part of `run_shared`: both norm maps (this rank's rows of A, its share of B) in one launch and the
        store of the share into the peers' maps."""
        check(self._lib.spamm_norms_shared(self._h, b_tile_begin, b_tile_count), "spamm_norms_shared")

    def upload_b_rows(self, b_rows, row_begin: int) -> None:
        """Rows [row_begin, row_begin + len(b_rows)) of B into the plan's copy of B."""
        rows = int(b_rows.shape[0])
        check(self._lib.spamm_upload_b_rows(self._h, _host_ptr(b_rows, rows * self.N * 4), row_begin, rows),
              "spamm_upload_b_rows")

    def multiply_b_resident(self, a_rows, tau: float, out=None, b_ready_event: int = 0):
        """`multiply` without the upload of B (the caller has assembled B on the GPU; `b_ready_event` is the handle of
        a CUDA event after which it is complete, 0 if it already is)."""
        if out is None:
            out = np.empty((self.rows, self.N), dtype=np.float32)
        st = SpammStats()
        check(self._lib.spamm_multiply_b_resident(self._h, _host_ptr(a_rows, self.rows * self.K * 4),
                                                  _host_ptr(out, self.rows * self.N * 4), float(tau),
                                                  C.c_void_p(b_ready_event), C.byref(st)), "spamm_multiply_b_resident")
        return out, st.as_dict()

    def compute_norm_a(self) -> None:
        check(self._lib.spamm_norm_a(self._h), "spamm_norm_a")

    def build_lists(self, tau: float) -> None:
        check(self._lib.spamm_build_lists(self._h, float(tau)), "spamm_build_lists")

    def pack(self) -> None:
        check(self._lib.spamm_pack(self._h), "spamm_pack")

    def gated_multiply(self) -> None:
        check(self._lib.spamm_gated_multiply(self._h), "spamm_gated_multiply")

    def run(self, tau: float) -> None:
        check(self._lib.spamm_run(self._h, float(tau)), "spamm_run")

    def set_precision(self, precision: str) -> None:
        """"half" (default: operands rounded to half, the reference's tensor-core build) or "split" (each operand
        as a sum of two halves, three tensor-core passes: float-level accuracy, the stand-in for the reference's
        float build)."""
        modes = {"half": 0, "split": 1}
        if precision not in modes:
            raise ValueError(f"precision must be one of {sorted(modes)}")
        check(self._lib.spamm_plan_set_precision(self._h, modes[precision]), "spamm_plan_set_precision")

    def clear_c_early(self) -> None:
        """Announce that lists, pack and multiply follow: C may be cleared now on the second stream (a speed hint)."""
        check(self._lib.spamm_clear_c_early(self._h), "spamm_clear_c_early")

    def finish(self, tau: float) -> None:
        """lists + pack + multiply in one call."""
        check(self._lib.spamm_finish(self._h, float(tau)), "spamm_finish")

    def sync(self) -> None:
        check(self._lib.spamm_sync(self._h), "spamm_sync")

    def b_rows(self, rank: Optional[int] = None) -> Tuple[int, int]:
        """(first row, number of rows) of B that rank `rank` (default: this one) brings to `multiply`."""
        r = self.rank if rank is None else rank
        if self.world == 1:
            return 0, self.K
        if self._share is not None:
            b0, b1 = r * self._share * TILE, (r + 1) * self._share * TILE
        else:                              # uneven: whole tile rows, the remainder to the first ranks
            k_tiles = -(-self.K // TILE)
            base, extra = divmod(k_tiles, self.world)
            b0 = (r * base + min(r, extra)) * TILE
            b1 = b0 + (base + (1 if r < extra else 0)) * TILE
        return min(b0, self.K), min(b1, self.K) - min(b0, self.K)

    def multiply(self, a_rows, b_rows, tau: float, out=None):
        """Host matrices in and out on every rank, each over its own PCIe link: this rank's rows of A, its rows
        `b_rows()` of B, its rows of C back (`out`, pinned for speed).  The shares of B are exchanged over NVLink
        (NCCL all-gather, in place in the plans' copies of B) while the rows of A already go up; the path then runs in
        chunks of rows with uploads, kernels and downloads overlapped.  Returns (rows of C, statistics of this rank).
        The reference copies all of A and all of B to every device (cuSpAMM.cu:449-450)."""
        if self.world == 1:
            return self.plan.multiply(a_rows, b_rows, tau, out=out)
        torch = self._torch
        r0, _ = self.b_rows()
        self.plan.upload_b_rows(b_rows, r0)
        if self._stream is None:
            self._stream = self.plan.torch_stream()
        if self._gather_stream is None:
            self._gather_stream = torch.cuda.Stream(priority=-5)
            self._gather_done = torch.cuda.Event()
        bfull = self.plan.as_tensor(BUF_B)
        self._gather_stream.wait_stream(self._stream)
        with torch.cuda.stream(self._gather_stream):
            if self._share is not None:
                rows = self._share * TILE
                self._dist.all_gather_into_tensor(bfull, bfull[self.rank * rows:(self.rank + 1) * rows], group=self.group)
            else:
                for r in range(self.world):
                    b0, n = self.b_rows(r)
                    if n:
                        self._dist.broadcast(bfull[b0:b0 + n], src=r, group=self.group)
            self._gather_done.record(self._gather_stream)
        return self.plan.multiply_b_resident(a_rows, tau, out=out, b_ready_event=self._gather_done.cuda_event)

    def run_timed(self, tau: float) -> dict:
        st = SpammStats()
        check(self._lib.spamm_run_timed(self._h, float(tau), C.byref(st)), "spamm_run_timed")
        return st.as_dict()

    def download_c(self, out=None):
        if out is None:
            out = np.empty((self.rows, self.N), dtype=np.float32)
        check(self._lib.spamm_download_c(self._h, _host_ptr(out, self.rows * self.N * 4)), "spamm_download_c")
        return out

    def multiply(self, a_rows, b, tau: float, out=None):
        """Host matrices in, host matrix out (the whole loop body of the reference driver plus the copies)."""
        if out is None:
            out = np.empty((self.rows, self.N), dtype=np.float32)
        st = SpammStats()
        check(self._lib.spamm_multiply(self._h, _host_ptr(a_rows, self.rows * self.K * 4),
                                       _host_ptr(b, self.K * self.N * 4), _host_ptr(out, self.rows * self.N * 4),
                                       float(tau), C.byref(st)), "spamm_multiply")
        return out, st.as_dict()

    # ---- readbacks for the parity tests
    def norm_a(self) -> np.ndarray:
        out = np.empty((self.row_tile_count, self.k_tiles), dtype=np.float32)
        check(self._lib.spamm_get_norm_a(self._h, out.ctypes.data), "spamm_get_norm_a")
        return out

    def norm_b(self) -> np.ndarray:
        out = np.empty((self.k_tiles, self.n_tiles), dtype=np.float32)
        check(self._lib.spamm_get_norm_b(self._h, out.ctypes.data), "spamm_get_norm_b")
        return out

    def counts(self) -> Tuple[np.ndarray, int]:
        out = np.empty((self.row_tile_count, self.n_tiles), dtype=np.int32)
        s = C.c_int64()
        check(self._lib.spamm_get_counts(self._h, out.ctypes.data, C.byref(s)), "spamm_get_counts")
        return out, int(s.value)

    def lists(self) -> Tuple[np.ndarray, np.ndarray]:
        """(offsets, k_idx): the per-C-tile skip lists the multiply kernel walks, in the reference's form."""
        tiles = self.row_tile_count * self.n_tiles
        offsets = np.zeros(tiles + 1, dtype=np.int64)
        check(self._lib.spamm_get_lists(self._h, offsets.ctypes.data, None), "spamm_get_lists")
        k_idx = np.empty(max(int(offsets[-1]), 1), dtype=np.int32)
        check(self._lib.spamm_get_lists(self._h, offsets.ctypes.data, k_idx.ctypes.data), "spamm_get_lists")
        return offsets, k_idx[: int(offsets[-1])]

    def error_norms(self, d_reference_ptr: int) -> Tuple[float, float, float]:
        """(||ref - C||_F, ||ref||_F, ||C||_F) against a device matrix of C's shape (tool.cu:6-24)."""
        out = (C.c_double * 3)()
        check(self._lib.spamm_error_norms(self._h, C.c_void_p(d_reference_ptr), out), "spamm_error_norms")
        return float(out[0]), float(out[1]), float(out[2])

    def count_valid(self, tau: float) -> Tuple[int, float]:
        """(count, sum of norm products): countValid of the reference (tool.cu:493-529) on the GPU."""
        c, s = C.c_int64(), C.c_double()
        check(self._lib.spamm_count_valid(self._h, float(tau), C.byref(c), C.byref(s)), "spamm_count_valid")
        return int(c.value), float(s.value)

    def tune_tau(self, expected_rate: float = 0.75, max_iters: int = 20, tolerance: float = 0.01):
        """(tau, rate, iterations): tuneValidRate of the reference (tool.cu:438-490, main.h:35-38)."""
        tau, rate, it = C.c_float(), C.c_double(), C.c_int()
        check(self._lib.spamm_tune_tau(self._h, expected_rate, max_iters, tolerance, C.byref(tau), C.byref(rate),
                                       C.byref(it)), "spamm_tune_tau")
        return float(tau.value), float(rate.value), int(it.value)

    def kernel_launches(self) -> int:
        return int(self._lib.spamm_kernel_launches(self._h))

    # ---- raw device memory, for moving data between GPUs
    def buffer(self, which: int) -> Tuple[int, int]:
        p, n = C.c_void_p(), C.c_size_t()
        check(self._lib.spamm_device_buffer(self._h, which, C.byref(p), C.byref(n)), "spamm_device_buffer")
        return int(p.value or 0), int(n.value)

    @property
    def stream_ptr(self) -> int:
        s = C.c_void_p()
        check(self._lib.spamm_stream(self._h, C.byref(s)), "spamm_stream")
        return int(s.value or 0)

    def as_tensor(self, which: int):
        """torch view (no copy) of one of the plan's float/int32 device buffers."""
        import torch

        ptr, nbytes = self.buffer(which)
        shapes = {
            BUF_A: ((self.row_tile_count * TILE, self.Kp), "<f4"),
            BUF_B: ((self.Kp, self.Np), "<f4"),
            BUF_C: ((self.row_tile_count * TILE, self.Np), "<f4"),
            BUF_NORM_A: ((self.row_tile_count, self.k_tiles), "<f4"),
            BUF_NORM_B: ((self.k_tiles, self.n_tiles), "<f4"),
            BUF_COUNTS: ((self.row_tile_count, self.n_tiles), "<i4"),
        }
        if which not in shapes:
            raise ValueError("no tensor view for this buffer")
        shape, typestr = shapes[which]
        if 0 in shape:
            dt = torch.float32 if typestr == "<f4" else torch.int32
            return torch.empty(shape, dtype=dt, device=f"cuda:{self.device}")
        return torch.as_tensor(_DeviceView(ptr, shape, typestr), device=f"cuda:{self.device}")

    def torch_stream(self):
        import torch

        return torch.cuda.ExternalStream(self.stream_ptr, device=f"cuda:{self.device}")


class SpammGroup:
    """Several GPUs driven by this one process: the reference's DEVICEDIM form (para.h:9, cuSpAMM.cu:404-451,470-537)
    through the group entry points of the C ABI.  Whole host matrices in and out; the library splits C by row blocks,
    uploads B by shares over every device's own PCIe link and exchanges shares and norm maps over NVLink."""

    def __init__(self, M: int, K: int, N: int, devices: Optional[Sequence[int]] = None, n_devices: Optional[int] = None):
        self._lib = _lib.load()
        if devices is None:
            devices = list(range(1 if n_devices is None else n_devices))
        self.devices = [int(d) for d in devices]
        self.M, self.K, self.N = M, K, N
        self._h = C.c_void_p()
        ids = (C.c_int * len(self.devices))(*self.devices)
        check(self._lib.spamm_group_create(C.byref(self._h), M, K, N, len(self.devices), ids), "spamm_group_create")
        self.plans = []
        for i, d in enumerate(self.devices):
            h = C.c_void_p()
            check(self._lib.spamm_group_plan(self._h, i, C.byref(h)), "spamm_group_plan")
            self.plans.append(SpammPlan._borrowed(h.value, d))

    def close(self) -> None:
        if getattr(self, "_h", None) and self._h.value:
            for p in self.plans:
                p.close()
            self._lib.spamm_group_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def upload(self, a=None, b=None) -> None:
        pa = _host_ptr(a, self.M * self.K * 4) if a is not None else 0
        pb = _host_ptr(b, self.K * self.N * 4) if b is not None else 0
        check(self._lib.spamm_group_upload(self._h, pa, pb), "spamm_group_upload")

    def run(self, tau: float) -> None:
        check(self._lib.spamm_group_run(self._h, float(tau)), "spamm_group_run")

    def sync(self) -> None:
        check(self._lib.spamm_group_sync(self._h), "spamm_group_sync")

    def download_c(self, out=None):
        if out is None:
            out = np.empty((self.M, self.N), dtype=np.float32)
        check(self._lib.spamm_group_download_c(self._h, _host_ptr(out, self.M * self.N * 4)), "spamm_group_download_c")
        return out

    def survivors(self) -> int:
        s = C.c_int64()
        check(self._lib.spamm_group_survivors(self._h, C.byref(s)), "spamm_group_survivors")
        return int(s.value)

    def multiply(self, a, b, tau: float, out=None):
        if out is None:
            out = np.empty((self.M, self.N), dtype=np.float32)
        st = SpammStats()
        check(self._lib.spamm_group_multiply(self._h, _host_ptr(a, self.M * self.K * 4), _host_ptr(b, self.K * self.N * 4),
                                             _host_ptr(out, self.M * self.N * 4), float(tau), C.byref(st)),
              "spamm_group_multiply")
        return out, st.as_dict()


class ShardedSpamm:
    """C sharded by row blocks over the ranks of a torch.distributed group (one process per GPU).

    Mirrors the reference's multi-device loop (cuSpAMM.cu:433-451, 470-537) with two changes the reference's
    own layout invites: B crosses PCIe once in all (by one rank and a broadcast, `distribute`, or in shares over
    every rank's own link and an all-gather, `multiply`) instead of once per device (cuSpAMM.cu:449-450), and every
    rank computes only its share of B's norm map, the shares being exchanged (`exchange="push"`: peer stores from
    a small kernel, one library call per step; `exchange="nccl"`: an NCCL all-gather on a side stream), instead of
    each device recomputing all of it (cuSpAMM.cu:486).

    `plan_factory(M, K, N, begin, count)` builds the per-rank plan (default: a `SpammPlan` on the current CUDA
    device); the tests pass a CPU stand-in to run the same orchestration over gloo.
    """

    def __init__(self, M: int, K: int, N: int, group=None, plan_factory=None, device: Optional[int] = None,
                 exchange: str = "push", blocks=None):
        import torch
        import torch.distributed as dist

        self._torch, self._dist = torch, dist
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.M, self.K, self.N = M, K, N
        self.Mp, self.Kp, self.Np = (-(-x // TILE) * TILE for x in (M, K, N))
        if blocks is None:
            blocks = row_blocks(-(-M // TILE), self.world)      # the reference's even split
        else:                                                   # e.g. from balanced_row_blocks
            blocks = [(int(b), int(c)) for b, c in blocks]
            ends = [b + c for b, c in blocks]
            if (len(blocks) != self.world or blocks[0][0] != 0 or ends[-1] != -(-M // TILE)
                    or any(c < 0 for _, c in blocks) or any(blocks[i + 1][0] != ends[i] for i in range(self.world - 1))):
                raise ValueError("blocks must tile the C tile rows contiguously, one block per rank")
        self.blocks = blocks
        self.row_tile_begin, self.row_tile_count = self.blocks[self.rank]
        if plan_factory is None:
            dev = torch.cuda.current_device() if device is None else device
            plan_factory = lambda M, K, N, b, c: SpammPlan(M, K, N, b, c, device=dev)  # noqa: E731
        self.plan = plan_factory(M, K, N, self.row_tile_begin, self.row_tile_count)
        k_tiles = -(-K // TILE)
        # equal shares of B's tile rows when they divide evenly, otherwise every rank computes the whole map
        self._share = (k_tiles // self.world) if (self.world > 1 and k_tiles % self.world == 0) else None
        self._nb = self._mine = self._stream = self._side = None
        self._nb_ptr = 0
        self._gather_stream = self._gather_done = None
        self._nccl = False
        # peer-to-peer exchange of B's norm-map shares (no collective in the step) when the plan offers it
        self._push = False
        if (exchange == "push" and self._share is not None and (self._share * -(-N // TILE)) % 4 == 0
                and hasattr(self.plan, "peer_handles")
                and self.world <= 8 and dist.get_backend(group) == "nccl"):
            mine = self.plan.peer_handles()
            everyone = [None] * self.world
            dist.all_gather_object(everyone, mine, group=group)
            self.plan.peer_attach(self.world, self.rank, b"".join(everyone))
            self._push = True

    def _on_stream(self):
        ts = getattr(self.plan, "torch_stream", None)
        if ts is None:
            import contextlib

            return contextlib.nullcontext()
        return self._torch.cuda.stream(ts())

    def distribute(self, a_rows, b=None, src: int = 0) -> None:
        """Every rank uploads its own rows of A; rank `src` uploads B, which is then broadcast to the others."""
        self.plan.upload(a_rows, b if self.rank == src else None)
        if self.world > 1:
            with self._on_stream():
                self._dist.broadcast(self.plan.as_tensor(BUF_B), src=src, group=self.group)

    def run(self, tau: float) -> None:
        """norm maps (B's shared between the ranks), lists, pack, multiply; asynchronous."""
        if self.world == 1 and hasattr(self.plan, "run"):
            self.plan.run(tau)
            return
        if self._share is None:
            self.plan.norms()
        elif self._push:
            # one library call for the whole step: the maps of this rank's rows of A and share of B in one launch, the
            # share stored into every GPU's map by a small kernel, then lists (which wait for the shares), pack, multiply
            self.plan.run_shared(tau, self.rank * self._share, self._share)
            return
        else:
            ptr = self.plan.buffer(BUF_NORM_B)[0] if hasattr(self.plan, "buffer") else 0
            if self._nb is None or ptr != self._nb_ptr:      # views and streams are built once: this runs every step
                self._nb_ptr = ptr                           # (again if the plan's current map of B has changed)
                self._nb = self.plan.as_tensor(BUF_NORM_B)
                self._mine = self._nb[self.rank * self._share:(self.rank + 1) * self._share]
                self._nccl = self._dist.get_backend(self.group) == "nccl"
                ts = getattr(self.plan, "torch_stream", None)
                self._stream = ts() if ts is not None else None
                # the exchange must outrank the plan's main stream (which is one step above the lowest priority), or
                # its few blocks queue behind the norm kernel's; the runtime clamps the value to the highest priority
                self._side = self._torch.cuda.Stream(priority=-5) if self._nccl else None
            nb, mine = self._nb, self._mine
            if self._nccl:
                # this rank's share of B's map first, then its exchange on a side stream while A's map is computed
                self.plan.norm_b_share(self.rank * self._share, self._share)
                self._side.wait_stream(self._stream)
                with self._torch.cuda.stream(self._side):
                    self._dist.all_gather_into_tensor(nb, mine, group=self.group)   # in place
                self.plan.compute_norm_a()
                self._clear_c_early()          # beside the exchange, not after it
                self._stream.wait_stream(self._side)
            else:
                self.plan.norms_share(self.rank * self._share, self._share)
                parts = [nb[r * self._share:(r + 1) * self._share] for r in range(self.world)]
                self._dist.all_gather(parts, mine.clone(), group=self.group)
        finish = getattr(self.plan, "finish", None)
        if finish is not None:
            finish(tau)
        else:
            self.plan.build_lists(tau)
            self.plan.pack()
            self.plan.gated_multiply()

    def _clear_c_early(self) -> None:
        f = getattr(self.plan, "clear_c_early", None)
        if f is not None:
            f()

    def b_rows(self, rank: Optional[int] = None) -> Tuple[int, int]:
        """(first row, number of rows) of B that rank `rank` (default: this one) brings to `multiply`."""
        r = self.rank if rank is None else rank
        if self.world == 1:
            return 0, self.K
        if self._share is not None:
            b0, b1 = r * self._share * TILE, (r + 1) * self._share * TILE
        else:                              # uneven: whole tile rows, the remainder to the first ranks
            k_tiles = -(-self.K // TILE)
            base, extra = divmod(k_tiles, self.world)
            b0 = (r * base + min(r, extra)) * TILE
            b1 = b0 + (base + (1 if r < extra else 0)) * TILE
        return min(b0, self.K), min(b1, self.K) - min(b0, self.K)

    def multiply(self, a_rows, b_rows, tau: float, out=None):
        """Host matrices in and out on every rank, each over its own PCIe link: this rank's rows of A, its rows
        `b_rows()` of B, its rows of C back (`out`, pinned for speed).  The shares of B are exchanged over NVLink
        (NCCL all-gather, in place in the plans' copies of B) while the rows of A already go up; the path then runs in
        chunks of rows with uploads, kernels and downloads overlapped.  Returns (rows of C, statistics of this rank).
        The reference copies all of A and all of B to every device (cuSpAMM.cu:449-450)."""
        if self.world == 1:
            return self.plan.multiply(a_rows, b_rows, tau, out=out)
        torch = self._torch
        r0, _ = self.b_rows()
        self.plan.upload_b_rows(b_rows, r0)
        if self._stream is None:
            self._stream = self.plan.torch_stream()
        if self._gather_stream is None:
            self._gather_stream = torch.cuda.Stream(priority=-5)
            self._gather_done = torch.cuda.Event()
        bfull = self.plan.as_tensor(BUF_B)
        self._gather_stream.wait_stream(self._stream)
        with torch.cuda.stream(self._gather_stream):
            if self._share is not None:
                rows = self._share * TILE
                self._dist.all_gather_into_tensor(bfull, bfull[self.rank * rows:(self.rank + 1) * rows], group=self.group)
            else:
                for r in range(self.world):
                    b0, n = self.b_rows(r)
                    if n:
                        self._dist.broadcast(bfull[b0:b0 + n], src=r, group=self.group)
            self._gather_done.record(self._gather_stream)
        return self.plan.multiply_b_resident(a_rows, tau, out=out, b_ready_event=self._gather_done.cuda_event)

    def run_timed(self, tau: float) -> dict:
        """One `run` with CUDA events between its parts (this rank's view, milliseconds); blocking."""
        torch = self._torch
        stream = self.plan.torch_stream()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        ev[0].record(stream)
        if self._share is None:
            self.plan.norms()
            ev[1].record(stream)
        elif self._push:
            self.plan.norms_shared(self.rank * self._share, self._share)
            ev[1].record(stream)       # the wait for the other GPUs' shares is inside the list build
        else:
            self.plan.norms_share(self.rank * self._share, self._share)
            ev[1].record(stream)
            nb = self.plan.as_tensor(BUF_NORM_B)
            mine = nb[self.rank * self._share:(self.rank + 1) * self._share]
            with torch.cuda.stream(stream):
                self._dist.all_gather_into_tensor(nb, mine, group=self.group)
        ev[2].record(stream)
        self.plan.build_lists(tau)
        ev[3].record(stream)
        self.plan.pack()
        ev[4].record(stream)
        self.plan.gated_multiply()
        ev[5].record(stream)
        self.plan.sync()
        names = ["ms_norm", "ms_allgather", "ms_lists", "ms_pack", "ms_multiply"]
        out = {n: ev[i].elapsed_time(ev[i + 1]) for i, n in enumerate(names)}
        out["ms_device_total"] = ev[0].elapsed_time(ev[5])
        out["exchange"] = "peer push" if self._push else ("nccl all-gather" if self._share is not None else "none")
        return out

    def sync(self) -> None:
        self.plan.sync()

    def survivors(self) -> int:
        """S summed over all ranks."""
        _, s = self.plan.counts()
        if self.world == 1:
            return s
        dev = self.plan.as_tensor(BUF_NORM_B).device
        t = self._torch.tensor([s], dtype=self._torch.int64, device=dev)
        self._dist.all_reduce(t, group=self.group)
        return int(t.item())

    def row_survivors(self) -> np.ndarray:
        """Surviving products per C tile row of the last step, for all tile rows, on every rank (the input of
        `balanced_row_blocks`)."""
        counts, _ = self.plan.counts()
        mine = counts.sum(axis=1).astype(np.int64)
        if self.world == 1:
            return mine
        parts = [None] * self.world
        self._dist.all_gather_object(parts, mine, group=self.group)
        return np.concatenate([np.asarray(x, dtype=np.int64) for x in parts])

    def gather_c(self, dst: int = 0):
        """Gathers the C slabs on rank `dst` (device to device), returns the full C there as a tensor, else None."""
        mine = self.plan.as_tensor(BUF_C)
        if self.world == 1:
            return mine
        equal = len({n for _, n in self.blocks}) == 1
        with self._on_stream():
            if self.rank == dst:
                full = self._torch.empty((self.Mp, self.Np), dtype=mine.dtype, device=mine.device)
                parts = [full[b * TILE:(b + n) * TILE] for b, n in self.blocks]
            else:
                full, parts = None, None
            if equal:
                self._dist.gather(mine, parts, dst=dst, group=self.group)
            elif self.rank == dst:
                # slabs of different heights: one receive per peer
                parts[dst].copy_(mine)
                reqs = [self._dist.irecv(parts[r], src=r, group=self.group)
                        for r in range(self.world) if r != dst and parts[r].numel()]
                for q in reqs:
                    q.wait()
            elif mine.numel():
                self._dist.send(mine, dst=dst, group=self.group)
        self.plan.sync()
        return full

    def close(self) -> None:
        close = getattr(self.plan, "close", None)
        if close:
            close()


# ---- generators (host side): csrc/generators.cpp through its own small library
from .hostgen import (gen_decay_alg, gen_decay_exp, gen_lattice, gen_ones, gen_signed_exp, gen_uniform,  # noqa: E402,F401
                      gen_uniform_alg)
