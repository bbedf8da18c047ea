#!/usr/bin/env python
"""Benchmark of the SpAMM hot path (norm maps -> skip lists -> half packing -> gated tensor-core multiply).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--n SIZE] [--tau TAU]
                    [--workload exp|alg|lattice|dense] [--precision half|split] [--partition auto|even|balanced]
                    [--exchange push|nccl] [--multiply-mode auto|one_sm|gated_pairs] [--no-sweep] [--no-cpu]
                    [--no-ref-kernels]

One "step" is one pass of the reference's timed region (cuSpAMM.cu:458-546) over matrices that are already
resident in HBM.  The default workload is the configuration the headline metric is quoted on: N=16384, exponential
decay a_ij = +-exp(-0.1|i-j|) with independent seeds for A and B, tau = 1e-6, plus a tau sweep reported beside it.
Under torchrun every rank owns one GPU and one block of C tile rows (strong scaling: the matrices stay the same).
Rank 0 prints one JSON line.

`--impl reference` times the CPU restatement of the reference's algorithm (the reference ships no CPU
implementation: its host loop is commented out, tool.cu:79-126) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAMBDA = 0.1
SEED_A, SEED_B = 1, 2
SWEEP_TAUS = [0.0, 1e-10, 1e-6, 1e-4, 1e-2]
TILE = 32
CPU_FULL_LIMIT = 1.0e11      # scalar multiply-adds the host loop is asked to do in full; above it, a sample of rows


# The benchmark workloads: name -> (description, default N, default tau)
WORKLOADS = {
    "exp": ("a_ij=+-exp(-0.1|i-j|), seeds 1/2", 16384, 1e-6),            # the headline
    "alg": ("a_ij=u_ij/(|i-j|^2+1), u in [-1,1), seeds 3/4", 16384, 1e-6),   # algebraic decay
    "lattice": ("a_ij=+-u*exp(-|r_i-r_j|) on an L^3 grid, u in [0.5,1), symmetric, seed 7, A=B", 32768, 1e-8),
    "dense": ("a_ij uniform in [-1,1), seeds 5/6", 16384, 0.0),            # nothing skipped
}
WORKLOAD = ["exp"]


def workload_name(n: int, tau: float) -> str:
    return f"N={n} fp32 A,B: {WORKLOADS[WORKLOAD[0]][0]}, tile 32, tau={tau:g}"


def config_dict(n: int, tau: float, world: int, **extra) -> dict:
    """The `config` object: the same keys in both arms."""
    cfg = {"workload": workload_name(n, tau), "survivors": None, "executed_fraction": None,
           "timed_region": "norm maps + skip lists + half packing + gated multiply, inputs resident in memory",
           "l2": "inputs (2*4*N^2 bytes) larger than L2, no flush needed", "parallelism": f"rowblock{world}",
           "partition": "even"}
    cfg.update(extra)
    return cfg


def read_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]),
                    "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


def read_traffic_ratio() -> float | None:
    """DRAM bytes per algorithmic byte of the norm-map kernel, from the committed ncu summary (None if absent)."""
    p = ROOT / "profiles" / "norm_map_traffic.json"
    try:
        return float(json.loads(p.read_text())["dram_bytes_per_algorithmic_byte"])
    except Exception:
        return None


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["reasons"] = sorted(reasons)
            out["samples"] = len(sm)
        return out


def pinned(shape):
    import torch

    t = torch.empty(shape, dtype=torch.float32, pin_memory=True)
    return t, t.numpy()


def generate_into(arr: np.ndarray, seed: int, row_begin: int, cols: int) -> None:
    """Rows [row_begin, row_begin+rows) of operand `seed` (SEED_A or SEED_B) of the selected workload, from the host
    generator library (plain C++; neither arm needs the GPU library for its inputs)."""
    from cuspamm_b200 import hostgen

    w, rows = WORKLOAD[0], arr.shape[0]
    first = seed == SEED_A
    if w == "exp":
        hostgen.fill("spamm_gen_signed_exp", arr, LAMBDA, seed, row_begin, rows, cols)
    elif w == "alg":
        hostgen.fill("spamm_gen_uniform_alg", arr, 3 if first else 4, row_begin, rows, cols)
    elif w == "dense":
        hostgen.fill("spamm_gen_uniform", arr, 5 if first else 6, row_begin, rows, cols)
    else:
        L = round(cols ** (1.0 / 3.0))
        if L ** 3 != cols:
            raise SystemExit("the lattice workload needs N = L^3 (e.g. 32768 = 32^3, 4096 = 16^3)")
        hostgen.fill("spamm_gen_lattice", arr, L, 7, row_begin, rows)


def sample_tile_rows(blocks, per_block: int = 3) -> list:
    """Tile rows of C to compare with the CPU checker: `per_block` rows spread evenly over every rank's block, the
    first and the last among them, so that every block boundary is covered."""
    rows = []
    for b, c in blocks:
        if c <= 0:
            continue
        k = min(per_block, c)
        rows.extend(sorted({b + (i * (c - 1)) // max(k - 1, 1) for i in range(k)}))
    return rows


# ------------------------------------------------------------------------------------------------ CPU leg

def cpu_step(O, A_rows, B, Ah_rows, Bh, tau, nA_full_rows=None):
    """One pass of the reference's timed region on the host for the given rows of A (a block of whole tile rows):
    norm maps, lists, gated product (inputs already rounded to half, as the reference rounds at generation time,
    tool.cu:418).  Returns (seconds, S, C rows)."""
    t0 = time.perf_counter()
    nA = O.norm_map(A_rows)
    nB = O.norm_map(B)
    counts, offsets, kidx = O.lists(nA, nB, tau)
    C = O.gated_multiply(Ah_rows, Bh, offsets, kidx)
    dt = time.perf_counter() - t0
    return dt, int(offsets[-1]), C


def cpu_sampled(O, n, tau, B, Bh, tile_rows):
    """The host loop on a sample of C tile rows (generated on demand): seconds, S of the sample, C rows, the rows'
    norm map.  The norm map of B is part of the time (it is needed whatever the sample)."""
    A_sub = np.empty((len(tile_rows) * TILE, n), dtype=np.float32)
    for i, r in enumerate(tile_rows):
        generate_into(A_sub[i * TILE:(i + 1) * TILE], SEED_A, r * TILE, n)
    Ah_sub = O.round_to_half(A_sub)
    dt, s, C = cpu_step(O, A_sub, B, Ah_sub, Bh, tau)
    return dt, s, C


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O

    O.set_num_threads(os.cpu_count() or 1)     # torchrun exports OMP_NUM_THREADS=1; this arm owns the host cores
    n, tau = args.n, args.tau
    B = np.empty((n, n), dtype=np.float32)
    generate_into(B, SEED_B, 0, n)
    Bh = O.round_to_half(B)
    T = n // TILE
    # how much is one step: the whole workload when the host can do it in a fraction of a second, else a sample of rows
    nB = O.norm_map(B)
    rows16 = sample_tile_rows([(0, T)], per_block=16)
    A_probe = np.empty((len(rows16) * TILE, n), dtype=np.float32)
    for i, r in enumerate(rows16):
        generate_into(A_probe[i * TILE:(i + 1) * TILE], SEED_A, r * TILE, n)
    s_probe = int(O.lists(O.norm_map(A_probe), nB, tau)[1][-1])
    est_total = s_probe / max(len(rows16), 1) * T
    full = est_total * 32768.0 <= CPU_FULL_LIMIT
    if full:
        A = np.empty((n, n), dtype=np.float32)
        generate_into(A, SEED_A, 0, n)
        Ah = O.round_to_half(A)
        sample = "whole workload per step (norm maps + lists + gated product, inputs pre-rounded to half)"
    else:
        # about 2e10 multiply-adds per step
        k = int(max(1, min(len(rows16), 2.0e10 / max(est_total / T * 32768.0, 1.0))))
        rows = rows16[:: max(1, len(rows16) // k)][:k]
        A = np.empty((len(rows) * TILE, n), dtype=np.float32)
        for i, r in enumerate(rows):
            generate_into(A[i * TILE:(i + 1) * TILE], SEED_A, r * TILE, n)
        Ah = O.round_to_half(A)
        sample = (f"{len(rows)} of {T} C tile rows per step (norm map of those rows of A and of all of B, lists, gated "
                  f"product); value = executed flops of the sample / its time")
    times, S = [], 0
    for i in range(args.warmup + args.steps):
        dt, S, _ = cpu_step(O, A, B, Ah, Bh, tau)
        if i >= args.warmup:
            times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    value = 65536.0 * S / (ms * 1e-3) / 1e12
    line = {
        "impl": "reference", "metric": "spamm_executed_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16xf16+f32", "data": "synthetic",
        "config": config_dict(n, tau, args.gpus, survivors=S if full else None,
                              executed_fraction=(S / T ** 3) if full else None),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": O.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ reference kernels

def time_reference_kernels(torch, plan_factory, steps: int = 3):
    """The reference's own kernels (unroll_get_Fnorm_FP16 + get_C_FP16_B32, cuSpAMM.cu:74-123,276-392) recompiled
    for this GPU, timed over its timed region next to this library on the same matrices: N=8192 (the largest size
    the reference's survivor count is right for, cuSpAMM.cu:328-333), exponential decay, tau 0 and 1e-6.  A reported
    baseline; the library's path does not depend on it."""
    import ctypes as C

    n = 8192
    path = ROOT / "oracle" / "_ref" / f"libref_{n}.so"
    if not path.exists():
        return {"unavailable": f"{path.name} not built (needs the reference sources at build time)"}
    try:
        lib = C.CDLL(str(path))
        lib.ref_timed_step_fp16.argtypes = [C.c_void_p] * 5 + [C.c_float]
        A = np.empty((n, n), dtype=np.float32)
        B = np.empty((n, n), dtype=np.float32)
        saved = WORKLOAD[0]
        WORKLOAD[0] = "exp"
        generate_into(A, SEED_A, 0, n)
        generate_into(B, SEED_B, 0, n)
        WORKLOAD[0] = saved
        dA, dB = torch.from_numpy(A).cuda().half(), torch.from_numpy(B).cuda().half()
        nA = torch.empty((n // 32, n // 32), dtype=torch.float32, device="cuda")
        nB = torch.empty_like(nA)
        dC = torch.empty((n, n), dtype=torch.float32, device="cuda")
        out = {"n": n, "matrices": "a_ij=+-exp(-0.1|i-j|), seeds 1/2, stored as half for the reference",
               "note": "reference: half inputs, its half-precision norm kernel, one block per C tile with WMMA; "
                       "library: float inputs, float norms, conversion on the GPU; both over norm maps + lists + multiply",
               "taus": []}
        with plan_factory(n) as p:
            p.upload(A, B)
            for tau in (0.0, 1e-6):
                torch.cuda.synchronize()
                if lib.ref_timed_step_fp16(dA.data_ptr(), nA.data_ptr(), dB.data_ptr(), nB.data_ptr(), dC.data_ptr(),
                                           tau) != 0:
                    return {"unavailable": "the reference's kernels did not launch on this GPU"}
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(steps):
                    lib.ref_timed_step_fp16(dA.data_ptr(), nA.data_ptr(), dB.data_ptr(), nB.data_ptr(), dC.data_ptr(),
                                            tau)
                e1.record()
                torch.cuda.synchronize()
                ms_ref = e0.elapsed_time(e1) / steps
                for _ in range(3):
                    p.run(tau)
                p.sync()
                st = [p.run_timed(tau) for _ in range(steps)]
                ms_lib = sum(s["ms_device_total"] for s in st) / steps
                S = int(st[-1]["survivors"])
                out["taus"].append({"tau": tau, "reference_ms": ms_ref, "library_ms": ms_lib, "speedup": ms_ref / ms_lib,
                                    "survivors_library": S,
                                    "library_executed_tflops": 65536.0 * S / (ms_lib * 1e-3) / 1e12,
                                    "reference_executed_tflops_at_library_count": 65536.0 * S / (ms_ref * 1e-3) / 1e12})
        del dA, dB, dC
        torch.cuda.empty_cache()
        return out
    except Exception as e:                      # a reported baseline, never a reason to lose the GPU numbers
        return {"unavailable": repr(e)}


# ------------------------------------------------------------------------------------------------ GPU leg

def run_ours(args):
    import torch
    import torch.distributed as dist

    from cuspamm_b200 import BUF_A, BUF_B, BUF_C, ShardedSpamm, SpammPlan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    n, tau = args.n, args.tau
    T = n // TILE
    peaks = read_peaks()

    def build(blocks=None):
        sh = ShardedSpamm(n, n, n, exchange=args.exchange, blocks=blocks)
        if args.precision != "half":
            sh.plan.set_precision(args.precision)
        if args.multiply_mode != "auto":
            sh.plan.set_multiply_mode(args.multiply_mode)
        a_t, a_np = pinned((sh.plan.rows, n))
        generate_into(a_np, SEED_A, sh.row_tile_begin * TILE, n)
        return sh, a_t, a_np

    sh, a_t, a_np = build()
    plan = sh.plan
    # B: rank 0 holds all of it on the host (it feeds `distribute` and the checker); every other rank holds the rows it
    # brings to the sharded host-to-host call
    if rank == 0:
        b_t, b_np = pinned((n, n))
        generate_into(b_np, SEED_B, 0, n)
    else:
        b_t, b_np = None, None
    sh.distribute(a_np, b_np)
    sh.sync()

    # ---- setup, outside the timed region like the reference's static split (cuSpAMM.cu:503,530): when the surviving
    # products are spread unevenly over the rows of C, move the block boundaries so that every GPU gets about the
    # same work (one untimed step with the even split measures the survivors per tile row)
    partition = "even"
    if world > 1 and args.partition != "even":
        from cuspamm_b200 import balanced_row_blocks

        sh.run(tau)
        sh.sync()
        per_row = sh.row_survivors().astype(np.float64)
        # a tile row's fixed cost (its share of the norm pass and of writing C) in units of one product's time
        base = 32 * 4 * (2 * n) / 6.5e12 / 0.175e-9
        weights = per_row + base
        load = lambda bl: max(weights[b:b + c].sum() for b, c in bl)       # noqa: E731
        blocks = balanced_row_blocks(weights, world)
        if blocks != sh.blocks and (args.partition == "balanced" or load(blocks) < 0.97 * load(sh.blocks)):
            imbalance = (load(sh.blocks) / (weights.sum() / world), load(blocks) / (weights.sum() / world))
            sh.close()
            del a_t, a_np
            sh, a_t, a_np = build(blocks)
            plan = sh.plan
            sh.distribute(a_np, b_np)
            sh.sync()
            partition = f"survivor-balanced (largest/mean block weight {imbalance[0]:.2f} -> {imbalance[1]:.2f})"
    rows = plan.rows

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = plan.torch_stream()
    issue_ms = [0.0]

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        t_issue = time.perf_counter()
        for _ in range(steps):
            fn()
        e1.record(stream)
        issue_ms[0] = (time.perf_counter() - t_issue) * 1e3 / steps     # host time to issue one step
        torch.cuda.synchronize()
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # ---- main timed region: K passes over resident inputs
    for _ in range(max(args.warmup, 3)):
        sh.run(tau)
    sh.sync()
    S = sh.survivors()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = plan.kernel_launches()
    if sampler:
        sampler.start()
    ms_step = timed(lambda: sh.run(tau), args.steps)
    clocks = sampler.stop() if sampler else None
    host_issue_ms = issue_ms[0]
    launches = plan.kernel_launches() - launches0
    sh.sync()

    # ---- the same steps once more with an event after every step: the fastest single step (rank-local)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(min(args.steps, 20) + 1)]
    barrier()
    marks[0].record(stream)
    for m in marks[1:]:
        sh.run(tau)
        m.record(stream)
    torch.cuda.synchronize()
    ms_min = min(a.elapsed_time(b) for a, b in zip(marks[:-1], marks[1:]))
    sh.sync()

    # ---- results of the timed configuration for the parity check (outside the timed region): every rank's sampled
    # tile rows of C and its list lengths
    tile_rows = sample_tile_rows(sh.blocks)
    mine = [r for r in tile_rows if sh.row_tile_begin <= r < sh.row_tile_begin + sh.row_tile_count]

    def grab_rows():
        c_dev = plan.as_tensor(BUF_C)
        with torch.cuda.stream(stream):
            parts = [c_dev[(r - sh.row_tile_begin) * TILE:(r - sh.row_tile_begin + 1) * TILE].cpu() for r in mine]
        torch.cuda.synchronize()
        counts, s_mine = plan.counts()
        got = {r: (parts[i].numpy(), int(counts[r - sh.row_tile_begin].sum())) for i, r in enumerate(mine)}
        if world == 1:
            return got, s_mine
        everyone = [None] * world
        dist.all_gather_object(everyone, (got, s_mine))
        merged = {}
        for g, _ in everyone:
            merged.update(g)
        return merged, sum(s for _, s in everyone)

    sampled_c, sampled_s_total = grab_rows()
    sampled_other = None
    if world > 1 and sh._share is not None and sh._push:
        # one more (untimed) step with the other exchange of B's norm-map shares, for the same check
        sh._push = False
        sh.run(tau)
        sh.sync()
        sampled_other, _ = grab_rows()
        sh._push = True
        sh.run(tau)
        sh.sync()

    # ---- per-phase times (same work, events between the phases; rank-local)
    phase = None
    if world == 1:
        acc = {}
        reps = max(3, min(args.steps, 10))
        for _ in range(reps):
            st = plan.run_timed(tau)
            for k, v in st.items():
                acc[k] = acc.get(k, 0.0) + v
        phase = {k: acc[k] / reps for k in ("ms_norm", "ms_lists", "ms_pack", "ms_multiply", "ms_device_total")}
        phase.update({k: int(st[k]) for k in ("steps", "packed_tiles_a", "packed_tiles_b")})
    elif sh._share is not None:
        acc = {}
        reps = max(3, min(args.steps, 10))
        exch = None
        for _ in range(reps):
            for k, v in sh.run_timed(tau).items():
                if isinstance(v, str):
                    exch = v
                else:
                    acc[k] = acc.get(k, 0.0) + v
        phase = {k: v / reps for k, v in acc.items()}      # rank 0's view
        phase["exchange"] = exch

    # ---- end to end through the public call with host buffers (pinned), every rank over its own PCIe link: its rows
    # of A and its share of B up, the shares exchanged over NVLink, its rows of C down
    e2e_steps = max(1, min(args.steps, 3))
    c_t, c_np = pinned((rows, n))
    if world == 1:
        bs_np = b_np
    else:
        r0, nrows = sh.b_rows()
        if rank == 0:
            bs_np = b_np[r0:r0 + nrows]
        else:
            bs_t, bs_np = pinned((nrows, n))
            generate_into(bs_np, SEED_B, r0, n)

    def e2e_step():
        sh.multiply(a_np, bs_np, tau, out=c_np)

    e2e_step()
    ms_e2e = timed(e2e_step, e2e_steps)
    # the host result of that call against the resident run's rows of C (same lists, same products)
    e2e_diff = 0.0
    for r in mine:
        lo = (r - sh.row_tile_begin) * TILE
        ref = sampled_c[r][0].astype(np.float64)
        den = float(np.linalg.norm(ref))
        d = float(np.linalg.norm(c_np[lo:lo + TILE].astype(np.float64) - ref))
        e2e_diff = max(e2e_diff, d / den if den else d)
    if world > 1:
        diffs = [None] * world
        dist.all_gather_object(diffs, e2e_diff)
        e2e_diff = max(diffs)

    # ---- the same with B uploaded by rank 0 alone and broadcast, and C gathered on rank 0 before it goes to the host
    ms_e2e_gather = None
    if world > 1:
        cf_t, _ = pinned((n, n)) if rank == 0 else (None, None)

        def e2e_gather_step():
            sh.distribute(a_np, b_np)
            sh.run(tau)
            full = sh.gather_c(0)
            if rank == 0:
                with torch.cuda.stream(stream):
                    cf_t.copy_(full, non_blocking=True)
                sh.sync()

        e2e_gather_step()
        ms_e2e_gather = timed(e2e_gather_step, max(1, min(e2e_steps, 2)))
        del cf_t
        sh.run(tau)
        sh.sync()

    # ---- the reference's comparator (run_cublas_time, tool.cu:153-224): the dense half GEMM of the library on the
    # same matrices, same box (fp16 in, fp32 accumulate), single GPU only
    dense_gemm = None
    if world == 1 and not args.no_sweep:
        with torch.cuda.stream(stream):
            a16 = plan.as_tensor(BUF_A).half()
            b16 = plan.as_tensor(BUF_B).half()
            for _ in range(3):
                c16 = torch.matmul(a16, b16)
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record(stream)
            for _ in range(5):
                c16 = torch.matmul(a16, b16)
            g1.record(stream)
        torch.cuda.synchronize()
        ms_gemm = g0.elapsed_time(g1) / 5
        dense_gemm = {"ms": ms_gemm, "tflops": 2.0 * n ** 3 / (ms_gemm * 1e-3) / 1e12,
                      "library": "cuBLAS through torch.matmul, fp16 inputs, fp16 output",
                      "spamm_speedup_over_dense": ms_gemm / ms_step}
        del a16, b16, c16
        torch.cuda.empty_cache()

    # ---- tau sweep (single GPU only; a few passes each)
    sweep = None
    if world == 1 and not args.no_sweep:
        sweep = []
        dense_c = None
        for t in SWEEP_TAUS:
            for _ in range(2):
                sh.run(t)
            sh.sync()
            reps = 3
            ms_t = timed(lambda: sh.run(t), reps)
            s_t = sh.survivors()
            st = plan.run_timed(t)
            if t == 0.0:
                dense_c = plan.as_tensor(BUF_C).clone()          # the dense product, kept for the error figures
            err = plan.error_norms(dense_c.data_ptr()) if dense_c is not None else None
            sweep.append({"tau": t, "ms": ms_t,
                          "err_vs_dense_rel_fro": (err[0] / err[1] if err and err[1] else None), "survivors": s_t,
                          "executed_fraction": s_t / T ** 3,
                          "executed_tflops": 65536.0 * s_t / (ms_t * 1e-3) / 1e12,
                          "ms_multiply": st["ms_multiply"], "ms_pack": st["ms_pack"], "ms_norm": st["ms_norm"],
                          "multiply_tflops": 65536.0 * s_t / (max(st["ms_multiply"], 1e-6) * 1e-3) / 1e12})
        del dense_c
        sh.run(tau)
        sh.sync()

    # ---- multi-GPU: the dense limit (tau = 0) beside the headline, where a step is milliseconds of tensor work
    dense_multi = None
    if world > 1 and not args.no_sweep:
        for _ in range(2):
            sh.run(0.0)
        sh.sync()
        ms_d = timed(lambda: sh.run(0.0), 3)
        s_d = sh.survivors()
        dense_multi = {"tau": 0.0, "ms": ms_d, "survivors": s_d, "executed_tflops": 65536.0 * s_d / (ms_d * 1e-3) / 1e12}
        sh.run(tau)
        sh.sync()

    ref_kernels = None
    if world == 1 and rank == 0 and not args.no_ref_kernels and not args.no_sweep:
        ref_kernels = time_reference_kernels(torch, lambda m: SpammPlan(m, m, m, device=local_rank))

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    value = 65536.0 * S / (ms_step * 1e-3) / 1e12
    line = {
        "metric": "spamm_executed_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16xf16+f32" if args.precision == "half" else "2xf16 split, 3 products, +f32",
        "data": "synthetic",
        "config": config_dict(n, tau, world, survivors=S, executed_fraction=S / T ** 3, partition=partition),
        "e2e": {"value": 65536.0 * S / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": 8 * n * n, "d2h_bytes_per_step": 4 * n * n, "steps": e2e_steps,
                "sampled_rows_rel_fro_vs_resident_run": e2e_diff,
                "path": ("spamm_multiply: B, then the rows of A in chunks, kernels and the rows of C overlapped" if world == 1
                         else "every rank, over its own PCIe link: its rows of A and 1/G of B up, the shares of B exchanged "
                              "over NVLink (NCCL all-gather), its rows of C down into its own pinned buffer; byte counts "
                              "are the totals over the ranks")},
        "gpu_launches": launches,
        "ms_per_step_min": ms_min,
        "host_issue_ms_per_step": host_issue_ms,
        "clocks": clocks,
    }
    if phase is not None and world > 1:
        line["phases_ms_rank0"] = phase
        # this rank's norm pass: its rows of A and its share of B, one launch
        share_rows = (sh._share or 0) * TILE
        norm_bytes = 4.0 * n * (rows + share_rows)
        ach = norm_bytes / (max(phase["ms_norm"], 1e-6) * 1e-3) / 1e9
        line["roofline"] = {"kernel": "norm_map_pair_kernel", "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"],
                            "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "traffic": None,
                            "peak_source": peaks["source"],
                            "note": "rank 0: 4*(its rows of A + its share of B's rows)*N bytes / the norm phase "
                                    "(norm launch + the small kernel that stores the share into the peers' maps)"}
        floor_ms = (norm_bytes + 4.0 * rows * n) / (peaks["hbm_gbs"] * 1e9) * 1e3
        line["hbm_floor_ms_per_rank"] = floor_ms
        line["cpu_baseline"] = {"see": "the n_gpus=1 line of the same run"}
    if dense_multi is not None:
        line["dense_tau0"] = dense_multi
    if dense_gemm is not None:
        line["dense_gemm"] = dense_gemm
    if ms_e2e_gather is not None:
        line["e2e_gather_on_rank0"] = {"value": 65536.0 * S / (ms_e2e_gather * 1e-3) / 1e12, "unit": "TFLOP/s",
                                       "ms_per_step": ms_e2e_gather,
                                       "note": "rank 0 uploads all of B and broadcasts it; C is gathered on rank 0 and "
                                               "copied to the host from there"}
    if phase is not None and world == 1:
        norm_bytes = 8.0 * n * n   # every float of A and of B read once
        # when the lists name most tiles the norm pass also writes every tile as half (2 bytes per element)
        converts_all = phase.get("packed_tiles_a", 0) + phase.get("packed_tiles_b", 0) == 2 * T ** 2 \
            and phase["ms_pack"] < 0.01
        if converts_all:
            norm_bytes += 4.0 * n * n
        achieved = norm_bytes / (phase["ms_norm"] * 1e-3) / 1e9
        ratio = None if converts_all else read_traffic_ratio()
        line["roofline"] = {"kernel": "norm_pack_pair_kernel" if converts_all else "norm_map_pair_kernel",
                            "bound": "hbm", "achieved": achieved,
                            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                            "traffic": (ratio * norm_bytes if ratio is not None else None),
                            "peak_source": peaks["source"],
                            "note": ("one launch per step reads A and B and writes both as half: achieved = "
                                     "6*(M*K+K*N) bytes / its duration" if converts_all else
                                     "one launch per step reads A and B: achieved = 4*(M*K+K*N) bytes / its duration")}
        line["phases_ms"] = phase
        # C is written either by the multiply kernel alone or, when few macro tiles have steps, by a memset that runs
        # beside the list build and the conversion plus the multiply of the busy macro tiles: one figure for both
        c_bytes = 4.0 * n * n
        ms_c = phase["ms_lists"] + phase["ms_pack"] + phase["ms_multiply"]
        line["c_write"] = {"bound": "hbm", "achieved": c_bytes / (ms_c * 1e-3) / 1e9, "unit": "GB/s",
                           "peak": peaks["hbm_gbs"], "frac": c_bytes / (ms_c * 1e-3) / 1e9 / peaks["hbm_gbs"],
                           "note": "4*M*N bytes / (lists + pack + multiply time): everything after the norm pass"}
        line["multiply_tensor"] = {"bound": "tensor", "achieved": 65536.0 * S / (phase["ms_multiply"] * 1e-3) / 1e12,
                                   "unit": "TFLOP/s", "peak": peaks["tflops_sustained"],
                                   "frac": 65536.0 * S / (phase["ms_multiply"] * 1e-3) / 1e12 / peaks["tflops_sustained"],
                                   "note": "executed flops / multiply phase, against the sustained dense figure"}
    if sweep is not None:
        line["tau_sweep"] = sweep
        dense = [s for s in sweep if s["tau"] == 0.0]
        if dense:
            line["dense_tensor"] = {"bound": "tensor", "achieved": dense[0]["multiply_tflops"], "unit": "TFLOP/s",
                                    "peak": peaks["tflops"], "frac": dense[0]["multiply_tflops"] / peaks["tflops"],
                                    "frac_of_sustained": dense[0]["multiply_tflops"] / peaks["tflops_sustained"],
                                    "vs_cublas_same_data": (dense_gemm["ms"] / dense[0]["ms_multiply"]
                                                            if dense_gemm else None),
                                    "note": "tau=0: every tile product executed; multiply phase of one step timed "
                                            "alone, so the burst figure is the denominator"}
    if ref_kernels is not None:
        line["ref_kernels"] = ref_kernels

    # ---- CPU checker: parity of the sampled rows (every world size and workload), and the host baseline (N=1 only)
    if not args.no_cpu:
        try:
            from oracle import oracle as O

            O.set_num_threads(os.cpu_count() or 1)
            B = np.ascontiguousarray(b_np)
            Bh = O.round_to_half(B)
            full = world == 1 and S * 32768.0 <= CPU_FULL_LIMIT
            # the sampled rows first
            dt_s, s_sample, C_sub = cpu_sampled(O, n, tau, B, Bh, tile_rows)
            s_gpu_sample = sum(sampled_c[r][1] for r in tile_rows)

            def rel(got):
                g = np.vstack([got[r][0] for r in tile_rows]).astype(np.float64)
                ref = C_sub.astype(np.float64)
                den = float(np.linalg.norm(ref))
                return float(np.linalg.norm(g - ref)) / den if den else float(np.linalg.norm(g - ref))

            parity = {"rows_checked": len(tile_rows) * TILE, "tile_rows": tile_rows,
                      "survivors_equal": s_sample == s_gpu_sample, "survivors_of_rows": s_sample,
                      "c_rel_fro": rel(sampled_c), "exchange": args.exchange if world > 1 else None}
            if sampled_other is not None:
                parity["other_exchange"] = {"exchange": "nccl", "c_rel_fro": rel(sampled_other),
                                            "survivors_equal": sum(sampled_other[r][1] for r in tile_rows) == s_sample}
            if full:
                A = np.empty((n, n), dtype=np.float32)
                generate_into(A, SEED_A, 0, n)
                Ah = O.round_to_half(A)
                cpu_step(O, A[:1024], B, Ah[:1024], Bh, tau)   # page in, spin up the threads
                dt, s_cpu, c_cpu = cpu_step(O, A, B, Ah, Bh, tau)
                line["cpu_baseline"] = {"value": 65536.0 * s_cpu / dt / 1e12, "unit": "TFLOP/s",
                                        "cores": O.num_threads(), "kind": "port", "ms": dt * 1e3,
                                        "sample": "whole workload, one pass (norm maps + lists + gated product, "
                                                  "inputs pre-rounded to half)"}
                num = float(np.linalg.norm((c_np - c_cpu).astype(np.float64)))
                den = float(np.linalg.norm(c_cpu.astype(np.float64)))
                parity.update({"survivors_equal": parity["survivors_equal"] and s_cpu == S, "survivors_total": s_cpu,
                               "c_rel_fro_whole_matrix": num / den if den else num,
                               "whole_matrix_from": "the end-to-end call's host result"})
            else:
                # the total count: the checker's list lengths on norm maps of all rows (generated block by block)
                nB = O.norm_map(B)
                s_total, blk = 0, 64
                buf = np.empty((blk * TILE, n), dtype=np.float32)
                for t0 in range(0, T, blk):
                    tn = min(blk, T - t0)
                    generate_into(buf[:tn * TILE], SEED_A, t0 * TILE, n)
                    s_total += int(O.lists(O.norm_map(buf[:tn * TILE]), nB, tau)[1][-1])
                parity.update({"survivors_equal": parity["survivors_equal"] and s_total == S,
                               "survivors_total": s_total})
                if world == 1:
                    line["cpu_baseline"] = {"value": 65536.0 * s_sample / dt_s / 1e12, "unit": "TFLOP/s",
                                            "cores": O.num_threads(), "kind": "port", "ms": dt_s * 1e3,
                                            "sample": f"{len(tile_rows)} of {T} C tile rows, one pass (norm map of those "
                                                      f"rows of A and of all of B, lists, gated product); value = "
                                                      f"executed flops of the sample / its time"}
            line["parity"] = parity
        except Exception as e:  # the baseline is a report, never a reason to lose the GPU numbers
            line["cpu_baseline"] = {"error": repr(e)}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="exp", choices=sorted(WORKLOADS))
    ap.add_argument("--n", type=int, default=None)
    ap.add_argument("--tau", type=float, default=None)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-ref-kernels", action="store_true",
                    help="skip timing the reference's own kernels (N=8192) beside the library")
    ap.add_argument("--precision", default="half", choices=["half", "split"],
                    help="half: the metric's configuration; split: the float-accuracy mode (three tensor-core passes)")
    ap.add_argument("--multiply-mode", default="auto", choices=["auto", "one_sm", "gated_pairs"],
                    help="which multiply kernels may run (auto: chosen from the counters of the previous step)")
    ap.add_argument("--partition", default="auto", choices=["auto", "even", "balanced"],
                    help="row blocks of C per GPU: even (the reference's), or moved so that the surviving products "
                         "are spread evenly (auto: only when that lowers the largest block's work by more than 3 %%)")
    ap.add_argument("--exchange", default="push", choices=["push", "nccl"],
                    help="multi-GPU: how B's norm-map shares travel (peer stores by a small kernel, or NCCL all-gather)")
    args = ap.parse_args()
    WORKLOAD[0] = args.workload
    if args.n is None:
        args.n = WORKLOADS[args.workload][1]
    if args.tau is None:
        args.tau = WORKLOADS[args.workload][2]
    if args.workload != "exp":
        args.no_sweep = True          # the tau sweep belongs to the headline workload
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
