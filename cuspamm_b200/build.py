"""Builds libspamm.so (sm_100a only) next to this file with nvcc.

Usage: ``python -m cuspamm_b200.build`` or ``cuspamm_b200.build.build_library()``.
The library is built in-tree so that it travels with the source tree to a GPU machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libspamm.so"
SOURCES = ["norm_map.cu", "skip_lists.cu", "pack_half.cu", "gated_multiply.cu", "gated_multiply_pair.cu", "gated_multiply_gpair.cu", "plan.cu", "group.cu", "extras.cu",
           "generators.cpp"]
HEADERS = [CSRC / "common.cuh", CSRC / "tc_utils.cuh", CSRC / "plan.cuh", PKG_DIR.parent / "include" / "spamm.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-O3,-Wall",
    "--fmad=true",
]


class NvccMissing(RuntimeError):
    pass


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise NvccMissing("nvcc not found; libspamm.so cannot be built")
    return exe


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compiles every source in csrc/ for sm_100a and links libspamm.so. Returns its path."""
    srcs = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    if not force and not _stale(LIB_PATH, list(srcs) + HEADERS):
        return LIB_PATH
    _nvcc()
    build_dir = PKG_DIR / "build"
    build_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for s in srcs:
        obj = build_dir / (s.name + ".o")
        objs.append(obj)
        if not force and not _stale(obj, [s] + HEADERS):
            continue
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(s), "-o", str(obj)]
        if ptxas_info and s.suffix == ".cu":
            cmd[1:1] = ["-Xptxas", "-v"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        procs.append((s, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for s, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s.name}:\n{out}")
        if (verbose or ptxas_info) and out.strip():
            print(out, file=sys.stderr)
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return LIB_PATH


GEN_LIB_PATH = PKG_DIR / "libspamm_gen.so"


def build_generators(force: bool = False) -> Path:
    """Builds the host-side input generators alone (g++, no CUDA) into libspamm_gen.so: what a process that only
    needs input matrices loads, e.g. the benchmark's CPU arm, which must not map the GPU library."""
    src = CSRC / "generators.cpp"
    header = PKG_DIR.parent / "include" / "spamm.h"
    if not force and not _stale(GEN_LIB_PATH, [src, header]):
        return GEN_LIB_PATH
    gxx = shutil.which("g++")
    if not gxx:
        if GEN_LIB_PATH.exists():
            return GEN_LIB_PATH
        raise RuntimeError("g++ not found; libspamm_gen.so cannot be built")
    cmd = [gxx, "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", str(src), "-o", str(GEN_LIB_PATH)]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"generator build failed:\n{r.stdout}")
    return GEN_LIB_PATH


def build_driver(verbose: bool = False) -> Path:
    """Builds the command-line driver `spamm_main` (same shape as the reference's `main`) against libspamm.so."""
    build_library()
    out = PKG_DIR / "spamm_main"
    src = CSRC / "spamm_main.cpp"
    if not _stale(out, [src, LIB_PATH] + HEADERS):
        return out
    cmd = [_nvcc(), "-O2", "-std=c++17", str(src), "-o", str(out), f"-L{PKG_DIR}", "-lspamm", "-lcudart",
           "-Xlinker", f"-rpath={PKG_DIR}", "-Xlinker", "-rpath=$ORIGIN"]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"driver build failed:\n{r.stdout}")
    return out


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(path)
    print(build_generators(force="--force" in sys.argv))
    print(build_driver(verbose=True))
