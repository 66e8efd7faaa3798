"""Build the two shared objects of the library with nvcc for sm_100a.

Counterpart of the reference's harness/build_so.py:25-26 (one `nvcc -shared` of the lib
source, written where the Python side ctypes-loads it). Here the output stays in-tree,
next to the sources:

    quadbit_b200/libquadbit_sparse_fp4.so    reference: /cache/sparse_fp4.so
    quadbit_b200/libquadbit_dense_nvfp4.so   reference: dense_nvfp4.so

Both come from the same translation units; the dense flavour only changes which block
size the shared symbol `quantize_act_nvfp4_2lvl` uses (per-16 instead of per-32), as the
reference's two libraries do. The CUDA runtime is linked statically and the driver API is
reached through cudaGetDriverEntryPoint, so the objects load on a machine without a GPU.

    python -m quadbit_b200.build_so [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
SOURCES = ["qb_abi.cu", "qb_quant.cu", "qb_compress.cu", "qb_gemm.cu", "qb_moe.cu", "qb_noalloc.cu", "qb_peak.cu", "qb_syncprobe.cu"]
HEADERS = ["qb_common.cuh", "qb_internal.h"]
FLAVOURS = {"sparse_fp4": [], "dense_nvfp4": ["-DQB_FLAVOUR_DENSE"]}
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-shared",
              "-Xcompiler", "-fPIC", "--cudart", "static"]


def so_path(flavour: str) -> Path:
    return PKG / f"libquadbit_{flavour}.so"


def _stale(target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    deps = [CSRC / f for f in SOURCES + HEADERS] + [PKG.parent / "include" / "quadbit_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    nvcc = os.environ.get("NVCC", "nvcc")
    out = {}
    procs = []
    for flavour, defs in FLAVOURS.items():
        target = so_path(flavour)
        out[flavour] = target
        if not force and not _stale(target):
            continue
        extra = os.environ.get("QB_NVCC_EXTRA", "").split()     # developer hook, e.g. -DQB_EXPERIMENT
        cmd = [nvcc, *NVCC_FLAGS, *defs, *extra, "-o", str(target), *[str(CSRC / s) for s in SOURCES]]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((flavour, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for flavour, p in procs:
        log, _ = p.communicate()
        if verbose or p.returncode != 0:
            print(log, flush=True)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed for {flavour} (exit {p.returncode})")
    return out


if __name__ == "__main__":
    paths = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    for k, v in paths.items():
        print(f"# built {v} ({v.stat().st_size} bytes)")
