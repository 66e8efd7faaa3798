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

import fcntl
import hashlib
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
SOURCES = ["qb_abi.cu", "qb_quant.cu", "qb_compress.cu", "qb_gemm.cu", "qb_moe.cu", "qb_noalloc.cu", "qb_peak.cu", "qb_peer.cu", "qb_glue.cu", "qb_ep.cu", "qb_gemv.cu"]
HEADERS = ["qb_common.cuh", "qb_internal.h"]
FLAVOURS = {"sparse_fp4": [], "dense_nvfp4": ["-DQB_FLAVOUR_DENSE"]}
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC"]
LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "--cudart", "static"]
FLAVOURED = {"qb_abi.cu"}          # the only translation unit that reads the flavour macro
OBJ = PKG / "build"


def so_path(flavour: str) -> Path:
    return PKG / f"libquadbit_{flavour}.so"


def _deps() -> list[Path]:
    return [CSRC / f for f in SOURCES + HEADERS] + [PKG.parent / "include" / "quadbit_b200.h"]


def _digest(paths, extra=()) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    for e in extra:
        h.update(str(e).encode())
    return h.hexdigest()


def _stamp(target: Path) -> Path:
    return target.with_name(target.name + ".srchash")


def _stale(target: Path) -> bool:
    """A library is current when the digest of the sources it was built from (stored beside it) matches the
    sources now; file times are not trusted (a copied tree has arbitrary ones)."""
    st = _stamp(target)
    if not target.exists() or not st.exists():
        return True
    return st.read_text().strip() != _digest(_deps(), NVCC_FLAGS + LINK_FLAGS)


def _obj_stale(obj: Path, src: Path, defs) -> bool:
    st = _stamp(obj)
    if not obj.exists() or not st.exists():
        return True
    hdrs = [CSRC / h for h in HEADERS] + [PKG.parent / "include" / "quadbit_b200.h"]
    return st.read_text().strip() != _digest([src] + hdrs, NVCC_FLAGS + list(defs))


def build(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    """One object per translation unit (compiled in parallel, shared by the two flavours except qb_abi.cu),
    then one link per flavour. Only stale objects are recompiled."""
    nvcc = os.environ.get("NVCC", "nvcc")
    out = {f: so_path(f) for f in FLAVOURS}
    if not force and not any(_stale(t) for t in out.values()):
        return out
    OBJ.mkdir(exist_ok=True)
    with open(OBJ / ".lock", "w") as lock:           # one builder at a time (ranks of a multi-process launch)
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not any(_stale(t) for t in out.values()):
            return out
        return _build_locked(nvcc, out, force, verbose)


def _build_locked(nvcc, out, force, verbose):
    jobs, objs = [], {f: [] for f in FLAVOURS}
    for src in SOURCES:
        variants = [(f, FLAVOURS[f]) for f in FLAVOURS] if src in FLAVOURED else [(None, [])]
        for flavour, defs in variants:
            obj = OBJ / (src.replace(".cu", "") + (f".{flavour}" if flavour else "") + ".o")
            for f in FLAVOURS:
                if flavour in (None, f):
                    objs[f].append(obj)
            if force or _obj_stale(obj, CSRC / src, defs):
                cmd = [nvcc, *NVCC_FLAGS, *defs, "-c", "-o", str(obj), str(CSRC / src)]
                if verbose:
                    cmd[1:1] = ["-Xptxas", "-v"]
                    print(" ".join(cmd), flush=True)
                hdrs = [CSRC / h for h in HEADERS] + [PKG.parent / "include" / "quadbit_b200.h"]
                jobs.append((src, obj, _digest([CSRC / src] + hdrs, NVCC_FLAGS + list(defs)), subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, obj, dig, p in jobs:
        log, _ = p.communicate()
        if verbose or p.returncode != 0:
            print(log, flush=True)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src} (exit {p.returncode})")
        _stamp(obj).write_text(dig)
    for flavour, target in out.items():
        cmd = [nvcc, *LINK_FLAGS, "-o", str(target), *[str(o) for o in objs[flavour]]]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            print(r.stdout, flush=True)
            raise RuntimeError(f"link failed for {flavour} (exit {r.returncode})")
        _stamp(target).write_text(_digest(_deps(), NVCC_FLAGS + LINK_FLAGS))
    return out


if __name__ == "__main__":
    paths = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    for k, v in paths.items():
        print(f"# built {v} ({v.stat().st_size} bytes)")
