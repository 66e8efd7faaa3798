"""The C-ABI boundary without a GPU: both shared objects load, export every function that
include/quadbit_b200.h declares, and the ctypes signatures used by the package agree with the
header's parameter counts. No compute entry point is called."""
import ctypes
import os
import re

import pytest

from quadbit_b200 import _lib, build_so

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "quadbit_b200.h")
DECL = re.compile(r"^\s*(?:const\s+char\s*\*|long\s+long|int|void\s*\*|void)\s*(\w+)\s*\(([^;{]*)\)\s*;", re.M | re.S)


def declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for name, params in DECL.findall(text):
        params = params.strip()
        out[name] = 0 if params in ("", "void") else params.count(",") + 1
    return out


@pytest.fixture(scope="module")
def libs():
    for flavour in build_so.FLAVOURS:
        if not build_so.so_path(flavour).exists():
            build_so.build()
            break
    return {f: ctypes.CDLL(str(build_so.so_path(f))) for f in build_so.FLAVOURS}


def test_header_declares_something():
    d = declared()
    assert len(d) >= 40
    for must in ("qb_gemm", "qb_quantize_act", "qb_compress_2to4", "sparse_fp4_mm_2lvl_t", "dense_nvfp4_mm", "moe_route"):
        assert must in d


def test_every_declared_symbol_is_exported(libs):
    for flavour, lib in libs.items():
        missing = [n for n in declared() if not hasattr(lib, n)]
        assert not missing, (flavour, missing)


def test_binding_table_matches_header():
    d = declared()
    undeclared = [n for n in _lib.EXPORTED if n not in d]
    assert not undeclared, undeclared
    unbound = [n for n in d if n not in _lib._SIGS]
    assert not unbound, unbound
    wrong = {n: (len(_lib._SIGS[n][0]), d[n]) for n in d if len(_lib._SIGS[n][0]) != d[n]}
    assert not wrong, wrong


def test_no_gpu_entry_points_answer(libs):
    lib = libs["sparse_fp4"]
    lib.qb_version.restype = ctypes.c_char_p
    assert lib.qb_version().decode().startswith("quadbit_b200")
    lib.qb_sf_atoms_bytes.restype = ctypes.c_longlong
    lib.qb_meta_native_bytes.restype = ctypes.c_longlong
    # 128 rows x 256 K: one 128x4 atom per 64 (dense, per-16) or 128 (sparse, per-32) K
    assert lib.qb_sf_atoms_bytes(128, 256, 16) == 4 * 512
    assert lib.qb_sf_atoms_bytes(128, 256, 32) == 2 * 512
    assert lib.qb_meta_native_bytes(128, 256) == 128 * 16
    lib.qb_gemm_splitk_static_max_elems.restype = ctypes.c_longlong
    assert lib.qb_gemm_splitk_static_max_elems() == 2 * 1024 * 1024
