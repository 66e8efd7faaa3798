"""ctypes binding of the two shared objects (the reference binds its .so the same way:
harness/quadbit_linear.py:51-63, harness/qb_vllm_plugin/qb_sm120_plugin.py:1124-1153).

There is no fallback: if the library cannot be built or loaded, import-time users get an
exception; nothing in this package computes on the CPU."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from functools import lru_cache

from . import build_so

P, I = c_void_p, c_int

_SIGS = {
    # reference symbols
    "sparse_fp4_mm": ([P] * 6 + [I] * 3, I),
    "sparse_fp4_mm_2lvl": ([P] * 6 + [I] * 3 + [P] * 2, I),
    "sparse_fp4_mm_2lvl_t": ([P] * 6 + [I] * 3 + [P] * 2, I),
    "quantize_act_nvfp4": ([P] * 3 + [I] * 2, None),
    "quantize_act_nvfp4b": ([P] * 3 + [I] * 2, None),
    "quantize_act_nvfp4_2lvl": ([P] * 4 + [I] * 2, None),
    "quantize_act_nvfp4_2lvl_s": ([P] * 4 + [I] * 2 + [P], None),
    "sparse_down_sk_2lvl": ([P] * 7 + [I] * 3 + [P] * 2 + [I], I),
    "sparse_moe_mm_2lvl": ([P] * 6 + [I] * 4 + [P] * 3 + [I, P], I),
    "sparse_moe_mm_2lvl_bw": ([P] * 6 + [I] * 4 + [P] * 5 + [I, P], I),
    "sparse_moe_mm_2lvl_scatter": ([P] * 5 + [I] * 4 + [P] * 7 + [I, P], I),
    "sparse_moe_gu_swiglu": ([P] * 5 + [I] * 4 + [P] * 6 + [I, I, P], I),
    "rmsnorm_nvfp4": ([P] * 6 + [I] * 2 + [c_float], None),
    "swiglu_nvfp4": ([P] * 4 + [I] * 2, None),
    "moe_route": ([P] * 4 + [I] * 2 + [P], I),
    "moe_combine_topk": ([P] * 3 + [I] * 4 + [P], I),
    "qb_init_func_attrs": ([], None),
    "qb_init_sk_attrs": ([], None),
    "qb_init_moe_attrs": ([], None),
    "qb_init_gusw_attrs": ([], None),
    "dense_nvfp4_mm": ([P] * 5 + [I] * 3 + [P] * 2, I),
    # native
    "qb_quantize_act": ([P] * 5 + [I] * 3 + [P], I),
    "qb_moe_route_fixed": ([P] * 4 + [I] * 3 + [P], I),
    "qb_moe_route_fixed_ex": ([P] * 4 + [I] * 4 + [P] * 4, I),
    "qb_gather_quantize_act": ([P] * 6 + [I] * 4 + [P], I),
    "qb_swiglu_quant_act": ([P] * 7 + [I] * 4 + [P], I),
    "qb_compress_2to4": ([P, I] + [P] * 6 + [I] * 2 + [P], I),
    "qb_compress_2to4_colnorm": ([P, I] + [P] * 7 + [I] * 2 + [P], I),
    "qb_dequant_fp4_blocks": ([P] * 4 + [I] * 3 + [c_longlong, P], I),
    "qb_pack_dense": ([P, I] + [P] * 4 + [I] * 2 + [P], I),
    "qb_relayout_sf": ([P] * 2 + [I] * 3 + [P], I),
    "qb_relayout_meta": ([P] * 2 + [I] * 2 + [P], I),
    "qb_sf_atoms_bytes": ([I] * 3, c_longlong),
    "qb_meta_native_bytes": ([I] * 2, c_longlong),
    "qb_gemm": ([P] * 12 + [I] * 8 + [P], I),
    "fused_swiglu_quant": ([P] * 4 + [I] * 2, None),
    "fused_swiglu_quant_2lvl": ([P] * 5 + [I] * 2, None),
    "rmsnorm_quant": ([P] * 4 + [I] * 2 + [c_float], None),
    "add_rmsnorm_quant": ([P] * 6 + [I] * 2 + [c_float], None),
    "qb_norm_quant": ([P] * 8 + [I] * 2 + [c_float, I, P], I),
    "fused_mlp_2lvl": ([P] * 17 + [I] * 5 + [P], I),
    "fused_mlp_2lvl_skdown": ([P] * 18 + [I] * 6 + [P], I),
    "qb_swiglu_quant": ([P] * 5 + [I] * 2 + [P], I),
    "qb_fused_mlp": ([P] * 18 + [I] * 7 + [P], I),
    "qb_gemm_decode": ([P] * 9 + [I] * 5 + [P], I),
    "qb_tile_weights": ([P] * 2 + [I] * 3 + [P], I),
    "qb_tiled_weight_bytes": ([I] * 3, c_longlong),
    "qb_gemm_decode_ws_bytes": ([I] * 3, c_longlong),
    "qb_linear_gemv": ([P] * 5 + [I] * 3 + [P], I),
    "qb_gemm_splitk_static": ([P] * 8 + [I] * 6 + [P], I),
    "qb_gemm_splitk_static_max_elems": ([], c_longlong),
    "qb_peer_alloc": ([P, c_longlong], I),
    "qb_peer_free": ([P], I),
    "qb_peer_export": ([P, P], I),
    "qb_peer_open": ([P, P], I),
    "qb_peer_close": ([P], I),
    "qb_peer_signal": ([P, I, I, I, P, P], I),
    "qb_ep_publish": ([P, P, c_longlong, P, P, I, I, P, P, I, I, P, P, P, P], I),
    "qb_moe_route_fixed_range": ([P] * 4 + [I] * 6 + [P] * 5, I),
    "qb_quantize_rows": ([P] * 4 + [I] * 4 + [P], I),
    "qb_gather_quantized": ([P] * 3 + [I, c_longlong] + [P] * 4 + [I] * 2 + [P] * 2, I),
    "qb_gather_quantize_act_peer": ([P, I, c_longlong] + [P] * 4 + [I] * 4 + [P, P], I),
    "qb_ep_combine": ([P] * 4 + [I] * 7 + [P], I),
    "qb_peer_wait": ([P, I, I, P, P], I),
    "qb_epoch_add": ([P, I, P], I),
    "qb_peer_status": ([P], I),
    "qb_gemm_rs": ([P] * 10 + [I] * 8 + [P, I, P], I),
    "qb_reduce_norm_quant": ([P, c_longlong, I] + [P] * 6 + [I] * 5 + [c_float, I, P, I, P, I, I, I, P, P, P], I),
    "qb_gemm_swiglu": ([P] * 12 + [I] * 6 + [P], I),
    "dense_fp4_mm": ([P] * 3 + [I] * 3, I),
    "dense_fp4_mm_sk": ([P] * 4 + [I] * 4, I),
    "qb_decode_tn": ([I], I),
    "dense_fp4_decode": ([P] * 3 + [I] * 3, I),
    "qb_encode_map": ([P, I, I, I], P),
    "qb_free_map": ([P], None),
    "dense_fp4_decode_cached": ([P] * 3 + [I] * 3, I),
    "dense_fp4_decode_cached_async": ([P] * 3 + [I] * 3, None),
    "sparse_fp4_mm_sk": ([P] * 7 + [I] * 4, I),
    "qb_register_weight": ([P, P, I, I, I, P], I),
    "qb_forget_weight": ([P], I),
    "qb_rope_inplace": ([P, P, I, I, c_longlong, I, P], I),
    "qb_mma_peak": ([I] * 4 + [P] * 3, I),
    "qb_status": ([P], I),
    "qb_last_error": ([], I),
    "qb_version": ([], ctypes.c_char_p),
}

EXPORTED = tuple(_SIGS)


@lru_cache(maxsize=None)
def load(flavour: str = "sparse_fp4") -> ctypes.CDLL:
    """Build (if stale or missing) and load libquadbit_<flavour>.so with argtypes set."""
    if flavour not in build_so.FLAVOURS:
        raise ValueError(f"unknown library flavour {flavour!r}")
    path = build_so.so_path(flavour)
    build_so.build()                 # recompiles only what is older than its sources
    lib = ctypes.CDLL(str(path))
    for name, (argtypes, restype) in _SIGS.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is missing
        fn.argtypes = argtypes
        fn.restype = restype
    return lib


class QuadbitError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise QuadbitError(f"{what} failed with code {rc}")
