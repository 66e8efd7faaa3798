"""Linear-method hook for a serving engine, the counterpart of the reference's vLLM plugin patch
(harness/qb_vllm_plugin/qb_sm120_plugin.py:1466-1534): the engine's linear method keeps its class and
its callers; `process_weights_after_loading(layer)` additionally packs the loaded weight once into the
two-level NVFP4 form, and `apply(layer, x, bias)` runs quantise + GEMM on it.

Nothing here imports the engine: `install()` takes the method class to patch (for vLLM that is e.g.
`vllm.model_executor.layers.linear.UnquantizedLinearMethod`), `install_vllm()` resolves that class by
name and fails loudly if the engine is not importable. There is no fallback to the engine's own GEMM for
layers that were packed; layers whose shape the kernels do not take (out or in not a multiple of 128)
are left to the engine and counted in STATS."""
from __future__ import annotations

from typing import Callable

import torch

STATS = {"sparse_layers": 0, "dense_layers": 0, "native_layers": 0, "calls": 0}


def _default_factory(mode: str) -> Callable[[torch.Tensor], object]:
    from .linear import DenseNVLinear, QuadbitLinear
    return (lambda w: QuadbitLinear(w, keep_ref_layout=False)) if mode == "sparse" else (lambda w: DenseNVLinear(w, keep_ref_layout=False))


def supported(weight: torch.Tensor) -> bool:
    return weight.dim() == 2 and weight.shape[0] % 128 == 0 and weight.shape[1] % 128 == 0


def install(method_cls, mode: str = "sparse", factory: Callable[[torch.Tensor], object] | None = None,
            select: Callable[[object], bool] | None = None):
    """Patch `method_cls.process_weights_after_loading` and `method_cls.apply` in place.

    mode: "sparse" (2:4-sparse two-level NVFP4, the reference's QuadbitLinear) or "dense".
    factory: weight [out, in] -> module with .forward(x); default builds QuadbitLinear / DenseNVLinear.
    select: layer -> bool, which layers to take (default: every layer with a supported 2-D weight).
    Returns a function that restores the original methods."""
    if mode not in ("sparse", "dense"):
        raise ValueError(f"mode {mode!r}")
    make = factory or _default_factory(mode)
    orig_pw = getattr(method_cls, "process_weights_after_loading", None)
    orig_apply = method_cls.apply

    def patched_pw(self, layer):
        if orig_pw is not None:
            orig_pw(self, layer)             # the engine's own bookkeeping first, as the reference plugin does
        w = getattr(layer, "weight", None)
        w = getattr(w, "data", w)
        if w is None or not supported(w) or (select is not None and not select(layer)):
            STATS["native_layers"] += 1
            return None
        layer._qb_linear = make(w)
        STATS["sparse_layers" if mode == "sparse" else "dense_layers"] += 1
        return None

    def patched_apply(self, layer, x, bias=None):
        lin = getattr(layer, "_qb_linear", None)
        if lin is None:
            return orig_apply(self, layer, x, bias)
        STATS["calls"] += 1
        out = lin.forward(x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16))
        out = out.to(x.dtype)
        return out + bias if bias is not None else out

    method_cls.process_weights_after_loading = patched_pw
    method_cls.apply = patched_apply

    def restore():
        if orig_pw is None:
            del method_cls.process_weights_after_loading
        else:
            method_cls.process_weights_after_loading = orig_pw
        method_cls.apply = orig_apply

    return restore


def install_vllm(mode: str = "sparse", method: str = "vllm.model_executor.layers.linear.UnquantizedLinearMethod", **kw):
    """Resolve a vLLM linear-method class by dotted name and patch it (raises ImportError without vLLM)."""
    import importlib
    mod_name, cls_name = method.rsplit(".", 1)
    cls = getattr(importlib.import_module(mod_name), cls_name)
    return install(cls, mode=mode, **kw)


def install_moe(method_cls, fmt: str = "mxfp4", act: str = "gptoss", fixed_capacity: bool = True,
                select: Callable[[object], bool] | None = None, release: bool = False):
    """Patch a fused-MoE method class the way the reference patches `GptOssMxfp4MoEMethod`
    (harness/qb_vllm_plugin/qb_sm120_plugin.py:2086-2498): after the engine's own
    `process_weights_after_loading(layer)`, the expert tensors of the layer are dequantised on the GPU, pruned 2:4 and
    packed once into a `SparseMoE`; `apply(layer, x, topk_weights, topk_ids, ...)` then runs the routed layer on it.

    fmt "mxfp4": `layer.w13_weight` [E, 2I, H/2] u8 + `layer.w13_weight_scale` [E, 2I, H/32] e8m0 with gate / up rows
    interleaved, `layer.w2_weight` [E, H, I/2] + `layer.w2_weight_scale` [E, H, I/32] (gpt-oss checkpoints);
    fmt "bf16": `layer.w13_weight` [E, 2I, H] (gate rows then up rows) and `layer.w2_weight` [E, H, I] as they are.
    `layer.w13_bias` [E, 2I] (same row order as the weight) and `layer.w2_bias` [E, H], when present, are applied in the
    epilogues of the grouped GEMMs as the reference does (qb_sm120_plugin.py:2192-2225, 2397-2400). An `expert_map`
    (expert-parallel engines passing local ids) is not supported and raises. The engine's expert tensors are released
    after packing when `release=True`. Layers that `select` rejects stay on the engine's path. Returns a function that
    restores the original methods."""
    if fmt not in ("mxfp4", "bf16"):
        raise ValueError(f"fmt {fmt!r}")
    from . import checkpoint as ck
    from .moe import SparseMoE
    orig_pw = getattr(method_cls, "process_weights_after_loading", None)
    orig_apply = method_cls.apply
    STATS.setdefault("moe_layers", 0)
    STATS.setdefault("moe_calls", 0)

    def patched_pw(self, layer):
        if orig_pw is not None:
            orig_pw(self, layer)
        if select is not None and not select(layer):
            STATS["native_layers"] += 1
            return None
        w13 = getattr(layer.w13_weight, "data", layer.w13_weight)
        w2 = getattr(layer.w2_weight, "data", layer.w2_weight)
        n_e = w13.shape[0]
        gus, dns = [], []
        for e in range(n_e):
            if fmt == "mxfp4":
                s13 = getattr(layer.w13_weight_scale, "data", layer.w13_weight_scale)
                s2 = getattr(layer.w2_weight_scale, "data", layer.w2_weight_scale)
                gate, up = ck.split_interleaved_gate_up(ck.mxfp4_to_bf16(w13[e], s13[e]))
                gus.append(torch.cat([gate, up], 0))
                dns.append(ck.mxfp4_to_bf16(w2[e], s2[e]))
            else:
                gus.append(w13[e].to(torch.bfloat16))
                dns.append(w2[e].to(torch.bfloat16))
        b13 = getattr(layer, "w13_bias", None)
        b2 = getattr(layer, "w2_bias", None)
        bgu = bdn = None
        if b13 is not None:
            b13 = getattr(b13, "data", b13)
            if fmt == "mxfp4":      # interleaved like the weight rows: gate = even, up = odd
                bgu = [torch.cat([b13[e][0::2], b13[e][1::2]], 0) for e in range(n_e)]
            else:
                bgu = [b13[e] for e in range(n_e)]
        if b2 is not None:
            b2 = getattr(b2, "data", b2)
            bdn = [b2[e] for e in range(n_e)]
        layer._qb_moe = SparseMoE(gus, dns, topk=1, act=act, fixed_capacity=fixed_capacity, b_gate_up=bgu, b_down=bdn)
        if release:                  # the packed copy replaces the engine's expert tensors
            for name in ("w13_weight", "w2_weight", "w13_weight_scale", "w2_weight_scale"):
                t = getattr(layer, name, None)
                if t is not None:
                    getattr(t, "data", t).set_(torch.empty(0, dtype=getattr(t, "data", t).dtype, device=getattr(t, "data", t).device))
        STATS["moe_layers"] += 1
        return None

    def patched_apply(self, layer, x, topk_weights, topk_ids, *args, **kw):
        moe = getattr(layer, "_qb_moe", None)
        if moe is None:
            return orig_apply(self, layer, x, topk_weights, topk_ids, *args, **kw)
        if kw.get("expert_map") is not None:
            raise NotImplementedError("install_moe: expert_map (engine-side expert parallelism) is not supported; "
                                      "use SparseMoE(expert_range=...) / forward_ep")
        STATS["moe_calls"] += 1
        moe.topk = topk_ids.shape[1]
        y = moe.forward(x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16), topk_ids, topk_weights)
        return y.to(x.dtype)

    method_cls.process_weights_after_loading = patched_pw
    method_cls.apply = patched_apply

    def restore():
        if orig_pw is None:
            del method_cls.process_weights_after_loading
        else:
            method_cls.process_weights_after_loading = orig_pw
        method_cls.apply = orig_apply

    return restore
