"""Fused 2:4-sparse SwiGLU MLP: the reference's `quadbit::fused_mlp` path
(harness/quadbit_serve.py:394-455: gate_up QBSparse + down QBSparse driven through one ctypes
call, fused_mlp_2lvl / fused_mlp_2lvl_skdown for tok <= 128).

Here one call to qb_fused_mlp launches four kernels on the current stream: quantise x,
gate/up GEMM (token-major), SwiGLU + two-level quantise, down GEMM. No padding to 128 tokens,
no host synchronisation; scratch comes from torch's caching allocator, so the call can be
captured in a CUDA graph after one warm-up call."""
from __future__ import annotations

import torch

from ._lib import check, load
from .linear import QuadbitLinear, _ptr, _stream


class FusedSparseMLP:
    """y = down( quant( silu(gate(x)) * up(x) ) ) with 2:4-sparse two-level NVFP4 weights.

    w_gate_up: [2*I, H] (gate rows first, as the reference concatenates them,
    harness/quadbit_linear.py:226), w_down: [H_out, I]."""

    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor, sk_splits: int = 8, sk_max_tok: int = 128):
        self.gu = QuadbitLinear(w_gate_up, keep_ref_layout=False)
        self.dn = QuadbitLinear(w_down, keep_ref_layout=False)
        assert self.gu.out_f == 2 * self.dn.in_f, "gate_up rows must be 2 * down in-features"
        self.lib = load("sparse_fp4")
        self.H, self.I, self.out_f = self.gu.in_f, self.dn.in_f, self.dn.out_f
        self.sk_splits, self.sk_max_tok = sk_splits, sk_max_tok

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.H).to(torch.bfloat16).contiguous()
        tok = x2.shape[0]
        dev = x2.device
        lib, H, I = self.lib, self.H, self.I
        u8 = torch.uint8
        Bb = torch.empty((tok, H // 2), dtype=u8, device=dev)
        sfx = torch.empty(lib.qb_sf_atoms_bytes(tok, H, 32), dtype=u8, device=dev)
        gBx = torch.empty((tok,), dtype=torch.float32, device=dev)
        Cgu = torch.empty((tok, 2 * I), dtype=torch.bfloat16, device=dev)
        Hb = torch.empty((tok, I // 2), dtype=u8, device=dev)
        sfh = torch.empty(lib.qb_sf_atoms_bytes(tok, I, 32), dtype=u8, device=dev)
        gH = torch.empty((tok,), dtype=torch.float32, device=dev)
        Cout = torch.empty((tok, self.out_f), dtype=torch.bfloat16, device=dev)
        splits = self.sk_splits if (tok <= self.sk_max_tok and self.sk_splits > 1) else 1
        Cf = torch.empty((tok, self.out_f), dtype=torch.float32, device=dev) if splits > 1 else None
        gu, dn = self.gu, self.dn
        check(lib.qb_fused_mlp(x2.data_ptr(), gu.At.data_ptr(), gu.sfa.data_ptr(), gu.meta_native.data_ptr(), gu.gA.data_ptr(),
                               dn.At.data_ptr(), dn.sfa.data_ptr(), dn.meta_native.data_ptr(), dn.gA.data_ptr(), Bb.data_ptr(),
                               sfx.data_ptr(), gBx.data_ptr(), Cgu.data_ptr(), Hb.data_ptr(), sfh.data_ptr(), gH.data_ptr(),
                               Cout.data_ptr(), _ptr(Cf), tok, H, I, 2 * I, self.out_f, splits, 1, _stream()), "qb_fused_mlp")
        return Cout.reshape(*lead, self.out_f)

    __call__ = forward


_REGISTRY: list[FusedSparseMLP] = []
_OP = None


def register_fused_mlp_op(mlps: list[FusedSparseMLP]):
    """Registers torch.ops.quadbit.fused_mlp(x, layer_idx, out_f) over `mlps`, the op the
    reference installs for vLLM's full-graph compile (harness/quadbit_serve.py:394-455): an
    opaque node whose kernels are baked into the CUDA graph at capture time."""
    global _OP
    _REGISTRY[:] = list(mlps)
    if _OP is None:
        @torch.library.custom_op("quadbit::fused_mlp", mutates_args=())
        def qb_fused_mlp(x: torch.Tensor, layer_idx: int, out_f: int) -> torch.Tensor:
            return _REGISTRY[layer_idx].forward(x)

        @qb_fused_mlp.register_fake
        def _(x, layer_idx, out_f):
            return x.new_empty((*x.shape[:-1], out_f))

        _OP = qb_fused_mlp
    return _OP
