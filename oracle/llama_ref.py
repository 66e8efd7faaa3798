"""CPU oracle of the Llama-architecture prefill forward with NVFP4 linears (TEST INFRASTRUCTURE, not product code).

Restates, in fp32 torch on the CPU, the forward the reference assembles from its pieces: attention projections on the
dense two-level NVFP4 path (harness/dense_e2e.py:99-113), the SwiGLU MLP on the 2:4-sparse path with the fused-MLP
arithmetic (harness/quadbit_serve.py:394-462, cuda/sparse_fp4_lib.cu:1133-1150), RMSNorm fused with the quantiser
(cuda/sparse_fp4_lib.cu:902-1011), attention itself in bf16 (harness/real_model.py:181-188). bf16 roundings sit where the
GPU path stores bf16: linear outputs, the residual stream, the attention output.

`world > 1` is the tensor-parallel oracle: column-parallel QKV / gate / up are exact row slices; the row-parallel
o_proj / down quantise each rank's K slice on its own (per-slice per-token global), round every rank's partial result
to bf16 and sum the partials in rank order in fp32 together with the residual. It is evaluated rank by rank in one
process. parity unpinned: the reference holds no golden vector for a whole forward; the pieces are pinned by
tests/golden/ref_fakequant.npz through oracle/fakequant.py."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import fakequant as fq


def make_weights(cfg, seed: int = 2, device="cpu", layers=None):
    """Random-init weights ~ N(0, 0.02), bf16, one generator per layer seeded (seed, layer) so any subset of layers or
    any tensor-parallel shard sees the same values. Norm weights are 1 + small noise so they matter in a comparison."""
    H, hd = cfg.hidden, cfg.head_dim
    out = {"layers": []}
    g = torch.Generator(device=device).manual_seed(seed)
    out["embed"] = (torch.randn(cfg.vocab, H, device=device, generator=g) * 0.02).to(torch.bfloat16)
    out["lm_head"] = (torch.randn(cfg.vocab, H, device=device, generator=g) * 0.02).to(torch.bfloat16)
    out["norm_f"] = (1 + 0.05 * torch.randn(H, device=device, generator=g)).to(torch.bfloat16)
    for li in range(cfg.n_layers if layers is None else layers):
        out["layers"].append(layer_weights(cfg, seed, li, device))
    return out


def layer_weights(cfg, seed: int, li: int, device="cpu"):
    H, hd, I = cfg.hidden, cfg.head_dim, cfg.intermediate
    g = torch.Generator(device=device).manual_seed(seed * 1000003 + li + 1)
    r = lambda *s: (torch.randn(*s, device=device, generator=g) * 0.02).to(torch.bfloat16)
    n = lambda: (1 + 0.05 * torch.randn(H, device=device, generator=g)).to(torch.bfloat16)
    return dict(wq=r(cfg.n_heads * hd, H), wk=r(cfg.n_kv_heads * hd, H), wv=r(cfg.n_kv_heads * hd, H), wo=r(H, cfg.n_heads * hd),
                w_gate=r(I, H), w_up=r(I, H), w_down=r(H, I), norm_attn=n(), norm_mlp=n())


def rope_tables(S: int, head_dim: int, theta: float):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(S, dtype=torch.float32), inv)
    return torch.cos(ang), torch.sin(ang)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B,S,h,hd]; rotate-half convention (first half with second half), tables [S, hd/2]."""
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def _bf(t):
    return t.to(torch.bfloat16).float()


def forward(ids: torch.Tensor, w: dict, cfg, world: int = 1):
    """ids [B,S] -> (final hidden states after the last norm [B*S, H] fp32, logits of the last token of every sequence
    [B, vocab] fp32)."""
    B, S = ids.shape
    H, hd, nh, nkv, I = cfg.hidden, cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.intermediate
    T = B * S
    cos, sin = rope_tables(S, hd, cfg.rope_theta)
    x = w["embed"][ids.reshape(-1)].float()                     # residual stream, bf16 values
    delta = None                                                # output of the previous block, added by the next norm
    for L in w["layers"]:
        # ---- attention block
        if delta is None:
            y, x16 = fq.rmsnorm_fp32(x, L["norm_attn"], cfg.rms_eps)
        else:
            y, x16 = _norm_tp(delta, x, L["norm_attn"], cfg.rms_eps)
        x = x16.float()
        xq = fq.act_dequant_2lvl(y, 16, round_bf16=False)
        attn = torch.zeros(T, nh * hd)
        for r in range(world):
            hq, hk = nh // world, nkv // world
            wq = L["wq"][r * hq * hd:(r + 1) * hq * hd].float()
            wk = L["wk"][r * hk * hd:(r + 1) * hk * hd].float()
            wv = L["wv"][r * hk * hd:(r + 1) * hk * hd].float()
            q = _bf(F.linear(xq, fq.dense_fp4_dequant(wq))).view(B, S, hq, hd)
            k = _bf(F.linear(xq, fq.dense_fp4_dequant(wk))).view(B, S, hk, hd)
            v = _bf(F.linear(xq, fq.dense_fp4_dequant(wv))).view(B, S, hk, hd)
            q, k = _bf(apply_rope(q, cos, sin)), _bf(apply_rope(k, cos, sin))
            rep = hq // hk
            kk, vv = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
            sc = torch.einsum("bshd,bthd->bhst", q, kk) / math.sqrt(hd)
            sc = sc.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
            o = torch.einsum("bhst,bthd->bshd", torch.softmax(sc, -1), vv)
            attn[:, r * hq * hd:(r + 1) * hq * hd] = _bf(o.reshape(T, hq * hd))
        ks = nh * hd // world
        delta = [_bf(F.linear(fq.act_dequant_2lvl(attn[:, r * ks:(r + 1) * ks], 16), fq.dense_fp4_dequant(L["wo"][:, r * ks:(r + 1) * ks].float())))
                 for r in range(world)]
        # ---- MLP block
        y, x16 = _norm_tp(delta, x, L["norm_mlp"], cfg.rms_eps)
        x = x16.float()
        yq = fq.act_dequant_2lvl(y, 32, round_bf16=False)
        isl = I // world
        parts = []
        for r in range(world):
            g = _bf(F.linear(yq, fq.sparse_fp4_dequant_2lvl(L["w_gate"][r * isl:(r + 1) * isl].float())))
            u = _bf(F.linear(yq, fq.sparse_fp4_dequant_2lvl(L["w_up"][r * isl:(r + 1) * isl].float())))
            h = (g / (1.0 + torch.exp(-g))) * u
            parts.append(_bf(F.linear(fq.act_dequant_2lvl(h, 32, round_bf16=False),
                                      fq.sparse_fp4_dequant_2lvl(L["w_down"][:, r * isl:(r + 1) * isl].float()))))
        delta = parts
    xf = _bf(_sum_in_order(delta) + x)
    hid = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w["norm_f"].float()
    last = _bf(hid).view(B, S, H)[:, -1]
    return hid, F.linear(last, w["lm_head"].float())


def _sum_in_order(parts):
    s = parts[0].clone()
    for p in parts[1:]:
        s = s + p
    return s


def _norm_tp(parts, x, wt, eps):
    """Tensor-parallel form of the fused residual add + RMSNorm: the bf16 partials of all ranks are summed in rank order
    in fp32, then the residual is added; the sum feeds the norm un-rounded and is stored as the new bf16 residual."""
    v = _sum_in_order(parts) + x
    y = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * wt.float()
    return y, v.to(torch.bfloat16)
