"""CPU oracle for the two-level NVFP4 hot path (TEST INFRASTRUCTURE, not product code).

This module restates, for CPU torch, the fake-quant / packing arithmetic that the
reference (vitali87/quadbit) defines as closures inside its Modal harness scripts.
Only tests, the smoke check and the CPU-baseline leg of the benchmark may import it;
the product path (quadbit_b200/) never does.

Pinning: tests/golden/*.npz hold outputs of the reference's own closures, extracted
from the reference sources by tests/golden/make_golden.py and executed on CPU; the
test-suite checks every function below against them bit for bit.

Reference sources followed (path:line inside the reference project):
  tables FP4/BND/UE4M3            harness/verify_sparse_2lvl.py:50-56
  q_fp4                           harness/verify_sparse_2lvl.py:58-59
  enc_ue4m3                       harness/verify_sparse_2lvl.py:61-73
  pair24                          harness/verify_sparse_2lvl.py:75-80
  sparse weight fake-quant        harness/verify_sparse_2lvl.py:82-91
  sparse weight pack              harness/verify_sparse_2lvl.py:108-122,
                                  harness/fused_moe.py:372-387 (zero-block guard)
  per-32 activation fake-quant    harness/verify_sparse_2lvl.py:100-106
  per-16 activation fake-quant    harness/recovery_worth.py:78-84
  dense weight fake-quant / pack  harness/recovery_worth.py:86-92, harness/dense_e2e.py:79-88
  packed-activation decode        harness/verify_sparse_2lvl.py:149-157
  linear                          harness/ab_sparse_semantics.py:118-124
  MoE routing / reference         harness/fused_moe.py:421-435, harness/moe_dist.py:133-135

Deliberate, documented choices where the reference leaves behaviour open:
  * pair-selection ties: torch.topk's tie order is unspecified; this oracle keeps the
    pair with the larger |w0|+|w1| and, on exact equality, the LOWER pair index
    (stable descending sort). `tie_groups()` reports how many groups are affected.
  * all-zero scale blocks: the divisor is clamped to 1e-30 before the divide
    (harness/fused_moe.py:381, harness/quadbit_serve.py:312-315), so the codes are 0
    instead of the 0/0 -> NaN -> code 7 of the unguarded expression. The same guard is
    applied to activations (zero padding rows).
  * scalar divisions (`/ 2688.0`, `/ 6.0`) are true IEEE fp32 divisions, as CPU torch
    computes them.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

# ---------------------------------------------------------------- tables
FP4 = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, 0, -.5, -1, -1.5, -2, -3, -4, -6], dtype=torch.float32)
BND = torch.tensor([.25, .75, 1.25, 1.75, 2.5, 3.5, 5.], dtype=torch.float32)
_c = torch.arange(128)
_e, _m = (_c >> 3) & 0xF, _c & 7
UE4M3 = torch.where(_e == 0, _m.float() * 0.001953125,
                    (1.0 + _m.float() / 8.0) * torch.exp2((_e - 7).float()))
GLOBAL_DIV = 2688.0  # 448 (e4m3 max) * 6 (e2m1 max)


def q_fp4(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> signed E2M1 code (int64). A magnitude exactly on a boundary takes the
    LOWER code (torch.bucketize, right=False)."""
    return torch.bucketize(v.abs(), BND) | ((v < 0).long() << 3)


def enc_ue4m3(s: torch.Tensor) -> torch.Tensor:
    """Positive fp32 scale -> UE4M3 code (int64), the reference's no-denormal encoder:
    round-half-even mantissa, biased<1 -> code 1, overflow / s>=480 -> 0x7f, s<=0 -> 0."""
    mant_f, e = torch.frexp(s.clamp_min(1e-30))
    mm = 2.0 * mant_f
    biased = (e - 1) + 7
    mant = torch.round((mm - 1.0) * 8.0).long()
    carry = mant == 8
    mant = torch.where(carry, torch.zeros_like(mant), mant)
    biased = torch.where(carry, biased + 1, biased)
    code = (biased.long() << 3) | mant
    code = torch.where(biased < 1, torch.ones_like(code), code)
    code = torch.where(biased > 15, torch.full_like(code, 0x7F), code)
    code = torch.where(s >= 480.0, torch.full_like(code, 0x7F), code)
    return torch.where(s > 0, code, torch.zeros_like(code))


# ---------------------------------------------------------------- 2:4 pair selection
def pair24(W: torch.Tensor, colnorm: torch.Tensor | None = None):
    """Pair-granular 2:4: in every group of 4 adjacent pairs keep the 2 with the largest
    |w0|+|w1|. Returns (Wg[out,ks,16,4,2], i01[out,ks,16,2] ascending, keptW, ks).
    colnorm [K] (activation column norms, Wanda) changes the importance to |w0|*c0 + |w1|*c1; an all-zero
    colnorm falls back to the magnitude (harness/qb_vllm_plugin/qb_sm120_plugin.py:1179-1190)."""
    out_f, in_f = W.shape
    ks = in_f // 128
    Wg = W.float().reshape(out_f, ks, 16, 4, 2)
    if colnorm is None or not bool((colnorm != 0).any()):
        imp = Wg.abs().sum(-1)
    else:
        imp = (Wg.abs() * colnorm.float().view(1, ks, 16, 4, 2)).sum(-1)
    order = torch.sort(imp, dim=-1, descending=True, stable=True).indices[..., :2]
    i01, _ = order.sort(dim=-1)
    keptW = torch.gather(Wg, 3, i01.unsqueeze(-1).expand(-1, -1, -1, -1, 2))
    return Wg, i01, keptW, ks


def tie_groups(W: torch.Tensor) -> int:
    """Number of 4-pair groups whose 2nd and 3rd largest importances are equal (the
    groups for which the reference's topk leaves the kept pair unspecified)."""
    out_f, in_f = W.shape
    imp = W.float().reshape(out_f, in_f // 8, 4, 2).abs().sum(-1)
    s = torch.sort(imp, dim=-1, descending=True).values
    return int((s[..., 1] == s[..., 2]).sum())


def _sparse_quant_core(W: torch.Tensor, colnorm: torch.Tensor | None = None):
    out_f, in_f = W.shape
    Wg, i01, keptW, ks = pair24(W, colnorm)
    gA = (keptW.abs().amax(dim=(1, 2, 3, 4), keepdim=True) / GLOBAL_DIV).clamp_min(1e-30).reshape(out_f, 1, 1)
    blk = keptW.reshape(out_f, ks, 4, 8, 2)
    scode = enc_ue4m3((blk.abs().amax(dim=(3, 4)) / 6.0) / gA)
    sdeq = UE4M3[scode] * gA
    kc = q_fp4(blk / sdeq.clamp_min(1e-30)[..., None, None])
    return i01, gA, scode, sdeq, kc, ks


def pack_weight_sparse_2lvl(W: torch.Tensor, colnorm: torch.Tensor | None = None):
    """[out,K] -> reference-layout packed tensors:
       Ac[out,K/4] u8 (byte = one kept pair, low nibble = even k),
       meta[K/128,out,2] i32 (group g: word g//8, bits 4*(g%8): i0|(i1<<2)),
       scaleA[K/128,out,4] u8 (one UE4M3 per 16 kept values = 32 logical K),
       gA[out] f32."""
    out_f, in_f = W.shape
    i01, gA, scode, sdeq, kc, ks = _sparse_quant_core(W, colnorm)
    Ac = (kc[..., 0] | (kc[..., 1] << 4)).reshape(out_f, ks * 32).to(torch.uint8).contiguous()
    nib = (i01[..., 0] | (i01[..., 1] << 2)).view(out_f, ks, 2, 8)
    sh = (torch.arange(8) * 4).view(1, 1, 1, 8)
    meta = (nib << sh).sum(-1).to(torch.int32).permute(1, 0, 2).contiguous()
    scaleA = scode.to(torch.uint8).permute(1, 0, 2).contiguous()
    return Ac, meta, scaleA, gA.reshape(out_f).float().contiguous()


def sparse_fp4_dequant_2lvl(W: torch.Tensor) -> torch.Tensor:
    """Dense fp32 [out,K] matrix that the packed sparse weight represents."""
    out_f, in_f = W.shape
    i01, gA, scode, sdeq, kc, ks = _sparse_quant_core(W)
    kd = (FP4[kc] * sdeq[..., None, None]).reshape(out_f, ks, 16, 2, 2)
    Wd = torch.zeros(out_f, ks, 16, 4, 2)
    Wd.scatter_(3, i01.unsqueeze(-1).expand(-1, -1, -1, -1, 2), kd)
    return Wd.reshape(out_f, in_f)


def unpack_weight_sparse_2lvl(Ac, meta, scaleA, gA) -> torch.Tensor:
    """Inverse of pack_weight_sparse_2lvl: dense fp32 [out,K] from the packed tensors."""
    out_f = Ac.shape[0]
    ks = meta.shape[0]
    codes = torch.stack([(Ac & 0xF).long(), (Ac >> 4).long()], -1).view(out_f, ks, 4, 8, 2)
    s = UE4M3[scaleA.permute(1, 0, 2).long()] * gA.view(out_f, 1, 1)            # [out,ks,4]
    kd = (FP4[codes] * s[..., None, None]).reshape(out_f, ks, 16, 2, 2)
    m = meta.permute(1, 0, 2).long() & 0xFFFFFFFF                                 # [out,ks,2]
    nib = (m.unsqueeze(-1) >> (torch.arange(8) * 4).view(1, 1, 1, 8)) & 0xF       # [out,ks,2,8]
    nib = nib.reshape(out_f, ks, 16)
    i01 = torch.stack([nib & 3, (nib >> 2) & 3], -1)
    Wd = torch.zeros(out_f, ks, 16, 4, 2)
    Wd.scatter_(3, i01.unsqueeze(-1).expand(-1, -1, -1, -1, 2), kd)
    return Wd.reshape(out_f, ks * 128)


# ---------------------------------------------------------------- dense weights
def nvfp4_pack(W: torch.Tensor):
    """[out,K] -> Ab[out,K/2] u8, SFA[K/128,out,8] u8 (per-16), gA[out] f32."""
    out_f, in_f = W.shape
    Wf = W.float()
    gA = (Wf.abs().amax(-1) / GLOBAL_DIV).clamp(min=1e-30)
    Wb = Wf.view(out_f, in_f // 16, 16)
    scode = enc_ue4m3((Wb.abs().amax(-1) / 6.0) / gA[:, None])
    sdeq = UE4M3[scode] * gA[:, None]
    q = q_fp4(Wb / sdeq.clamp_min(1e-30)[..., None]).view(out_f, in_f)
    Ab = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8).contiguous()
    SFA = scode.view(out_f, in_f // 128, 8).permute(1, 0, 2).contiguous().to(torch.uint8)
    return Ab, SFA, gA.contiguous()


def dense_fp4_dequant(W: torch.Tensor) -> torch.Tensor:
    out_f, in_f = W.shape
    Wf = W.float()
    gA = (Wf.abs().amax(-1, keepdim=True) / GLOBAL_DIV).clamp_min(1e-30)
    b = Wf.view(out_f, in_f // 16, 16)
    sdeq = UE4M3[enc_ue4m3((b.abs().amax(-1) / 6.0) / gA)] * gA
    return (FP4[q_fp4(b / sdeq.clamp_min(1e-30)[..., None])] * sdeq[..., None]).reshape(out_f, in_f)


def unpack_weight_dense(Ab, SFA, gA) -> torch.Tensor:
    out_f = Ab.shape[0]
    in_f = Ab.shape[1] * 2
    codes = torch.empty(out_f, in_f, dtype=torch.long)
    codes[:, 0::2] = (Ab & 0xF).long()
    codes[:, 1::2] = (Ab >> 4).long()
    s = UE4M3[SFA.permute(1, 0, 2).reshape(out_f, in_f // 16).long()] * gA[:, None]
    return FP4[codes] * s.repeat_interleave(16, dim=1)


# ---------------------------------------------------------------- activations
def act_quant_2lvl(x: torch.Tensor, block: int, round_bf16: bool = True):
    """bf16-rounded [tok,K] -> (Bbytes[tok,K/2] u8, scale[K/128,tok,128/block] u8, g[tok] f32).
    block = 32 for the sparse path, 16 for the dense path."""
    i = x.shape[-1]
    b = (x.to(torch.bfloat16).float() if round_bf16 else x.float()).reshape(-1, i)
    t = b.shape[0]
    g = (b.abs().amax(-1, keepdim=True) / GLOBAL_DIV).clamp_min(1e-30)
    bb = b.reshape(t, i // block, block)
    code = enc_ue4m3((bb.abs().amax(-1) / 6.0) / g)
    sdeq = UE4M3[code] * g
    q = q_fp4(bb / sdeq.clamp_min(1e-30)[..., None]).reshape(t, i)
    Bbytes = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8).contiguous()
    per = 128 // block
    scale = code.view(t, i // 128, per).permute(1, 0, 2).contiguous().to(torch.uint8)
    return Bbytes, scale, g.reshape(t).contiguous()


def act_dequant_2lvl(x: torch.Tensor, block: int, round_bf16: bool = True) -> torch.Tensor:
    """Fake-quant of activations: act_2lvl_deq_p32 (block=32) / act_fp4_dequant (block=16).
    round_bf16=False quantises fp32 values directly (the fused SwiGLU quantiser's input)."""
    lead = x.shape[:-1]
    i = x.shape[-1]
    b = (x.to(torch.bfloat16).float() if round_bf16 else x.float()).reshape(-1, i)
    g = (b.abs().amax(-1, keepdim=True) / GLOBAL_DIV).clamp_min(1e-30)
    bb = b.reshape(b.shape[0], i // block, block)
    sdeq = UE4M3[enc_ue4m3((bb.abs().amax(-1) / 6.0) / g)] * g
    return (FP4[q_fp4(bb / sdeq.clamp_min(1e-30)[..., None])] * sdeq[..., None]).reshape(*lead, i)


def act_quant_1lvl(x: torch.Tensor, block: int, round_bf16: bool = True):
    """Single-level quantiser (no global): code = enc(amax/6), as quant_act /
    quant_act_nv (cuda/sparse_fp4_lib.cu:704-732, cuda/dense_nvfp4_fast_lib.cu:175-206)
    restated with the same guard/tie rules as the two-level oracle."""
    i = x.shape[-1]
    b = (x.to(torch.bfloat16).float() if round_bf16 else x.float()).reshape(-1, i)
    t = b.shape[0]
    bb = b.reshape(t, i // block, block)
    code = enc_ue4m3(bb.abs().amax(-1) / 6.0)
    sdeq = UE4M3[code]
    q = q_fp4(bb / sdeq.clamp_min(1e-30)[..., None]).reshape(t, i)
    Bbytes = (q[:, 0::2] | (q[:, 1::2] << 4)).to(torch.uint8).contiguous()
    per = 128 // block
    scale = code.view(t, i // 128, per).permute(1, 0, 2).contiguous().to(torch.uint8)
    return Bbytes, scale


def unpack_act(Bbytes, scale, g, block: int) -> torch.Tensor:
    """Dequantise exactly what the GEMM sees for the activations."""
    t = Bbytes.shape[0]
    in_f = Bbytes.shape[1] * 2
    codes = torch.empty(t, in_f, dtype=torch.long)
    codes[:, 0::2] = (Bbytes & 0xF).long()
    codes[:, 1::2] = (Bbytes >> 4).long()
    sc = scale.permute(1, 0, 2).reshape(t, in_f // block).long()
    local = UE4M3[sc].repeat_interleave(block, dim=1)
    if g is not None:
        local = local * g[:, None]          # same product order as the fake-quant (sdeq = UE4M3[code]*g)
    return FP4[codes] * local


# ---------------------------------------------------------------- linear
def linear_sparse(x: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    """fp32 result of the 2:4-sparse two-level NVFP4 linear: y = act_deq32(x) @ Wdeq^T."""
    return F.linear(act_dequant_2lvl(x.float(), 32), sparse_fp4_dequant_2lvl(W.float()))


def linear_dense(x: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    return F.linear(act_dequant_2lvl(x.float(), 16), dense_fp4_dequant(W.float()))


def rmsnorm_fp32(x: torch.Tensor, w: torch.Tensor, eps: float, res: torch.Tensor | None = None):
    """fp32 RMSNorm of bf16 inputs as the fused quantisers compute it (cuda/sparse_fp4_lib.cu:902-1011):
    v = x (+ res); y = v * rsqrt(mean(v^2) + eps) * w. Returns (y, bf16(v))."""
    v = x.to(torch.bfloat16).float()
    if res is not None:
        v = v + res.to(torch.bfloat16).float()
    y = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.to(torch.bfloat16).float()
    return y, v.to(torch.bfloat16)


def fused_mlp_sparse(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """Reference arithmetic of the fused SwiGLU MLP (cuda/sparse_fp4_lib.cu:1133-1150 with
    swiglu_amax / swiglu_quant_g :837-884): gate/up linear rounded to bf16, h = silu(g)*u in
    fp32, two-level per-32 fake-quant of h, down linear. w_gate_up rows: gate then up."""
    I = w_down.shape[1]
    gu = linear_sparse(x, w_gate_up).to(torch.bfloat16).float()
    g, u = gu[..., :I], gu[..., I:]
    h = (g / (1.0 + torch.exp(-g))) * u
    return F.linear(act_dequant_2lvl(h, 32, round_bf16=False), sparse_fp4_dequant_2lvl(w_down.float()))


# ---------------------------------------------------------------- native (tcgen05) layouts
def sf_to_atoms(scale_ref: torch.Tensor) -> torch.Tensor:
    """Reference step-major scales [K/128, rows, P] (P = 4 per-32 or 8 per-16) ->
    the 128x4 scale-factor atoms the block-scaled tensor-core instruction reads:
    [ceil(rows/128), Kp*P/512, 512] u8 with byte (r%32)*16 + (r//32)*4 + c inside an atom,
    atom j covering 4 consecutive scale columns. Rows are zero padded to 128 and K to a
    multiple of 256 (Kp)."""
    ks, rows, P = scale_ref.shape
    rp = (rows + 127) // 128 * 128
    kp = (ks + 1) // 2 * 2
    s = torch.zeros(kp, rp, P, dtype=torch.uint8)
    s[:ks, :rows] = scale_ref
    s = s.permute(1, 0, 2).reshape(rp, kp * P)                       # [rows, ncol]
    s = s.view(rp // 128, 4, 32, kp * P // 4, 4)                     # [rb, r1, r0, atom, c]
    return s.permute(0, 3, 2, 1, 4).contiguous().view(rp // 128, kp * P // 4, 512)


def meta_to_native(meta_ref: torch.Tensor) -> torch.Tensor:
    """Reference metadata [K/128, out, 2] i32 -> [out/128, Kp/256, 128, 16] u8: per 128-row
    block and 256 logical K, 16 bytes per row (group g of a 128-K step at bits 4g); K is
    zero padded to a multiple of 256."""
    ks, out_f, _ = meta_ref.shape
    kp = (ks + 1) // 2 * 2
    mp = torch.zeros(kp, out_f, 2, dtype=torch.int32)
    mp[:ks] = meta_ref
    m = mp.permute(1, 0, 2).contiguous().view(torch.uint8).view(out_f, kp // 2, 16)
    return m.view(out_f // 128, 128, kp // 2, 16).permute(0, 2, 1, 3).contiguous()


# ---------------------------------------------------------------- MoE
def route_topk(logits: torch.Tensor, topk: int):
    """softmax -> top-k -> renormalise (harness/moe_dist.py:133-135 without the 1.5 gain)."""
    p = torch.softmax(logits.float(), -1)
    w, idx = p.topk(topk, dim=-1)
    return idx, w / w.sum(-1, keepdim=True)


def build_routing(assign: torch.Tensor, e: int, bn: int = 128):
    """Sort routed slots by expert, pad every expert segment to a multiple of bn rows.
    Returns (src[r_pad] (-1 = padding), eblk[r_pad/bn] i32, r_pad)."""
    order = torch.argsort(assign, stable=True)
    counts = torch.bincount(assign, minlength=e)
    padc = (counts + bn - 1) // bn * bn
    r_pad = int(padc.sum())
    src = torch.full((r_pad,), -1, dtype=torch.long)
    eblk = torch.zeros(r_pad // bn, dtype=torch.int32)
    off = 0
    oi = 0
    for ex in range(e):
        ce, pe = int(counts[ex]), int(padc[ex])
        if pe == 0:
            continue
        src[off:off + ce] = order[oi:oi + ce]
        oi += ce
        eblk[off // bn:(off + pe) // bn] = ex
        off += pe
    return src, eblk, r_pad


def moe_seg_linear(x_rows: torch.Tensor, eblk: torch.Tensor, W_experts, bn: int = 128) -> torch.Tensor:
    """Per-expert reference of the segmented GEMM: rows of block b use expert eblk[b]."""
    out = torch.zeros(x_rows.shape[0], W_experts[0].shape[0])
    deq = {}
    for b in range(eblk.numel()):
        ex = int(eblk[b])
        if ex not in deq:
            deq[ex] = sparse_fp4_dequant_2lvl(W_experts[ex].float())
        xs = x_rows[b * bn:(b + 1) * bn]
        out[b * bn:(b + 1) * bn] = F.linear(act_dequant_2lvl(xs.float(), 32), deq[ex])
    return out


# ---------------------------------------------------------------- checkpoint block formats
def mxfp4_dequant(w_u8: torch.Tensor, s_u8: torch.Tensor) -> torch.Tensor:
    """gpt-oss MXFP4 expert weight -> bf16: w [out, in/2] u8 (low nibble = even column), s [out, in/32] u8 e8m0
    (multiplier 2^(raw-127)); harness/qb_vllm_plugin/qb_sm120_plugin.py:2089-2100."""
    b = w_u8.to(torch.int32) & 0xFF
    out_f, inb = b.shape
    codes = torch.empty(out_f, inb * 2, dtype=torch.long)
    codes[:, 0::2] = b & 0xF
    codes[:, 1::2] = (b >> 4) & 0xF
    mult = torch.exp2(s_u8.float() - 127.0)
    return (FP4[codes].view(out_f, s_u8.shape[-1], 32) * mult[:, :, None]).reshape(out_f, inb * 2).to(torch.bfloat16)


def nvfp4_ckpt_dequant(w_u8: torch.Tensor, scale_e4m3_u8: torch.Tensor, s2: float, group: int = 16) -> torch.Tensor:
    """modelopt NVFP4 weight -> bf16: FP4[nibble] * e4m3fn block scale [out, in/group] (given as raw bytes) * per-tensor
    fp32 scale, products in that order in fp32; harness/qb_vllm_plugin/qb_sm120_plugin.py:70-95."""
    b = w_u8.to(torch.int32) & 0xFF
    out_f, inb = b.shape
    k = inb * 2
    codes = torch.empty(out_f, k, dtype=torch.long)
    codes[:, 0::2] = b & 0xF
    codes[:, 1::2] = (b >> 4) & 0xF
    bs = scale_e4m3_u8.view(torch.float8_e4m3fn).float().repeat_interleave(group, dim=1)[:, :k]
    return (FP4[codes] * bs * torch.tensor(s2, dtype=torch.float32)).to(torch.bfloat16)
