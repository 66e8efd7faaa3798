"""Llama-architecture prefill forward on the NVFP4 kernels, tensor-parallel over the GPUs of one box.

What the reference assembles for its end-to-end runs, here as one module: attention projections on the dense two-level
NVFP4 GEMM (harness/dense_e2e.py:99-113), the SwiGLU MLP on the 2:4-sparse GEMM with the fused-MLP arithmetic
(harness/quadbit_serve.py:394-462), RMSNorm fused with the quantiser in front of both (cuda/sparse_fp4_lib.cu:902-1011),
attention math in bf16 (harness/real_model.py:181-188). Embedding, RoPE, attention and the final norm / logits are plain
torch (host layer); every linear, quantiser and norm in the layer stack is a kernel of this library.

Tensor parallelism (world = number of GPUs, one process each) with the residual stream sharded by tokens:

    N1   reduce(down partials of the previous layer) + residual + RMSNorm + per-16 quantise of this rank's token rows,
         the packed rows stored into EVERY rank's gathered array                      (qb_reduce_norm_quant)
    QKV  dense GEMM on all tokens, this rank's heads: column-parallel, no exchange      (qb_gemm)
    attention over this rank's heads (torch SDPA), per-16 quantise of its output        (qb_quantize_act)
    O    dense GEMM over this rank's K slice, partial rows stored into the owner's slot (qb_gemm_rs)
    N2   reduce(o_proj partials) + residual + RMSNorm + per-32 quantise, stored to all  (qb_reduce_norm_quant)
    GU   2:4-sparse GEMM, this rank's gate and up rows, column-parallel                 (qb_gemm)
    SwiGLU + per-32 quantise of the local intermediate slice                            (qb_swiglu_quant)
    D    2:4-sparse GEMM over this rank's K slice, partial rows stored into the owners  (qb_gemm_rs)

so per layer the NVLink carries two reduce-scatters of bf16 partials (issued by GEMM epilogues, overlapping the MMAs) and
two all-gathers of QUANTISED activations (0.56 bytes per value instead of 2), and no NCCL call. `comm="nccl"` runs the
same arithmetic with all_to_all_single / all_gather_into_tensor in place of the peer stores (the baseline the fused
form is measured against, and the fallback when peer mapping is unavailable). The row-parallel GEMMs quantise each
rank's K slice on its own (per-slice token global), the partials are bf16 and are summed in rank order: see
oracle/llama_ref.py for the arithmetic this is tested against."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from ._lib import check, load
from .linear import DenseNVLinear, QuadbitLinear, _stream
from .tp import TPContext, ptr_array


@dataclass
class LlamaConfig:
    n_layers: int = 32
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 14336
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    vocab: int = 128256


def random_layer(cfg: LlamaConfig, seed: int, li: int, device) -> dict:
    """One layer of random-init weights ~ N(0, 0.02) in bf16 (norm weights 1 + small noise), from a generator seeded by
    (seed, layer): any rank generates the same full matrices and slices its shard."""
    H, hd, I = cfg.hidden, cfg.head_dim, cfg.intermediate
    g = torch.Generator(device=device).manual_seed(seed * 1000003 + li + 1)
    r = lambda *s: (torch.randn(*s, device=device, generator=g) * 0.02).to(torch.bfloat16)
    n = lambda: (1 + 0.05 * torch.randn(H, device=device, generator=g)).to(torch.bfloat16)
    return dict(wq=r(cfg.n_heads * hd, H), wk=r(cfg.n_kv_heads * hd, H), wv=r(cfg.n_kv_heads * hd, H), wo=r(H, cfg.n_heads * hd),
                w_gate=r(I, H), w_up=r(I, H), w_down=r(H, I), norm_attn=n(), norm_mlp=n())


def random_weights(cfg: LlamaConfig, seed: int, device) -> dict:
    """Random-init model: embedding, lm_head, final norm and a per-layer generator (layers are built and packed one at a
    time, so the bf16 matrices of only one layer exist at once)."""
    g = torch.Generator(device=device).manual_seed(seed)
    H = cfg.hidden
    return dict(embed=(torch.randn(cfg.vocab, H, device=device, generator=g) * 0.02).to(torch.bfloat16),
                lm_head=(torch.randn(cfg.vocab, H, device=device, generator=g) * 0.02).to(torch.bfloat16),
                norm_f=(1 + 0.05 * torch.randn(H, device=device, generator=g)).to(torch.bfloat16),
                layers=lambda li: random_layer(cfg, seed, li, device))


def shard_layer(L: dict, cfg: LlamaConfig, rank: int, world: int) -> dict:
    """This rank's slices of one layer's bf16 weights: heads (q, k, v rows; o_proj columns) and intermediate features
    (gate, up rows; down columns)."""
    hd = cfg.head_dim
    hq, hk, isl = cfg.n_heads // world * hd, cfg.n_kv_heads // world * hd, cfg.intermediate // world
    qkv = torch.cat([L["wq"][rank * hq:(rank + 1) * hq], L["wk"][rank * hk:(rank + 1) * hk], L["wv"][rank * hk:(rank + 1) * hk]], 0)
    gu = torch.cat([L["w_gate"][rank * isl:(rank + 1) * isl], L["w_up"][rank * isl:(rank + 1) * isl]], 0)
    return dict(qkv=qkv.contiguous(), wo=L["wo"][:, rank * hq:(rank + 1) * hq].contiguous(), gate_up=gu.contiguous(),
                down=L["w_down"][:, rank * isl:(rank + 1) * isl].contiguous(), norm_attn=L["norm_attn"], norm_mlp=L["norm_mlp"])


class _Layer:
    def __init__(self, W: dict, interleave_gu: bool = False):
        self.qkv = DenseNVLinear(W["qkv"], keep_ref_layout=False)
        self.wo = DenseNVLinear(W["wo"], keep_ref_layout=False)
        gu = W["gate_up"]
        if interleave_gu:            # rows as (gate, up) pairs for the fused SwiGLU epilogue
            half = gu.shape[0] // 2
            gu = torch.stack([gu[:half], gu[half:]], 1).reshape(gu.shape[0], gu.shape[1]).contiguous()
        self.gu = QuadbitLinear(gu, keep_ref_layout=False)
        self.dn = QuadbitLinear(W["down"], keep_ref_layout=False)
        self.norm_attn = W["norm_attn"].to(torch.bfloat16).contiguous()
        self.norm_mlp = W["norm_mlp"].to(torch.bfloat16).contiguous()


class LlamaPrefill:
    """One rank of the model. `weights`: dict as oracle-side `make_weights` builds it (embed, lm_head, norm_f, layers =
    list of per-layer dicts or a callable layer index -> dict, so full-size layers can be generated and packed one at a
    time). `ctx`: a TPContext for world > 1 with comm="peer". fuse_swiglu: SwiGLU and the quantiser of its result run in the
    epilogue of the gate/up GEMM (qb_gemm_swiglu): the [tokens, 2 * intermediate] bf16 round trip and one kernel per layer
    disappear, at the price of a different arithmetic for h (formed from the fp32 accumulators, quantised with one scale per
    32 features and no per-token global, as the reference's fused MoE GEMM does) - off by default, the default matches the
    reference's fused_mlp_2lvl."""

    def __init__(self, cfg: LlamaConfig, weights: dict, rank: int = 0, world: int = 1, group=None, comm: str = "peer",
                 ctx: TPContext | None = None, device=None, fuse_swiglu: bool = False):
        assert cfg.n_heads % world == 0 and cfg.n_kv_heads % world == 0 and cfg.intermediate % (128 * world) == 0
        assert comm in ("peer", "nccl")
        self.cfg, self.rank, self.world, self.group, self.comm = cfg, rank, world, group, comm
        self.lib = load("sparse_fp4")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.embed = weights["embed"].to(self.device)
        self.lm_head = weights["lm_head"].to(self.device)
        self.norm_f = weights["norm_f"].to(self.device)
        layers = weights["layers"]
        n = cfg.n_layers
        self.layers = []
        for li in range(n):
            L = layers(li) if callable(layers) else layers[li]
            self.layers.append(_Layer(shard_layer({k: v.to(self.device) for k, v in L.items()}, cfg, rank, world), fuse_swiglu))
        self.fuse_swiglu = fuse_swiglu
        self.ctx = ctx
        self._rope = {}
        self.timings = None
        self._marks = []
        self._last_idx = {}
        self._graph = self._graph_key = self._graph_out = self._ids_static = None
        self.capture = None          # set to a dict to keep the intermediate tensors of the LAST layer run (tests)

    # ------------------------------------------------------------------ pieces
    def _rope_table(self, S: int) -> torch.Tensor:
        """fp32 [S, 128] = cos | sin of pos * theta^(-2i/128); computed on the host so that every device (and the CPU
        oracle) uses the same bits."""
        if S not in self._rope:
            hd = self.cfg.head_dim
            inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
            ang = torch.outer(torch.arange(S, dtype=torch.float32), inv)
            self._rope[S] = torch.cat([torch.cos(ang), torch.sin(ang)], 1).contiguous().to(self.device)
        return self._rope[S]

    def _attention(self, qkv: torch.Tensor, B: int, S: int) -> torch.Tensor:
        """qkv [T, (hq + 2 hk) * hd] bf16 of this rank's heads -> [T, hq * hd] bf16: RoPE in place on the q and k heads
        (qb_rope_inplace), then causal GQA attention in bf16 (torch SDPA)."""
        cfg = self.cfg
        hd, hq, hk = cfg.head_dim, cfg.n_heads // self.world, cfg.n_kv_heads // self.world
        assert hd == 128
        check(self.lib.qb_rope_inplace(qkv.data_ptr(), self._rope_table(S).data_ptr(), B * S, S, qkv.shape[1], hq + hk, _stream()),
              "qb_rope_inplace")
        q = qkv[:, : hq * hd].view(B, S, hq, hd)
        k = qkv[:, hq * hd:(hq + hk) * hd].view(B, S, hk, hd)
        v = qkv[:, (hq + hk) * hd:].view(B, S, hk, hd)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True)
        return o.transpose(1, 2).reshape(B * S, hq * hd)

    def _gemm(self, lin, Bb: int, sfb: int, gB: int, tok: int, out: torch.Tensor):
        dense = isinstance(lin, DenseNVLinear)
        out_f, in_f = (lin.out, lin.inn) if dense else (lin.out_f, lin.in_f)
        check(self.lib.qb_gemm(lin.At.data_ptr(), Bb, lin.sfa.data_ptr(), sfb, 0 if dense else lin.meta_native.data_ptr(), lin.gA.data_ptr(),
                               gB, out.data_ptr(), 0, 0, 0, 0, out_f, out_f, tok, in_f, 2 if dense else 3, 1, 1, 0, _stream()), "qb_gemm")

    def _row_parallel(self, lin, q, tok: int, k: int) -> torch.Tensor | None:
        """Row-parallel GEMM on the quantised local K slice q = (Bb, atoms, g). world 1: returns [tok, out]. Otherwise the
        partial rows go to the owners' slots (set k) and None is returned."""
        dense = isinstance(lin, DenseNVLinear)
        out_f, in_f = (lin.out, lin.inn) if dense else (lin.out_f, lin.in_f)
        Bb, sfb, gB = q
        gp = gB.data_ptr() if gB is not None else 0
        if self.world == 1:
            out = torch.empty((tok, out_f), dtype=torch.bfloat16, device=self.device)
            self._gemm(lin, Bb.data_ptr(), sfb.data_ptr(), gp, tok, out)
            return out
        ctx = self.ctx
        if self.comm == "nccl":
            import torch.distributed as dist
            part = torch.empty((tok, out_f), dtype=torch.bfloat16, device=self.device)
            self._gemm(lin, Bb.data_ptr(), sfb.data_ptr(), gp, tok, part)
            dist.all_to_all_single(ctx.slots_view(k), part.view(self.world, ctx.Tl, out_f), group=self.group)
            return None
        check(self.lib.qb_gemm_rs(lin.At.data_ptr(), Bb.data_ptr(), lin.sfa.data_ptr(), sfb.data_ptr(),
                                  0 if dense else lin.meta_native.data_ptr(), lin.gA.data_ptr(), gp, ctx.slot_out_ptrs(k),
                                  ctx.flag_ptrs(ctx.FLAG_SLOT[k]), ctx.done[k:].data_ptr(), out_f, tok, in_f, 2 if dense else 3, self.world,
                                  self.rank, ctx.Tl, 0, ctx.epoch.data_ptr(), 0, _stream()), "qb_gemm_rs")
        return None

    def _norm_quant(self, src, k, res, wt, block: int, T: int):
        """Fused reduce + residual add + RMSNorm + quantiser of this rank's rows. src: bf16 [Tl, H] tensor (world 1, or the
        embedding rows of the first layer) or None = this rank's slots `k`. Returns (new residual or None, (Bb ptr, atoms
        ptr, g ptr) of the quantised activations of ALL T tokens as the following column-parallel GEMM reads them)."""
        lib, H, W = self.lib, self.cfg.hidden, self.world
        Tl = T // W
        hout = torch.empty((Tl, H), dtype=torch.bfloat16, device=self.device) if res is not None else None
        hp = hout.data_ptr() if hout is not None else 0
        rp = res.data_ptr() if res is not None else 0
        if W == 1:
            Bb = torch.empty((T, H // 2), dtype=torch.uint8, device=self.device)
            sf = torch.empty(lib.qb_sf_atoms_bytes(T, H, block), dtype=torch.uint8, device=self.device)
            g = torch.empty((T,), dtype=torch.float32, device=self.device)
            check(lib.qb_reduce_norm_quant(src.data_ptr(), 0, 1, rp, wt.data_ptr(), hp, ptr_array([Bb.data_ptr()]), ptr_array([sf.data_ptr()]),
                                           ptr_array([g.data_ptr()]), 0, 0, T, T, H, self.cfg.rms_eps, block, 0, 0, None, 0, 0, 0, 0, 0, _stream()),
                  "qb_reduce_norm_quant")
            self._keep = (Bb, sf, g)
            return hout, (Bb.data_ptr(), sf.data_ptr(), g.data_ptr())
        ctx = self.ctx
        if src is None:
            s0, stride, nsrc = ctx.slots_view(k).data_ptr(), Tl * H, W
        else:
            s0, stride, nsrc = src.data_ptr(), 0, 1
        if self.comm == "nccl":
            import torch.distributed as dist
            Bl = torch.empty((Tl, H // 2), dtype=torch.uint8, device=self.device)
            sl = torch.empty(lib.qb_sf_atoms_bytes(Tl, H, block), dtype=torch.uint8, device=self.device)
            gl = torch.empty((Tl,), dtype=torch.float32, device=self.device)
            check(lib.qb_reduce_norm_quant(s0, stride, nsrc, rp, wt.data_ptr(), hp, ptr_array([Bl.data_ptr()]), ptr_array([sl.data_ptr()]),
                                           ptr_array([gl.data_ptr()]), 0, 0, Tl, Tl, H, self.cfg.rms_eps, block, 0, 0, None, 0, 0, 0, 0, 0, _stream()),
                  "qb_reduce_norm_quant")
            Bb = torch.empty((T, H // 2), dtype=torch.uint8, device=self.device)
            sf = torch.empty(lib.qb_sf_atoms_bytes(T, H, block), dtype=torch.uint8, device=self.device)
            g = torch.empty((T,), dtype=torch.float32, device=self.device)
            dist.all_gather_into_tensor(Bb, Bl, group=self.group)
            dist.all_gather_into_tensor(sf, sl, group=self.group)        # atoms are 128-row-block major: rank chunks concatenate
            dist.all_gather_into_tensor(g, gl, group=self.group)
            self._keep = (Bb, sf, g)
            return hout, (Bb.data_ptr(), sf.data_ptr(), g.data_ptr())
        fw = ctx.FLAG_GATHER[block]
        wait_ptr = ctx.flag_own(ctx.FLAG_SLOT[k]) if src is None else 0
        Bv, Sv, Gv = ctx.gathered_ptrs(block)
        check(lib.qb_reduce_norm_quant(s0, stride, nsrc, rp, wt.data_ptr(), hp, Bv, Sv, Gv, W, self.rank * Tl, T, Tl, H, self.cfg.rms_eps,
                                       block, wait_ptr, 0, ctx.flag_ptrs(fw), W, self.rank, 0, ctx.done[2 + (block == 32):].data_ptr(),
                                       ctx.epoch.data_ptr(), _stream()), "qb_reduce_norm_quant")
        return hout, ("gathered", block)

    def _resolve(self, q, block: int):
        """Pointers of the gathered activations; with peer stores, first wait until every rank's rows have landed."""
        if isinstance(q[0], str):
            ctx = self.ctx
            check(self.lib.qb_peer_wait(ctx.flag_own(ctx.FLAG_GATHER[block]), self.world, 0, ctx.epoch.data_ptr(), _stream()), "qb_peer_wait")
            return ctx.gathered_own(block)
        return q

    # ------------------------------------------------------------------ forward
    def forward_steps(self, ids: torch.Tensor):
        """Generator over the forward: yields after every kernel that other ranks wait for (so that a single process can
        drive several emulated ranks in lock step); the last value is (hidden_local [T/world, H] bf16, logits [B, vocab])."""
        cfg, lib, W = self.cfg, self.lib, self.world
        B, S = ids.shape
        T, H, I = B * S, cfg.hidden, cfg.intermediate // W
        Tl = T // W
        r0 = self.rank * Tl
        self._mark("start")
        x = self.embed[ids.reshape(-1)[r0:r0 + Tl]]                                # residual stream, this rank's rows (ids on the device)
        res, q16 = self._norm_quant(x, None, None, self.layers[0].norm_attn, 16, T)
        self._mark("embed+norm_quant")
        yield None
        for li, L in enumerate(self.layers):
            Bb, sf, g = self._resolve(q16, 16)
            if W > 1 and self.comm == "peer":
                self.ctx.bump(_stream())         # every flag written in this layer carries the new epoch
            self._cap_gathered("q16", (Bb, sf, g), 16, T)
            self._cap("x_attn_in", x)
            qkv = torch.empty((T, L.qkv.out), dtype=torch.bfloat16, device=self.device)
            self._gemm(L.qkv, Bb, sf, g, T, qkv)
            self._mark("qkv_gemm")
            self._cap("qkv", qkv)
            attn = self._attention(qkv, B, S)
            self._mark("rope+attention")
            self._cap("attn", attn)
            aq = self._quantize(attn, 16)
            self._mark("act_quant")
            o = self._row_parallel(L.wo, aq, T, 0)
            self._mark("o_proj_gemm")
            yield None
            if self.capture is not None:
                if W > 1 and self.comm == "peer":          # test aid: the partials must have landed before they are copied
                    check(lib.qb_peer_wait(self.ctx.flag_own(0), W, 0, self.ctx.epoch.data_ptr(), _stream()), "qb_peer_wait")
                self._cap("o_parts", o.unsqueeze(0) if W == 1 else self.ctx.slots_view(0))
            x, q32 = self._norm_quant(o, 0, x, L.norm_mlp, 32, T)
            self._mark("reduce+norm_quant")
            yield None
            self._cap("x_mlp_in", x)
            Bb, sf, g = self._resolve(q32, 32)
            self._cap_gathered("q32", (Bb, sf, g), 32, T)
            Hb = torch.empty((T, I // 2), dtype=torch.uint8, device=self.device)
            sfh = torch.empty(lib.qb_sf_atoms_bytes(T, I, 32), dtype=torch.uint8, device=self.device)
            if self.fuse_swiglu:
                gH = None
                check(lib.qb_gemm_swiglu(L.gu.At.data_ptr(), Bb, L.gu.sfa.data_ptr(), sf, L.gu.meta_native.data_ptr(), L.gu.gA.data_ptr(), g, 0, 0,
                                         Hb.data_ptr(), sfh.data_ptr(), 0, 2 * I, 2 * I, T, H, 3, 1, _stream()), "qb_gemm_swiglu")
                self._mark("gate_up_gemm")
            else:
                cgu = torch.empty((T, 2 * I), dtype=torch.bfloat16, device=self.device)
                self._gemm(L.gu, Bb, sf, g, T, cgu)
                self._mark("gate_up_gemm")
                self._cap("cgu", cgu)
                gH = torch.empty((T,), dtype=torch.float32, device=self.device)
                check(lib.qb_swiglu_quant(cgu.data_ptr(), Hb.data_ptr(), 0, sfh.data_ptr(), gH.data_ptr(), T, I, _stream()), "qb_swiglu_quant")
                self._mark("swiglu_quant")
            d = self._row_parallel(L.dn, (Hb, sfh, gH), T, 1)
            self._mark("down_gemm")
            yield None
            if self.capture is not None:
                if W > 1 and self.comm == "peer":
                    check(lib.qb_peer_wait(self.ctx.flag_own(1), W, 0, self.ctx.epoch.data_ptr(), _stream()), "qb_peer_wait")
                self._cap("d_parts", d.unsqueeze(0) if W == 1 else self.ctx.slots_view(1))
            if li + 1 < len(self.layers):
                x, q16 = self._norm_quant(d, 1, x, self.layers[li + 1].norm_attn, 16, T)
                self._mark("reduce+norm_quant")
                yield None
        # final: sum of the last partials + residual -> bf16 -> RMSNorm -> logits of the last token of every sequence
        if W == 1:
            v = (d.float() + x.float())
        else:
            ctx = self.ctx
            if self.comm == "peer":
                check(lib.qb_peer_wait(ctx.flag_own(ctx.FLAG_SLOT[1]), W, 0, ctx.epoch.data_ptr(), _stream()), "qb_peer_wait")
            sl = ctx.slots_view(1).float()
            v = sl[0]
            for s in range(1, W):
                v = v + sl[s]
            v = v + x.float()
        xf = v.to(torch.bfloat16).float()
        hid = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * self.norm_f.float()).to(torch.bfloat16)
        # rows of the last token of every sequence that this rank owns (static index tensors, cached per shape)
        src_idx, dst_idx = self._last_index(B, S, r0, Tl)
        last = torch.zeros((B, H), dtype=torch.float32, device=self.device)
        if src_idx.numel():
            last.index_copy_(0, dst_idx, hid.index_select(0, src_idx).float())
        self._last_rows = last
        self._mark("final_norm")
        yield hid, last

    def _last_index(self, B: int, S: int, r0: int, Tl: int):
        key = (B, S, r0, Tl)
        if key not in self._last_idx:
            own = [(b * S + S - 1 - r0, b) for b in range(B) if r0 <= b * S + S - 1 < r0 + Tl]
            self._last_idx[key] = (torch.tensor([o[0] for o in own], dtype=torch.long, device=self.device),
                                   torch.tensor([o[1] for o in own], dtype=torch.long, device=self.device))
        return self._last_idx[key]

    def _finish(self, hid: torch.Tensor, last: torch.Tensor):
        """Sum the last-token rows over the ranks (every rank filled the ones it owns) and take the logits."""
        if self.world > 1 and torch.distributed.is_initialized():
            last = last.clone()
            torch.distributed.all_reduce(last, group=self.group)
        return hid, (last.to(torch.bfloat16) @ self.lm_head.t()).float()

    def _mark(self, name: str):
        """With `self.timings` set to a dict, the device time between consecutive marks is added to timings[name]
        (events are resolved by `finish_timings`)."""
        if self.timings is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._marks.append((name, ev))

    def finish_timings(self):
        torch.cuda.synchronize()
        for (_, e0), (name, e1) in zip(self._marks[:-1], self._marks[1:]):
            self.timings[name] = self.timings.get(name, 0.0) + e0.elapsed_time(e1)
        self._marks = []
        return self.timings

    def _cap(self, name: str, t):
        if self.capture is not None:
            self.capture[name] = t.clone() if isinstance(t, torch.Tensor) else t

    def _cap_gathered(self, name: str, q, block: int, T: int):
        """Copy of the quantised activations a column-parallel GEMM is about to read: (Bbytes, atoms, g)."""
        if self.capture is None:
            return
        from .tp import view_u8
        H = self.cfg.hidden
        nb, ns = T * H // 2, self.lib.qb_sf_atoms_bytes(T, H, block)
        self.capture[name] = (view_u8(q[0], nb, self.device).clone().view(T, H // 2), view_u8(q[1], ns, self.device).clone(),
                              view_u8(q[2], T * 4, self.device).clone().view(torch.float32))

    def _quantize(self, x: torch.Tensor, block: int):
        lib = self.lib
        tok, K = x.shape
        Bb = torch.empty((tok, K // 2), dtype=torch.uint8, device=self.device)
        sf = (torch.zeros if K % 256 else torch.empty)(lib.qb_sf_atoms_bytes(tok, K, block), dtype=torch.uint8, device=self.device)
        g = torch.empty((tok,), dtype=torch.float32, device=self.device)
        check(lib.qb_quantize_act(x.data_ptr(), Bb.data_ptr(), 0, sf.data_ptr(), g.data_ptr(), tok, K, block, _stream()), "qb_quantize_act")
        return Bb, sf, g

    def forward(self, ids: torch.Tensor):
        out = None
        for out in self.forward_steps(ids.to(self.device)):
            pass
        return self._finish(*out)

    __call__ = forward

    def forward_graphed(self, ids: torch.Tensor):
        """`forward` with the whole layer stack replayed from one CUDA graph (captured on the first call for a shape, after
        two eager warm-up runs). The cross-GPU flag values are read from the device epoch when the kernels run, so the
        captured arguments stay valid; every rank must make the same sequence of calls."""
        key = tuple(ids.shape)
        if self._graph is None or self._graph_key != key:
            self._graph = None
            self._ids_static = ids.to(self.device).clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    for out in self.forward_steps(self._ids_static):
                        pass
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for out in self.forward_steps(self._ids_static):
                    pass
            self._graph, self._graph_key, self._graph_out = g, key, out
        self._ids_static.copy_(ids.to(self.device))
        self._graph.replay()
        return self._finish(*self._graph_out)


def forward_emulated(models, ids: torch.Tensor):
    """Drive `world` ranks that share one GPU in lock step (see tp.TPContext.emulated). Returns the list of per-rank
    (hidden_local, logits); the last-token rows are summed here in place of the all-reduce."""
    gens = [m.forward_steps(ids.to(m.device)) for m in models]
    outs = [None] * len(models)
    for step in zip(*gens):
        outs = list(step)
    last = sum(o[1] for o in outs)
    return [(o[0], (last.to(torch.bfloat16) @ m.lm_head.t()).float()) for o, m in zip(outs, models)]
