"""Sparse-NVFP4 MoE helpers with the contract of the reference's `fused_moe.py` entry point and
of the plugin's `_load_sparse_moe()` namespace (harness/fused_moe.py:372-435,
harness/qb_vllm_plugin/qb_sm120_plugin.py:1124-1368): pack / stack / quant_act / seg_gemm /
build_routing / route / seg_bw / combine, on the sm_100a library.

Expert weights are packed on the GPU and stacked along the output-feature axis; routed rows are
sorted by expert and every expert segment is padded to 128 rows, so one grouped GEMM launch
covers all experts (`eblk[row_block] -> expert`)."""
from __future__ import annotations

from types import SimpleNamespace

import torch

from ._lib import check, load
from .linear import _ptr, _stream, quantize_act, sf_atoms_empty

BN = 128   # routed-row block (reference: _BN, harness/fused_moe.py:352)


def pad_w(W: torch.Tensor) -> torch.Tensor:
    """Zero-pad [out,in] to out%256, in%128 (harness/fused_moe.py:444-448)."""
    out_f, in_f = W.shape
    outp, inp = (out_f + 255) // 256 * 256, (in_f + 127) // 128 * 128
    if (outp, inp) == (out_f, in_f):
        return W
    Wp = W.new_zeros(outp, inp)
    Wp[:out_f, :in_f] = W
    return Wp


def pack(lib, w: torch.Tensor):
    """[out,in] -> native packed expert weight (Ac, meta_native, sfa atoms, gA)."""
    w = w.contiguous()
    if w.dtype not in (torch.float32, torch.bfloat16):
        w = w.float()
    out_f, in_f = w.shape
    dev = w.device
    z = torch.zeros if in_f % 256 else torch.empty
    Ac = torch.empty((out_f, in_f // 4), dtype=torch.uint8, device=dev)
    meta = z(lib.qb_meta_native_bytes(out_f, in_f), dtype=torch.uint8, device=dev)
    sfa = z(lib.qb_sf_atoms_bytes(out_f, in_f, 32), dtype=torch.uint8, device=dev)
    gA = torch.empty((out_f,), dtype=torch.float32, device=dev)
    check(lib.qb_compress_2to4(w.data_ptr(), 1 if w.dtype == torch.bfloat16 else 0, Ac.data_ptr(), 0, meta.data_ptr(), 0,
                               sfa.data_ptr(), gA.data_ptr(), out_f, in_f, _stream()), "qb_compress_2to4")
    return Ac, meta, sfa, gA


def stack(packs):
    """Concatenate per-expert packs along the output-feature axis (every native array is
    row-block major, so this is a plain cat; out%128 per expert)."""
    return tuple(torch.cat([p[i] for p in packs], 0).contiguous() for i in range(4))


def build_routing(assign: torch.Tensor, e: int, with_pos: bool = False):
    """Sort routed slots by expert and pad segments to BN rows: (src, eblk, r_pad), as
    harness/fused_moe.py:421-435 but without the per-expert host loop. with_pos also returns
    pos[i] = padded row of routed slot i (the inverse of src on its valid entries)."""
    dev = assign.device
    order = torch.argsort(assign.to(torch.int16) if e < 32768 else assign, stable=True)    # 16-bit keys: 2 radix passes instead of 8
    counts = torch.bincount(assign, minlength=e)
    padc = (counts + BN - 1) // BN * BN
    poff = torch.cumsum(padc, 0) - padc
    r_pad = int(padc.sum().item())
    src = torch.full((r_pad,), -1, dtype=torch.long, device=dev)
    coff = torch.cumsum(counts, 0) - counts
    sorted_e = assign[order]
    within = torch.arange(order.numel(), device=dev) - coff[sorted_e]
    dst = poff[sorted_e] + within
    src[dst] = order
    eblk = torch.repeat_interleave(torch.arange(e, device=dev, dtype=torch.int32), (padc // BN))
    if with_pos:
        pos = torch.empty_like(order)
        pos[order] = dst
        return src, eblk.contiguous(), r_pad, pos
    return src, eblk.contiguous(), r_pad


def fixed_capacity(n: int, e: int, align: int = BN) -> int:
    """Rows that always hold n routed slots of e experts with every segment padded to `align` rows."""
    return (n + e * (align - 1) + align - 1) // align * align


def build_routing_fixed(assign: torch.Tensor, e: int):
    """`build_routing` without a host read: the padded row count is the worst case `fixed_capacity(n, e)`, blocks
    beyond the used ones carry expert id -1 (the grouped GEMM skips them) and their rows src = -1. Everything
    stays on the device with static shapes, so the layer can be captured in a CUDA graph (the reference's
    graph-safe fixed-capacity routing: route_fixed_cap, harness/qb_vllm_plugin/qb_sm120_plugin.py:1271-1315).
    Returns (src [r_cap], eblk [r_cap/BN], r_cap, pos [n])."""
    dev = assign.device
    n = assign.numel()
    r_cap = fixed_capacity(n, e)
    order = torch.argsort(assign.to(torch.int16) if e < 32768 else assign, stable=True)    # 16-bit keys: 2 radix passes instead of 8
    counts = torch.zeros(e, dtype=torch.long, device=dev).scatter_add_(0, assign, torch.ones_like(assign))
    padc = (counts + BN - 1) // BN * BN
    pend = torch.cumsum(padc, 0)
    poff = pend - padc
    coff = torch.cumsum(counts, 0) - counts
    sorted_e = assign[order]
    within = torch.arange(n, device=dev) - coff[sorted_e]
    dst = poff[sorted_e] + within
    src = torch.full((r_cap,), -1, dtype=torch.long, device=dev)
    src[dst] = order
    pos = torch.empty_like(order)
    pos[order] = dst
    blk0 = torch.arange(r_cap // BN, device=dev) * BN
    eb = torch.bucketize(blk0, pend, right=True)                 # expert whose padded segment holds the block
    eblk = torch.where(eb < e, eb, torch.full_like(eb, -1)).to(torch.int32)
    return src, eblk.contiguous(), r_cap, pos


def route_fixed_kernel(lib, assign: torch.Tensor, e: int):
    """`build_routing_fixed` as one kernel launch (qb_moe_route_fixed): same segments, capacity and expert-block table;
    the order of the rows inside an expert's segment follows the kernel's atomics."""
    dev = assign.device
    n = assign.numel()
    r_cap = fixed_capacity(n, e)
    assign = assign.long().contiguous()
    src = torch.empty((r_cap,), dtype=torch.long, device=dev)
    pos = torch.empty((n,), dtype=torch.long, device=dev)
    eblk = torch.empty((r_cap // BN,), dtype=torch.int32, device=dev)
    check(lib.qb_moe_route_fixed(assign.data_ptr(), src.data_ptr(), pos.data_ptr(), eblk.data_ptr(), n, e, r_cap, _stream()),
          "qb_moe_route_fixed")
    return src, eblk, r_cap, pos


def seg_gemm(lib, x_rows: torch.Tensor, w, mpe: int, in_f: int, eblk: torch.Tensor, bias=None, row_w=None):
    """Quantise routed rows and run the grouped GEMM: [r_pad, mpe] bf16 (token-major);
    with bias / row_w the epilogue computes (acc + bias[expert]) * row_w[row]."""
    Ac, meta, sfa, gA = w
    r = x_rows.shape[0]
    Bb, sfb, gB = quantize_act(lib, x_rows, 32, True)
    C = torch.empty((r, mpe), dtype=torch.bfloat16, device=x_rows.device)
    mode = 3 if (bias is not None or row_w is not None) else 1
    check(lib.qb_gemm(Ac.data_ptr(), Bb.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), meta.data_ptr(), gA.data_ptr(), gB.data_ptr(),
                      C.data_ptr(), 0, eblk.data_ptr(), _ptr(bias), _ptr(row_w), Ac.shape[0], mpe, r, in_f, 1, mode, 1, 128,
                      _stream()), "qb_gemm(grouped)")
    return C


def seg_gemm_q(lib, Bb, sfb, gB, w, mpe: int, in_f: int, eblk: torch.Tensor, bias=None, row_w=None, out=None, tile: int = 128):
    """Grouped GEMM on already quantised routed rows (Bb [r, in_f/2], scale atoms, gB [r]); out: optional [r, mpe] bf16.
    tile = 256 needs every expert's rows padded to 256."""
    Ac, meta, sfa, gA = w
    r = Bb.shape[0]
    C = out if out is not None else torch.empty((r, mpe), dtype=torch.bfloat16, device=Bb.device)
    mode = 3 if (bias is not None or row_w is not None) else 1
    check(lib.qb_gemm(Ac.data_ptr(), Bb.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), meta.data_ptr(), gA.data_ptr(), _ptr(gB),
                      C.data_ptr(), 0, eblk.data_ptr(), _ptr(bias), _ptr(row_w), Ac.shape[0], mpe, r, in_f, 1, mode, 1, tile,
                      _stream()), "qb_gemm(grouped)")
    return C


def combine(lib, dbuf: torch.Tensor, inverse: torch.Tensor, t: int, H: int, topk: int):
    y = torch.empty((t, H), dtype=torch.bfloat16, device=dbuf.device)
    check(lib.moe_combine_topk(dbuf.data_ptr(), inverse.data_ptr(), y.data_ptr(), t, H, topk, dbuf.shape[1], _stream()),
          "moe_combine_topk")
    return y


def swiglu(gate, up):
    """gpt-oss clamped SwiGLU (harness/fused_moe.py:450-452)."""
    gate = gate.clamp(max=7.0)
    up = up.clamp(-7.0, 7.0)
    return (gate * torch.sigmoid(1.702 * gate)) * (up + 1.0)


class SparseMoE:
    """Top-k routed SwiGLU MoE layer on 2:4-sparse NVFP4 experts: route -> gather -> grouped
    gate/up GEMM -> SwiGLU -> grouped down GEMM with the routing weight in the epilogue ->
    top-k combine. `experts` (optional) restricts the layer to a contiguous expert range
    [e0, e1) for expert parallelism; slots of other experts are skipped."""

    def __init__(self, w_gate_up: list[torch.Tensor], w_down: list[torch.Tensor], topk: int, act: str = "silu",
                 expert_range: tuple[int, int] | None = None, n_experts_total: int | None = None, fixed_capacity: bool = False,
                 b_gate_up: list[torch.Tensor] | None = None, b_down: list[torch.Tensor] | None = None, fused_gu: bool = False):
        self.lib = lib = load("sparse_fp4")
        self.E = len(w_gate_up)
        self.topk, self.act = topk, act
        self.H = w_gate_up[0].shape[1]
        self.I = w_down[0].shape[1]
        self.Hp = (self.H + 127) // 128 * 128
        self.Ip = (self.I + 127) // 128 * 128
        self.mpe_gu = (2 * self.Ip + 255) // 256 * 256       # multiples of 256: the grouped GEMM then runs on the CTA-pair kernel
        self.mpe_dn = (self.H + 255) // 256 * 256
        # fused_gu: SwiGLU + single-level per-32 quantiser of h run in the epilogue of the gate/up GEMM (qb_gemm_swiglu, the
        # reference's fused GEMM1, cuda/sparse_fp4_lib.cu:1679-1868): the gate/up rows are stored as (gate, up) pairs, the bf16
        # [rows, 2*Ip] intermediate and the SwiGLU kernel disappear, and h carries no per-row global (as in the reference's
        # MoE path). Without it h is quantised two-level by a separate kernel.
        self.fused_gu = fused_gu
        gus, dns = [], []
        for wg, wd in zip(w_gate_up, w_down):
            g = wg.new_zeros(self.mpe_gu, self.Hp)
            if fused_gu:                                           # row 2i = gate i, row 2i + 1 = up i
                g[0: 2 * self.I: 2, : self.H] = wg[: self.I]
                g[1: 2 * self.I: 2, : self.H] = wg[self.I:]
            else:                                                  # gate rows [0,I), up rows [Ip, Ip+I)
                g[: self.I, : self.H] = wg[: self.I]
                g[self.Ip: self.Ip + self.I, : self.H] = wg[self.I:]
            d = wd.new_zeros(self.mpe_dn, self.Ip)
            d[: self.H, : self.I] = wd
            gus.append(pack(lib, g))
            dns.append(pack(lib, d))
        self.w_gu, self.w_dn = stack(gus), stack(dns)
        # optional expert biases (gpt-oss: w13_bias [2I] gate then up, w2_bias [H]); applied in the epilogues of the
        # grouped GEMMs: gate/up + bias before SwiGLU, (down + bias) * routing weight (the reference's gu_bias / bias,
        # harness/qb_vllm_plugin/qb_sm120_plugin.py:2192-2225,2397-2400). Rows are padded like the weights.
        self.b_gu = self.b_dn = None
        if b_gate_up is not None:
            b = w_gate_up[0].new_zeros((self.E, self.mpe_gu), dtype=torch.bfloat16)
            for e, be in enumerate(b_gate_up):
                if fused_gu:
                    b[e, 0: 2 * self.I: 2] = be[: self.I].to(torch.bfloat16)
                    b[e, 1: 2 * self.I: 2] = be[self.I:].to(torch.bfloat16)
                else:
                    b[e, : self.I] = be[: self.I].to(torch.bfloat16)
                    b[e, self.Ip: self.Ip + self.I] = be[self.I:].to(torch.bfloat16)
            self.b_gu = b.contiguous()
        if b_down is not None:
            b = w_down[0].new_zeros((self.E, self.mpe_dn), dtype=torch.bfloat16)
            for e, be in enumerate(b_down):
                b[e, : self.H] = be.to(torch.bfloat16)
            self.b_dn = b.contiguous()
        self.e0, self.e1 = expert_range if expert_range else (0, self.E)
        self.E_total = n_experts_total or self.E
        # fixed_capacity: route into the worst-case number of padded rows instead of reading the exact count back
        # from the device; `forward` then issues no host read and can be captured in a CUDA graph
        self.fixed_capacity = fixed_capacity
        # Rows every expert's segment is padded to in the one-kernel fixed-capacity routing. The CTA-pair MMA takes as long for
        # a 128-token tile as for a 256-token one, so with segments padded to 256 an expert with 129..256 rows costs one
        # tile instead of two (and 257..384 two instead of three); the padding rows cost the quantisers next to nothing.
        self.row_align = 256

    def _side_stream(self, dev):
        st = getattr(self, "_side", None)
        if st is None or st.device != torch.device(dev):
            st = self._side = torch.cuda.Stream(device=dev)
        return st

    def quantize_tokens(self, x: torch.Tensor, out=None):
        """x [T, H] bf16 -> (codes [T, Hp/2] u8, scales [Hp/128, T, 4] u8, globals [T] f32): the layer's input quantiser
        (two-level, per-32), hidden size zero-padded to Hp. `out`: optional (codes ptr, scales ptr, globals ptr) to write to."""
        x = x.to(torch.bfloat16).contiguous()
        if self.H % 8:                           # the quantiser reads 16-byte chunks
            x = torch.nn.functional.pad(x, (0, self.Hp - self.H))
        T = x.shape[0]
        if out is None:
            Bq = torch.empty((T, self.Hp // 2), dtype=torch.uint8, device=x.device)
            sq = torch.empty((self.Hp // 128, T, 4), dtype=torch.uint8, device=x.device)
            gq = torch.empty((T,), dtype=torch.float32, device=x.device)
            ptrs = (Bq.data_ptr(), sq.data_ptr(), gq.data_ptr())
        else:
            Bq = sq = gq = None
            ptrs = out
        if T:
            check(self.lib.qb_quantize_rows(x.data_ptr(), ptrs[0], ptrs[1], ptrs[2], T, self.Hp, x.shape[1], 32, _stream()), "qb_quantize_rows")
        return Bq, sq, gq

    def _run_padded(self, x, src: torch.Tensor, eblk: torch.Tensor, r_pad: int, rw: torch.Tensor, peer_x=None, d_out=None,
                    n_used=None, tile: int = 128, xq=None) -> torch.Tensor:
        """The four kernels of the layer on a routed, padded batch: src [r_pad] = row of x for every padded row (-1 =
        padding), eblk = expert of every 128-row block, rw [r_pad] = routing weight of every row. Returns
        d [r_pad, mpe_dn] bf16 = expert(row) * weight."""
        lib = self.lib
        dev = src.device
        nu = n_used.data_ptr() if n_used is not None else 0       # device int: rows in use (fixed-capacity routing), else all
        Bb = torch.empty((r_pad, self.Hp // 2), dtype=torch.uint8, device=dev)
        sfb = sf_atoms_empty(lib, r_pad, self.Hp, 32, dev)
        gB = torch.empty((r_pad,), dtype=torch.float32, device=dev)
        # Every token is quantised ONCE; its routed slots copy the packed row (codes, scales, global): a token with top-k
        # slots is not quantised k times, and what moves (over NVLink, with peers) is 0.53 bytes per value instead of 2.
        if peer_x is not None:
            # src holds GLOBAL token rows; the quantised rows are pulled from the ranks that hold them
            # (peer_x = (code pointers, scale pointers, global pointers, rows per rank, number of ranks))
            qc, qs, qg, rows_per_rank, nr = peer_x
        else:
            from .tp import ptr_array
            rows_per_rank, nr = max(x.shape[0], 1), 1
            Bq, sq, gq = xq if xq is not None else self.quantize_tokens(x)       # xq: quantised by the caller (beside the routing)
            qc, qs, qg = ptr_array([Bq.data_ptr()]), ptr_array([sq.data_ptr()]), ptr_array([gq.data_ptr()])
        check(lib.qb_gather_quantized(qc, qs, qg, nr, rows_per_rank, src.data_ptr(), Bb.data_ptr(), sfb.data_ptr(), gB.data_ptr(), r_pad,
                                      self.Hp, nu, _stream()), "qb_gather_quantized")
        Hb = torch.empty((r_pad, self.Ip // 2), dtype=torch.uint8, device=dev)
        sfh = sf_atoms_empty(lib, r_pad, self.Ip, 32, dev)
        if self.fused_gu:
            Ac, meta, sfa, gA = self.w_gu
            assert self.mpe_gu == 2 * self.Ip
            check(lib.qb_gemm_swiglu(Ac.data_ptr(), Bb.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), meta.data_ptr(), gA.data_ptr(), gB.data_ptr(),
                                     eblk.data_ptr(), _ptr(self.b_gu), Hb.data_ptr(), sfh.data_ptr(), 0, Ac.shape[0], self.mpe_gu, r_pad, self.Hp,
                                     1, 0 if self.act == "gptoss" else 1, _stream()), "qb_gemm_swiglu")
            return seg_gemm_q(lib, Hb, sfh, None, self.w_dn, self.mpe_dn, self.Ip, eblk, bias=self.b_dn, row_w=rw, out=d_out, tile=tile)
        gu = seg_gemm_q(lib, Bb, sfb, gB, self.w_gu, self.mpe_gu, self.Hp, eblk, bias=self.b_gu, tile=tile)   # [r_pad, 2*Ip]: gate | up
        gH = torch.empty((r_pad,), dtype=torch.float32, device=dev)
        check(lib.qb_swiglu_quant_act(gu.data_ptr(), Hb.data_ptr(), 0, sfh.data_ptr(), gH.data_ptr(), src.data_ptr(), nu, r_pad, self.Ip, 0,
                                      0 if self.act == "gptoss" else 1, _stream()), "qb_swiglu_quant_act")
        return seg_gemm_q(lib, Hb, sfh, gH, self.w_dn, self.mpe_dn, self.Ip, eblk, bias=self.b_dn, row_w=rw, out=d_out, tile=tile)  # [r_pad, mpe_dn]

    def _expert_rows_padded(self, rows_in: torch.Tensor, assign: torch.Tensor, row_w: torch.Tensor, row_of=None):
        """Routed rows through this layer's experts in the padded, expert-sorted row order of the grouped GEMM:
        returns (d [r_pad, mpe_dn] bf16 = expert(row) * weight, pos [n] = padded row of routed row i).
        Routed row i is rows_in[i], or rows_in[row_of[i]] when row_of is given (tokens are then not copied
        once per routed slot before the gather). Four kernels between the routing and the result: gather + pad +
        quantise, grouped gate/up GEMM, SwiGLU + quantise, grouped down GEMM with the routing weight in its epilogue."""
        dev = rows_in.device
        if self.fixed_capacity:
            src, eblk, r_pad, pos = route_fixed_kernel(self.lib, assign, self.e1 - self.e0)
        else:
            src, eblk, r_pad, pos = build_routing(assign.long(), self.e1 - self.e0, with_pos=True)
        if row_of is not None:
            src = torch.where(src >= 0, row_of[src.clamp_min(0)], src)
        rw = torch.zeros((r_pad + 1,), dtype=torch.float32, device=dev)
        # an expert id outside the layer's range has no row (pos = -1, fixed-capacity routing): its weight goes to a spare slot
        rw[torch.where(pos >= 0, pos, torch.full_like(pos, r_pad))] = row_w.float()
        return self._run_padded(rows_in, src, eblk, r_pad, rw[:r_pad]), pos

    def expert_rows(self, rows_in: torch.Tensor, assign: torch.Tensor, row_w: torch.Tensor) -> torch.Tensor:
        """rows_in [n,H] bf16, assign [n] local expert ids, row_w [n] routing weights -> [n,H] bf16 =
        expert(row) * weight, in the order of rows_in. Every row is quantised on its own and summed over K
        in a fixed order, so the result of a row does not depend on which other rows share the call (what
        makes the expert-parallel layer equal the 1-GPU one)."""
        if rows_in.shape[0] == 0:
            return torch.zeros((0, self.H), dtype=torch.bfloat16, device=rows_in.device)
        d, pos = self._expert_rows_padded(rows_in, assign, row_w)
        out = torch.index_select(d[:, : self.H], 0, pos.clamp_min(0))          # one pass: gathers the H valid features of each row
        return out * (pos >= 0).unsqueeze(1).to(out.dtype)                    # an id outside the expert range contributes nothing

    def forward(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
        """x [T,H] bf16, topk_idx [T,topk] global expert ids, topk_w [T,topk] -> [T,H] bf16
        (the partial sum over this rank's experts under expert parallelism)."""
        T = x.shape[0]
        dev = x.device
        assign_g = topk_idx.reshape(-1).long()
        if self.e0 == 0 and self.e1 == self.E_total and self.fixed_capacity:
            # routing, token row of every padded row, routing weight of every row and the combine table in one launch
            n, e = assign_g.numel(), self.E
            al = self.row_align
            # the token quantiser does not depend on the routing: it runs on a second stream beside the routing kernel
            # (fork / join with events, which a CUDA-graph capture records as parallel branches)
            main = torch.cuda.current_stream()
            side = self._side_stream(dev)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                xq = self.quantize_tokens(x)
            for t in xq:
                t.record_stream(main)
            r_cap = fixed_capacity(n, e, al)
            src = torch.empty((r_cap,), dtype=torch.long, device=dev)
            pos = torch.empty((n,), dtype=torch.long, device=dev)
            eblk = torch.empty((r_cap // BN,), dtype=torch.int32, device=dev)
            rw = torch.empty((r_cap,), dtype=torch.float32, device=dev)
            inverse = torch.empty((n,), dtype=torch.int32, device=dev)
            w_in = topk_w.reshape(-1).float().contiguous()
            n_used = torch.empty((1,), dtype=torch.int32, device=dev)
            check(self.lib.qb_moe_route_fixed_range(assign_g.contiguous().data_ptr(), src.data_ptr(), pos.data_ptr(), eblk.data_ptr(), n, 0, e,
                                                    r_cap, self.topk, al, w_in.data_ptr(), rw.data_ptr(), inverse.data_ptr(),
                                                    n_used.data_ptr(), _stream()), "qb_moe_route_fixed_range")
            main.wait_stream(side)
            d = self._run_padded(x, src, eblk, r_cap, rw, n_used=n_used, tile=al, xq=xq)
            return combine(self.lib, d, inverse, T, self.H, self.topk)
        if self.e0 == 0 and self.e1 == self.E_total:
            slots = torch.arange(assign_g.numel(), device=dev)
        else:
            local = (assign_g >= self.e0) & (assign_g < self.e1)
            slots = torch.nonzero(local).squeeze(1)                      # routed slots owned here
            if slots.numel() == 0:
                return torch.zeros((T, self.H), dtype=torch.bfloat16, device=dev)
        d, pos = self._expert_rows_padded(x, assign_g[slots] - self.e0, topk_w.reshape(-1)[slots], row_of=slots // self.topk)
        inverse = torch.full((T * self.topk,), -1, dtype=torch.int32, device=dev)
        inverse[slots] = pos.int()
        return combine(self.lib, d, inverse, T, self.H, self.topk)

    def forward_ep(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, group=None) -> torch.Tensor:
        """Expert-parallel layer over the ranks of `group`: this rank holds experts [e0, e1) and its own
        tokens x [T_local,H]; routed rows travel to their expert's rank and back with two all-to-all
        exchanges (`dist.ep_moe`), the top-k sum runs at home. Equals `forward` of a 1-rank layer."""
        from . import dist as qd
        return qd.ep_moe(x, topk_idx, topk_w, self.E_total, self.expert_rows,
                         lambda d, inverse, T: combine(self.lib, d, inverse, T, self.H, self.topk), group)

    # ------------------------------------------------------------------ expert parallelism by peer loads
    def ep_capacity(self, T: int) -> int:
        """Routed rows a rank must be able to hold when all T * topk slots could land on its experts."""
        return fixed_capacity(T * self.topk, self.e1 - self.e0, self.row_align)

    def make_ep_context(self, T: int, rank: int, world: int, group=None, emulate=None):
        from .tp import EPContext
        width = self.Hp if self.H % 8 else self.H
        if emulate is not None:
            return emulate
        return EPContext(T, width, self.topk, self.mpe_dn, self.ep_capacity(T), rank, world, group)

    def forward_ep_peer_steps(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, ctx):
        """Expert-parallel layer without a collective library and without a host read (a generator that yields where
        other ranks are waited for, so that one process can drive emulated ranks; the last value is y [T_local, H]).

        This rank holds experts [e0, e1) and tokens x [T_local, H]. (1) Every rank quantises its tokens once into a
        peer-visible buffer and stores its routing (expert ids, weights) into the replicated tables of all ranks. (2) Every
        rank routes ALL slots onto its own experts with the one-kernel fixed-capacity routing, pulls the QUANTISED rows it
        needs from their home ranks (qb_gather_quantized), and runs its experts. (3) Every rank combines the
        top-k rows of its own tokens, reading them from the experts' owners. Flags carry the device epoch, so the whole
        layer has fixed kernel arguments (CUDA-graph replay). Equals `forward` of a 1-rank layer."""
        lib, W, rank = self.lib, ctx.world, ctx.rank
        T, Tl, topk = ctx.T, ctx.Tl, self.topk
        dev = x.device
        epr = self.e1 - self.e0
        assert x.shape[0] == Tl and self.E_total == epr * W and self.e0 == rank * epr
        idx = topk_idx.reshape(-1).long().contiguous()
        w = topk_w.reshape(-1).float().contiguous()
        n = T * topk
        ep = ctx.epoch.data_ptr()
        ctx.bump(_stream())
        # this rank's tokens, quantised once, straight into its peer-visible buffer: codes | scales | globals
        off_sf = (Tl * (self.Hp // 2) + 255) // 256 * 256
        off_g = off_sf + ((self.Hp // 128) * Tl * 4 + 255) // 256 * 256
        assert off_g + Tl * 4 <= ctx.sizes[0]
        self.quantize_tokens(x, out=(ctx.own(0), ctx.own(0, off_sf), ctx.own(0, off_g)))
        check(lib.qb_ep_publish(0, 0, 0, idx.data_ptr(), w.data_ptr(), Tl * topk, rank * Tl * topk,
                                ctx.ptrs(1), ctx.ptrs(1, ctx.off_w), W, rank, ctx.flag_ptrs(ctx.FLAG_PUBLISHED), ep, ctx.done.data_ptr(),
                                _stream()), "qb_ep_publish")
        yield None
        check(lib.qb_peer_wait(ctx.flag_own(ctx.FLAG_PUBLISHED), W, 0, ep, _stream()), "qb_peer_wait")
        r_cap = ctx.r_cap
        src = torch.empty((r_cap,), dtype=torch.long, device=dev)
        pos = torch.empty((n,), dtype=torch.long, device=dev)
        eblk = torch.empty((r_cap // BN,), dtype=torch.int32, device=dev)
        rw = torch.empty((r_cap,), dtype=torch.float32, device=dev)
        n_used = torch.empty((1,), dtype=torch.int32, device=dev)
        assert r_cap == self.ep_capacity(T)
        check(lib.qb_moe_route_fixed_range(ctx.own(1), src.data_ptr(), pos.data_ptr(), eblk.data_ptr(), n, self.e0, epr, r_cap, topk,
                                           self.row_align, ctx.own(1, ctx.off_w), rw.data_ptr(), ctx.own(3), n_used.data_ptr(), _stream()),
              "qb_moe_route_fixed_range")
        d_out = ctx.own_tensor(2)[: r_cap * self.mpe_dn * 2].view(torch.bfloat16).view(r_cap, self.mpe_dn)
        self._run_padded(None, src, eblk, r_cap, rw, peer_x=(ctx.ptrs(0), ctx.ptrs(0, off_sf), ctx.ptrs(0, off_g), Tl, W), d_out=d_out,
                         n_used=n_used, tile=self.row_align)
        check(lib.qb_peer_signal(ctx.flag_ptrs(ctx.FLAG_OUTPUT), W, rank, 0, ep, _stream()), "qb_peer_signal")
        yield None
        check(lib.qb_peer_wait(ctx.flag_own(ctx.FLAG_OUTPUT), W, 0, ep, _stream()), "qb_peer_wait")
        y = torch.empty((Tl, self.H), dtype=torch.bfloat16, device=dev)
        check(lib.qb_ep_combine(ctx.ptrs(2), ctx.ptrs(3), idx.data_ptr(), y.data_ptr(), Tl, rank * Tl, self.H, topk, self.mpe_dn, epr, W,
                                _stream()), "qb_ep_combine")
        yield y

    def forward_ep_peer(self, x, topk_idx, topk_w, ctx):
        y = None
        for y in self.forward_ep_peer_steps(x, topk_idx, topk_w, ctx):
            pass
        return y

    __call__ = forward


def load_sparse_moe():
    """Namespace with the names of the plugin's `_load_sparse_moe()` (qb_sm120_plugin.py:1364-1368)."""
    lib = load("sparse_fp4")
    return SimpleNamespace(lib=lib, pack=lambda w: pack(lib, w), stack=stack,
                           quant_act=lambda x, in_f=None: quantize_act(lib, x, 32, True),
                           seg_gemm=lambda x, w, mpe, in_f, eblk: seg_gemm(lib, x, w, mpe, in_f, eblk),
                           seg_bw=lambda x, w, mpe, in_f, eblk, row_w, bias=None: seg_gemm(lib, x, w, mpe, in_f, eblk, bias, row_w),
                           build_routing=build_routing, combine=lambda d, inv, t, H, topk: combine(lib, d, inv, t, H, topk),
                           pad_w=pad_w, swiglu=swiglu)
