"""GPU parity of the reference-named entry points that fuse a tail into the grouped MoE GEMM
(sparse_moe_mm_2lvl_scatter, sparse_moe_gu_swiglu, cuda/sparse_fp4_lib.cu:1649,1875) and of the dense
library's per-16 glue (rmsnorm_nvfp4, swiglu_nvfp4, cuda/dense_nvfp4_fast_lib.cu:251,274), against
the CPU oracle. Tolerances as in the other GPU tests: bf16 outputs |y - ref| / (|ref| + 1) < 6e-3; the
quantisers behind a device exp / rsqrt may differ from the oracle on codes that sit on a rounding
boundary (mismatch fraction < 5e-3)."""
import pytest
import torch

from oracle import fakequant as fq

pytestmark = pytest.mark.gpu


def S():
    return torch.cuda.current_stream().cuda_stream


@pytest.fixture(scope="module")
def lib():
    import quadbit_b200 as qb
    return qb.load("sparse_fp4")


def _routed_problem(E, Mpe, K, T, topk, seed):
    torch.manual_seed(seed)
    Ws = [torch.randn(Mpe, K) * 0.02 for _ in range(E)]
    packs = [fq.pack_weight_sparse_2lvl(w) for w in Ws]
    dev = dict(Ac=torch.cat([p[0] for p in packs], 0).cuda(), meta=torch.cat([p[1] for p in packs], 1).contiguous().cuda(),
               scaleA=torch.cat([p[2] for p in packs], 1).contiguous().cuda(), gA=torch.cat([p[3] for p in packs], 0).cuda())
    x = torch.randn(T, K)
    idx, w = fq.route_topk(torch.randn(T, E), topk)
    src, eblk, r_pad = fq.build_routing(idx.reshape(-1), E)
    rows = torch.zeros(r_pad, K)
    valid = src >= 0
    rows[valid] = x[src[valid] // topk]
    return Ws, dev, rows, src, valid, eblk, r_pad, w


def _quantise_rows(lib, rows, r_pad, K):
    xb = rows.to(torch.bfloat16).cuda()
    Bb = torch.empty((r_pad, K // 2), dtype=torch.uint8, device="cuda")
    sB = torch.empty((K // 128, r_pad, 4), dtype=torch.uint8, device="cuda")
    gB = torch.empty((r_pad,), dtype=torch.float32, device="cuda")
    lib.quantize_act_nvfp4_2lvl_s(xb.data_ptr(), Bb.data_ptr(), sB.data_ptr(), gB.data_ptr(), r_pad, K, S())
    return Bb, sB, gB


@pytest.mark.parametrize("Hout", [256, 200])
def test_scatter_entry_adds_bias_weight_into_token_rows(lib, Hout):
    """Out[tok] += (down + bias[expert]) * weight over the routed rows, padding rows skipped and padded
    features (f >= Hout) left out; twice in a row to cover the reused scratch buffer."""
    E, Mpe, K, T, topk = 4, 256, 512, 80, 2
    Ws, d, rows, src, valid, eblk, r_pad, w = _routed_problem(E, Mpe, K, T, topk, 11)
    Bb, sB, gB = _quantise_rows(lib, rows, r_pad, K)
    bias = (torch.randn(E, Hout) * 0.1).to(torch.bfloat16)
    sc_w = torch.zeros(r_pad)
    sc_w[valid] = w.reshape(-1)[src[valid]]
    sc_tok = torch.full((r_pad,), -1, dtype=torch.int32)
    sc_tok[valid] = (src[valid] // topk).int()
    eb, bias_d, sc_w_d, sc_tok_d = eblk.cuda(), bias.cuda(), sc_w.cuda(), sc_tok.cuda()
    ref_rows = fq.moe_seg_linear(rows, eblk, Ws)[:, :Hout]
    eidx = eblk.long().repeat_interleave(128)
    contrib = (ref_rows + bias.float()[eidx]) * sc_w[:, None]
    ref = torch.zeros(T, Hout)
    ref.index_add_(0, sc_tok[valid].long(), contrib[valid])
    for _ in range(2):
        Out = torch.zeros((T, Hout), dtype=torch.float32, device="cuda")
        rc = lib.sparse_moe_mm_2lvl_scatter(d["Ac"].data_ptr(), Bb.data_ptr(), d["scaleA"].data_ptr(), sB.data_ptr(), d["meta"].data_ptr(),
                                            E * Mpe, Mpe, r_pad, K, d["gA"].data_ptr(), gB.data_ptr(), eb.data_ptr(), sc_tok_d.data_ptr(),
                                            sc_w_d.data_ptr(), bias_d.data_ptr(), Out.data_ptr(), Hout, S())
        assert rc == 0 and lib.qb_status(S()) == 0
        err = ((Out.cpu() - ref).abs() / (ref.abs() + 1.0)).max().item()
        assert err < 6e-3, err


def test_bias_weight_entry_with_padded_features(lib):
    """sparse_moe_mm_2lvl_bw with Hout < Mpe: the bias is [E][Hout] and padded features get none."""
    E, Mpe, K, T, topk, Hout = 3, 256, 256, 50, 2, 192
    Ws, d, rows, src, valid, eblk, r_pad, w = _routed_problem(E, Mpe, K, T, topk, 12)
    Bb, sB, gB = _quantise_rows(lib, rows, r_pad, K)
    bias = (torch.randn(E, Hout) * 0.1).to(torch.bfloat16)
    sc_w = torch.zeros(r_pad)
    sc_w[valid] = w.reshape(-1)[src[valid]]
    eb, bias_d, sc_w_d = eblk.cuda(), bias.cuda(), sc_w.cuda()
    C = torch.empty((r_pad, Mpe), dtype=torch.bfloat16, device="cuda")
    rc = lib.sparse_moe_mm_2lvl_bw(d["Ac"].data_ptr(), Bb.data_ptr(), d["scaleA"].data_ptr(), sB.data_ptr(), d["meta"].data_ptr(), C.data_ptr(),
                                   E * Mpe, Mpe, r_pad, K, d["gA"].data_ptr(), gB.data_ptr(), eb.data_ptr(), sc_w_d.data_ptr(),
                                   bias_d.data_ptr(), Hout, S())
    assert rc == 0 and lib.qb_status(S()) == 0
    ref = fq.moe_seg_linear(rows, eblk, Ws)
    bpad = torch.zeros(E, Mpe)
    bpad[:, :Hout] = bias.float()
    ref = (ref + bpad[eblk.long().repeat_interleave(128)]) * sc_w[:, None]
    err = ((C.float().cpu() - ref).abs() / (ref.abs() + 1.0)).max().item()
    assert err < 6e-3, err


@pytest.mark.parametrize("act", [0, 1])
def test_gate_up_swiglu_entry_matches_unfused_path(lib, act):
    """sparse_moe_gu_swiglu == grouped GEMM (+ bias) -> SwiGLU over interleaved (gate, up) rows -> single-level
    per-32 quantiser, checked against the oracle applied to the bf16 output of the plain grouped entry."""
    E, Ih, K, T, topk = 3, 128, 512, 70, 2
    Mpe = 2 * Ih
    Ws, d, rows, src, valid, eblk, r_pad, w = _routed_problem(E, Mpe, K, T, topk, 13 + act)
    Bb, sB, gB = _quantise_rows(lib, rows, r_pad, K)
    eb = eblk.cuda()
    bias = (torch.randn(E, Mpe) * 0.2).to(torch.bfloat16)
    bias_d = bias.cuda()
    ones = torch.ones(r_pad, device="cuda")
    Cgu = torch.empty((r_pad, Mpe), dtype=torch.bfloat16, device="cuda")
    assert lib.sparse_moe_mm_2lvl_bw(d["Ac"].data_ptr(), Bb.data_ptr(), d["scaleA"].data_ptr(), sB.data_ptr(), d["meta"].data_ptr(),
                                     Cgu.data_ptr(), E * Mpe, Mpe, r_pad, K, d["gA"].data_ptr(), gB.data_ptr(), eb.data_ptr(),
                                     ones.data_ptr(), bias_d.data_ptr(), Mpe, S()) == 0
    Hw = torch.empty((r_pad, Ih // 2), dtype=torch.uint8, device="cuda")
    sH = torch.empty((Ih // 128, r_pad, 4), dtype=torch.uint8, device="cuda")
    rc = lib.sparse_moe_gu_swiglu(d["Ac"].data_ptr(), Bb.data_ptr(), d["scaleA"].data_ptr(), sB.data_ptr(), d["meta"].data_ptr(),
                                  E * Mpe, Mpe, r_pad, K, d["gA"].data_ptr(), gB.data_ptr(), eb.data_ptr(), bias_d.data_ptr(),
                                  Hw.data_ptr(), sH.data_ptr(), Ih, act, S())
    assert rc == 0 and lib.qb_status(S()) == 0
    gu = Cgu.float().cpu()
    ref_gu = fq.moe_seg_linear(rows, eblk, Ws) + bias.float()[eblk.long().repeat_interleave(128)]
    assert ((gu - ref_gu).abs() / (ref_gu.abs() + 1.0)).max().item() < 6e-3
    g, u = gu[:, 0::2], gu[:, 1::2]
    if act == 0:
        g = g.clamp(max=7.0)
        u = u.clamp(-7.0, 7.0)
        h = (g / (1.0 + torch.exp(-1.702 * g))) * (u + 1.0)
    else:
        h = (g / (1.0 + torch.exp(-g))) * u
    eB, eS = fq.act_quant_1lvl(h, 32, round_bf16=False)
    want = fq.unpack_act(eB, eS, None, 32)
    deq = fq.unpack_act(Hw.cpu(), sH.cpu(), None, 32)
    assert (deq != want).float().mean().item() < 5e-3
    # single-level scales bottom out at 2^-9, so small h quantise coarsely: compare with the oracle's own error
    assert ((deq - h).norm() / h.norm()).item() < 1.02 * ((want - h).norm() / h.norm()).item() + 1e-3


def test_dense_library_glue_per16():
    """rmsnorm_nvfp4 (with and without the residual add) and swiglu_nvfp4: per-16 single-level."""
    import quadbit_b200 as qb
    lib = qb.load("dense_nvfp4")
    torch.manual_seed(5)
    tok, H, eps = 37, 1024, 1e-5
    x = torch.randn(tok, H).to(torch.bfloat16)
    r = torch.randn(tok, H).to(torch.bfloat16)
    wt = (1 + 0.1 * torch.randn(H)).to(torch.bfloat16)
    xd, rd, wd = x.cuda(), r.cuda(), wt.cuda()
    for add in (False, True):
        Bb = torch.empty((tok, H // 2), dtype=torch.uint8, device="cuda")
        SFB = torch.empty((H // 128, tok, 8), dtype=torch.uint8, device="cuda")
        hout = torch.empty((tok, H), dtype=torch.bfloat16, device="cuda")
        lib.rmsnorm_nvfp4(xd.data_ptr(), rd.data_ptr() if add else 0, wd.data_ptr(), hout.data_ptr() if add else 0, Bb.data_ptr(),
                          SFB.data_ptr(), tok, H, eps)
        assert lib.qb_last_error() == 0 and lib.qb_status(0) == 0
        y, v16 = fq.rmsnorm_fp32(x, wt, eps, r if add else None)
        if add:
            assert torch.equal(hout.cpu(), v16)
        eB, eS = fq.act_quant_1lvl(y, 16, round_bf16=False)
        deq = fq.unpack_act(Bb.cpu(), SFB.cpu(), None, 16)
        want = fq.unpack_act(eB, eS, None, 16)
        assert (deq != want).float().mean().item() < 5e-3
        assert ((deq - y).norm() / y.norm()).item() < 0.12
    batch, hidden = 72, 512
    g = (torch.randn(hidden, batch) * 1.5).to(torch.bfloat16)
    u = (torch.randn(hidden, batch) * 1.5).to(torch.bfloat16)
    gd, ud = g.cuda(), u.cuda()
    Hb = torch.empty((batch, hidden // 2), dtype=torch.uint8, device="cuda")
    SFH = torch.empty((hidden // 128, batch, 8), dtype=torch.uint8, device="cuda")
    lib.swiglu_nvfp4(gd.data_ptr(), ud.data_ptr(), Hb.data_ptr(), SFH.data_ptr(), batch, hidden)
    assert lib.qb_last_error() == 0 and lib.qb_status(0) == 0
    gf, uf = g.float().t(), u.float().t()
    h = (gf / (1.0 + torch.exp(-gf))) * uf
    eB, eS = fq.act_quant_1lvl(h, 16, round_bf16=False)
    want = fq.unpack_act(eB, eS, None, 16)
    deq = fq.unpack_act(Hb.cpu(), SFH.cpu(), None, 16)
    assert (deq != want).float().mean().item() < 5e-3
    assert ((deq - h).norm() / h.norm()).item() < 0.12


def test_plugin_namespace_with_reference_layouts():
    """`load_sparse_moe_reference_layout()` carries the 14 names of the plugin's `_load_sparse_moe()` namespace with its
    signatures: pack -> stack -> route / route_fixed_cap -> quant_into -> seg_into / seg_bw / down_scatter / gu_swiglu -> combine."""
    import quadbit_b200.moe as qmoe
    sp = qmoe.load_sparse_moe_reference_layout()
    for name in ("lib pack stack quant_act seg_gemm build_routing quant_into seg_into route_fixed_cap gu_swiglu down_scatter seg_bw "
                 "combine route").split():
        assert hasattr(sp, name), name
    torch.manual_seed(17)
    E, Mpe, K, T, topk = 4, 256, 256, 60, 2
    Ws = [torch.randn(Mpe, K) * 0.02 for _ in range(E)]
    packs = [sp.pack(w.cuda()) for w in Ws]
    for p, w in zip(packs, Ws):                                   # the CUDA packer equals the oracle's, bit for bit
        for a, b in zip(p, fq.pack_weight_sparse_2lvl(w)):
            assert torch.equal(a.cpu(), b)
    w = sp.stack(packs)
    x = torch.randn(T, K)
    idx, wt = fq.route_topk(torch.randn(T, E), topk)
    assign = idx.reshape(-1).cuda()
    src, eblk, r_pad = sp.build_routing(assign, E)
    src2, eblk2, _ = sp.route(assign, E, r_pad)
    assert torch.equal(eblk2, eblk) and torch.equal(torch.sort(src2.view(-1, 128), 1).values, torch.sort(src.view(-1, 128), 1).values)
    valid = src >= 0
    rows = torch.zeros(r_pad, K, device="cuda", dtype=torch.bfloat16)
    rows[valid] = x.cuda().bfloat16()[src[valid] // topk]
    c = sp.seg_gemm(rows, w, Mpe, K, eblk)
    ref = fq.moe_seg_linear(rows.float().cpu(), eblk.cpu(), Ws)
    assert ((c.float().cpu() - ref).abs() / (ref.abs() + 1.0)).max().item() < 6e-3
    bb, sb, gb = sp.quant_act(rows)
    c2 = torch.empty_like(c)
    sp.seg_into(w, bb, sb, gb, c2, Mpe, K, eblk)
    assert torch.equal(c, c2)
    # weighted rows (seg_bw) + combine == fused scatter (down_scatter)
    sc_w = torch.zeros(r_pad, device="cuda")
    sc_w[valid] = wt.reshape(-1).cuda()[src[valid]]
    cbw = torch.empty_like(c)
    # the plugin's seg_bw / down_scatter run the down GEMM on single-level rows (gB = 1): quantise accordingly
    sb1 = torch.empty_like(sb)
    bb1 = torch.empty_like(bb)
    sp.lib.quantize_act_nvfp4(rows.data_ptr(), bb1.data_ptr(), sb1.data_ptr(), r_pad, K)
    sp.seg_bw(w, bb1, sb1, cbw, Mpe, r_pad, K, eblk, sc_w, None, Mpe)
    inverse = torch.full((T * topk,), -1, dtype=torch.int32, device="cuda")
    inverse[src[valid]] = torch.nonzero(valid).squeeze(1).int()
    y = torch.empty((T, Mpe), dtype=torch.bfloat16, device="cuda")
    sp.combine(cbw, inverse, y, T, Mpe, topk, Mpe)
    sc_tok = torch.full((r_pad,), -1, dtype=torch.int32, device="cuda")
    sc_tok[valid] = (src[valid] // topk).int()
    out = torch.zeros((T, Mpe), dtype=torch.float32, device="cuda")
    sp.down_scatter(w, bb1, sb1, out, Mpe, r_pad, K, eblk, sc_tok, sc_w, None, Mpe)
    assert sp.lib.qb_status(0) == 0
    assert ((out.cpu() - y.float().cpu()).abs() / (y.float().cpu().abs() + 1.0)).max().item() < 6e-3
    # fixed capacity: every expert owns cap rows, nothing dropped when cap is large enough
    cap = 128
    fsrc, feblk, dropped = sp.route_fixed_cap(assign, E, cap)
    assert int(dropped) == 0 and fsrc.numel() == E * cap and torch.equal(feblk.cpu(), torch.arange(E, dtype=torch.int32))
    for e in range(E):
        seg = fsrc[e * cap:(e + 1) * cap]
        got = torch.sort(seg[seg >= 0]).values
        assert torch.equal(got, torch.nonzero(assign == e).squeeze(1))
