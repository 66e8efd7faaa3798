"""GPU parity of the reference-named entry points that fuse a tail into the grouped MoE GEMM
(sparse_moe_mm_2lvl_scatter, sparse_moe_gu_swiglu, cuda/sparse_fp4_lib.cu:1649,1875) and of the dense
library's per-16 glue (rmsnorm_nvfp4, swiglu_nvfp4, cuda/dense_nvfp4_fast_lib.cu:251,274), against
the CPU oracle. Tolerances as in the other GPU tests: bf16 outputs |y - ref| / (|ref| + 1) < 6e-3; the
quantisers behind a device exp / rsqrt may differ from the oracle only on codes that sit within 1e-5 of a rounding
boundary (tests/_parity.py)."""
import pytest
import torch

from oracle import fakequant as fq
from tests._parity import assert_codes_explained

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
    # the fused entry forms h from the fp32 accumulators (no bf16 rounding of gate / up in between), as the reference's
    # fused kernel does: the oracle is the fp32 fake-quant linear; codes may differ where the accumulation order of the
    # tensor core moves a quotient across a boundary (relative distance <= 2e-4)
    g, u = ref_gu[:, 0::2], ref_gu[:, 1::2]
    if act == 0:
        g = g.clamp(max=7.0)
        u = u.clamp(-7.0, 7.0)
        h = (g / (1.0 + torch.exp(-1.702 * g))) * (u + 1.0)
    else:
        h = (g / (1.0 + torch.exp(-g))) * u
    eB, eS = fq.act_quant_1lvl(h, 32, round_bf16=False)
    want = fq.unpack_act(eB, eS, None, 32)
    deq = fq.unpack_act(Hw.cpu(), sH.cpu(), None, 32)
    assert_codes_explained(h, Hw, sH, None, 32, tol=2e-4, max_scale_flips=5e-3)
    # single-level scales bottom out at 2^-9, so small h quantise coarsely: compare with the oracle's own error
    assert ((deq - h).norm() / h.norm()).item() < 1.02 * ((want - h).norm() / h.norm()).item() + 1e-3


@pytest.mark.parametrize("tok,grouped", [(256, False), (640, False), (384, True)])
def test_native_fused_gate_up_swiglu_epilogue(lib, tok, grouped):
    """qb_gemm_swiglu: gate/up GEMM (interleaved rows) with SwiGLU + single-level per-32 quantiser in the epilogue, plain
    (the 128- and 256-token tiles of the CTA-pair kernel) and grouped, scale codes in both layouts."""
    import quadbit_b200.moe as qmoe
    torch.manual_seed(tok)
    Ih, K, E = 256, 512, 3 if grouped else 1
    out_f = 2 * Ih
    Ws = [torch.randn(out_f, K) * 0.05 for _ in range(E)]          # rows: (gate_0, up_0, gate_1, up_1, ...)
    x = torch.randn(tok, K)
    bias = (torch.randn(E, out_f) * 0.2).to(torch.bfloat16)
    packs = [qmoe.pack(lib, w.cuda()) for w in Ws]
    Ac, meta, sfa, gA = qmoe.stack(packs)
    import quadbit_b200 as qb
    Bb, sfb, gB = qb.quantize_act(lib, x.cuda().bfloat16(), 32, True)
    eblk = torch.tensor([i % E for i in range(tok // 128)], dtype=torch.int32) if grouped else None
    Hb = torch.zeros((tok, Ih // 2), dtype=torch.uint8, device="cuda")
    atoms = torch.zeros(lib.qb_sf_atoms_bytes(tok, Ih, 32), dtype=torch.uint8, device="cuda")
    sref = torch.zeros((Ih // 128, tok, 4), dtype=torch.uint8, device="cuda")
    for act in (1, 0):
        rc = lib.qb_gemm_swiglu(Ac.data_ptr(), Bb.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), meta.data_ptr(), gA.data_ptr(), gB.data_ptr(),
                                eblk.cuda().data_ptr() if grouped else 0, bias.cuda().data_ptr(), Hb.data_ptr(), atoms.data_ptr(), sref.data_ptr(),
                                E * out_f, out_f, tok, K, 1, act, S())
        assert rc == 0 and lib.qb_status(S()) == 0
        xq = fq.act_dequant_2lvl(x, 32)
        gu = torch.empty(tok, out_f)
        for b in range(tok // 128):
            e = int(eblk[b]) if grouped else 0
            gu[b * 128:(b + 1) * 128] = torch.nn.functional.linear(xq[b * 128:(b + 1) * 128], fq.sparse_fp4_dequant_2lvl(Ws[e])) + bias[e].float()
        g, u = gu[:, 0::2], gu[:, 1::2]
        if act == 0:
            g, u = g.clamp(max=7.0), u.clamp(-7.0, 7.0)
            h = (g / (1.0 + torch.exp(-1.702 * g))) * (u + 1.0)
        else:
            h = (g / (1.0 + torch.exp(-g))) * u
        assert_codes_explained(h, Hb, sref, None, 32, tol=2e-4, max_scale_flips=5e-3)
        mask = fq.sf_to_atoms(torch.ones(Ih // 128, tok, 4, dtype=torch.uint8)).view(-1).bool()
        assert torch.equal(atoms.cpu()[mask], fq.sf_to_atoms(sref.cpu()).view(-1)[mask])
    d = torch.zeros(16, dtype=torch.uint8, device="cuda").data_ptr()
    assert lib.qb_gemm_swiglu(d, d, d, d, d, 0, 0, 0, 0, d, d, 0, 384, 384, 256, 512, 1, 1, S()) == 1001        # out % 256
    assert lib.qb_gemm_swiglu(d, d, d, d, d, 0, 0, 0, 0, d, d, 0, 512, 512, 64, 512, 1, 1, S()) == 1001         # tok < 128


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
        deq = fq.unpack_act(Bb.cpu(), SFB.cpu(), None, 16)
        assert_codes_explained(y, Bb, SFB, None, 16)
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
    deq = fq.unpack_act(Hb.cpu(), SFH.cpu(), None, 16)
    assert_codes_explained(h, Hb, SFH, None, 16)
    assert ((deq - h).norm() / h.norm()).item() < 0.12


def test_reference_named_moe_entries_chain(lib):
    """The MoE entry points a caller of the reference library binds, in the order its plugin drives them
    (harness/qb_vllm_plugin/qb_sm120_plugin.py:1203-1368): CUDA packer in the reference layout -> moe_route ->
    quantize_act_nvfp4_2lvl_s -> sparse_moe_mm_2lvl -> sparse_moe_mm_2lvl_bw + moe_combine_topk ==
    sparse_moe_mm_2lvl_scatter."""
    torch.manual_seed(17)
    E, Mpe, K, T, topk = 4, 256, 256, 60, 2
    Ws = [torch.randn(Mpe, K) * 0.02 for _ in range(E)]
    packs = []
    for w in Ws:
        wd = w.cuda()
        ac = torch.empty((Mpe, K // 4), dtype=torch.uint8, device="cuda")
        meta = torch.empty((K // 128, Mpe, 2), dtype=torch.int32, device="cuda")
        sa = torch.empty((K // 128, Mpe, 4), dtype=torch.uint8, device="cuda")
        ga = torch.empty((Mpe,), dtype=torch.float32, device="cuda")
        assert lib.qb_compress_2to4(wd.data_ptr(), 0, ac.data_ptr(), meta.data_ptr(), 0, sa.data_ptr(), 0, ga.data_ptr(), Mpe, K, S()) == 0
        for a, b in zip((ac, meta, sa, ga), fq.pack_weight_sparse_2lvl(w)):      # equals the oracle's packer, bit for bit
            assert torch.equal(a.cpu(), b)
        packs.append((ac, meta, sa, ga))
    Ac = torch.cat([p[0] for p in packs], 0).contiguous()
    meta = torch.cat([p[1] for p in packs], 1).contiguous()
    scaleA = torch.cat([p[2] for p in packs], 1).contiguous()
    gA = torch.cat([p[3] for p in packs], 0).contiguous()
    x = torch.randn(T, K)
    idx, wt = fq.route_topk(torch.randn(T, E), topk)
    assign = idx.reshape(-1)
    src_o, eblk_o, r_pad = fq.build_routing(assign, E)
    # moe_route: padded segment offsets in, slot of every padded row out (order inside a segment is the kernel's)
    counts = torch.bincount(assign, minlength=E)
    padc = (counts + 127) // 128 * 128
    poff = (torch.cumsum(padc, 0) - padc).cuda()
    ai = assign.int().cuda()
    src = torch.full((r_pad,), -1, dtype=torch.int32, device="cuda")
    counter = torch.empty(E, dtype=torch.int32, device="cuda")
    assert lib.moe_route(ai.data_ptr(), poff.data_ptr(), counter.data_ptr(), src.data_ptr(), ai.numel(), E, S()) == 0
    src = src.long().cpu()
    assert torch.equal(torch.sort(src.view(-1, 128), 1).values, torch.sort(src_o.view(-1, 128), 1).values)
    eblk = eblk_o.cuda()
    valid = src >= 0
    rows = torch.zeros(r_pad, K)
    rows[valid] = x.to(torch.bfloat16).float()[src[valid] // topk]
    Bb, sB, gB = _quantise_rows(lib, rows, r_pad, K)
    c = torch.empty((r_pad, Mpe), dtype=torch.bfloat16, device="cuda")
    assert lib.sparse_moe_mm_2lvl(Ac.data_ptr(), Bb.data_ptr(), scaleA.data_ptr(), sB.data_ptr(), meta.data_ptr(), c.data_ptr(),
                                  E * Mpe, Mpe, r_pad, K, gA.data_ptr(), gB.data_ptr(), eblk.data_ptr(), 1, S()) == 0
    ref = fq.moe_seg_linear(rows, eblk_o, Ws)
    assert ((c.float().cpu() - ref).abs() / (ref.abs() + 1.0)).max().item() < 6e-3
    # weighted rows (bw entry) + combine == fused scatter entry; both run on single-level rows (gB = 1), as the plugin's down GEMM
    rows_d = rows.to(torch.bfloat16).cuda()
    bb1 = torch.empty_like(Bb)
    sb1 = torch.empty_like(sB)
    lib.quantize_act_nvfp4(rows_d.data_ptr(), bb1.data_ptr(), sb1.data_ptr(), r_pad, K)
    sc_w = torch.zeros(r_pad)
    sc_w[valid] = wt.reshape(-1)[src[valid]]
    sc_w = sc_w.cuda()
    cbw = torch.empty_like(c)
    assert lib.sparse_moe_mm_2lvl_bw(Ac.data_ptr(), bb1.data_ptr(), scaleA.data_ptr(), sb1.data_ptr(), meta.data_ptr(), cbw.data_ptr(),
                                     E * Mpe, Mpe, r_pad, K, gA.data_ptr(), 0, eblk.data_ptr(), sc_w.data_ptr(), 0, Mpe, S()) == 0
    inverse = torch.full((T * topk,), -1, dtype=torch.int32)
    inverse[src[valid]] = torch.nonzero(valid).squeeze(1).int()
    inverse = inverse.cuda()
    y = torch.empty((T, Mpe), dtype=torch.bfloat16, device="cuda")
    assert lib.moe_combine_topk(cbw.data_ptr(), inverse.data_ptr(), y.data_ptr(), T, Mpe, topk, Mpe, S()) == 0
    sc_tok = torch.full((r_pad,), -1, dtype=torch.int32)
    sc_tok[valid] = (src[valid] // topk).int()
    sc_tok = sc_tok.cuda()
    out = torch.zeros((T, Mpe), dtype=torch.float32, device="cuda")
    assert lib.sparse_moe_mm_2lvl_scatter(Ac.data_ptr(), bb1.data_ptr(), scaleA.data_ptr(), sb1.data_ptr(), meta.data_ptr(), E * Mpe, Mpe,
                                          r_pad, K, gA.data_ptr(), 0, eblk.data_ptr(), sc_tok.data_ptr(), sc_w.data_ptr(), 0,
                                          out.data_ptr(), Mpe, S()) == 0
    assert lib.qb_status(0) == 0
    assert ((out.cpu() - y.float().cpu()).abs() / (y.float().cpu().abs() + 1.0)).max().item() < 6e-3
