"""GPU parity of the tcgen05 GEMM (dense and 2:4-sparse, plain / token-major / split-K /
grouped) through the C-ABI, against the CPU oracle.

Error metrics (stated once, used below):
  * fp32 accumulators (out_mode 2) vs the float64 dot product of the oracle-dequantised
    operands:  |d - ref| / (|ref| + rms(ref))  <= 1e-3   (accumulation order only; rms(ref)
    keeps cancelling sums from blowing up a purely relative figure);
  * bf16 outputs vs the oracle's fp32 fake-quant linear:  |y - ref| / (|ref| + 1) < 6e-3, the
    reference's own gate (harness/quadbit_linear.py:175-179, cuda/pack_verify.cu:283-285):
    bf16 rounding alone is 2^-8 = 3.9e-3 relative."""
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


def acc_err(D, ref):
    D = D.double().cpu()
    ref = ref.double()
    assert torch.isfinite(D).all()
    return ((D - ref).abs() / (ref.abs() + ref.pow(2).mean().sqrt())).max().item()


def bf16_err(y, ref):
    y = y.float().cpu()
    assert torch.isfinite(y).all()
    return ((y - ref).abs() / (ref.abs() + 1.0)).max().item()


def native_operands(W, x, sparse):
    """Oracle-packed operands moved to the GPU in the layouts qb_gemm takes."""
    if sparse:
        A, meta, sA, gA = fq.pack_weight_sparse_2lvl(W)
        Wd = fq.unpack_weight_sparse_2lvl(A, meta, sA, gA)
        mn = fq.meta_to_native(meta).cuda()
    else:
        A, sA, gA = fq.nvfp4_pack(W)
        Wd = fq.unpack_weight_dense(A, sA, gA)
        mn = None
    blk = 32 if sparse else 16
    Bb, sB, gB = fq.act_quant_2lvl(x, blk)
    xd = fq.unpack_act(Bb, sB, gB, blk)
    return dict(A=A.cuda(), B=Bb.cuda(), sfa=fq.sf_to_atoms(sA).cuda(), sfb=fq.sf_to_atoms(sB).cuda(), meta=mn, gA=gA.cuda(),
                gB=gB.cuda(), Wd=Wd, xd=xd, sA=sA, sB=sB, meta_ref=meta if sparse else None)


def gemm(lib, ops, out_f, tok, K, sparse, mode, splits=1, bn=0, use_globals=True, eblk=None, a_rows=None, bias=None, row_w=None):
    a_rows = a_rows or out_f
    shape = (tok, out_f) if mode in (1, 3) else (out_f, tok)
    C = torch.full(shape, float("nan"), dtype=torch.float32 if mode == 2 else torch.bfloat16, device="cuda")
    Cf = torch.empty((tok, out_f), dtype=torch.float32, device="cuda") if splits > 1 else None
    p = lambda t: 0 if t is None else t.data_ptr()
    rc = lib.qb_gemm(p(ops["A"]), p(ops["B"]), p(ops["sfa"]), p(ops["sfb"]), p(ops["meta"]),
                     p(ops["gA"]) if use_globals else 0, p(ops["gB"]) if use_globals else 0, p(C), p(Cf), p(eblk), p(bias),
                     p(row_w), a_rows, out_f, tok, K, int(sparse), mode, splits, bn, S())
    assert rc == 0, rc
    assert lib.qb_status(S()) == 0
    return C


CASES = [(128, 128, 256, 0), (256, 384, 1024, 128), (256, 512, 1024, 256), (384, 200, 1152, 0), (128, 1, 512, 0),
         (256, 16, 2048, 16), (128, 64, 4096, 64), (512, 100, 768, 64), (1024, 640, 2048, 256)]


@pytest.mark.parametrize("sparse", [1, 0])
@pytest.mark.parametrize("out_f,tok,K,bn", CASES)
def test_gemm_fp32_accumulators(lib, sparse, out_f, tok, K, bn):
    torch.manual_seed(out_f + tok + K)
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    ops = native_operands(W, x, sparse)
    D = gemm(lib, ops, out_f, tok, K, sparse, 2, bn=bn)
    # raw accumulators exclude the globals: compare with dequantised operands / (gA, gB)
    ref = (ops["Wd"].double() / ops["gA"].cpu().double()[:, None]) @ (ops["xd"].double() / ops["gB"].cpu().double()[:, None]).t()
    assert acc_err(D, ref) <= 1e-3


@pytest.mark.parametrize("sparse", [1, 0])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("out_f,tok,K,bn", CASES)
def test_gemm_bf16_outputs_match_fake_quant(lib, sparse, mode, out_f, tok, K, bn):
    torch.manual_seed(out_f + tok + K + 1)
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    ops = native_operands(W, x, sparse)
    C = gemm(lib, ops, out_f, tok, K, sparse, mode, bn=bn)
    ref = (fq.linear_sparse if sparse else fq.linear_dense)(x, W)          # [tok, out]
    y = C if mode == 1 else C.t()
    assert bf16_err(y, ref) < 6e-3


PAIR_CASES = [(256, 128, 256, 512), (512, 768, 1024, 512), (256, 300, 1152, 512), (1024, 512, 4096, 0), (768, 1000, 2048, 0),
              (256, 256, 512, 384), (512, 640, 1024, 384),
              (256, 192, 256, 576), (512, 768, 2048, 576), (256, 1000, 1152, 576), (768, 4096, 4096, 576), (512, 130, 512, 576),
              (1024, 2048, 8448, 0), (512, 1536, 12288, 512)]


@pytest.mark.parametrize("sparse", [1, 0])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("out_f,tok,K,bn", PAIR_CASES)
def test_cta_pair_kernel_matches_fake_quant(lib, sparse, mode, out_f, tok, K, bn):
    """The prefill kernel (tcgen05.mma.cta_group::2; bn 512 / 576 / 384 select its 256- / 192- / 128-token
    tile, bn 0 lets the library choose the 256-token tile for tok >= 512) against the oracle and against the single-CTA
    kernel, which must agree bit for bit (same products, same fp32 accumulation per K block)."""
    torch.manual_seed(out_f + tok + K + 7)
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    ops = native_operands(W, x, sparse)
    C = gemm(lib, ops, out_f, tok, K, sparse, mode, bn=bn)
    ref = (fq.linear_sparse if sparse else fq.linear_dense)(x, W)
    y = C if mode == 1 else C.t()
    assert bf16_err(y, ref) < 6e-3
    C1 = gemm(lib, ops, out_f, tok, K, sparse, mode, bn=128)
    assert bf16_err(C, C1.float().cpu()) < 6e-3


@pytest.mark.parametrize("sparse", [1, 0])
def test_token_major_output_is_bitwise_transpose(lib, sparse):
    """Reference check (harness/verify_sparse_2lvl.py:196-197): the zero-copy [tok,out] output
    must equal .t() of the [out,tok] output bit for bit."""
    torch.manual_seed(11)
    out_f, tok, K = 512, 384, 1024
    ops = native_operands(torch.randn(out_f, K) * 0.02, torch.randn(tok, K), sparse)
    C0 = gemm(lib, ops, out_f, tok, K, sparse, 0)
    C1 = gemm(lib, ops, out_f, tok, K, sparse, 1)
    assert torch.equal(C0.t().contiguous(), C1)


@pytest.mark.parametrize("sparse", [1, 0])
@pytest.mark.parametrize("out_f,tok,K,splits", [(256, 16, 4096, 4), (128, 64, 14336, 8), (512, 1, 2048, 3), (256, 128, 1024, 2),
                                                (128, 256, 2304, 5)])
def test_split_k_matches_single_pass(lib, sparse, out_f, tok, K, splits):
    torch.manual_seed(K + splits)
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    ops = native_operands(W, x, sparse)
    y = gemm(lib, ops, out_f, tok, K, sparse, 1, splits=splits)
    ref = (fq.linear_sparse if sparse else fq.linear_dense)(x, W)
    assert bf16_err(y, ref) < 6e-3
    y0 = gemm(lib, ops, out_f, tok, K, sparse, 0, splits=splits)
    assert bf16_err(y0.t(), ref) < 6e-3


@pytest.mark.parametrize("sparse", [1, 0])
@pytest.mark.parametrize("out_f,tok,K", [(4096, 1, 4096), (512, 16, 14336), (1024, 64, 2048), (256, 128, 4096), (384, 200, 1152),
                                          (14336, 16, 512)])
def test_decode_gemm_single_launch_split_k(lib, sparse, out_f, tok, K):
    """qb_gemm_decode: K split over CTAs, partial sums in per-split slabs, last arriver reduces.
    Two calls on one workspace: the arrival counters must be left clean by the first call."""
    torch.manual_seed(out_f + tok + K + 3)
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    ops = native_operands(W, x, sparse)
    ref = (fq.linear_sparse if sparse else fq.linear_dense)(x, W)
    ws = torch.zeros(lib.qb_gemm_decode_ws_bytes(out_f, tok, K), dtype=torch.uint8, device="cuda")
    p = lambda t: 0 if t is None else t.data_ptr()
    for mode in (1, 0, 1):
        C = torch.full((tok, out_f) if mode == 1 else (out_f, tok), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.qb_gemm_decode(p(ops["A"]), p(ops["B"]), p(ops["sfa"]), p(ops["sfb"]), p(ops["meta"]), p(ops["gA"]), p(ops["gB"]),
                                p(C), p(ws), out_f, tok, K, sparse, mode, S())
        assert rc == 0 and lib.qb_status(S()) == 0
        assert bf16_err(C if mode == 1 else C.t(), ref) < 6e-3
    ntile = (out_f // 128) * 4 * 2
    assert int(ws[: ntile * 4].view(torch.int32).abs().sum()) == 0


@pytest.mark.parametrize("sparse", [1, 0])
@pytest.mark.parametrize("out_f,tok,K", [(4096, 64, 14336), (4096, 128, 4096), (768, 200, 2304)])
def test_decode_split_k_inside_a_cluster_is_reproducible(lib, sparse, out_f, tok, K):
    """Shapes whose K splits fit the GPU as one wave of clusters: the partial tiles are summed in distributed shared
    memory in split order, so two calls give the same bits (the workspace form adds at the L2 in arrival order), the
    workspace is not touched, and the result meets the oracle like every other path."""
    torch.manual_seed(out_f + tok + K + 9)
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    ops = native_operands(W, x, sparse)
    ref = (fq.linear_sparse if sparse else fq.linear_dense)(x, W)
    ws = torch.zeros(lib.qb_gemm_decode_ws_bytes(out_f, tok, K), dtype=torch.uint8, device="cuda")
    p = lambda t: 0 if t is None else t.data_ptr()
    outs = []
    for _ in range(3):
        C = torch.full((tok, out_f), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.qb_gemm_decode(p(ops["A"]), p(ops["B"]), p(ops["sfa"]), p(ops["sfb"]), p(ops["meta"]), p(ops["gA"]), p(ops["gB"]),
                                p(C), p(ws), out_f, tok, K, sparse, 1, S())
        assert rc == 0 and lib.qb_status(S()) == 0
        outs.append(C.clone())
    assert bf16_err(outs[0], ref) < 6e-3
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert int(ws.view(torch.int32).abs().sum()) == 0


def test_all_ones_known_answer(lib):
    """Reference KAT (harness/run_torch.py:60-74): all-ones operands, unit scales, pairs {0,1}
    kept -> every output is exactly K/2."""
    out_f, tok, K = 256, 128, 512
    ops = dict(A=torch.full((out_f, K // 4), 0x22, dtype=torch.uint8).cuda(),
               B=torch.full((tok, K // 2), 0x22, dtype=torch.uint8).cuda(),
               sfa=fq.sf_to_atoms(torch.full((K // 128, out_f, 4), 0x38, dtype=torch.uint8)).cuda(),
               sfb=fq.sf_to_atoms(torch.full((K // 128, tok, 4), 0x38, dtype=torch.uint8)).cuda(),
               meta=fq.meta_to_native(torch.full((K // 128, out_f, 2), 0x44444444, dtype=torch.int32)).cuda(), gA=None, gB=None)
    C = gemm(lib, ops, out_f, tok, K, 1, 0, use_globals=False)
    assert torch.equal(C.float().cpu(), torch.full((out_f, tok), K / 2))


def test_reference_named_entry_points(lib):
    """The reference's own ctypes call sequence (harness/verify_sparse_2lvl.py:124-147) with
    reference-layout tensors: quantize_act_nvfp4_2lvl + sparse_fp4_mm_2lvl / _t / sk."""
    torch.manual_seed(2)
    out_f, tok, K = 512, 256, 1024
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    Ac, meta, scaleA, gA = [t.cuda() for t in fq.pack_weight_sparse_2lvl(W)]
    xb = x.to(torch.bfloat16).cuda()
    Bb = torch.empty((tok, K // 2), dtype=torch.uint8, device="cuda")
    sB = torch.empty((K // 128, tok, 4), dtype=torch.uint8, device="cuda")
    gB = torch.empty((tok,), dtype=torch.float32, device="cuda")
    lib.quantize_act_nvfp4_2lvl(xb.data_ptr(), Bb.data_ptr(), sB.data_ptr(), gB.data_ptr(), tok, K)
    assert lib.qb_last_error() == 0
    C = torch.empty((out_f, tok), dtype=torch.bfloat16, device="cuda")
    Ct = torch.empty((tok, out_f), dtype=torch.bfloat16, device="cuda")
    args = (Ac.data_ptr(), Bb.data_ptr(), scaleA.data_ptr(), sB.data_ptr(), meta.data_ptr())
    assert lib.sparse_fp4_mm_2lvl(*args, C.data_ptr(), out_f, tok, K, gA.data_ptr(), gB.data_ptr()) == 0
    assert lib.sparse_fp4_mm_2lvl_t(*args, Ct.data_ptr(), out_f, tok, K, gA.data_ptr(), gB.data_ptr()) == 0
    assert torch.equal(C.t().contiguous(), Ct)
    ref = fq.linear_sparse(x, W)
    assert bf16_err(Ct, ref) < 6e-3
    Csk = torch.empty((tok, out_f), dtype=torch.bfloat16, device="cuda")
    Cf = torch.empty((tok, out_f), dtype=torch.float32, device="cuda")
    assert lib.sparse_down_sk_2lvl(*args, Csk.data_ptr(), Cf.data_ptr(), out_f, tok, K, gA.data_ptr(), gB.data_ptr(), 4) == 0
    assert bf16_err(Csk, ref) < 6e-3
    # single-level entry: no globals -> compare with the packed operands' own dequant
    C1 = torch.empty((out_f, tok), dtype=torch.bfloat16, device="cuda")
    assert lib.sparse_fp4_mm(*args, C1.data_ptr(), out_f, tok, K) == 0
    Wl = fq.unpack_weight_sparse_2lvl(Ac.cpu(), meta.cpu(), scaleA.cpu(), torch.ones(out_f))
    xl = fq.unpack_act(Bb.cpu(), sB.cpu(), None, 32)
    ref1 = xl @ Wl.t()
    assert ((C1.t().float().cpu() - ref1).abs() / (ref1.abs() + ref1.abs().mean())).max() < 6e-3


def test_reference_named_dense_entry_point():
    import quadbit_b200 as qb
    lib = qb.load("dense_nvfp4")
    torch.manual_seed(4)
    out_f, tok, K = 256, 512, 1024
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    Ab, SFA, gA = [t.cuda() for t in fq.nvfp4_pack(W)]
    xb = x.to(torch.bfloat16).cuda()
    Bb = torch.empty((tok, K // 2), dtype=torch.uint8, device="cuda")
    SFB = torch.empty((K // 128, tok, 8), dtype=torch.uint8, device="cuda")
    gB = torch.empty((tok,), dtype=torch.float32, device="cuda")
    lib.quantize_act_nvfp4_2lvl(xb.data_ptr(), Bb.data_ptr(), SFB.data_ptr(), gB.data_ptr(), tok, K)
    C = torch.empty((out_f, tok), dtype=torch.bfloat16, device="cuda")
    assert lib.dense_nvfp4_mm(Ab.data_ptr(), Bb.data_ptr(), SFA.data_ptr(), SFB.data_ptr(), C.data_ptr(), out_f, tok, K,
                              gA.data_ptr(), gB.data_ptr()) == 0
    assert bf16_err(C.t(), fq.linear_dense(x, W)) < 6e-3


def test_module_api_any_token_count(lib):
    """QuadbitLinear / DenseNVLinear forward with token counts that are not tile multiples
    (the reference pads to 128, harness/quadbit_linear.py:146-152)."""
    import quadbit_b200 as qb
    torch.manual_seed(6)
    W = torch.randn(256, 512) * 0.02
    ql = qb.QuadbitLinear(W.cuda())
    dl = qb.DenseNVLinear(W.cuda())
    for tok in (1, 7, 100, 129, 300):
        x = torch.randn(tok, 512)
        y = ql.forward(x.cuda().bfloat16())
        assert y.shape == (tok, 256) and bf16_err(y, fq.linear_sparse(x, W)) < 6e-3
        yd = dl.forward(x.cuda().bfloat16())
        assert yd.shape == (tok, 256) and bf16_err(yd, fq.linear_dense(x, W)) < 6e-3
    x3 = torch.randn(2, 5, 512)
    assert ql.forward(x3.cuda().bfloat16()).shape == (2, 5, 256)
    assert qb.load("sparse_fp4").qb_status(0) == 0


def test_grouped_moe_gemm_matches_per_expert_reference(lib):
    """Segmented GEMM over routed rows (reference: matmul_sp_moe via sparse_moe_mm_2lvl,
    checked as harness/moe_seg.py does against a per-expert loop), plus the bias * routing
    weight epilogue, through the reference-named entry points."""
    torch.manual_seed(8)
    E, Mpe, K, T, topk = 4, 256, 512, 96, 2
    Ws = [torch.randn(Mpe, K) * 0.02 for _ in range(E)]
    packs = [fq.pack_weight_sparse_2lvl(w) for w in Ws]
    Ac = torch.cat([p[0] for p in packs], 0).cuda()
    meta = torch.cat([p[1] for p in packs], 1).contiguous().cuda()
    scaleA = torch.cat([p[2] for p in packs], 1).contiguous().cuda()
    gA = torch.cat([p[3] for p in packs], 0).cuda()
    x = torch.randn(T, K)
    idx, w = fq.route_topk(torch.randn(T, E), topk)
    assign = idx.reshape(-1)
    src, eblk, r_pad = fq.build_routing(assign, E)
    rows = torch.zeros(r_pad, K)
    valid = src >= 0
    rows[valid] = x[src[valid] // topk]
    xb = rows.to(torch.bfloat16).cuda()
    Bb = torch.empty((r_pad, K // 2), dtype=torch.uint8, device="cuda")
    sB = torch.empty((K // 128, r_pad, 4), dtype=torch.uint8, device="cuda")
    gB = torch.empty((r_pad,), dtype=torch.float32, device="cuda")
    lib.quantize_act_nvfp4_2lvl_s(xb.data_ptr(), Bb.data_ptr(), sB.data_ptr(), gB.data_ptr(), r_pad, K, S())
    C = torch.empty((r_pad, Mpe), dtype=torch.bfloat16, device="cuda")
    eb = eblk.cuda()
    rc = lib.sparse_moe_mm_2lvl(Ac.data_ptr(), Bb.data_ptr(), scaleA.data_ptr(), sB.data_ptr(), meta.data_ptr(), C.data_ptr(),
                                E * Mpe, Mpe, r_pad, K, gA.data_ptr(), gB.data_ptr(), eb.data_ptr(), 1, S())
    assert rc == 0 and lib.qb_status(S()) == 0
    ref = fq.moe_seg_linear(rows, eblk, Ws)
    assert bf16_err(C, ref) < 6e-3
    C0 = torch.empty((Mpe, r_pad), dtype=torch.bfloat16, device="cuda")
    assert lib.sparse_moe_mm_2lvl(Ac.data_ptr(), Bb.data_ptr(), scaleA.data_ptr(), sB.data_ptr(), meta.data_ptr(), C0.data_ptr(),
                                  E * Mpe, Mpe, r_pad, K, gA.data_ptr(), gB.data_ptr(), eb.data_ptr(), 0, 0) == 0
    assert torch.equal(C0.t().contiguous(), C)
    # bias + routing weight epilogue
    bias = (torch.randn(E, Mpe) * 0.1).to(torch.bfloat16)
    sc_w = torch.zeros(r_pad)
    sc_w[valid] = w.reshape(-1)[src[valid]]
    Cbw = torch.empty((r_pad, Mpe), dtype=torch.bfloat16, device="cuda")
    sc_w_d, bias_d = sc_w.cuda(), bias.cuda()
    rc = lib.sparse_moe_mm_2lvl_bw(Ac.data_ptr(), Bb.data_ptr(), scaleA.data_ptr(), sB.data_ptr(), meta.data_ptr(), Cbw.data_ptr(),
                                   E * Mpe, Mpe, r_pad, K, gA.data_ptr(), gB.data_ptr(), eb.data_ptr(), sc_w_d.data_ptr(),
                                   bias_d.data_ptr(), Mpe, S())
    assert rc == 0 and lib.qb_status(S()) == 0
    eidx = eblk.long().repeat_interleave(128)
    refbw = (ref + bias.float()[eidx]) * sc_w[:, None]
    assert bf16_err(Cbw, refbw) < 6e-3
    # combine: y[t] = sum_k Cbw[inverse[t,k]]
    inverse = torch.full((T * topk,), -1, dtype=torch.int32)
    inverse[src[valid]] = torch.nonzero(valid).squeeze(1).int()
    y = torch.empty((T, Mpe), dtype=torch.bfloat16, device="cuda")
    inverse_d = inverse.cuda()
    assert lib.moe_combine_topk(Cbw.data_ptr(), inverse_d.data_ptr(), y.data_ptr(), T, Mpe, topk, Mpe, S()) == 0
    torch.cuda.synchronize()
    yref = Cbw.float().cpu()[inverse.long().view(T, topk)].sum(1)
    assert bf16_err(y, yref) < 6e-3


def test_moe_route_kernel_groups_slots(lib):
    """Reference check (harness/fused_moe.py:718-726): every routed slot is placed exactly once
    inside its expert's padded segment."""
    torch.manual_seed(9)
    E, N = 8, 1000
    assign = torch.randint(0, E, (N,), dtype=torch.int32)
    assign[::17] = -1
    counts = torch.bincount(assign[assign >= 0].long(), minlength=E)
    padc = (counts + 127) // 128 * 128
    poff = torch.cumsum(padc, 0) - padc
    r_pad = int(padc.sum())
    src = torch.full((r_pad,), -1, dtype=torch.int32, device="cuda")
    counter = torch.empty(E, dtype=torch.int32, device="cuda")
    assign_d, poff_d = assign.cuda(), poff.cuda()
    assert lib.moe_route(assign_d.data_ptr(), poff_d.data_ptr(), counter.data_ptr(), src.data_ptr(), N, E, S()) == 0
    torch.cuda.synchronize()
    src = src.cpu()
    assert torch.equal(counter.cpu().long(), counts)
    placed = src[src >= 0]
    assert placed.numel() == int((assign >= 0).sum()) and placed.unique().numel() == placed.numel()
    for e in range(E):
        seg = src[int(poff[e]): int(poff[e] + counts[e])]
        assert (seg >= 0).all() and (assign[seg.long()] == e).all()


# ----------------------------------------------------------------------------- tiled weight layout
def tiled_reference(A: torch.Tensor, sparse: int) -> torch.Tensor:
    """[rows][row_bytes] -> [rows/128][ceil(K/256)][128][64 or 128] with a zero tail, on the CPU."""
    rows, rb = A.shape
    a_row = 64 if sparse else 128
    kblocks = (rb + a_row - 1) // a_row
    P = torch.zeros((rows, kblocks * a_row), dtype=torch.uint8)
    P[:, :rb] = A
    return P.view(rows // 128, 128, kblocks, a_row).permute(0, 2, 1, 3).contiguous().view(-1)


@pytest.mark.parametrize("sparse", [1, 0])
@pytest.mark.parametrize("rows,K", [(128, 128), (256, 384), (512, 1024), (1024, 4096)])
def test_tile_weights_is_the_permutation(lib, sparse, rows, K):
    torch.manual_seed(rows + K)
    A = torch.randint(0, 256, (rows, K // 4 if sparse else K // 2), dtype=torch.uint8)
    n = lib.qb_tiled_weight_bytes(rows, K, sparse)
    ref = tiled_reference(A, sparse)
    assert n == ref.numel()
    Ad = A.cuda()
    At = torch.full((n,), 0xAB, dtype=torch.uint8, device="cuda")
    assert lib.qb_tile_weights(Ad.data_ptr(), At.data_ptr(), rows, K, sparse, S()) == 0
    torch.cuda.synchronize()
    assert torch.equal(At.cpu(), ref)


@pytest.mark.parametrize("sparse", [1, 0])
@pytest.mark.parametrize("out_f,tok,K,bn,splits", [(256, 16, 1024, 16, 1), (512, 200, 768, 0, 1), (1024, 512, 2048, 512, 1),
                                                  (512, 640, 1024, 0, 1), (256, 16, 2048, 16, 4)])
def test_gemm_tiled_weights_bitwise_equal(lib, sparse, out_f, tok, K, bn, splits):
    torch.manual_seed(out_f + tok + K + 7)
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    ops = native_operands(W, x, sparse)
    Cr = gemm(lib, ops, out_f, tok, K, sparse, 1, splits=splits, bn=bn)
    At = torch.empty(lib.qb_tiled_weight_bytes(out_f, K, sparse), dtype=torch.uint8, device="cuda")
    assert lib.qb_tile_weights(ops["A"].data_ptr(), At.data_ptr(), out_f, K, sparse, S()) == 0
    ops_t = dict(ops)
    ops_t["A"] = At
    Ct = gemm(lib, ops_t, out_f, tok, K, int(sparse) | 2, 1, splits=splits, bn=bn)
    if splits == 1:
        assert torch.equal(Cr, Ct)
    else:   # atomic split-K adds in arrival order
        assert (Cr.float() - Ct.float()).abs().max() <= 2e-2 * Cr.float().abs().max()


@pytest.mark.parametrize("name,out_f,K", [("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 14336, 4096), ("down", 4096, 14336)])
def test_prefill_set_at_full_size(lib, name, out_f, K):
    """The Llama-3-8B prefill shapes at 4096 tokens, 2:4-sparse, through the module API: (a) the CTA-pair kernel and
    the single-CTA kernel, two independent schedules of the same products, give the same bf16 matrix; (b) the
    first 48 tokens against the CPU oracle's fake-quant linear (bf16 gate 6e-3); (c) the compressor's output
    against the oracle's packer on the first 256 weight rows, bit for bit."""
    import quadbit_b200 as qb
    tok = 4096
    g = torch.Generator().manual_seed(out_f * 7 + K)
    W = (torch.randn(out_f, K, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(tok, K, generator=g).to(torch.bfloat16)
    lin = qb.QuadbitLinear(W.cuda())
    Bb, sB, gB = lin.pack_act(x.cuda())
    y_pair = lin.run(Bb, sB, tok, gB, out_t=True, bn=512)
    y_one = lin.run(Bb, sB, tok, gB, out_t=True, bn=128)
    assert lib.qb_status(S()) == 0
    assert torch.equal(y_pair, y_one)
    ref = fq.linear_sparse(x[:48].float(), W.float())
    assert bf16_err(y_pair[:48], ref) < 6e-3
    Wf = W[:256].float()
    ties = fq.tie_groups(Wf)
    eAc, emeta, escale, egA = fq.pack_weight_sparse_2lvl(Wf)
    same_rows = (lin.Ac[:256].cpu() == eAc).all(1)
    # bf16 weights tie at the keep boundary in a few groups, where both sides keep the lower pair index
    assert bool(same_rows.all()), (name, int((~same_rows).sum()), ties)
    assert torch.equal(lin.meta[:, :256].cpu(), emeta) and torch.equal(lin.scaleA[:, :256].cpu(), escale)
    assert torch.equal(lin.gA[:256].cpu(), egA)


@pytest.mark.parametrize("sparse", [1, 0])
def test_pair_kernel_output_inside_a_larger_buffer(lib, sparse):
    """The 256-token tile stores its token-major output with TMA (16-token x 32-feature boxes, clipped at the ragged end):
    an output that starts 16 or 48 bytes into a larger buffer must get the same bytes as a fresh output, and nothing may be
    written outside it."""
    out_f, tok, K = 512, 600, 1024
    torch.manual_seed(5)
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    ops = native_operands(W, x, sparse)
    ref = gemm(lib, ops, out_f, tok, K, sparse, 1, bn=512)
    p = lambda t: 0 if t is None else t.data_ptr()
    buf = torch.full((tok * out_f + 64,), float("nan"), dtype=torch.bfloat16, device="cuda")
    for off in (8, 24):                                  # elements: 16 and 48 bytes into the buffer
        buf.fill_(float("nan"))
        C = buf[off: off + tok * out_f].view(tok, out_f)
        rc = lib.qb_gemm(p(ops["A"]), p(ops["B"]), p(ops["sfa"]), p(ops["sfb"]), p(ops["meta"]), p(ops["gA"]), p(ops["gB"]), C.data_ptr(),
                         0, 0, 0, 0, out_f, out_f, tok, K, int(sparse), 1, 1, 512, S())
        assert rc == 0 and lib.qb_status(S()) == 0
        assert torch.equal(C, ref)
        assert bool(torch.isnan(buf[:off]).all()) and bool(torch.isnan(buf[off + tok * out_f:]).all())    # nothing written outside
