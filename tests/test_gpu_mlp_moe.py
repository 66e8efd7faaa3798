"""GPU parity of the fused SwiGLU MLP and the MoE layer against the CPU oracle."""
import pytest
import torch

from oracle import fakequant as fq
from tests._parity import assert_codes_explained

pytestmark = pytest.mark.gpu


def S():
    return torch.cuda.current_stream().cuda_stream


def rel(y, ref):
    y = y.float().cpu()
    assert torch.isfinite(y).all()
    return ((y - ref).norm() / ref.norm()).item()


def test_swiglu_quant_kernel_against_oracle():
    """One-pass SwiGLU + two-level quantiser: globals exact up to exp rounding, every code that differs from
    the oracle's sits within 1e-5 of a rounding boundary, dequantised values at the FP4 quantisation floor."""
    import quadbit_b200 as qb
    lib = qb.load("sparse_fp4")
    torch.manual_seed(0)
    for tok, I in ((5, 256), (37, 2944), (16, 14336)):
        cgu = (torch.randn(tok, 2 * I) * 1.5).to(torch.bfloat16)
        g, u = cgu[:, :I].float(), cgu[:, I:].float()
        h = (g / (1.0 + torch.exp(-g))) * u
        d = cgu.cuda()
        Hb = torch.empty((tok, I // 2), dtype=torch.uint8, device="cuda")
        sref = torch.empty((I // 128, tok, 4), dtype=torch.uint8, device="cuda")
        atoms = torch.zeros(lib.qb_sf_atoms_bytes(tok, I, 32), dtype=torch.uint8, device="cuda")
        gH = torch.empty(tok, device="cuda")
        assert lib.qb_swiglu_quant(d.data_ptr(), Hb.data_ptr(), sref.data_ptr(), atoms.data_ptr(), gH.data_ptr(), tok, I, S()) == 0
        assert lib.qb_status(S()) == 0
        deq = fq.unpack_act(Hb.cpu(), sref.cpu(), gH.cpu(), 32)
        assert_codes_explained(h, Hb, sref, gH, 32)                # exp() rounding moves boundary cases only
        assert ((deq - h).norm() / h.norm()).item() < 0.12           # FP4 floor
        mask = fq.sf_to_atoms(torch.ones(I // 128, tok, 4, dtype=torch.uint8)).view(-1).bool()
        assert torch.equal(atoms.cpu()[mask], fq.sf_to_atoms(sref.cpu()).view(-1)[mask])


@pytest.mark.parametrize("tok", [1, 48, 300])
def test_fused_mlp_matches_oracle(tok):
    import quadbit_b200 as qb
    torch.manual_seed(tok)
    H, I = 512, 768
    wgu = torch.randn(2 * I, H) * 0.05
    wdn = torch.randn(H, I) * 0.05
    x = torch.randn(tok, H)
    mlp = qb.FusedSparseMLP(wgu.cuda(), wdn.cuda())
    y = mlp.forward(x.cuda().bfloat16())
    assert mlp.lib.qb_status(0) == 0
    ref = fq.fused_mlp_sparse(x, wgu, wdn)
    assert y.shape == (tok, H) and rel(y, ref) < 0.02       # reference gate: RED < 0.02 (harness/verify_sparse_2lvl.py:211)
    # unfused composition through the module API gives the same thing
    gu = mlp.gu.forward(x.cuda().bfloat16()).float()
    h = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
    Bb, sfb, gB = qb.quantize_act(mlp.lib, h.to(torch.bfloat16), 32, True)
    y2 = mlp.dn.run(Bb, sfb, tok, gB, out_t=True)
    assert rel(y2, ref) < 0.05      # h takes an extra bf16 rounding on this path


def test_fused_mlp_reference_named_entry_points():
    """fused_mlp_2lvl / fused_mlp_2lvl_skdown with reference-layout weights and the reference's
    scratch sizes (harness/quadbit_serve.py:427-450)."""
    import quadbit_b200 as qb
    lib = qb.load("sparse_fp4")
    torch.manual_seed(3)
    H, I, tp = 512, 768, 128
    wgu = torch.randn(2 * I, H) * 0.05
    wdn = torch.randn(H, I) * 0.05
    x = torch.randn(tp, H)
    gu = [t.cuda() for t in fq.pack_weight_sparse_2lvl(wgu)]
    dn = [t.cuda() for t in fq.pack_weight_sparse_2lvl(wdn)]
    dev = "cuda"
    x2 = x.to(torch.bfloat16).cuda()
    Bb = torch.empty((tp, H // 2), dtype=torch.uint8, device=dev)
    sBg = torch.empty((H // 128, tp, 4), dtype=torch.uint8, device=dev)
    gBg = torch.empty((tp,), dtype=torch.float32, device=dev)
    Cgu = torch.empty((2 * I, tp), dtype=torch.bfloat16, device=dev)
    Hb = torch.empty((tp, I // 2), dtype=torch.uint8, device=dev)
    sH = torch.empty((I // 128, tp, 4), dtype=torch.uint8, device=dev)
    gH = torch.empty((tp,), dtype=torch.float32, device=dev)
    ref = fq.fused_mlp_sparse(x, wgu, wdn)
    for sk in (False, True):
        Cout = torch.full((tp, H), float("nan"), dtype=torch.bfloat16, device=dev)
        args = [x2.data_ptr(), gu[0].data_ptr(), gu[2].data_ptr(), gu[1].data_ptr(), gu[3].data_ptr(), dn[0].data_ptr(),
                dn[2].data_ptr(), dn[1].data_ptr(), dn[3].data_ptr(), Bb.data_ptr(), sBg.data_ptr(), gBg.data_ptr(), Cgu.data_ptr(),
                Hb.data_ptr(), sH.data_ptr(), gH.data_ptr(), Cout.data_ptr()]
        if sk:
            Cf = torch.empty((H * tp,), dtype=torch.float32, device=dev)
            rc = lib.fused_mlp_2lvl_skdown(*args, Cf.data_ptr(), tp, H, I, 2 * I, H, 3, S())
        else:
            rc = lib.fused_mlp_2lvl(*args, tp, H, I, 2 * I, H, S())
        assert rc == 0 and lib.qb_status(S()) == 0
        assert rel(Cout, ref) < 0.02


def test_fused_mlp_custom_op_and_graph_capture():
    """quadbit::fused_mlp custom op; the call is capturable in a CUDA graph and replays to the
    same result (reference checks: harness/p4_capture.py, quadbit_serve.py graph_probe)."""
    import quadbit_b200 as qb
    torch.manual_seed(5)
    H, I, tok = 256, 512, 64
    mlp = qb.FusedSparseMLP((torch.randn(2 * I, H) * 0.05).cuda(), (torch.randn(H, I) * 0.05).cuda())
    qb.register_fused_mlp_op([mlp])
    x = torch.randn(tok, H, device="cuda").bfloat16()
    y_eager = torch.ops.quadbit.fused_mlp(x, 0, H)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        mlp.forward(x)
        stream.synchronize()
        gph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gph, stream=stream):
            y_graph = mlp.forward(x)
        gph.replay()
        stream.synchronize()
    assert torch.equal(y_graph, y_eager)
    assert mlp.lib.qb_status(0) == 0


def moe_reference(x, wgu, wdn, idx, w, act_fn):
    T, H = x.shape
    y = torch.zeros(T, wdn[0].shape[0])
    for e in range(len(wgu)):
        sel = (idx == e)
        toks = torch.nonzero(sel.any(1)).squeeze(1)
        if toks.numel() == 0:
            continue
        I = wdn[e].shape[1]
        gu = fq.linear_sparse(x[toks], wgu[e]).to(torch.bfloat16).float()
        h = act_fn(gu[:, :I], gu[:, I:]).to(torch.bfloat16).float()
        d = fq.linear_sparse(h, wdn[e])
        wt = (w * sel)[toks].sum(1, keepdim=True)
        y[toks] += (d * wt).to(torch.bfloat16).float()
    return y


@pytest.mark.parametrize("H,I,E,topk,T", [(256, 384, 8, 2, 200), (384, 256, 4, 4, 64)])
def test_moe_layer_matches_per_expert_reference(H, I, E, topk, T):
    """Routed MoE layer (route, gather, grouped GEMMs, weight epilogue, combine) against a
    per-expert loop of the oracle (reference: harness/fused_moe.py:503-613 cosine gates)."""
    import quadbit_b200 as qb
    torch.manual_seed(E + T)
    wgu = [torch.randn(2 * I, H) * 0.05 for _ in range(E)]
    wdn = [torch.randn(H, I) * 0.05 for _ in range(E)]
    x = torch.randn(T, H)
    idx, w = fq.route_topk(torch.randn(T, E), topk)
    moe = qb.SparseMoE([t.cuda() for t in wgu], [t.cuda() for t in wdn], topk)
    y = moe.forward(x.cuda().bfloat16(), idx.cuda(), w.cuda())
    assert moe.lib.qb_status(0) == 0
    ref = moe_reference(x, wgu, wdn, idx, w, lambda g, u: torch.nn.functional.silu(g) * u)
    cos = torch.nn.functional.cosine_similarity(y.float().cpu().flatten(), ref.flatten(), dim=0).item()
    assert cos > 0.999 and rel(y, ref) < 0.03
    # expert-parallel shards sum to the full layer (reference: harness/p4_m3c.py, moe_dist.py:199-206)
    parts = []
    for r in range(2):
        e0, e1 = r * E // 2, (r + 1) * E // 2
        sh = qb.SparseMoE([t.cuda() for t in wgu[e0:e1]], [t.cuda() for t in wdn[e0:e1]], topk, expert_range=(e0, e1),
                          n_experts_total=E)
        parts.append(sh.forward(x.cuda().bfloat16(), idx.cuda(), w.cuda()).float())
    assert rel(parts[0] + parts[1], ref) < 0.03


@pytest.mark.parametrize("act", ["silu", "gptoss"])
def test_moe_layer_fused_gate_up_epilogue(act):
    """SparseMoE(fused_gu=True): SwiGLU + single-level quantiser of h in the epilogue of the grouped gate/up GEMM (the
    reference's fused GEMM1 arithmetic: h from the fp32 accumulators, one UE4M3 scale per 32 features, no per-row global),
    against a per-expert loop of the oracle with that arithmetic."""
    import quadbit_b200 as qb
    torch.manual_seed(31)
    H, I, E, topk, T = 256, 384, 4, 2, 200
    wgu = [torch.randn(2 * I, H) * 0.5 for _ in range(E)]         # large enough that h sits well inside the UE4M3 range
    wdn = [torch.randn(H, I) * 0.05 for _ in range(E)]
    x = torch.randn(T, H)
    idx, w = fq.route_topk(torch.randn(T, E), topk)
    moe = qb.SparseMoE([t.cuda() for t in wgu], [t.cuda() for t in wdn], topk, act=act, fused_gu=True)
    for fixed in (False, True):
        moe.fixed_capacity = fixed
        y = moe.forward(x.cuda().bfloat16(), idx.cuda(), w.cuda())
        assert moe.lib.qb_status(0) == 0
        ref = torch.zeros(T, H)
        for e in range(E):
            sel = idx == e
            toks = torch.nonzero(sel.any(1)).squeeze(1)
            if toks.numel() == 0:
                continue
            gu = fq.linear_sparse(x[toks], wgu[e])
            g, u = gu[:, :I], gu[:, I:]
            if act == "gptoss":
                g, u = g.clamp(max=7.0), u.clamp(-7.0, 7.0)
                h = (g * torch.sigmoid(1.702 * g)) * (u + 1.0)
            else:
                h = torch.nn.functional.silu(g) * u
            hq = fq.unpack_act(*fq.act_quant_1lvl(h, 32, round_bf16=False), None, 32)
            d = torch.nn.functional.linear(hq, fq.sparse_fp4_dequant_2lvl(wdn[e]))
            wt = (w * sel)[toks].sum(1, keepdim=True)
            ref[toks] += (d * wt).to(torch.bfloat16).float()
        cos = torch.nn.functional.cosine_similarity(y.float().cpu().flatten(), ref.flatten(), dim=0).item()
        assert cos > 0.999 and rel(y, ref) < 0.03, (fixed, cos, rel(y, ref))


def test_build_routing_matches_reference_helper():
    import quadbit_b200.moe as moe
    torch.manual_seed(1)
    assign = torch.randint(0, 8, (300,))
    src, eblk, r_pad = moe.build_routing(assign.cuda(), 8)
    esrc, eeblk, erp = fq.build_routing(assign, 8)
    assert r_pad == erp and torch.equal(src.cpu(), esrc) and torch.equal(eblk.cpu(), eeblk)


def test_moe_forward_ep_single_rank_equals_forward():
    """Without a process group the all-to-all layer degenerates to sort -> experts -> unsort -> combine and
    must give the bits of `forward` (rows are computed independently of their neighbours)."""
    import quadbit_b200 as qb
    torch.manual_seed(21)
    H, I, E, topk, T = 256, 256, 4, 2, 150
    wgu = [torch.randn(2 * I, H) * 0.05 for _ in range(E)]
    wdn = [torch.randn(H, I) * 0.05 for _ in range(E)]
    x = torch.randn(T, H).cuda().bfloat16()
    idx, w = fq.route_topk(torch.randn(T, E), topk)
    moe = qb.SparseMoE([t.cuda() for t in wgu], [t.cuda() for t in wdn], topk)
    y = moe.forward(x, idx.cuda(), w.cuda())
    y_ep = moe.forward_ep(x, idx.cuda(), w.cuda())
    assert moe.lib.qb_status(0) == 0
    assert torch.equal(y, y_ep)


def _ep_problem(seed=23):
    torch.manual_seed(seed)
    H, I, E, topk, T = 256, 256, 4, 2, 256
    wgu = [torch.randn(2 * I, H) * 0.05 for _ in range(E)]
    wdn = [torch.randn(H, I) * 0.05 for _ in range(E)]
    x = torch.randn(T, H).to(torch.bfloat16)
    idx, w = fq.route_topk(torch.randn(T, E), topk)
    return H, I, E, topk, T, wgu, wdn, x, idx, w


def test_moe_expert_parallel_by_peer_loads_two_ranks_on_one_gpu():
    """forward_ep_peer with both ranks in this process (buffers are plain allocations, ranks driven in lock step so that a
    waiting kernel always follows its producers): routing tables replicated by stores, token rows pulled by the fused
    gather + quantise, expert outputs pulled by the combine. Must equal the 1-rank layer bit for bit, twice in a row."""
    import quadbit_b200 as qb
    from quadbit_b200.tp import EPContext
    H, I, E, topk, T, wgu, wdn, x, idx, w = _ep_problem()
    full = qb.SparseMoE([t.cuda() for t in wgu], [t.cuda() for t in wdn], topk, fixed_capacity=True)
    y_ref = full.forward(x.cuda(), idx.cuda(), w.cuda())
    world, Tl = 2, T // 2
    moes = [qb.SparseMoE([t.cuda() for t in wgu[r * 2:(r + 1) * 2]], [t.cuda() for t in wdn[r * 2:(r + 1) * 2]], topk,
                         expert_range=(r * 2, (r + 1) * 2), n_experts_total=E) for r in range(world)]
    ctxs = EPContext.emulated(T, H, topk, moes[0].mpe_dn, moes[0].ep_capacity(T), world, torch.device("cuda"))
    for it in range(2):
        gens = [m.forward_ep_peer_steps(x[r * Tl:(r + 1) * Tl].cuda(), idx[r * Tl:(r + 1) * Tl].cuda(), w[r * Tl:(r + 1) * Tl].cuda(), ctxs[r])
                for r, m in enumerate(moes)]
        outs = None
        for step in zip(*gens):
            outs = step
        assert full.lib.qb_status(0) == 0 and full.lib.qb_peer_status(0) == 0
        y = torch.cat(list(outs), 0)
        assert torch.equal(y, y_ref), it


def _ep_peer_gpu_worker(rank, world, port, ret):
    import os
    import torch.distributed as dist
    import quadbit_b200 as qb
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    H, I, E, topk, T, wgu, wdn, x, idx, w = _ep_problem()
    epr, Tl = E // world, T // world
    moe = qb.SparseMoE([t.cuda() for t in wgu[rank * epr:(rank + 1) * epr]], [t.cuda() for t in wdn[rank * epr:(rank + 1) * epr]], topk,
                       expert_range=(rank * epr, (rank + 1) * epr), n_experts_total=E)
    ctx = moe.make_ep_context(T, rank, world)
    dist.barrier()
    xs, ids, ws = x[rank * Tl:(rank + 1) * Tl].cuda(), idx[rank * Tl:(rank + 1) * Tl].cuda(), w[rank * Tl:(rank + 1) * Tl].cuda()
    for _ in range(3):
        y = moe.forward_ep_peer(xs, ids, ws, ctx)
    torch.cuda.synchronize()
    assert moe.lib.qb_status(0) == 0 and moe.lib.qb_peer_status(0) == 0
    ret[rank] = y.cpu()
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_moe_expert_parallel_by_peer_loads_two_gpus():
    import torch.multiprocessing as mp
    import quadbit_b200 as qb
    H, I, E, topk, T, wgu, wdn, x, idx, w = _ep_problem()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_ep_peer_gpu_worker, args=(2, 29541, ret), nprocs=2, join=True)
    full = qb.SparseMoE([t.cuda() for t in wgu], [t.cuda() for t in wdn], topk, fixed_capacity=True)
    y_ref = full.forward(x.cuda(), idx.cuda(), w.cuda()).cpu()
    assert torch.equal(torch.cat([ret[0], ret[1]], 0), y_ref)


def _ep_gpu_worker(rank, world, port, ret):
    import os
    import torch.distributed as dist
    import quadbit_b200 as qb
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    torch.manual_seed(22)
    H, I, E, topk, T = 256, 256, 8, 2, 256
    wgu = [torch.randn(2 * I, H) * 0.05 for _ in range(E)]
    wdn = [torch.randn(H, I) * 0.05 for _ in range(E)]
    x = torch.randn(T, H).cuda().bfloat16()
    idx, w = fq.route_topk(torch.randn(T, E), topk)
    idx, w = idx.cuda(), w.cuda()
    full = qb.SparseMoE([t.cuda() for t in wgu], [t.cuda() for t in wdn], topk).forward(x, idx, w)
    e0, e1 = rank * E // world, (rank + 1) * E // world
    sh = qb.SparseMoE([t.cuda() for t in wgu[e0:e1]], [t.cuda() for t in wdn[e0:e1]], topk, expert_range=(e0, e1), n_experts_total=E)
    tl = T // world
    mine = slice(rank * tl, (rank + 1) * tl)
    y = sh.forward_ep(x[mine], idx[mine], w[mine])
    ok = torch.equal(y, full[mine]) and sh.lib.qb_status(0) == 0
    ret.put((rank, bool(ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_moe_forward_ep_two_gpus_equals_one_gpu():
    """Expert-parallel NCCL all-to-all dispatch / combine over two GPUs against the 1-GPU layer, bit for bit
    (reference check: harness/moe_dist.py:199-206 compares the distributed output with the single-GPU one)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_ep_gpu_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(ret.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert got[0] and got[1]


def test_moe_fixed_capacity_routing_equals_exact_and_captures_in_a_graph():
    """Fixed-capacity routing (unused 128-row blocks carry expert id -1 and are skipped by the grouped GEMM) gives the
    bits of the exact-size routing, with no host read, so the whole layer replays from a CUDA graph."""
    import quadbit_b200 as qb
    import quadbit_b200.moe as qmoe
    torch.manual_seed(23)
    for H, I, E, topk, T in ((256, 256, 8, 2, 300), (384, 128, 4, 4, 96)):      # pair-kernel and single-CTA grouped forms
        wgu = [torch.randn(2 * I, H).cuda() * 0.05 for _ in range(E)]
        wdn = [torch.randn(H, I).cuda() * 0.05 for _ in range(E)]
        x = torch.randn(T, H).cuda().bfloat16()
        idx, w = fq.route_topk(torch.randn(T, E), topk)
        idx, w = idx.cuda(), w.cuda()
        exact = qb.SparseMoE(wgu, wdn, topk)
        fixed = qb.SparseMoE(wgu, wdn, topk, fixed_capacity=True)
        y = exact.forward(x, idx, w)
        yf = fixed.forward(x, idx, w)
        assert torch.equal(y, yf)
        src, eblk, r_cap, pos = qmoe.build_routing_fixed(idx.reshape(-1).long(), E)
        esrc, eeblk, r_pad = qmoe.build_routing(idx.reshape(-1).long(), E)
        assert r_cap >= r_pad and torch.equal(src[:r_pad], esrc) and bool((src[r_pad:] == -1).all())
        assert torch.equal(eblk[: r_pad // 128], eeblk) and bool((eblk[r_pad // 128:] == -1).all())
        # capture and replay with new inputs of the same shape
        sx, si, sw = x.clone(), idx.clone(), w.clone()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                fixed.forward(sx, si, sw)
        torch.cuda.current_stream().wait_stream(s)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = fixed.forward(sx, si, sw)
        x2 = torch.randn(T, H).cuda().bfloat16()
        idx2, w2 = fq.route_topk(torch.randn(T, E), topk)
        sx.copy_(x2); si.copy_(idx2.cuda()); sw.copy_(w2.cuda())
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, exact.forward(x2, idx2.cuda(), w2.cuda()))
        assert exact.lib.qb_status(0) == 0


def test_route_fixed_kernel_matches_torch_routing_up_to_row_order():
    import quadbit_b200 as qb
    import quadbit_b200.moe as qmoe
    lib = qb.load("sparse_fp4")
    torch.manual_seed(29)
    for n, e in ((1, 1), (300, 8), (5000, 128), (40000, 64)):
        assign = torch.randint(0, e, (n,), device="cuda")
        if e > 4:
            assign[assign == 3] = 2                                  # an expert without rows
        src, eblk, r_cap, pos = qmoe.route_fixed_kernel(lib, assign, e)
        tsrc, teblk, tcap, tpos = qmoe.build_routing_fixed(assign, e)
        assert r_cap == tcap and torch.equal(eblk, teblk)
        # padding in the same rows (segment tails), every slot placed exactly once, in a block of its own expert
        assert torch.equal(src < 0, tsrc < 0)
        valid = src >= 0
        assert torch.equal(torch.sort(src[valid]).values, torch.arange(n, device="cuda"))
        assert torch.equal(pos[src[valid]], torch.nonzero(valid).squeeze(1))
        assert torch.equal(assign[src[valid]].int(), eblk[torch.nonzero(valid).squeeze(1) // 128])
        assert int(valid.sum()) == n and lib.qb_status(0) == 0


def test_route_fixed_range_with_segments_padded_to_256():
    """qb_moe_route_fixed_range(align = 256): every expert's segment is a multiple of 256 rows, the two 128-row blocks of
    a 256-row tile carry the same expert, the slot -> row table and the count of rows in use agree with the segments,
    slots of experts outside [e_base, e_base + e) get no row."""
    import quadbit_b200 as qb
    import quadbit_b200.moe as qmoe
    lib = qb.load("sparse_fp4")
    torch.manual_seed(31)
    dev = "cuda"
    for n, e_total, e_base, e in ((7, 4, 0, 4), (4096, 16, 4, 8), (32768, 128, 0, 128), (9000, 64, 48, 16)):
        assign = torch.randint(0, e_total, (n,), device=dev)
        w_in = torch.rand(n, device=dev)
        r_cap = qmoe.fixed_capacity(n, e, 256)
        src = torch.empty(r_cap, dtype=torch.long, device=dev)
        pos = torch.empty(n, dtype=torch.long, device=dev)
        eblk = torch.empty(r_cap // 128, dtype=torch.int32, device=dev)
        rw = torch.empty(r_cap, dtype=torch.float32, device=dev)
        inverse = torch.empty(n, dtype=torch.int32, device=dev)
        n_used = torch.zeros(1, dtype=torch.int32, device=dev)
        assert lib.qb_moe_route_fixed_range(assign.data_ptr(), src.data_ptr(), pos.data_ptr(), eblk.data_ptr(), n, e_base, e, r_cap, 1, 256,
                                            w_in.data_ptr(), rw.data_ptr(), inverse.data_ptr(), n_used.data_ptr(), S()) == 0
        torch.cuda.synchronize()
        local = (assign >= e_base) & (assign < e_base + e)
        counts = torch.bincount((assign[local] - e_base), minlength=e)
        padded = (counts + 255) // 256 * 256
        assert int(n_used.item()) == int(padded.sum())
        want_eblk = torch.repeat_interleave(torch.arange(e, device=dev, dtype=torch.int32), (padded // 128))
        used_blocks = int(padded.sum()) // 128
        assert torch.equal(eblk[:used_blocks], want_eblk) and bool((eblk[used_blocks:] == -1).all())
        assert torch.equal(eblk[0::2], eblk[1::2])
        assert bool((pos[~local] == -1).all()) and torch.equal(pos.int(), inverse)
        rows = pos[local]
        assert rows.unique().numel() == rows.numel()                          # every local slot has a row of its own
        assert torch.equal(src[rows], torch.nonzero(local).squeeze(1))       # ... which points back at the slot
        assert torch.equal(eblk[rows // 128].long(), assign[local] - e_base)   # ... inside its expert's segment
        assert torch.equal(rw[rows], w_in[local])
        mask = torch.ones(r_cap, dtype=torch.bool, device=dev)
        mask[rows] = False
        assert bool((src[mask] == -1).all()) and bool((rw[mask] == 0).all())    # padding and unused capacity
        assert lib.qb_status(0) == 0


def test_dispatch_of_quantised_rows_equals_gather_then_quantise():
    """qb_quantize_rows + qb_gather_quantized (every token quantised once, routed slots copy the packed row) must give the
    routed batch of qb_gather_quantize_act_peer (gather of bf16 rows fused into their quantiser) bit for bit, with the
    rows split over two source buffers as in an expert-parallel layer."""
    import quadbit_b200 as qb
    from quadbit_b200.tp import ptr_array
    lib = qb.load("sparse_fp4")
    torch.manual_seed(33)
    dev = "cuda"
    for T, H, K, R in ((64, 256, 256, 300), (1000, 2880, 2944, 4096)):
        x = (torch.randn(T, H, device=dev) * 2).to(torch.bfloat16)
        x[3] = 0                                                              # an all-zero token
        src = torch.randint(0, T, (R,), device=dev)
        src[torch.rand(R, device=dev) < 0.2] = -1                            # padding rows
        half = T // 2
        xs = [x[:half].contiguous(), x[half:].contiguous()]
        # reference: gather + quantise of every routed row
        Bb0 = torch.zeros(R, K // 2, dtype=torch.uint8, device=dev)
        sf0 = torch.zeros(lib.qb_sf_atoms_bytes(R, K, 32), dtype=torch.uint8, device=dev)
        g0 = torch.zeros(R, dtype=torch.float32, device=dev)
        assert lib.qb_gather_quantize_act_peer(ptr_array([t.data_ptr() for t in xs]), 2, half, src.data_ptr(), Bb0.data_ptr(), sf0.data_ptr(),
                                               g0.data_ptr(), R, K, H, 32, 0, S()) == 0
        # tokens quantised once per buffer, then the packed rows are copied
        q = []
        for t in xs:
            Bq = torch.empty(half, K // 2, dtype=torch.uint8, device=dev)
            sq = torch.empty(K // 128, half, 4, dtype=torch.uint8, device=dev)
            gq = torch.empty(half, dtype=torch.float32, device=dev)
            assert lib.qb_quantize_rows(t.data_ptr(), Bq.data_ptr(), sq.data_ptr(), gq.data_ptr(), half, K, H, 32, S()) == 0
            q.append((Bq, sq, gq))
        Bb1 = torch.zeros_like(Bb0)
        sf1 = torch.zeros_like(sf0)
        g1 = torch.zeros_like(g0)
        assert lib.qb_gather_quantized(ptr_array([a[0].data_ptr() for a in q]), ptr_array([a[1].data_ptr() for a in q]),
                                       ptr_array([a[2].data_ptr() for a in q]), 2, half, src.data_ptr(), Bb1.data_ptr(), sf1.data_ptr(),
                                       g1.data_ptr(), R, K, 0, S()) == 0
        torch.cuda.synchronize()
        assert torch.equal(Bb0, Bb1) and torch.equal(sf0, sf1) and torch.equal(g0, g1)
        assert lib.qb_status(0) == 0
