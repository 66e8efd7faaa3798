"""Llama-architecture prefill forward (configs[3] of the benchmark, at a reduced size the CPU oracle finishes in seconds):
1 GPU against oracle/llama_ref.py, the tensor-parallel data path (GEMM + reduce-scatter by peer stores, reduce + norm +
quantise + all-gather by peer stores) with two ranks emulated on one GPU against the tensor-parallel oracle, and on two real
GPUs (peer-mapped memory) against the NCCL form of the same arithmetic.

Parity is checked stage by stage (`staged_check`): each stage of the oracle is fed the GPU's own output of the stage before,
with the gates of the kernel tests (quantiser codes explained by rounding boundaries, GEMM outputs within 6e-3, residual
stream bit for bit). End to end, a forward chains FP4 quantisers and only agrees at the level of the 4-bit rounding noise."""
import os

import pytest
import torch

from oracle import llama_ref

pytestmark = pytest.mark.gpu


def small_cfg():
    from quadbit_b200.llama import LlamaConfig
    return LlamaConfig(n_layers=2, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, intermediate=1024, vocab=512)


def close(a, b):
    a, b = a.float().cpu(), b.float().cpu()
    assert torch.isfinite(a).all()
    rel = ((a - b).norm() / b.norm()).item()
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    return rel, cos


def atoms_to_sf(atoms: torch.Tensor, rows: int, K: int, block: int) -> torch.Tensor:
    """Inverse of fakequant.sf_to_atoms: scale-factor atoms -> reference layout [K/128, rows, 128/block]."""
    P = 128 // block
    kp = (K // 128 + 1) // 2 * 2
    rp = (rows + 127) // 128 * 128
    a = atoms.cpu().view(rp // 128, kp * P // 4, 32, 4, 4)                    # [rb, atom, r0, r1, c]
    s = a.permute(0, 3, 2, 1, 4).reshape(rp, kp, P)[:rows, : K // 128]
    return s.permute(1, 0, 2).contiguous()


def bf16_err(y, ref):
    y = y.float().cpu()
    assert torch.isfinite(y).all()
    return ((y - ref).abs() / (ref.abs() + 1.0)).max().item()


def staged_check(cfg, w, ids, caps, world):
    """Stage-by-stage parity of ONE layer: every stage of the oracle is fed the GPU's own output of the stage before, so a
    code that falls the other way at one quantiser is not amplified by the next ones. caps[r] = captured tensors of rank r.
    Gates: quantisers by tests/_parity.assert_codes_explained (every differing code within 1e-5 of a rounding boundary),
    GEMM outputs |y - ref| / (|ref| + 1) < 6e-3, bf16 attention relative L2 < 1e-2, the residual stream bit for bit."""
    import torch.nn.functional as F
    from oracle import fakequant as fq
    from tests._parity import assert_codes_explained
    L = w["layers"][0]
    B, S = ids.shape
    T, H, hd, I = B * S, cfg.hidden, cfg.head_dim, cfg.intermediate
    Tl = T // world
    hq, hk, isl = cfg.n_heads // world, cfg.n_kv_heads // world, I // world
    x0 = w["embed"][ids.reshape(-1)]
    # 1. first norm + per-16 quantiser: identical gathered arrays on every rank
    Bb, atoms, g = caps[0]["q16"]
    for c in caps[1:]:
        assert all(torch.equal(a, b) for a, b in zip(c["q16"], caps[0]["q16"]))
    s16 = atoms_to_sf(atoms, T, H, 16)
    y, _ = fq.rmsnorm_fp32(x0, L["norm_attn"], cfg.rms_eps)
    assert_codes_explained(y, Bb, s16, g, 16)
    xq = fq.unpack_act(Bb.cpu(), s16, g.cpu(), 16)
    cos, sin = llama_ref.rope_tables(S, hd, cfg.rope_theta)
    o_sum = torch.zeros(T, H)
    for r, c in enumerate(caps):
        # 2. column-parallel QKV of this rank's heads
        Wr = torch.cat([L["wq"][r * hq * hd:(r + 1) * hq * hd], L["wk"][r * hk * hd:(r + 1) * hk * hd], L["wv"][r * hk * hd:(r + 1) * hk * hd]], 0)
        assert bf16_err(c["qkv"], F.linear(xq, fq.dense_fp4_dequant(Wr.float()))) < 6e-3
        # 3. RoPE + causal GQA attention from the GPU's own qkv
        qkv = c["qkv"].float().cpu()
        q = llama_ref.apply_rope(qkv[:, : hq * hd].view(B, S, hq, hd), cos, sin)
        k = llama_ref.apply_rope(qkv[:, hq * hd:(hq + hk) * hd].view(B, S, hk, hd), cos, sin)
        v = qkv[:, (hq + hk) * hd:].view(B, S, hk, hd)
        kk, vv = k.repeat_interleave(hq // hk, 2), v.repeat_interleave(hq // hk, 2)
        sc = torch.einsum("bshd,bthd->bhst", q, kk) / hd ** 0.5
        sc = sc.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
        assert sc[torch.isfinite(sc)].std() > 0.3    # the scores are far from uniform: RoPE and the head mapping matter
        ref_a = torch.einsum("bhst,bthd->bshd", torch.softmax(sc, -1), vv).reshape(T, hq * hd)
        got_a = c["attn"].float().cpu()
        assert ((got_a - ref_a).norm() / ref_a.norm()).item() < 1e-2
        # 4. row-parallel o_proj over this rank's K slice: the partial rows sit in the owners' slot r
        ks = hq * hd
        ref_o = F.linear(fq.act_dequant_2lvl(got_a, 16), fq.dense_fp4_dequant(L["wo"][:, r * ks:(r + 1) * ks].float()))
        got_o = torch.cat([caps[own]["o_parts"][r] for own in range(world)], 0) if world > 1 else c["o_parts"][0]
        assert bf16_err(got_o, ref_o) < 6e-3
        o_sum += got_o.float().cpu()
    # 5. reduce + residual + norm + per-32 quantiser (rows of rank r), gathered arrays identical everywhere
    for c in caps[1:]:
        assert all(torch.equal(a, b) for a, b in zip(c["q32"], caps[0]["q32"]))
    vsum = o_sum + x0.float()
    x1 = torch.cat([c["x_mlp_in"] for c in caps], 0).cpu()
    assert torch.equal(x1, vsum.to(torch.bfloat16))                         # new residual stream, bit for bit
    y2 = vsum * torch.rsqrt(vsum.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * L["norm_mlp"].float()
    Bb2, atoms2, g2 = caps[0]["q32"]
    s32 = atoms_to_sf(atoms2, T, H, 32)
    assert_codes_explained(y2, Bb2, s32, g2, 32)
    yq = fq.unpack_act(Bb2.cpu(), s32, g2.cpu(), 32)
    d_sum = torch.zeros(T, H)
    for r, c in enumerate(caps):
        # 6. column-parallel gate / up, 7. SwiGLU + quantiser + row-parallel down over this rank's slice
        Wgu = torch.cat([L["w_gate"][r * isl:(r + 1) * isl], L["w_up"][r * isl:(r + 1) * isl]], 0)
        assert bf16_err(c["cgu"], F.linear(yq, fq.sparse_fp4_dequant_2lvl(Wgu.float()))) < 6e-3
        gu = c["cgu"].float().cpu()
        gt, up = gu[:, :isl], gu[:, isl:]
        h = (gt / (1.0 + torch.exp(-gt))) * up
        ref_d = F.linear(fq.act_dequant_2lvl(h, 32, round_bf16=False), fq.sparse_fp4_dequant_2lvl(L["w_down"][:, r * isl:(r + 1) * isl].float()))
        got_d = torch.cat([caps[own]["d_parts"][r] for own in range(world)], 0) if world > 1 else c["d_parts"][0]
        assert bf16_err(got_d, ref_d) < 6e-3
        d_sum += got_d.float().cpu()
    return (d_sum + x1.float()).to(torch.bfloat16).float()


def scaled_weights(cfg):
    """Oracle-side random weights with the q / k projections scaled up so that attention scores are O(1)."""
    w = llama_ref.make_weights(cfg, seed=2)
    for L in w["layers"]:
        L["wq"] = (L["wq"].float() * 3).to(torch.bfloat16)
        L["wk"] = (L["wk"].float() * 3).to(torch.bfloat16)
    return w


def final_hidden(cfg, w, xf):
    hid = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * w["norm_f"].float()
    return hid


def test_forward_stage_by_stage_one_gpu():
    from quadbit_b200.llama import LlamaPrefill
    cfg = small_cfg()
    cfg.n_layers = 1
    w = scaled_weights(cfg)
    ids = torch.randint(0, cfg.vocab, (2, 128), generator=torch.Generator().manual_seed(5))
    model = LlamaPrefill(cfg, w)
    model.capture = cap = {}
    hid, logits = model(ids)
    assert model.lib.qb_status(0) == 0 and model.lib.qb_peer_status(0) == 0
    xf = staged_check(cfg, w, ids, [cap], 1)
    ref_h = final_hidden(cfg, w, xf)
    assert ((hid.float().cpu() - ref_h).abs() / (ref_h.abs() + 1.0)).max().item() < 1e-2
    ref_l = torch.nn.functional.linear(ref_h.to(torch.bfloat16).float().view(2, 128, -1)[:, -1], w["lm_head"].float())
    rel, cos = close(logits, ref_l)
    assert rel < 2e-2 and cos > 0.999, (rel, cos)


def test_forward_end_to_end_one_gpu():
    """Two layers end to end against the oracle. A forward chains FP4 quantisers, so a bf16 rounding that falls the other
    way (RoPE and attention run in bf16 on the GPU, in fp32 in the oracle) re-draws part of the rounding noise of everything
    downstream: the two agree at the level of that noise (about 10 % per element at 4 bits), which still separates a
    correct forward from a wrong one (cosine ~ 0 for a wrong head mapping or layer order)."""
    from quadbit_b200.llama import LlamaPrefill
    cfg = small_cfg()
    w = llama_ref.make_weights(cfg, seed=2)
    ids = torch.randint(0, cfg.vocab, (2, 128), generator=torch.Generator().manual_seed(5))
    model = LlamaPrefill(cfg, w)
    hid, logits = model(ids)
    assert model.lib.qb_status(0) == 0 and model.lib.qb_peer_status(0) == 0
    ref_h, ref_l = llama_ref.forward(ids, w, cfg)
    rel, cos = close(hid, ref_h)
    assert rel < 0.25 and cos > 0.97, (rel, cos)
    hid2, _ = model(ids)
    assert torch.equal(hid, hid2)                 # a second call reuses nothing stale
    for _ in range(2):                            # the CUDA-graph replay gives the same bits
        hid3, logits3 = model.forward_graphed(ids)
        assert torch.equal(hid, hid3) and torch.equal(logits, logits3)


def test_tensor_parallel_data_path_two_ranks_on_one_gpu():
    """Both ranks in this process, buffers plain allocations: every fused kernel of the multi-GPU path runs (peer-store
    epilogue, flag publication, bounded flag waits, multi-source reduce, fan-out stores), launched in an order in which a
    waiting kernel always follows its producers. Checked stage by stage against the tensor-parallel oracle arithmetic."""
    from quadbit_b200.llama import LlamaPrefill, forward_emulated
    from quadbit_b200.tp import TPContext
    cfg = small_cfg()
    cfg.n_layers = 1
    w = scaled_weights(cfg)
    ids = torch.randint(0, cfg.vocab, (2, 128), generator=torch.Generator().manual_seed(5))
    T = ids.numel()
    ctxs = TPContext.emulated(T, cfg.hidden, 2, torch.device("cuda"))
    models = [LlamaPrefill(cfg, w, rank=r, world=2, ctx=ctxs[r]) for r in range(2)]
    for it in range(2):                                  # twice: flags count up, buffers are reused
        caps = [{}, {}]
        for m, c in zip(models, caps):
            m.capture = c
        outs = forward_emulated(models, ids)
        assert models[0].lib.qb_status(0) == 0 and models[0].lib.qb_peer_status(0) == 0
        xf = staged_check(cfg, w, ids, caps, 2)
        ref_h = final_hidden(cfg, w, xf)
        hid = torch.cat([o[0] for o in outs], 0)
        assert ((hid.float().cpu() - ref_h).abs() / (ref_h.abs() + 1.0)).max().item() < 1e-2, it
    # two layers end to end against the tensor-parallel oracle, at the level of the FP4 rounding noise (see the 1-GPU test)
    cfg2 = small_cfg()
    w2 = llama_ref.make_weights(cfg2, seed=2)
    ctxs = TPContext.emulated(T, cfg2.hidden, 2, torch.device("cuda"))
    models = [LlamaPrefill(cfg2, w2, rank=r, world=2, ctx=ctxs[r]) for r in range(2)]
    outs = forward_emulated(models, ids)
    hid = torch.cat([o[0] for o in outs], 0)
    ref_h, _ = llama_ref.forward(ids, w2, cfg2, world=2)
    rel, cos = close(hid, ref_h)
    assert rel < 0.25 and cos > 0.97, (rel, cos)


def _tp_worker(rank, world, port, ret):
    import torch.distributed as dist
    from quadbit_b200.llama import LlamaPrefill
    from quadbit_b200.tp import TPContext
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    cfg = small_cfg()
    w = llama_ref.make_weights(cfg, seed=2)
    ids = torch.randint(0, cfg.vocab, (2, 128), generator=torch.Generator().manual_seed(5))
    ctx = TPContext(ids.numel(), cfg.hidden, rank, world)
    dist.barrier()
    res = {}
    for comm in ("peer", "nccl"):
        model = LlamaPrefill(cfg, w, rank=rank, world=world, comm=comm, ctx=ctx)
        for _ in range(2):
            hid, logits = model(ids)
        if comm == "peer":                      # replayed from a CUDA graph: same bits, flags keep counting
            for _ in range(2):
                hid_g, logits_g = model.forward_graphed(ids)
            assert torch.equal(hid_g, hid) and torch.equal(logits_g, logits)
        torch.cuda.synchronize()
        assert model.lib.qb_status(0) == 0 and model.lib.qb_peer_status(0) == 0
        res[comm] = (hid.cpu(), logits.cpu())
        dist.barrier()
    ret[rank] = res
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_two_gpus_peer_equals_nccl_and_oracle():
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_tp_worker, args=(world, 29531, ret), nprocs=world, join=True)
    cfg = small_cfg()
    w = llama_ref.make_weights(cfg, seed=2)
    ids = torch.randint(0, cfg.vocab, (2, 128), generator=torch.Generator().manual_seed(5))
    ref_h, ref_l = llama_ref.forward(ids, w, cfg, world=2)
    hid_peer = torch.cat([ret[r]["peer"][0] for r in range(world)], 0)
    hid_nccl = torch.cat([ret[r]["nccl"][0] for r in range(world)], 0)
    assert torch.equal(hid_peer, hid_nccl)               # same arithmetic, two transports
    assert torch.equal(ret[0]["peer"][1], ret[1]["peer"][1])
    rel, cos = close(hid_peer, ref_h)
    assert rel < 0.25 and cos > 0.97, (rel, cos)
