"""Llama-architecture prefill forward (configs[3] of the benchmark, at a reduced size the CPU oracle finishes in seconds):
1 GPU against oracle/llama_ref.py, the tensor-parallel data path (GEMM + reduce-scatter by peer stores, reduce + norm +
quantise + all-gather by peer stores) with two ranks emulated on one GPU against the tensor-parallel oracle, and on two real
GPUs (peer-mapped memory) against the NCCL form of the same arithmetic.

Tolerance: the forward chains quantisers, so one bf16 rounding that falls the other way moves a few E2M1 codes downstream;
final hidden states and logits must agree with the oracle to relative L2 error < 0.05 and cosine > 0.998."""
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


def test_forward_matches_oracle_one_gpu():
    from quadbit_b200.llama import LlamaPrefill
    cfg = small_cfg()
    w = llama_ref.make_weights(cfg, seed=2)
    ids = torch.randint(0, cfg.vocab, (2, 128), generator=torch.Generator().manual_seed(5))
    model = LlamaPrefill(cfg, w)
    hid, logits = model(ids)
    assert model.lib.qb_status(0) == 0 and model.lib.qb_peer_status(0) == 0
    ref_h, ref_l = llama_ref.forward(ids, w, cfg)
    rel, cos = close(hid, ref_h)
    assert rel < 0.05 and cos > 0.998, (rel, cos)
    rel, cos = close(logits, ref_l)
    assert rel < 0.05 and cos > 0.998, (rel, cos)
    # a second call reuses nothing stale
    hid2, _ = model(ids)
    assert torch.equal(hid, hid2)


def test_tensor_parallel_data_path_two_ranks_on_one_gpu():
    """Both ranks in this process, buffers plain allocations: every fused kernel of the multi-GPU path runs (peer-store
    epilogue, flag publication, bounded flag waits, multi-source reduce, fan-out stores), launched in an order in which a
    waiting kernel always follows its producers."""
    from quadbit_b200.llama import LlamaPrefill, forward_emulated
    from quadbit_b200.tp import TPContext
    cfg = small_cfg()
    w = llama_ref.make_weights(cfg, seed=2)
    ids = torch.randint(0, cfg.vocab, (2, 128), generator=torch.Generator().manual_seed(5))
    T = ids.numel()
    ctxs = TPContext.emulated(T, cfg.hidden, 2, torch.device("cuda"))
    models = [LlamaPrefill(cfg, w, rank=r, world=2, ctx=ctxs[r]) for r in range(2)]
    for it in range(2):                                  # twice: flags count up, buffers are reused
        outs = forward_emulated(models, ids)
        assert models[0].lib.qb_status(0) == 0 and models[0].lib.qb_peer_status(0) == 0
        hid = torch.cat([o[0] for o in outs], 0)
        ref_h, ref_l = llama_ref.forward(ids, w, cfg, world=2)
        rel, cos = close(hid, ref_h)
        assert rel < 0.05 and cos > 0.998, (it, rel, cos)
        rel, cos = close(outs[0][1], ref_l)
        assert rel < 0.05 and cos > 0.998, (it, rel, cos)
    # and the tensor-parallel result agrees with the one-rank model at the level of the FP4 rounding noise (the
    # row-parallel linears quantise each K slice against its own token maximum, so the noise is drawn differently)
    one_h, _ = llama_ref.forward(ids, w, cfg, world=1)
    rel, cos = close(hid, one_h)
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
    assert rel < 0.05 and cos > 0.998, (rel, cos)
    rel, cos = close(ret[0]["peer"][1], ref_l)
    assert rel < 0.05 and cos > 0.998, (rel, cos)
