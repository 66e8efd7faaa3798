"""world_size-2 gloo tests (CPU) of the sharding logic used for N > 1: column-parallel shards are
bit-identical slices, row-parallel and expert-parallel partials all-reduce to the 1-rank result."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import fakequant as fq
from quadbit_b200 import dist as qd


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    torch.set_num_threads(2)
    tok, K, out_f = 24, 512, 256
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    full = fq.linear_sparse(x, W)
    # column parallel: shard rows are exactly the rows of the full result
    y_col = qd.column_parallel_linear(x, qd.column_shard(W, rank, world), fq.linear_sparse, gather=True)
    ok_col = torch.equal(y_col, full)
    # row parallel: per-slice quantisation globals differ from the 1-rank pack, so equality is to tolerance
    y_row = qd.row_parallel_linear(x, qd.row_shard(W, rank, world), fq.linear_sparse, rank, world)
    err_row = ((y_row - full).norm() / full.norm()).item()
    # expert parallel: partial MoE outputs sum to the full layer
    E, topk = 4, 2
    Ws = [torch.randn(128, K) * 0.02 for _ in range(E)]
    idx, w = fq.route_topk(torch.randn(tok, E), topk)

    def moe(e0, e1):
        y = torch.zeros(tok, 128)
        for e in range(e0, e1):
            sel = (idx == e)
            t = torch.nonzero(sel.any(1)).squeeze(1)
            if t.numel():
                y[t] += fq.linear_sparse(x[t], Ws[e]) * (w * sel)[t].sum(1, keepdim=True)
        return y

    e0, e1 = qd.expert_range(E, rank, world)
    y_ep = qd.all_reduce_sum(moe(e0, e1))
    err_ep = (y_ep - moe(0, E)).abs().max().item()
    if rank == 0:
        ret.put((ok_col, err_row, err_ep))
    dist.barrier()
    dist.destroy_process_group()


def test_tp_ep_sharding_world2_gloo():
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    ok_col, err_row, err_ep = ret.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok_col
    # each K slice is quantised against its own row/token maxima, so the two results carry
    # independent FP4 rounding noise (about 9 % each against the unquantised product)
    assert err_row < 0.15
    assert err_ep < 1e-5


def _ep_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(3)
    torch.set_num_threads(2)
    T, K, H, E, topk = 40, 256, 128, 4, 2
    Ws = [torch.randn(H, K) * 0.02 for _ in range(E)]
    x = torch.randn(T, K)
    idx, w = fq.route_topk(torch.randn(T, E), topk)
    idx[:5] = torch.tensor([2, 3])           # uneven split sizes: the first tokens all go to rank 1's experts
    e0, _ = qd.expert_range(E, rank, world)

    def expert_rows(rows, local_e, weight):
        out = torch.zeros(rows.shape[0], H)
        for e in local_e.unique().tolist():
            sel = local_e == e
            out[sel] = fq.linear_sparse(rows[sel], Ws[e0 + e]) * weight[sel, None]
        return out

    tl = T // world
    mine = slice(rank * tl, (rank + 1) * tl)
    y = qd.ep_moe(x[mine], idx[mine], w[mine], E, expert_rows)
    full = torch.zeros(T, H)
    for e in range(E):
        sel = idx == e
        t = torch.nonzero(sel.any(1)).squeeze(1)
        full[t] += fq.linear_sparse(x[t], Ws[e]) * (w * sel)[t].sum(1, keepdim=True)
    ret.put((rank, (y - full[mine]).abs().max().item()))
    dist.barrier()
    dist.destroy_process_group()


def test_ep_all_to_all_dispatch_combine_world2_gloo():
    """Tokens and experts both sharded over two ranks: rows go to their expert's rank and come back
    (uneven split sizes included); every rank's slice equals the single-process layer."""
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(ret.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got[0] < 1e-5 and got[1] < 1e-5


def test_ep_single_process_is_plain_topk_sum():
    torch.manual_seed(4)
    T, K, H, E, topk = 12, 256, 128, 4, 2
    Ws = [torch.randn(H, K) * 0.02 for _ in range(E)]
    x = torch.randn(T, K)
    idx, w = fq.route_topk(torch.randn(T, E), topk)
    fn = lambda rows, le, wt: torch.stack([fq.linear_sparse(rows[i:i + 1], Ws[int(le[i])])[0] * wt[i] for i in range(rows.shape[0])])
    y = qd.ep_moe(x, idx, w, E, fn)
    ref = torch.zeros(T, H)
    for t in range(T):
        for k in range(topk):
            ref[t] += fq.linear_sparse(x[t:t + 1], Ws[int(idx[t, k])])[0] * w[t, k]
    assert (y - ref).abs().max().item() < 1e-5


def test_shard_shapes_stay_tile_aligned():
    for out_f, K in ((6144, 4096), (14336, 4096), (4096, 14336), (4096, 4096)):
        W = torch.empty(out_f, K)
        for world in (2, 4, 8):
            assert qd.column_shard(W, world - 1, world).shape == (out_f // world, K)
            assert qd.row_shard(W, 0, world).shape == (out_f, K // world)
            assert (K // world) % 256 == 0 and (out_f // world) % 128 == 0
