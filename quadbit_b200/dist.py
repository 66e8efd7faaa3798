"""Tensor- and expert-parallel sharding of the NVFP4 linears over one node
(one process per GPU, torch.distributed; NCCL on GPUs, gloo in the CPU tests).

The reference has one distributed script, expert parallel with an all-reduce of the partial
[T,H] outputs (harness/moe_dist.py:123,161-162); tensor parallelism it leaves to vLLM. Here:

  column-parallel (QKV, gate, up): rank r owns output rows [r*out/W, (r+1)*out/W). Per-row
      weight globals make each shard bit-identical to the same rows of the unsharded pack;
      no communication.
  row-parallel (o_proj, down): rank r owns K columns [r*K/W, (r+1)*K/W) (a multiple of 256 so
      packed tensors split on stage boundaries); every rank produces a full [tok,out] partial
      and the partials are summed with one all-reduce.
  expert-parallel: rank r owns experts [r*E/W, (r+1)*E/W). Either every rank sees all tokens and the
      partial [T,H] outputs are summed with one all-reduce (`SparseMoE(expert_range=...)`, the
      reference's form), or tokens are sharded too and routed rows travel to their expert's rank and
      back with two all-to-all exchanges (`ep_moe`).

The compute is injected (`linear_fn(x, W_shard) -> y`) so the same helpers run the CUDA
modules on GPUs and the CPU oracle in the gloo tests."""
from __future__ import annotations

import torch
import torch.distributed as dist


def column_shard(W: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    out_f = W.shape[0]
    assert out_f % (128 * world) == 0, "output features must split into 128-row tiles per rank"
    n = out_f // world
    return W[rank * n:(rank + 1) * n].contiguous()


def row_shard(W: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    K = W.shape[1]
    assert K % (256 * world) == 0, "K must split into 256-deep stages per rank"
    n = K // world
    return W[:, rank * n:(rank + 1) * n].contiguous()


def expert_range(n_experts: int, rank: int, world: int) -> tuple[int, int]:
    assert n_experts % world == 0
    n = n_experts // world
    return rank * n, (rank + 1) * n


def column_parallel_linear(x: torch.Tensor, W_shard: torch.Tensor, linear_fn, gather: bool = False):
    """y_shard = linear_fn(x, W_shard) [tok, out/W]; with gather=True all-gathers to [tok,out]."""
    y = linear_fn(x, W_shard)
    if not gather or not dist.is_initialized() or dist.get_world_size() == 1:
        return y
    parts = [torch.empty_like(y) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, y.contiguous())
    return torch.cat(parts, dim=-1)


def row_parallel_linear(x: torch.Tensor, W_shard: torch.Tensor, linear_fn, rank: int, world: int):
    """x [tok,K] replicated; each rank multiplies its K slice and the partials are all-reduced."""
    n = x.shape[-1] // world
    y = linear_fn(x[..., rank * n:(rank + 1) * n].contiguous(), W_shard)
    if dist.is_initialized() and world > 1:
        dist.all_reduce(y)
    return y


def all_reduce_sum(t: torch.Tensor) -> torch.Tensor:
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t)
    return t


def ep_moe(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, n_experts: int, expert_rows_fn, combine_fn=None,
           group=None) -> torch.Tensor:
    """Expert-parallel MoE layer with all-to-all dispatch and combine.

    x [T_local,H] are this rank's tokens, topk_idx / topk_w [T_local,topk] their global expert ids and
    routing weights; rank r owns experts [r*E/W, (r+1)*E/W). Routed slots are sorted by expert (hence by
    destination rank), rows + local expert id + routing weight go out in one all-to-all per tensor,
    `expert_rows_fn(rows, local_expert, weight) -> [n,H]` runs on the owner, the weighted outputs come
    back in a second all-to-all in the order they were sent, and the top-k rows of every token are summed
    at home by `combine_fn(d, inverse, T)` (default: fp32 sum in slot order, rounded to x.dtype).
    Split sizes are exchanged first (one small all-to-all and a host read: NCCL needs them on the host)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    assert n_experts % world == 0
    epr = n_experts // world
    T, topk = topk_idx.shape
    flat_e = topk_idx.reshape(-1).long()
    order = torch.argsort(flat_e.to(torch.int16) if n_experts < 32768 else flat_e, stable=True)
    send_e = flat_e[order]
    send_rows = x[order // topk].contiguous()
    send_w = topk_w.reshape(-1)[order].float().contiguous()
    if world > 1:
        send_counts = torch.bincount(send_e // epr, minlength=world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        n_recv = sum(rc)
        recv_rows = x.new_empty((n_recv, x.shape[1]))
        dist.all_to_all_single(recv_rows, send_rows, rc, sc, group=group)
        meta_out = torch.stack([(send_e - (send_e // epr) * epr).float(), send_w], 1).contiguous()   # local expert id, weight
        meta_in = meta_out.new_empty((n_recv, 2))
        dist.all_to_all_single(meta_in, meta_out, rc, sc, group=group)
        recv_e, recv_w = meta_in[:, 0].long(), meta_in[:, 1].contiguous()
    else:
        sc = rc = None
        recv_rows, recv_e, recv_w = send_rows, send_e - rank * epr, send_w
    out = expert_rows_fn(recv_rows, recv_e, recv_w).contiguous()
    if world > 1:
        back = out.new_empty((send_rows.shape[0], out.shape[1]))
        dist.all_to_all_single(back, out, sc, rc, group=group)
    else:
        back = out
    inverse = torch.empty((T * topk,), dtype=torch.int32, device=x.device)
    inverse[order] = torch.arange(T * topk, dtype=torch.int32, device=x.device)
    if combine_fn is not None:
        return combine_fn(back, inverse, T)
    return back.float()[inverse.long().view(T, topk)].sum(1).to(x.dtype)
