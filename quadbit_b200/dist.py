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
  expert-parallel: rank r owns experts [r*E/W, (r+1)*E/W); partial [T,H] outputs are summed
      with one all-reduce (`SparseMoE(expert_range=...)`).

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
