"""Multi-GPU forms of the two shardable pieces of the path (one process per GPU).

* Whole-model weight quantization needs no exchange: ``model_quant.shard_plan`` partitions the
  tensors, every rank quantizes its share.
* The MX linear shards by output columns (rows of the ``[N, K]`` weight): every rank holds the
  codes and scales of its rows, activations are replicated, each rank computes ``Y[:, n0:n1]`` and
  the shards are exchanged with one all-gather.  Shards are cut on multiples of the GEMM's 256-wide
  output tile so that no rank computes a partial tile twice.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["column_shards", "shard_weight", "column_parallel_linear_mx"]

TILE_N = 256


def column_shards(n: int, world_size: int, tile: int = TILE_N) -> List[Tuple[int, int]]:
    """``[(n0, n1)]`` per rank: contiguous column ranges covering ``[0, n)``, cut on multiples of
    ``tile`` and balanced to within one tile (a rank may get an empty range when there are fewer
    tiles than ranks)."""
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    tiles = -(-n // tile)
    out, t0 = [], 0
    for r in range(world_size):
        cnt = tiles // world_size + (1 if r < tiles % world_size else 0)
        n0, n1 = min(t0 * tile, n), min((t0 + cnt) * tile, n)
        out.append((n0, n1))
        t0 += cnt
    return out


def shard_weight(w_codes: torch.Tensor, w_scale: torch.Tensor, rank: int, world_size: int):
    """Rows of the ``[N, K]`` weight codes and ``[N, K/block]`` scales this rank owns."""
    n0, n1 = column_shards(w_codes.shape[0], world_size)[rank]
    return w_codes[n0:n1].contiguous(), w_scale[n0:n1].contiguous()


def column_parallel_linear_mx(x_codes, x_scale, w_codes_shard, w_scale_shard, n_total: int, block_size: int,
                              group=None, bias_shard: Optional[torch.Tensor] = None,
                              gemm: Optional[Callable] = None) -> torch.Tensor:
    """``linear_mx`` with the weight sharded by output columns over ``group``.  Returns the full
    ``[..., n_total]`` result on every rank.  ``gemm`` defaults to ``torch.ops.quantized_ops.linear_mx``
    (tests on CPU pass a stand-in so that the exchange logic runs under gloo)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    shards = column_shards(n_total, world)
    n0, n1 = shards[rank]
    if w_codes_shard.shape[0] != n1 - n0:
        raise ValueError(f"rank {rank} holds {w_codes_shard.shape[0]} weight rows, its shard is {n1 - n0}")
    if gemm is None:
        gemm = torch.ops.quantized_ops.linear_mx
    lead = x_codes.shape[:-1]
    m = 1
    for d in lead:
        m *= d
    if n1 > n0:
        y_local = gemm(x_codes, w_codes_shard, bias_shard, input_scale=x_scale, weight_scale=w_scale_shard,
                       block_size=block_size).reshape(m, n1 - n0)
    else:
        y_local = x_codes.new_empty((m, 0))
    if world == 1:
        return y_local.reshape(*lead, n_total)
    # equal-sized exchange buffers: shards differ by at most one tile
    width = max(b - a for a, b in shards)
    send = y_local if y_local.shape[1] == width else torch.nn.functional.pad(y_local, (0, width - y_local.shape[1]))
    recv = torch.empty((world * m, width), dtype=send.dtype, device=send.device)
    dist.all_gather_into_tensor(recv, send.contiguous(), group=group)
    recv = recv.view(world, m, width)
    out = torch.empty((m, n_total), dtype=send.dtype, device=send.device)
    for r, (a, b) in enumerate(shards):
        if b > a:
            out[:, a:b] = recv[r, :, : b - a]
    return out.reshape(*lead, n_total)
