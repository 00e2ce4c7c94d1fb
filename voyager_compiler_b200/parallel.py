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


class P2PColumnParallelLinearMX:
    """Column-sharded ``linear_mx`` whose all-gather is fused into the GEMM epilogue: the output
    ``[M, n_total]`` lives in peer-mapped (symmetric) memory on every rank and each rank's GEMM
    writes its column range into its own copy and into every peer's copy with plain stores over
    NVLink (``vq_gemm_bf16_tn_scatter``).  Two stream-ordered barriers per call order the writes
    against the peers' reads.  The weight shard is dequantised once at construction (weights are
    static); activations are dequantised per call by this package's dequantize kernel."""

    def __init__(self, w_codes_shard, w_scale_shard, n_total: int, block_size: int, max_rows: int, group=None,
                 bias_shard: Optional[torch.Tensor] = None):
        import torch.distributed._symmetric_memory as symm_mem
        from . import ops

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.n_total, self.block, self.max_rows = n_total, block_size, max_rows
        self.n0, self.n1 = column_shards(n_total, self.world)[self.rank]
        if w_codes_shard.shape[0] != self.n1 - self.n0:
            raise ValueError("weight shard does not match this rank's column range")
        if w_codes_shard.dtype != torch.bfloat16:
            raise NotImplementedError("the peer-to-peer linear takes bfloat16 operands")
        self.w = ops.dequantize(w_codes_shard, w_scale_shard, None, None, block_size).contiguous()
        self.bias = bias_shard.contiguous() if bias_shard is not None else None
        dev = w_codes_shard.device
        self.y = symm_mem.empty(max_rows, n_total, dtype=torch.bfloat16, device=dev)
        self.handle = symm_mem.rendezvous(self.y, self.group)
        ptrs = list(self.handle.buffer_ptrs)
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        import ctypes as C
        self._ptrs = (C.c_void_p * len(order))(*[ptrs[r] for r in order])
        self._status = torch.zeros(1, dtype=torch.int32, device=dev)

    def __call__(self, x_codes, x_scale) -> torch.Tensor:
        from . import _lib, ops
        m = x_codes.numel() // x_codes.shape[-1]
        if m > self.max_rows:
            raise ValueError(f"{m} rows exceed the {self.max_rows} this object was sized for")
        k = x_codes.shape[-1]
        xd = ops.dequantize(x_codes.reshape(m, k), x_scale.reshape(m, -1), None, None, self.block).contiguous()
        self.handle.barrier(channel=0)        # every rank is done reading the previous result
        if self.n1 > self.n0:
            rc = _lib.lib.vq_gemm_bf16_tn_scatter(
                xd.data_ptr(), self.w.data_ptr(), self.bias.data_ptr() if self.bias is not None else None, self._ptrs,
                self.world, self.n_total, self.n0, m, self.n1 - self.n0, k, self._status.data_ptr(),
                torch.cuda.current_stream(xd.device).cuda_stream)
            _lib.check(rc, "P2PColumnParallelLinearMX")
        self.handle.barrier(channel=1)        # every rank's column range has landed everywhere
        return self.y[:m].reshape(*x_codes.shape[:-1], self.n_total)

    def status(self) -> int:
        v = int(self._status.item())
        self._status.zero_()
        return v
