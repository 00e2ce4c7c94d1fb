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

__all__ = ["column_shards", "shard_weight", "column_parallel_linear_mx", "ColumnParallelLinearMX", "P2PColumnParallelLinearMX"]

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


class ColumnParallelLinearMX:
    """``linear_mx`` with the weight sharded by output columns over ``group`` and the result exchanged with
    NCCL all-gathers, prepared once per weight shard (the decoded weight pieces are found again on the next
    call).  With ``chunks`` > 1 the shard's columns are cut into that many pieces (multiples of the GEMM's
    256-wide tile): while the GEMM of piece ``c + 1`` runs on the caller's stream, piece ``c`` is gathered and
    copied into place on a side stream.  This is the library-collective form of the exchange;
    :class:`P2PColumnParallelLinearMX`, which stores from the GEMM epilogue into the peers' memory, is the fast one.  Returns the full ``[..., n_total]`` result on every rank.  ``gemm`` defaults to
    ``torch.ops.quantized_ops.linear_mx`` (tests on CPU pass a stand-in so the exchange logic runs under gloo)."""

    def __init__(self, w_codes_shard, w_scale_shard, n_total: int, block_size: int, group=None,
                 bias_shard: Optional[torch.Tensor] = None, gemm: Optional[Callable] = None, chunks: Optional[int] = None):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.n_total, self.block = n_total, block_size
        self.shards = column_shards(n_total, self.world)
        n0, n1 = self.shards[self.rank]
        if w_codes_shard.shape[0] != n1 - n0:
            raise ValueError(f"rank {self.rank} holds {w_codes_shard.shape[0]} weight rows, its shard is {n1 - n0}")
        self.gemm = gemm if gemm is not None else torch.ops.quantized_ops.linear_mx
        self.width = max(b - a for a, b in self.shards)                 # equal-sized exchange buffers
        tiles = -(-self.width // TILE_N)
        if chunks is None:
            # one piece: measured on 4 x B200 the cfg5 linear takes 0.84 ms in one piece and 1.08 ms in four --
            # every piece adds a GEMM, a collective and a copy per rank to the launch queue, and at these sizes
            # (11 MB per piece and rank) the host cannot queue them as fast as the GPU retires them
            chunks = 1
        chunks = max(1, min(int(chunks), tiles))
        per = -(-tiles // chunks) * TILE_N
        # piece c covers shard-local columns [c * per, (c + 1) * per); the views are kept so that the decoded
        # copies of the weight pieces are found again on the next call
        self.pieces = []
        for c0 in range(0, self.width, per):
            c1 = min(c0 + per, self.width)
            lo, hi = min(c0, n1 - n0), min(c1, n1 - n0)
            self.pieces.append((c0, c1, w_codes_shard[lo:hi], w_scale_shard[lo:hi] if w_scale_shard is not None else None,
                                bias_shard[lo:hi] if bias_shard is not None else None))
        self._side = torch.cuda.Stream(w_codes_shard.device) if w_codes_shard.is_cuda and self.world > 1 else None

    def __call__(self, x_codes, x_scale) -> torch.Tensor:
        lead = x_codes.shape[:-1]
        m = 1
        for d in lead:
            m *= d
        out = torch.empty((m, self.n_total), dtype=x_codes.dtype, device=x_codes.device)
        main = torch.cuda.current_stream(x_codes.device) if self._side is not None else None
        for c0, c1, wq, ws, bias in self.pieces:
            w = c1 - c0
            if wq.shape[0]:
                y = self.gemm(x_codes, wq, bias, input_scale=x_scale, weight_scale=ws, block_size=self.block).reshape(m, wq.shape[0])
            else:
                y = x_codes.new_empty((m, 0))
            if self.world == 1:
                out[:, c0:c0 + y.shape[1]] = y
                continue
            send = y if y.shape[1] == w else torch.nn.functional.pad(y, (0, w - y.shape[1]))
            recv = torch.empty((self.world, m, w), dtype=send.dtype, device=send.device)
            if self._side is not None:
                ready = torch.cuda.Event()
                ready.record(main)
                with torch.cuda.stream(self._side):
                    self._side.wait_event(ready)
                    self._exchange(send.contiguous(), recv, out, c0, w)
                send.record_stream(self._side)
                recv.record_stream(self._side)
            else:
                self._exchange(send.contiguous(), recv, out, c0, w)
        if self._side is not None:
            main.wait_stream(self._side)
        return out.reshape(*lead, self.n_total)

    def _exchange(self, send, recv, out, c0, w):
        dist.all_gather_into_tensor(recv.view(self.world * recv.shape[1], w), send, group=self.group)
        for r, (a, b) in enumerate(self.shards):
            lo, hi = min(a + c0, b), min(a + c0 + w, b)
            if hi > lo:
                out[:, lo:hi] = recv[r, :, : hi - lo]


def column_parallel_linear_mx(x_codes, x_scale, w_codes_shard, w_scale_shard, n_total: int, block_size: int,
                              group=None, bias_shard: Optional[torch.Tensor] = None,
                              gemm: Optional[Callable] = None, chunks: Optional[int] = None) -> torch.Tensor:
    """One call of :class:`ColumnParallelLinearMX` (which is the form to keep when the same weight shard is
    used again: it reuses the decoded weight pieces and its side stream)."""
    return ColumnParallelLinearMX(w_codes_shard, w_scale_shard, n_total, block_size, group, bias_shard, gemm, chunks)(x_codes, x_scale)


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
        # own copy first, then the peers starting with the next rank: at any moment the ranks write to
        # different destinations instead of all starting on rank 0's memory
        order = [(self.rank + d) % self.world for d in range(self.world)]
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
