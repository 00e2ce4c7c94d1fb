"""Whole-model MX weight quantization: many tensors, one kernel launch.

Upstream quantizes the parameters of a converted model one by one with ``calculate_mx_qparam``
followed by ``quantize`` (src/voyager_compiler/quantization/quantize_pt2e.py:485-500), each a
chain of full-size torch passes.  Here every parameter that shares dtype, block size and table
goes through ``vq_quantize_mx_multi``: a single persistent launch that reads each weight once and
writes packed codes (4 or 8 bits) plus one fp32 scale per block, or -- for drop-in use -- the same
float ``(scale, codes)`` pair the upstream ops return.

Layer-wise sharding over several GPUs is plain partitioning: :func:`shard_plan` gives every
rank a subset of the tensors (and a row range of tensors worth splitting) balanced by element
count; no collective is needed because blocks never cross rows.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from .qtables import exp_tables, table_handle

__all__ = ["PackedMX", "quantize_tensors_mx", "MXQuantPlan", "ChannelQuant", "ChannelQuantPlan", "quantize_tensors_per_channel", "dequantize_packed", "unpack_codes", "dequantize_packed_reference", "shard_plan",
           "HostPipeline"]

_DT = {torch.float32: _lib.VQ_F32, torch.bfloat16: _lib.VQ_BF16}
_workspaces: Dict[Tuple[str, int], torch.Tensor] = {}


@dataclass
class PackedMX:
    """Packed result for one tensor.  ``codes``: uint8, ``code_bits`` per element along the last
    axis (two per byte for 4 bits, even element in the low nibble).  ``scale``: fp32, one per
    block.  ``levels``: fp32 value of each code (host tensor); value = levels[code] * scale."""
    codes: torch.Tensor
    scale: torch.Tensor
    shape: Tuple[int, ...]
    block: int
    code_bits: int
    levels: torch.Tensor
    exp_e8: Optional[torch.Tensor] = None

    def levels_on(self, device) -> torch.Tensor:
        """fp32 levels on ``device`` (copied once per device and kept)."""
        cache = self.__dict__.setdefault("_levels_dev", {})
        key = str(device)
        t = cache.get(key)
        if t is None:
            t = cache[key] = self.levels.to(device, torch.float32).contiguous()
        return t


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (str(device), torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _check_block_multiple(tensors, idx, device, block):
    for i in idx:
        t = tensors[i]
        if t.device != device:
            raise ValueError("all tensors must live on one device")
        if t.ndim < 1 or t.shape[-1] % block:
            raise NotImplementedError(
                f"tensor {i}: last dimension {tuple(t.shape)} must be a multiple of the block ({block})")


def _build_items(tensors, idx, dt, device, block, code_bits, float_outputs, want_exp, levels, results, in_place=False):
    """Descriptors and freshly allocated outputs for the tensors ``idx`` (all of dtype ``dt``).
    Fills ``results`` and returns ``(items, inputs kept alive)``.  ``in_place``: the tensors are read
    where they are (they must be contiguous) instead of through ``.contiguous()`` copies."""
    items = (_lib.VqMxItem * len(idx))()
    keep = []

    def source(i):
        t = tensors[i]
        if in_place and not t.is_contiguous():
            raise ValueError(f"tensor {i} must be contiguous (the plan reads it in place)")
        return t.contiguous()

    if float_outputs:
        for k, i in enumerate(idx):
            t = tensors[i]
            x = source(i)
            sc = torch.empty(tuple(t.shape[:-1]) + (t.shape[-1] // block,), dtype=dt, device=device)
            cd = torch.empty_like(x)
            items[k].input, items[k].n = x.data_ptr(), x.numel()
            items[k].out_scale, items[k].out_codes = sc.data_ptr(), cd.data_ptr()
            results[i] = (sc, cd)
            keep.append(x)
        return items, keep
    # one allocation per output kind for the whole group; the per-tensor results are views
    # (16-byte aligned segments), which keeps the host cost of a call low for many tensors
    per_byte = 8 // code_bits
    nel = [tensors[i].numel() for i in idx]
    cbytes = [(n // per_byte + 15) // 16 * 16 for n in nel]
    nblk = [n // block for n in nel]
    codes_all = torch.empty(sum(cbytes), dtype=torch.uint8, device=device)
    scale_all = torch.empty(sum(nblk), dtype=torch.float32, device=device)
    exp_all = torch.empty(sum(nblk), dtype=torch.int8, device=device) if want_exp else None
    cviews, sviews = codes_all.split(cbytes), scale_all.split(nblk)
    eviews = exp_all.split(nblk) if want_exp else None
    cbase, sbase = codes_all.data_ptr(), scale_all.data_ptr()
    ebase = exp_all.data_ptr() if want_exp else 0
    coff = soff = 0
    for k, i in enumerate(idx):
        t = tensors[i]
        x = source(i)
        lead = tuple(t.shape[:-1])
        items[k].input, items[k].n = x.data_ptr(), nel[k]
        items[k].scale_f32, items[k].codes = sbase + 4 * soff, cbase + coff
        if want_exp:
            items[k].exp_e8 = ebase + soff
        cd = cviews[k][:nel[k] // per_byte].view(lead + (t.shape[-1] // per_byte,))
        sc = sviews[k].view(lead + (t.shape[-1] // block,))
        ex = eviews[k].view(lead + (t.shape[-1] // block,)) if want_exp else None
        results[i] = PackedMX(cd, sc, tuple(t.shape), block, code_bits, levels, ex)
        coff += cbytes[k]
        soff += nblk[k]
        keep.append(x)
    return items, keep


def _tables_for(qmap, scale_qmap, device, float_outputs, code_bits):
    tab = table_handle(qmap, device)
    if not float_outputs:
        if code_bits not in (4, 8):
            raise ValueError("code_bits must be 4 or 8")
        tab.with_codes()
        if code_bits == 4 and tab.levels.numel() > 16:
            raise ValueError(f"table has {tab.levels.numel()} levels; 4-bit codes hold 16")
    stab = table_handle(scale_qmap, device, allow_runs=False) if scale_qmap is not None else None
    return tab, stab


def quantize_tensors_mx(tensors: Sequence[torch.Tensor], qmap, block: int, quant_max: float,
                        force_scale_power_of_two: bool = False, scale_qmap=None, code_bits: Optional[int] = 4,
                        float_outputs: bool = False, want_exp: bool = False):
    """Quantize every tensor (blocks of ``block`` along the last, contiguous axis) in one launch
    per dtype.  ``qmap``: a 65 536-entry table tensor, a numpy pattern array or an upstream dtype
    string.  Returns a list of :class:`PackedMX` (``code_bits`` 4 or 8), or, with
    ``float_outputs=True``, a list of ``(scale, codes)`` float tensors exactly as
    ``torch.ops.quantized_ops.quantize_mx`` returns them."""
    if not tensors:
        return []
    device = tensors[0].device
    if device.type != "cuda":
        raise RuntimeError("quantize_tensors_mx: CUDA tensors only; there is no CPU path")
    results: List = [None] * len(tensors)
    with torch.cuda.device(device):
        tab, stab = _tables_for(qmap, scale_qmap, device, float_outputs, code_bits)
        stream = torch.cuda.current_stream(device).cuda_stream
        for dt in (torch.bfloat16, torch.float32):
            idx = [i for i, t in enumerate(tensors) if t.dtype == dt]
            if not idx:
                continue
            exp = exp_tables(dt, quant_max, device) if force_scale_power_of_two else None
            _check_block_multiple(tensors, idx, device, block)
            items, keep = _build_items(tensors, idx, dt, device, block, code_bits, float_outputs, want_exp,
                                       None if float_outputs else tab.levels, results)
            need = _lib.lib.vq_quantize_mx_multi_workspace(len(idx))
            ws = _workspace(device, need)
            _lib.check(_lib.lib.vq_quantize_mx_multi(
                items, len(idx), _DT[dt], block, float(quant_max), 1 if force_scale_power_of_two else 0,
                exp.ptr() if exp is not None else None, stab.ptr() if stab is not None else None, tab.ptr(),
                0 if float_outputs else code_bits, ws.data_ptr(), ws.numel(), stream), "quantize_tensors_mx")
            del keep
    return results


class MXQuantPlan:
    """:func:`quantize_tensors_mx` prepared once: outputs, descriptors, tables and the launch shape
    are fixed at construction, so :meth:`run` is one library call -- one kernel launch -- per dtype
    with no allocation, no descriptor copy and no Python work that grows with the tensor count.
    For passes that repeat over the same parameters (weights re-quantized every calibration or
    training step, the shards of a whole-model pass).  The tensors are read where they are when
    ``run()`` executes, so they must be contiguous and stay alive; ``results`` (one
    :class:`PackedMX`, or one ``(scale, codes)`` pair with ``float_outputs``, per tensor) is
    overwritten by every run."""

    def __init__(self, tensors: Sequence[torch.Tensor], qmap, block: int, quant_max: float,
                 force_scale_power_of_two: bool = False, scale_qmap=None, code_bits: Optional[int] = 4,
                 float_outputs: bool = False, want_exp: bool = False):
        if not tensors:
            raise ValueError("no tensors")
        device = tensors[0].device
        if device.type != "cuda":
            raise RuntimeError("MXQuantPlan: CUDA tensors only; there is no CPU path")
        self.device = device
        self.results: List = [None] * len(tensors)
        self._plans: List[C.c_void_p] = []
        self._keep = []
        with torch.cuda.device(device):
            self._tab, self._stab = _tables_for(qmap, scale_qmap, device, float_outputs, code_bits)
            stream = torch.cuda.current_stream(device).cuda_stream
            for dt in (torch.bfloat16, torch.float32):
                idx = [i for i, t in enumerate(tensors) if t.dtype == dt]
                if not idx:
                    continue
                exp = exp_tables(dt, quant_max, device) if force_scale_power_of_two else None
                _check_block_multiple(tensors, idx, device, block)
                items, keep = _build_items(tensors, idx, dt, device, block, code_bits, float_outputs, want_exp,
                                           None if float_outputs else self._tab.levels, self.results, in_place=True)
                ws = torch.empty(max(_lib.lib.vq_quantize_mx_multi_workspace(len(idx)), 16), dtype=torch.uint8, device=device)
                handle = C.c_void_p()
                _lib.check(_lib.lib.vq_mx_plan_create(
                    items, len(idx), _DT[dt], block, float(quant_max), 1 if force_scale_power_of_two else 0,
                    exp.ptr() if exp is not None else None, self._stab.ptr() if self._stab is not None else None,
                    self._tab.ptr(), 0 if float_outputs else code_bits, ws.data_ptr(), ws.numel(), stream,
                    C.byref(handle)), "MXQuantPlan")
                self._plans.append(handle)
                self._keep.append((keep, ws, exp))

    def run(self) -> List:
        """Queue the pass on the current stream of the plan's device; returns ``results``."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        run, check = _lib.lib.vq_mx_plan_run, _lib.check
        with torch.cuda.device(self.device):
            for h in self._plans:
                check(run(h, stream), "MXQuantPlan.run")
        return self.results

    def close(self) -> None:
        for h in self._plans:
            _lib.lib.vq_mx_plan_destroy(h)
        self._plans = []

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass


@dataclass
class ChannelQuant:
    """Per-channel result for one tensor (fields not asked for are ``None``).  ``scale`` and ``amax``
    have the keepdim shape ``[C, 1, ...]`` upstream's observer produces; ``values`` is what
    ``quantize`` returns, ``dequant`` what ``dequantize(values, scale)`` returns."""
    scale: Optional[torch.Tensor]
    amax: Optional[torch.Tensor]
    values: Optional[torch.Tensor]
    codes: Optional[torch.Tensor]
    dequant: Optional[torch.Tensor]
    levels: Optional[torch.Tensor] = None


class ChannelQuantPlan:
    """Outputs and launch descriptors of a per-channel pass, prepared once: ``run()`` is then one
    library call per dtype (no allocation), for weights that are re-quantized every step
    (calibration, quantization-aware training).  ``results`` holds one :class:`ChannelQuant` per
    tensor; the tensors are read where they are at the time of ``run()``."""

    def __init__(self, tensors: Sequence[torch.Tensor], qmap, quant_max: float, *, scales=None,
                 want_values: bool = False, want_codes: bool = False, want_dequant: bool = True,
                 want_amax: bool = False):
        if not tensors:
            raise ValueError("no tensors")
        device = tensors[0].device
        if device.type != "cuda":
            raise RuntimeError("quantize_tensors_per_channel: CUDA tensors only; there is no CPU path")
        if not (want_values or want_codes or want_dequant or want_amax):
            raise ValueError("nothing to compute")
        self.device = device
        self.quant_max = float(quant_max)
        self.results: List = [None] * len(tensors)
        self._groups = []
        self._keep = []
        with torch.cuda.device(device):
            self._tab = table_handle(qmap, device)
            try:
                self._tab.with_codes()          # code table + levels by (code, sign): the pipelined kernel's tables
            except ValueError:
                if want_codes:
                    raise
            for dt in (torch.bfloat16, torch.float32):
                idx = [i for i, t in enumerate(tensors) if t.dtype == dt]
                if not idx:
                    continue
                items = (_lib.VqChannelItem * len(idx))()
                for k, i in enumerate(idx):
                    t = tensors[i]
                    if t.device != device or t.ndim < 1:
                        raise ValueError("all tensors must live on one device and have a channel axis")
                    if not t.is_contiguous():
                        raise ValueError("tensors must be contiguous (the plan reads them in place)")
                    ch = t.shape[0]
                    kd = (ch,) + (1,) * (t.ndim - 1)
                    r = ChannelQuant(None, None, None, None, None, self._tab.levels if want_codes else None)
                    items[k].input = t.data_ptr()
                    items[k].channels = ch
                    items[k].length = t.numel() // ch if ch else 1
                    if scales is not None:
                        sc = scales[i].to(dt).reshape(ch).contiguous()
                        self._keep.append(sc)
                        items[k].scale_in = sc.data_ptr()
                        r.scale = sc.reshape(kd)
                    else:
                        r.scale = torch.empty(kd, dtype=dt, device=device)
                        items[k].scale_out = r.scale.data_ptr()
                    if want_amax:
                        r.amax = torch.empty(kd, dtype=dt, device=device)
                        items[k].amax_out = r.amax.data_ptr()
                    if want_values:
                        r.values = torch.empty_like(t)
                        items[k].values = r.values.data_ptr()
                    if want_codes:
                        r.codes = torch.empty(t.shape, dtype=torch.uint8, device=device)
                        items[k].codes = r.codes.data_ptr()
                    if want_dequant:
                        r.dequant = torch.empty_like(t)
                        items[k].dequant = r.dequant.data_ptr()
                    self.results[i] = r
                    self._keep.append(t)
                need = _lib.lib.vq_channel_quantize_multi_workspace(items, len(idx))
                ws = torch.empty(max(need, 16), dtype=torch.uint8, device=device)
                handle = C.c_void_p()
                _lib.check(_lib.lib.vq_channel_plan_create(items, len(idx), _DT[dt], self.quant_max, self._tab.ptr(),
                                                           ws.data_ptr(), ws.numel(),
                                                           torch.cuda.current_stream(device).cuda_stream, C.byref(handle)),
                           "quantize_tensors_per_channel")
                self._groups.append((handle, ws))

    def run(self) -> List[ChannelQuant]:
        """One kernel launch per dtype on the current stream (descriptors were uploaded at construction)."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            for handle, _ in self._groups:
                _lib.check(_lib.lib.vq_channel_plan_run(handle, stream), "quantize_tensors_per_channel")
        return self.results

    def close(self) -> None:
        for handle, _ in self._groups:
            _lib.lib.vq_channel_plan_destroy(handle)
        self._groups = []

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass


def quantize_tensors_per_channel(tensors: Sequence[torch.Tensor], qmap, quant_max: float, *, scales=None,
                                 want_values: bool = False, want_codes: bool = False, want_dequant: bool = True,
                                 want_amax: bool = False) -> List[ChannelQuant]:
    """Per-output-channel (axis 0) quantization of many weight tensors in one launch per dtype:
    ``scale = amax(|w|, all axes but 0) / quant_max`` (1 where that amax is 0, NaN or Inf; upstream
    ``FusedAmaxObsFakeQuantize`` after its history has settled, fake_quantize.py:320-333), then
    ``quantize(w, scale, qmap=qmap)`` and ``dequantize(q, scale)`` -- amax, divide, table lookup and
    multiply fused, the channel read from HBM once.  ``scales``: optional list of per-channel
    scales (observer state) to use instead of the amax rule."""
    if not tensors:
        return []
    return ChannelQuantPlan([t.contiguous() for t in tensors], qmap, quant_max, scales=scales, want_values=want_values,
                            want_codes=want_codes, want_dequant=want_dequant, want_amax=want_amax).run()


def dequantize_packed(p: PackedMX, dtype=torch.float32, use_exponent: bool = False) -> torch.Tensor:
    """``levels[code] * scale`` with the packed-storage kernel; ``use_exponent`` takes the E8
    exponents instead of the fp32 scales (power-of-two scales only)."""
    if dtype not in _DT:
        raise NotImplementedError(f"dequantize_packed: dtype {dtype}")
    dev = p.codes.device
    out = torch.empty(p.shape, dtype=dtype, device=dev)
    n = out.numel()
    if n == 0:
        return out
    if use_exponent and p.exp_e8 is None:
        raise ValueError("this PackedMX carries no exponents")
    with torch.cuda.device(dev):
        levels = p.levels_on(dev)
        rc = _lib.lib.vq_dequantize_packed(
            p.codes.data_ptr(), p.code_bits, levels.data_ptr(), levels.numel(),
            None if use_exponent else p.scale.data_ptr(), p.exp_e8.data_ptr() if use_exponent else None,
            n, p.block, out.data_ptr(), _DT[dtype], torch.cuda.current_stream(dev).cuda_stream)
        _lib.check(rc, "dequantize_packed")
    return out


def unpack_codes(p: PackedMX) -> torch.Tensor:
    """uint8 code of every element, shape ``p.shape`` (torch ops; a test and debugging helper)."""
    c = p.codes
    if p.code_bits == 8:
        return c.reshape(p.shape)
    lo, hi = c & 0xF, c >> 4
    return torch.stack([lo, hi], dim=-1).reshape(p.shape)


def dequantize_packed_reference(p: PackedMX, dtype=torch.float32) -> torch.Tensor:
    """``levels[code] * scale`` with torch ops (a test helper, not a product kernel)."""
    codes = unpack_codes(p).long()
    vals = p.levels.to(codes.device)[codes]
    s = torch.repeat_interleave(p.scale, p.block, dim=-1)
    return (vals * s).to(dtype)


# ---------------------------------------------------------------------------------------------
def shard_plan(sizes: Sequence[int], rows: Sequence[int], world_size: int, split_threshold: float = 0.5):
    """Balanced assignment of tensors to ranks.  ``sizes[i]`` elements, ``rows[i]`` rows of tensor
    i.  Tensors larger than ``split_threshold`` x the per-rank share are cut by rows into
    ``world_size`` pieces; the rest are placed greedily, largest first, on the least loaded rank.
    Returns ``plan[rank] = [(tensor index, row_begin, row_end), ...]``; every row of every tensor
    appears exactly once."""
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    total = sum(sizes)
    share = total / world_size
    plan: List[List[Tuple[int, int, int]]] = [[] for _ in range(world_size)]
    load = [0.0] * world_size
    whole = []
    for i, (n, r) in enumerate(zip(sizes, rows)):
        if world_size > 1 and n > split_threshold * share and r >= world_size:
            per_row = n // r
            for k in range(world_size):
                b, e = r * k // world_size, r * (k + 1) // world_size
                if e > b:
                    plan[k].append((i, b, e))
                    load[k] += (e - b) * per_row
        else:
            whole.append(i)
    for i in sorted(whole, key=lambda j: -sizes[j]):
        k = min(range(world_size), key=lambda r_: load[r_])
        plan[k].append((i, 0, rows[i]))
        load[k] += sizes[i]
    for p in plan:
        p.sort()
    return plan


class HostPipeline:
    """Quantize tensors that live in pinned HOST memory and return packed results in pinned host
    memory: host->device copies, the fused kernel and device->host copies run on three streams,
    chunk by chunk, so the transfers overlap the kernel."""

    def __init__(self, device, qmap, block: int, quant_max: float, force_scale_power_of_two: bool = False,
                 code_bits: int = 4, chunk_bytes: int = 1 << 30, chunks_in_flight: int = 3):
        self.device = torch.device(device)
        self.chunks_in_flight = max(1, int(chunks_in_flight))
        self.qmap, self.block, self.quant_max = qmap, block, quant_max
        self.pow2, self.code_bits, self.chunk_bytes = force_scale_power_of_two, code_bits, chunk_bytes
        self.s_in = torch.cuda.Stream(self.device)
        self.s_k = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    @staticmethod
    def chunk_plan(nbytes: Sequence[int], chunk_bytes: int) -> List[List[int]]:
        """Consecutive tensors grouped until a group reaches ``chunk_bytes``; every index once, in order."""
        chunks, cur, size = [], [], 0
        for i, n in enumerate(nbytes):
            cur.append(i)
            size += n
            if size >= chunk_bytes:
                chunks.append(cur)
                cur, size = [], 0
        if cur:
            chunks.append(cur)
        return chunks

    def run(self, host_tensors: Sequence[torch.Tensor], host_out: Optional[List[Tuple[torch.Tensor, torch.Tensor]]] = None):
        """Returns ``[(codes_host, scale_host), ...]``; ``host_out`` supplies preallocated pinned
        destinations.  Synchronises the three streams before returning.  At most
        ``chunks_in_flight`` chunks (inputs + packed results) are resident on the device at a time:
        the host waits for the oldest chunk's copy-out before it queues another one."""
        dev = self.device
        chunks = self.chunk_plan([t.numel() * t.element_size() for t in host_tensors], self.chunk_bytes)
        outs: List = [None] * len(host_tensors)
        self.h2d_bytes = self.d2h_bytes = 0
        in_flight: List = []
        for ch in chunks:
            if len(in_flight) >= self.chunks_in_flight:
                in_flight.pop(0).synchronize()
            with torch.cuda.stream(self.s_in):
                dev_in = [host_tensors[i].to(dev, non_blocking=True) for i in ch]
                ev_in = torch.cuda.Event()
                ev_in.record(self.s_in)
            self.h2d_bytes += sum(host_tensors[i].numel() * host_tensors[i].element_size() for i in ch)
            with torch.cuda.stream(self.s_k):
                self.s_k.wait_event(ev_in)
                packed = quantize_tensors_mx(dev_in, self.qmap, self.block, self.quant_max, self.pow2,
                                             code_bits=self.code_bits)
                ev_k = torch.cuda.Event()
                ev_k.record(self.s_k)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_k)
                for i, p in zip(ch, packed):
                    if host_out is not None:
                        hc, hs = host_out[i]
                    else:
                        hc = torch.empty(p.codes.shape, dtype=torch.uint8, pin_memory=True)
                        hs = torch.empty(p.scale.shape, dtype=torch.float32, pin_memory=True)
                    hc.copy_(p.codes, non_blocking=True)
                    hs.copy_(p.scale, non_blocking=True)
                    outs[i] = (hc, hs)
                    self.d2h_bytes += hc.numel() + hs.numel() * 4
            # tensors allocated on one stream and used on another must outlive that use
            for t in dev_in:
                t.record_stream(self.s_k)
            for p in packed:
                p.codes.record_stream(self.s_out)
                p.scale.record_stream(self.s_out)
            ev_out = torch.cuda.Event()
            ev_out.record(self.s_out)
            in_flight.append(ev_out)
            del dev_in, packed
        self.s_in.synchronize()
        self.s_k.synchronize()
        self.s_out.synchronize()
        return outs
