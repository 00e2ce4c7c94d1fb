"""Device-resident descriptions of lookup tables and of the shared-exponent rule.

``table_handle(qmap, device)`` turns the 65 536-entry ``qmap`` tensor an op receives into the
``vq_table`` the kernels take: the table is copied to the host once, analysed
(:func:`voyager_compiler_b200.tables.analyse_table`) and cached, keyed by the tensor's storage
pointer and version counter.

``exp_tables(dtype, quant_max, device)`` derives, once per (dtype, floor(log2 quant_max)), the
tables with which the kernels reproduce ``floor(log2(amax)) - floor(log2(quant_max))`` and
``2 ** e`` exactly as torch's CPU arithmetic evaluates them in that dtype
(src/voyager_compiler/quantization/mx_utils.py:42-47, ops/quantized.py:471-488): the exponent
field of amax is exact, and the only places where the rounded ``log2`` floors one higher sit just
below each power of two, so one threshold per binary exponent describes the CPU result fully.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import threading
from collections import OrderedDict
from typing import Optional

import numpy as np
import torch

from . import _lib, tables

__all__ = ["TableHandle", "table_handle", "exp_tables", "ExpTables", "set_table_policy", "clear_caches"]

_lock = threading.Lock()
_table_cache: "OrderedDict[tuple, TableHandle]" = OrderedDict()
_exp_cache: dict = {}
_CACHE_MAX = 128

# Tables with at most this many runs use the run-start binary search instead of the staged LUT.
_policy = {"runs_max": int(os.environ.get("VOYAGER_B200_RUNS_MAX", "0")),
           "allow_int": os.environ.get("VOYAGER_B200_NO_INT", "0") != "1"}


def set_table_policy(runs_max: Optional[int] = None, allow_int: Optional[bool] = None) -> None:
    """Choose how tables are evaluated: tables with <= ``runs_max`` runs use the binary search
    (0 disables it); ``allow_int`` enables the arithmetic path for integer round-and-clamp tables."""
    with _lock:
        if runs_max is not None:
            _policy["runs_max"] = int(runs_max)
        if allow_int is not None:
            _policy["allow_int"] = bool(allow_int)
        _table_cache.clear()


def clear_caches() -> None:
    with _lock:
        _table_cache.clear()
        _exp_cache.clear()


def _dev_u16(arr: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(arr, dtype=np.uint16).view(np.int16).copy()).to(device)


class TableHandle:
    """Owns the device buffers behind one ``vq_table``."""

    def __init__(self, lut16_host: np.ndarray, device: torch.device, source: Optional[torch.Tensor] = None,
                 allow_runs: bool = True):
        self.source = source            # keeps the storage alive so the cache key cannot be recycled
        self.device = device
        self.analysis = tables.analyse_table(lut16_host)
        an = self.analysis
        self.lut16 = _dev_u16(an.lut16, device)
        self._lut8 = None
        self._levels = None
        self._run = None
        self.c = _lib.VqTable()
        self.c.lut16 = self.lut16.data_ptr()
        self.c.nan_uniform = 1 if an.nan_consistent else 0
        self.c.flat_tiny = 1 if an.flat_tiny else 0
        if an.is_int and _policy["allow_int"]:
            self.c.kind = _lib.TABLE_INT
            self.c.lo, self.c.hi = an.lo, an.hi
        elif allow_runs and an.n_runs and an.n_runs <= _policy["runs_max"] and an.nan_consistent:
            self._use_runs()
        else:
            self.c.kind = _lib.TABLE_LUT16

    def _use_runs(self):
        an = self.analysis
        keys = an.run_keys if an.run_keys.size else np.zeros(1, dtype=np.uint16)
        self._run = (_dev_u16(keys, self.device), _dev_u16(an.run_vals, self.device))
        self.c.kind = _lib.TABLE_RUNS
        self.c.n_runs = an.n_runs
        self.c.run_keys = self._run[0].data_ptr()
        self.c.run_vals = self._run[1].data_ptr()
        self.c.nan_val, self.c.pinf_val, self.c.ninf_val = an.nan_val, an.pinf_val, an.ninf_val

    @property
    def kind(self) -> int:
        return self.c.kind

    def with_codes(self) -> "TableHandle":
        """Make packed codes available (``lut8`` / ``run_codes``); see tables.code_table."""
        if self._lut8 is None:
            an = self.analysis
            codes, levels = tables.code_table(an.lut16)
            self._levels = torch.from_numpy(levels.copy())
            self._lut8 = torch.from_numpy(codes.copy()).to(self.device)
            if self.c.kind != _lib.TABLE_INT:
                self.c.lut8 = self._lut8.data_ptr()
                lv2 = tables.levels_by_code_and_sign(an.lut16, codes)
                if lv2 is not None:
                    self._levels2 = torch.from_numpy(lv2).to(self.device)
                    self.c.levels2 = self._levels2.data_ptr()
            if self.c.kind == _lib.TABLE_RUNS:
                rc = codes[an.run_first]
                self._run_codes = torch.from_numpy(np.ascontiguousarray(rc)).to(self.device)
                self.c.run_codes = self._run_codes.data_ptr()
                self.c.nan_code, self.c.pinf_code, self.c.ninf_code = int(codes[0xFFFF]), int(codes[0x7F80]), int(codes[0xFF80])
        return self

    @property
    def levels(self) -> torch.Tensor:
        """fp32 value of every packed code (host tensor)."""
        self.with_codes()
        return self._levels

    def ptr(self):
        return C.byref(self.c)


def _to_bits_host(qmap: torch.Tensor) -> np.ndarray:
    if qmap.numel() != 1 << 16:
        raise ValueError(f"a lookup table must have 65536 entries, got {qmap.numel()}")
    # entries are stored into a bf16 result tensor by the reference, i.e. cast to bf16
    t = qmap.detach().reshape(-1).to(torch.bfloat16).cpu().contiguous()
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def table_handle(qmap, device, allow_runs: bool = True) -> TableHandle:
    """Cached ``TableHandle`` for a table tensor (any device, bf16 / float / integer entries),
    a numpy uint16[65536] array of bf16 patterns, or an upstream dtype string such as ``"int8"``.
    ``allow_runs=False`` keeps the table out of the binary-search form (scale tables are read once
    per block from global memory, where the search has nothing to gain)."""
    device = torch.device(device)
    if isinstance(qmap, str):
        key = ("name", qmap, str(device), allow_runs)
    elif isinstance(qmap, np.ndarray):
        key = ("np", qmap.tobytes(), str(device), allow_runs)
    else:
        key = ("t", qmap.data_ptr(), qmap._version, qmap.dtype, str(qmap.device), tuple(qmap.shape), str(device),
               allow_runs)
    with _lock:
        h = _table_cache.get(key)
        if h is not None:
            _table_cache.move_to_end(key)
            return h
    if isinstance(qmap, str):
        h = TableHandle(tables.build_table(qmap), device, allow_runs=allow_runs)
    elif isinstance(qmap, np.ndarray):
        h = TableHandle(qmap, device, allow_runs=allow_runs)
    else:
        h = TableHandle(_to_bits_host(qmap), device, source=qmap, allow_runs=allow_runs)
    with _lock:
        _table_cache[key] = h
        while len(_table_cache) > _CACHE_MAX:
            _table_cache.popitem(last=False)
    return h


# ---------------------------------------------------------------------------------------------
class ExpTables:
    def __init__(self, bump_at: torch.Tensor, scale_of: torch.Tensor):
        self.bump_at, self.scale_of = bump_at, scale_of
        self.c = _lib.VqExpTables()
        self.c.bump_at = bump_at.data_ptr()
        self.c.scale_of = scale_of.data_ptr()

    def ptr(self):
        return C.byref(self.c)


def _bits_to_dtype(bits: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """int64 fp32 bit patterns -> CPU tensor of ``dtype`` (bf16 patterns have zero low halves)."""
    f = bits.to(torch.int32).view(torch.float32)
    return f if dtype == torch.float32 else f.to(torch.bfloat16)


def derive_exp_tables_host(dtype: torch.dtype, floor_log2_qmax: int):
    """(bump_at uint32[277], scale_of fp32[278]) computed with torch CPU arithmetic in ``dtype``."""
    step = 1 if dtype == torch.float32 else 1 << 16
    window = 128
    bump = np.zeros(277, dtype=np.uint32)
    cand, owner, nxt_of = [], [], []
    for i in range(277):
        e = i - 149
        nxt = 0x7F800000 if e == 127 else ((e + 1 + 127) << 23 if e + 1 >= -126 else 1 << (e + 1 + 149))
        first = (e + 127) << 23 if e >= -126 else 1 << (e + 149)
        lo = max(first, nxt - window * step)
        lo = (lo + step - 1) // step * step
        pats = np.arange(lo, nxt, step, dtype=np.int64)
        cand.append(pats)
        owner.append(np.full(pats.shape, i))
        bump[i] = nxt
    cand_all = np.concatenate(cand)
    owner_all = np.concatenate(owner)
    v = _bits_to_dtype(torch.from_numpy(cand_all), dtype)
    # one large tensor, so the vectorised log2 the ops use on real data is the one sampled here
    fl = torch.floor(torch.log2(v)).float().numpy()
    bumped = fl > (owner_all - 149)
    for i in range(277):
        sel = owner_all == i
        if not sel.any():
            continue
        b = bumped[sel]
        if b.any():
            first_true = int(np.argmax(b))
            if not b[first_true:].all():
                raise RuntimeError("log2 of this torch build is not monotone near a power of two")
            if first_true == 0 and cand_all[sel][0] != ((i - 149 + 127) << 23 if i - 149 >= -126 else 1 << i):
                raise RuntimeError("search window below a power of two is too small")
            bump[i] = np.uint32(cand_all[sel][first_true])
    e_all = torch.arange(-149, 129, dtype=torch.float32).to(dtype)
    s = 2 ** (e_all - floor_log2_qmax)
    s = torch.where(s > 0.0, s, 1.0)
    return bump, s.float().numpy().copy()


def exp_tables(dtype: torch.dtype, quant_max: float, device) -> ExpTables:
    device = torch.device(device)
    fl = math.floor(math.log2(quant_max))
    key = (dtype, fl, str(device))
    with _lock:
        t = _exp_cache.get(key)
    if t is None:
        bump, scale = derive_exp_tables_host(dtype, fl)
        t = ExpTables(torch.from_numpy(bump.view(np.int32).copy()).to(device), torch.from_numpy(scale).to(device))
        with _lock:
            _exp_cache[key] = t
    return t


_pow2_stay_cache: dict = {}


def derive_pow2_stay_host() -> np.ndarray:
    """For every biased fp32 exponent E, the number of consecutive values ``2^(E-127) * (1 + m 2^-23)``, m = 0, 1, ...,
    for which ``ceil(log2(x))`` evaluated in the CPU's fp32 arithmetic is still ``E - 127`` (the logarithm of a value
    just above a power of two rounds to the integer).  This is what ``2 ** ceil(log2(scale))`` of the observer
    (quantization/fake_quantize.py:339-340) depends on; uint8[256], entries 0 and 255 unused."""
    span = 256
    e = np.arange(1, 255, dtype=np.uint32)
    bits = (e[:, None] << 23) | np.arange(span, dtype=np.uint32)[None, :]
    x = torch.from_numpy(bits.view(np.float32).copy())
    same = torch.ceil(torch.log2(x)) == torch.from_numpy((e.astype(np.int64) - 127).astype(np.float32))[:, None]
    # length of the leading run of True in every row
    stay = torch.cumprod(same.to(torch.int64), dim=1).sum(dim=1)
    if int(stay.max()) >= span or int(stay.min()) < 1:
        raise RuntimeError("unexpected log2 behaviour on this host")
    out = np.zeros(256, dtype=np.uint8)
    out[1:255] = stay.numpy().astype(np.uint8)
    return out


def pow2_stay_table(device) -> torch.Tensor:
    device = torch.device(device)
    key = str(device)
    with _lock:
        t = _pow2_stay_cache.get(key)
    if t is None:
        t = torch.from_numpy(derive_pow2_stay_host()).to(device)
        with _lock:
            _pow2_stay_cache[key] = t
    return t
