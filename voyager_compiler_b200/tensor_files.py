"""Tensor files next to upstream's dump (src/voyager_compiler/codegen/transform/bufferize/emit.py:143-175:
one raw float32 ``<name>.bin`` per tensor, written by a thread pool; ``flush_tensor_files`` waits for them).

``save_tensor`` writes that same float32 file.  ``save_packed`` writes a quantized weight in the form the
kernels of this package produce it (:class:`~voyager_compiler_b200.model_quant.PackedMX`): ``<name>.codes.bin``
(uint8, ``code_bits`` per element, low nibble first), ``<name>.scales.bin`` (float32, one per block),
``<name>.levels.bin`` (float32 value of every code) and ``<name>.json`` (shape, block, code_bits), i.e.
4.5 bits per element for NF4 with blocks of 64 instead of 32.  ``load_packed`` reads it back and
``model_quant.dequantize_packed`` turns it into the float tensor upstream's file would hold.  Device-to-host
copies run on the caller's stream into pinned buffers; the file writes are handed to a thread pool.
"""
from __future__ import annotations

import json
import os
from concurrent.futures import ThreadPoolExecutor
from typing import List

import numpy as np
import torch

_executor = ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 4))
_pending: List = []


def _host_copy(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().contiguous()
    if t.device.type != "cuda":
        return t
    host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
    host.copy_(t, non_blocking=True)
    return host


def _write(arrays, event):
    if event is not None:
        event.synchronize()                      # the copies above were queued on the caller's stream
    for filename, host in arrays:
        if isinstance(host, (bytes, str)):
            with open(filename, "w" if isinstance(host, str) else "wb") as f:
                f.write(host)
        else:
            host.numpy().tofile(filename)


def _submit(arrays, device):
    event = None
    if device is not None and device.type == "cuda":
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(device))
    _pending.append(_executor.submit(_write, arrays, event))


def save_tensor(tensor: torch.Tensor, filename: str) -> None:
    """Raw float32 file, as upstream's ``_save_tensor`` writes it (emit.py:158-164); asynchronous."""
    t = tensor.detach()
    t = t.to(torch.float32) if t.dtype != torch.float32 else t
    _submit([(filename, _host_copy(t))], tensor.device)


def save_packed(packed, basename: str) -> None:
    """Packed codes + block scales + levels + a JSON header under ``basename``.*; asynchronous."""
    meta = {"shape": list(packed.shape), "block": int(packed.block), "code_bits": int(packed.code_bits),
            "levels": int(packed.levels.numel()), "format": "voyager_b200.packed_mx.v1"}
    arrays = [(basename + ".codes.bin", _host_copy(packed.codes)),
              (basename + ".scales.bin", _host_copy(packed.scale.to(torch.float32))),
              (basename + ".levels.bin", _host_copy(packed.levels.to(torch.float32))),
              (basename + ".json", json.dumps(meta))]
    _submit(arrays, packed.codes.device)


def flush_tensor_files() -> None:
    """Wait until every queued file is on disk (emit.py:167-175); re-raises a failed write."""
    while _pending:
        _pending.pop().result()


def load_packed(basename: str, device="cpu"):
    """The :class:`PackedMX` that ``save_packed`` wrote (scales as float32)."""
    from .model_quant import PackedMX
    with open(basename + ".json") as f:
        meta = json.load(f)
    if meta.get("format") != "voyager_b200.packed_mx.v1":
        raise ValueError(f"{basename}.json: not a packed tensor header")
    shape = tuple(meta["shape"])
    n = int(np.prod(shape)) if shape else 1
    codes = torch.from_numpy(np.fromfile(basename + ".codes.bin", dtype=np.uint8))
    want = n * meta["code_bits"] // 8
    if codes.numel() != want:
        raise ValueError(f"{basename}.codes.bin: {codes.numel()} bytes, expected {want}")
    scale = torch.from_numpy(np.fromfile(basename + ".scales.bin", dtype=np.float32))
    levels = torch.from_numpy(np.fromfile(basename + ".levels.bin", dtype=np.float32))
    last = shape[-1] if shape else 1
    nblk = -(-last // meta["block"])
    codes = codes.reshape(shape[:-1] + (last * meta["code_bits"] // 8,)).to(device)
    scale = scale.reshape(shape[:-1] + (nblk,)).to(device)
    return PackedMX(codes=codes, scale=scale, shape=shape, block=meta["block"], code_bits=meta["code_bits"], levels=levels)
