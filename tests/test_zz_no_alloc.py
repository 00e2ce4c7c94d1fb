"""The allocation-free multi-tensor entry point (built-in descriptor workspace).

For callers that cannot allocate device memory at quantization time (plug-ins inside a closed
memory pool, serving loops with pre-sized buffers).  Called straight through the C ABI with ctypes;
its outputs must be bit-identical to those of the workspace-taking entry point, on two calls in a
row (the second call reuses the array the first one filled).  Collected last so that a run stopping
at the first failure has already exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(dev):
    from voyager_compiler_b200 import _lib, qtables
    lib = _lib.lib
    fn = lib.vq_quantize_mx_multi_static
    fn.argtypes = [C.POINTER(_lib.VqMxItem), C.c_int, C.c_int, C.c_int64, C.c_double, C.c_int,
                   C.POINTER(_lib.VqExpTables), C.POINTER(_lib.VqTable), C.POINTER(_lib.VqTable), C.c_int, C.c_void_p]
    fn.restype = C.c_int
    lib.vq_quantize_mx_multi_static_max_items.restype = C.c_int
    tab = qtables.table_handle("nf4", dev).with_codes()
    return _lib, lib, fn, tab


def _items(_lib, tensors, outs):
    items = (_lib.VqMxItem * len(tensors))()
    for k, (t, (codes, scale)) in enumerate(zip(tensors, outs)):
        items[k].input = t.data_ptr()
        items[k].n = t.numel()
        items[k].codes = codes.data_ptr()
        items[k].scale_f32 = scale.data_ptr()
    return items


def _alloc_outs(tensors):
    return [(torch.zeros(t.numel() // 2, dtype=torch.uint8, device=t.device),
             torch.zeros(t.numel() // 64, dtype=torch.float32, device=t.device)) for t in tensors]


def test_static_workspace_matches_workspace_entry_point_twice():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    _lib, lib, fn, tab = _setup(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for call, seed in enumerate((11, 12)):                      # two calls in a row, different data
        g = torch.Generator(device=dev); g.manual_seed(seed)
        shapes = [(64, 256), (3, 64), (129, 1024), (1, 4096)] if call == 0 else [(17, 128), (256, 512)]
        tensors = [(torch.randn(s, generator=g, device=dev) * 0.02).to(torch.bfloat16) for s in shapes]
        ref_outs, got_outs = _alloc_outs(tensors), _alloc_outs(tensors)
        ws = torch.empty(lib.vq_quantize_mx_multi_workspace(len(tensors)) + 256, dtype=torch.uint8, device=dev)
        rc = lib.vq_quantize_mx_multi(_items(_lib, tensors, ref_outs), len(tensors), _lib.VQ_BF16, 64, 1.0, 0, None, None,
                                      tab.ptr(), 4, ws.data_ptr(), ws.numel(), stream)
        _lib.check(rc, "vq_quantize_mx_multi")
        rc = fn(_items(_lib, tensors, got_outs), len(tensors), _lib.VQ_BF16, 64, 1.0, 0, None, None, tab.ptr(), 4, stream)
        _lib.check(rc, "vq_quantize_mx_multi_static")
        torch.cuda.synchronize()
        for (rc_, rs), (gc, gs) in zip(ref_outs, got_outs):
            assert torch.equal(gc, rc_) and torch.equal(gs.view(torch.int32), rs.view(torch.int32))
            assert int(gc.max()) > 0                              # the kernel really wrote codes


def test_static_workspace_rejects_too_many_tensors():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    _lib, lib, fn, tab = _setup(dev)
    limit = lib.vq_quantize_mx_multi_static_max_items()
    assert limit == 1024
    items = (_lib.VqMxItem * (limit + 1))()
    rc = fn(items, limit + 1, _lib.VQ_BF16, 64, 1.0, 0, None, None, tab.ptr(), 4, None)
    assert rc == -1 and b"1024" in lib.vq_last_error()
