"""The allocation-free multi-tensor entry point (descriptor scratch built into the library).

Who needs it: code that quantizes from a place where device memory cannot be requested -- a
plug-in called inside another framework's forward pass while that framework's memory pool is
closed, a serving loop whose buffers were all sized at start-up, a worker thread that must never
wait on the allocator's lock.  ``vq_quantize_mx_multi`` wants a caller-provided scratch buffer for
the tensor descriptors; ``vq_quantize_mx_multi_static`` keeps that scratch in a fixed array inside
the library (1024 tensors at most per call) and so asks for nothing.

The test drives it straight through the C ABI with more than 32 tensors per call: only then do the
descriptors travel through the scratch array (fewer ride in the kernel parameters and would leave
the array untouched).  Two calls in a row use different tensor counts and shapes, so the second
one overwrites what the first left behind.  Outputs must be bit-identical to the entry point that
takes a workspace, and to the CPU oracle.  The file name makes pytest collect it last, so a run
that stops at the first failure has already exercised everything else; it also passes when run on
its own in a fresh process (nothing here depends on state left by other tests).
"""
import ctypes as C
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))

pytestmark = pytest.mark.gpu

SHAPES = [(64, 256), (3, 64), (129, 1024), (1, 4096), (17, 128), (256, 512), (33, 192)]


def _setup(dev):
    from voyager_compiler_b200 import _lib, qtables
    tab = qtables.table_handle("nf4", dev).with_codes()
    return _lib, _lib.lib, _lib.lib.vq_quantize_mx_multi_static, tab


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


def _unpack(codes):
    return torch.stack([codes & 0xF, codes >> 4], dim=-1).reshape(-1)


@pytest.mark.parametrize("generic", [False, True])
def test_static_scratch_matches_workspace_entry_point_twice(generic, monkeypatch):
    import voyager_oracle as vo
    from golden_util import golden_table, same_bits

    if generic:                                   # the unspecialised kernel reads the scratch for any tensor count
        monkeypatch.setenv("VOYAGER_B200_GENERIC_MX", "1")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    _lib, lib, fn, tab = _setup(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    tab_v = golden_table("nf4")
    for call, (count, seed, first) in enumerate(((48, 11, 0), (35, 12, 3))):   # different counts, different shapes
        g = torch.Generator().manual_seed(seed)
        host = [(torch.randn(SHAPES[(first + i) % len(SHAPES)], generator=g) * 0.02).to(torch.bfloat16) for i in range(count)]
        host[2].view(-1)[:64] = 0                                              # an all-zero block
        tensors = [h.to(dev) for h in host]
        ref_outs, got_outs = _alloc_outs(tensors), _alloc_outs(tensors)
        ws = torch.empty(lib.vq_quantize_mx_multi_workspace(count) + 256, dtype=torch.uint8, device=dev)
        rc = lib.vq_quantize_mx_multi(_items(_lib, tensors, ref_outs), count, _lib.VQ_BF16, 64, 1.0, 0, None, None,
                                      tab.ptr(), 4, ws.data_ptr(), ws.numel(), stream)
        _lib.check(rc, "vq_quantize_mx_multi")
        rc = fn(_items(_lib, tensors, got_outs), count, _lib.VQ_BF16, 64, 1.0, 0, None, None, tab.ptr(), 4, stream)
        _lib.check(rc, "vq_quantize_mx_multi_static")
        torch.cuda.synchronize()
        for k, ((rc_, rs), (gc, gs)) in enumerate(zip(ref_outs, got_outs)):
            assert torch.equal(gc, rc_) and torch.equal(gs.view(torch.int32), rs.view(torch.int32)), (call, k)
            assert int(gc.max()) > 0                                           # the kernel really wrote codes
        for k in (0, 2, count - 1):                                            # and both agree with the CPU oracle
            s_ref = vo.mx_scale(host[k], (-1,), 64, 1.0, False)
            v_ref = vo.quantize(host[k], s_ref, None, (-1,), 64, tab_v).float().reshape(-1)
            assert same_bits(got_outs[k][1].reshape(s_ref.shape), s_ref.float())[0]
            assert torch.equal(tab.levels[_unpack(got_outs[k][0]).cpu().long()], v_ref)


def test_static_scratch_rejects_too_many_tensors():
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    _lib, lib, fn, tab = _setup(dev)
    limit = lib.vq_quantize_mx_multi_static_max_items()
    assert limit == 1024
    items = (_lib.VqMxItem * (limit + 1))()
    rc = fn(items, limit + 1, _lib.VQ_BF16, 64, 1.0, 0, None, None, tab.ptr(), 4, None)
    assert rc == -1 and b"1024" in lib.vq_last_error()
