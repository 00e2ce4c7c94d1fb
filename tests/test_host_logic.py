"""Host-side logic that needs no GPU: ABI surface, scale layouts, exponent tables."""
import math
import os
import re
import sys

import numpy as np
import pytest
import torch

import voyager_compiler_b200 as vb
from voyager_compiler_b200 import _lib, ops, qtables
from golden_util import cases, materialize

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import voyager_oracle as vo  # noqa: E402


def test_library_exports_every_declared_symbol():
    text = open(os.path.join(ROOT, "include", "voyager_b200.h")).read()
    names = re.findall(r"VQ_API\s+[\w\s\*]+?\b(vq_\w+)\s*\(", text)
    assert len(names) >= 8
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in the header but not exported"
    assert _lib.lib.vq_version() == _lib.ABI_VERSION


def test_fastdiv_selfcheck():
    rng = np.random.default_rng(0)
    for d in [1, 2, 3, 7, 32, 64, 4096, 11008, 2 ** 31 - 1] + rng.integers(1, 2 ** 31, 200).tolist():
        for n in [0, 1, d - 1, d, d + 1, 2 ** 31 - 1] + rng.integers(0, 2 ** 31, 50).tolist():
            if 0 <= n < 2 ** 31:
                assert _lib.lib.vq_selftest_fastdiv(int(d), int(n)) == 0


def test_cpu_tensors_are_rejected_loudly():
    x = torch.randn(4, 32)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.quantized_ops.quantize(x, torch.ones(1), None, None, None, torch.zeros(65536, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        vb.quantize(x, torch.ones(1), qmap=torch.zeros(65536, dtype=torch.bfloat16))


def test_quantize_requires_qmap():
    with pytest.raises(AssertionError):
        vb.quantize(torch.randn(2), torch.ones(1))


def test_meta_shapes():
    m = torch.empty(6, 70, device="meta")
    q = torch.empty(65536, device="meta", dtype=torch.bfloat16)
    if vb.REGISTERED_AS != "def":
        pytest.skip("upstream composite provides the meta kernels")
    s, c = torch.ops.quantized_ops.quantize_mx(m, q, (-1,), 32, 127.0, True)
    assert s.shape == (6, 3) and c.shape == (6, 70)
    assert torch.ops.quantized_ops.calculate_mx_qparam(m, (0,), 32, 127.0).shape == (1, 70)
    y = torch.ops.quantized_ops.linear_mx(torch.empty(5, 64, device="meta"), torch.empty(48, 64, device="meta"))
    assert y.shape == (5, 48)


# ------------------------------------------------------------------------------ scale layouts
def _layout_indices(lay, shape):
    """Scale index of every element according to a vq_scale_layout (numpy model of the kernel)."""
    n = math.prod(shape)
    i = np.arange(n, dtype=np.int64)
    if lay.mode == _lib.SCALE_SCALAR:
        return np.zeros(n, dtype=np.int64)
    if lay.mode == _lib.SCALE_ROWBLOCK:
        K = lay.K
        bs = min(lay.block, K)
        nb = -(-K // bs)
        return (i // K) * nb + (i % K) // bs
    idx = np.zeros(n, dtype=np.int64)
    rem = i.copy()
    for d in range(lay.ndim - 1, -1, -1):
        c = rem % lay.size[d]
        rem //= lay.size[d]
        idx += (c // lay.div[d]) * lay.stride[d]
    return idx


LAYOUT_CASES = [
    ((16, 96), (16, 3), 32), ((3, 40), (3, 2), 32), ((5, 8), (5, 1), 32), ((8, 4, 3, 3), (8, 1, 1, 1), None),
    ((12, 20), (12, 1), None), ((12, 20), (1, 20), None), ((12, 20), (1,), None), ((12, 20), (), None),
    ((12, 20), (3, 20), 4), ((12, 20), (3, 5), 4), ((2, 70, 12), (2, 3, 12), 32), ((2, 40, 3, 5), (2, 3, 3, 5), 16),
    ((6, 50), (6, 4), 16), ((1, 1, 64), (1, 1, 2), 32), ((4, 1, 64), (4, 1, 2), 32), ((7,), (1,), 8), ((64,), (2,), 32),
    ((2, 3, 4), (3, 1), None),
]


@pytest.mark.parametrize("shape,sshape,bs", LAYOUT_CASES)
def test_layout_matches_expand(shape, sshape, bs):
    n_s = math.prod(sshape)
    scale = torch.arange(n_s, dtype=torch.float32).reshape(sshape)
    want = vo.spread_scale(scale, shape, bs) if bs is not None else scale.expand(shape)
    lay = ops._layout("t", shape, scale, bs)
    got = _layout_indices(lay, shape)
    assert (got == want.reshape(-1).numpy().astype(np.int64)).all(), (lay.mode, got[:20])


def test_layout_rejects_uncovered_dims():
    with pytest.raises(RuntimeError):
        ops._layout("t", (4, 64), torch.ones(4, 1), 32)


# ------------------------------------------------------------------------------ exponent tables
def _model_pow2_scale(amax_f32: np.ndarray, bump: np.ndarray, scale_of: np.ndarray) -> np.ndarray:
    """numpy model of the kernel's power-of-two scale rule (block_scale in csrc/vq_common.cuh)."""
    bits = amax_f32.view(np.uint32).astype(np.int64)
    out = np.empty(bits.shape, dtype=np.float32)
    for k, b in enumerate(bits):
        if b > 0x7F800000:
            out[k] = 1.0
        elif b == 0x7F800000:
            out[k] = np.inf
        else:
            if b == 0:
                b = 0x00800000
            e = (b >> 23) - 127 if b >= 0x00800000 else (int(b).bit_length() - 1) - 149
            i = e + 149
            i += 1 if b >= int(bump[i]) else 0
            out[k] = scale_of[i]
    return out


@pytest.mark.parametrize("case_name", ["mxs_sweep_bf16", "mxs_sweep_bf16_q1", "mxs_sweep_f32", "mxs_sweep_f32_q448",
                                       "mxs_f32_edges_pow2", "mxs_bf16_edges_pow2"])
def test_exp_tables_reproduce_upstream_scales(case_name):
    case = next(c for c in cases("calculate_mx_qparam") if c["name"] == case_name)
    t, p, expected = materialize(case)
    x = t["input"]
    bump, scale_of = qtables.derive_exp_tables_host(x.dtype, math.floor(math.log2(p["quant_max"])))
    bs = p["block_size"]
    xa = x.abs().float()
    # torch.max semantics: NaN wins
    blocks = xa.reshape(xa.shape[0], -1, min(bs, xa.shape[1]))
    amax = torch.where(torch.isnan(blocks).any(-1), torch.tensor(float("nan")), blocks.amax(-1))
    got = _model_pow2_scale(amax.reshape(-1).numpy().copy(), bump, scale_of)
    want = expected[0].float().reshape(-1).numpy()
    assert (got.view(np.uint32) == want.view(np.uint32)).all()


def test_exp_tables_shape_and_bounds():
    for dt in (torch.float32, torch.bfloat16):
        bump, scale_of = qtables.derive_exp_tables_host(dt, 6)
        assert bump.shape == (277,) and scale_of.shape == (278,)
        assert scale_of[149 + 6] == 1.0            # amax in [64,128) -> 2^(6-6)
        assert (scale_of > 0).all()
    # all-zero block: amax is replaced by 2^-126 -> 2^-132 (a subnormal) in fp32, and in bf16 too
    b32, s32 = qtables.derive_exp_tables_host(torch.float32, 6)
    assert s32[149 - 126] == np.float32(2.0 ** -132)


def test_reciprocal_quotient_rounds_like_division_for_8bit_significands():
    """The bf16 kernels compute x / scale as x * rcp(scale) and round to bf16.  For operands with
    8-bit significands this equals rounding the IEEE fp32 quotient, for every reciprocal within one
    ulp of 1 / scale: checked here over all significand pairs (the argument is exponent-free)."""
    import numpy as np
    mx = np.arange(1, 256, dtype=np.float32)[:, None]
    ms = np.arange(128, 256, dtype=np.float32)[None, :]
    exact = torch.from_numpy((mx / ms).astype(np.float32)).to(torch.bfloat16)
    r = (np.float32(1.0) / ms).astype(np.float32)
    for cand in (r, np.nextafter(r, np.float32(0)), np.nextafter(r, np.float32(2))):
        q = torch.from_numpy((mx * cand).astype(np.float32)).to(torch.bfloat16)
        assert torch.equal(q.view(torch.int16), exact.view(torch.int16))
    # distance of every quotient from the nearest bf16 rounding boundary, relative: > 2^-17
    q64 = (mx.astype(np.float64) / ms.astype(np.float64))
    f = q64 / 2.0 ** np.floor(np.log2(q64))              # in [1, 2)
    t = f * 256.0                                        # boundaries are the odd integers
    odd = 2.0 * np.floor(t / 2.0) + 1.0
    assert (np.abs(t - odd) / t).min() > 2.0 ** -17


def test_flat_tiny_flag_of_tables():
    from voyager_compiler_b200 import tables
    assert tables.analyse_table(tables.build_table("nf4")).flat_tiny
    assert tables.analyse_table(tables.build_table("int8")).flat_tiny
    assert tables.analyse_table(tables.build_table("posit8_1")).flat_tiny
    # -0 maps to +0 but a tiny negative to -0: the zone is not constant, the kernels keep the scan
    assert not tables.analyse_table(tables.build_table("fp8_e4m3")).flat_tiny
    ident = np.arange(1 << 16, dtype=np.uint16)
    assert not tables.analyse_table(ident).flat_tiny


def test_observer_entry_points_reject_bad_arguments_before_any_launch():
    """Argument checks of the observer kernels' C ABI: an invalid dtype or size is refused with a message and a
    negative status, before the device is touched (so this runs without a GPU)."""
    lib = _lib.lib
    lib.vq_last_error.restype = __import__("ctypes").c_char_p
    assert lib.vq_exp_histogram(None, 7, 16, None, None, None, 0, None) < 0
    assert b"dtype" in lib.vq_last_error()
    assert lib.vq_exp_histogram(None, _lib.VQ_F32, -1, None, None, None, 0, None) < 0
    assert lib.vq_outlier_split(None, 7, 16, None, None, None, None) < 0
    assert lib.vq_outlier_split(None, _lib.VQ_BF16, 16, None, None, None, None) < 0           # null threshold / counter
    assert lib.vq_outlier_merge(None, None, 9, 4, None, None, None) < 0
    assert lib.vq_outlier_merge(None, None, _lib.VQ_F32, -4, None, None, None) < 0
    assert lib.vq_group_affine_fake_quantize(None, 7, 2, 64, 32, 0.0, 15.0, None, None, None, None, None) < 0
    assert lib.vq_group_affine_fake_quantize(None, _lib.VQ_F32, 2, 64, 0, 0.0, 15.0, None, None, None, None, None) < 0
    assert lib.vq_group_affine_fake_quantize(None, _lib.VQ_F32, 2, 64, 32, 15.0, 15.0, None, None, None, None, None) < 0
    assert b"quant_max" in lib.vq_last_error()
    # empty inputs are a no-op
    assert lib.vq_group_affine_fake_quantize(None, _lib.VQ_F32, 0, 64, 32, 0.0, 15.0, None, None, None, None, None) == 0
    assert lib.vq_outlier_merge(None, None, _lib.VQ_F32, 0, torch.zeros(1).data_ptr(), None, None) == 0


def test_module_accepts_every_upstream_scheme_and_option():
    """Constructor parity with fake_quantize.py:216-307: no scheme or option is refused any more (construction needs no GPU)."""
    from voyager_compiler_b200 import fake_quantize as fq
    m = fq.FusedAmaxObsFakeQuantize("int8", qscheme="group_wise_affine", quant_min=0.0, quant_max=255.0, ch_axis=-1, block_size=32)
    assert isinstance(m.calculate_qparams(), tuple) and len(m.calculate_qparams()) == 2
    m = fq.FusedAmaxObsFakeQuantize("int8", qscheme="per_tensor_symmetric", quant_max=127.0, amax_history_len=4,
                                    record_histogram=True, outlier_pct=0.01, outlier_ema_decay=0.5)
    assert m.histogram.shape == (254,) and m.outlier_threshold.numel() == 0 and m.outlier_ema_decay == 0.5
    assert m.max_outlier_pct == 0.0
    m = fq.FusedAmaxObsFakeQuantize("int8", qscheme="microscaling", quant_max=127.0, ch_axis=-1, block_size=32, outlier_threshold=6.0)
    assert m.outlier_threshold == 6.0
    with pytest.raises(AssertionError):
        fq.FusedAmaxObsFakeQuantize("int8", qscheme="per_tensor_symmetric", quant_max=127.0, outlier_pct=0.1, outlier_threshold=1.0)


def test_nvtx_wrapper_is_only_installed_on_request(monkeypatch):
    from voyager_compiler_b200 import ops

    def op(x, y=1):
        """doc"""
        return x + y
    monkeypatch.delenv("VOYAGER_B200_NVTX", raising=False)
    assert ops._traced("vmap", op) is op                      # default: the function itself, no wrapper
    monkeypatch.setenv("VOYAGER_B200_NVTX", "1")
    wrapped = ops._traced("vmap", op)
    assert wrapped is not op and wrapped.__doc__ == "doc" and wrapped.__wrapped__ is op
