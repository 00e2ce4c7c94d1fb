"""GPU parity: every upstream fixture replayed through torch.ops.quantized_ops on CUDA tensors.

Codes, scales and element-wise results must be bit-identical to the upstream CPU outputs (NaN
matching NaN); the GEMMs must be within 1e-2 relative Frobenius error."""
import os
import sys

import pytest
import torch

import voyager_compiler_b200 as vb
from golden_util import case_ids, cases, run_case, same_bits

pytestmark = pytest.mark.gpu

CONTRACTIONS = ("linear_mx", "matmul_mx", "conv2d_mx")
ELEMENTWISE = [c for c in cases() if c["op"] not in CONTRACTIONS]
GEMMS = [c for c in cases() if c["op"] in CONTRACTIONS]
POLICIES = {
    "default": dict(runs_max=0, allow_int=True),
    "lut": dict(runs_max=0, allow_int=False),
    "runs": dict(runs_max=512, allow_int=False),
}


@pytest.fixture(params=list(POLICIES))
def policy(request):
    vb.set_table_policy(**POLICIES[request.param])
    yield request.param
    vb.set_table_policy(**POLICIES["default"])


@pytest.mark.parametrize("case", ELEMENTWISE, ids=[c["name"] for c in ELEMENTWISE])
def test_fixture_bit_exact_on_cuda(case, policy):
    before = vb._lib.launch_count()
    outs, expected = run_case(case, torch.ops.quantized_ops, device="cuda")
    torch.cuda.synchronize()
    assert vb._lib.launch_count() > before, "no kernel of this library was launched"
    assert len(outs) == len(expected)
    for o, e in zip(outs, expected):
        assert o.is_cuda and o.is_contiguous()
        ok, msg = same_bits(o, e)
        assert ok, f"{case['name']} [{policy}]: {msg}"


@pytest.mark.parametrize("case", [c for c in ELEMENTWISE if c["op"] in ("vmap", "quantize", "dequantize")],
                         ids=[c["name"] for c in ELEMENTWISE if c["op"] in ("vmap", "quantize", "dequantize")])
def test_generic_elementwise_kernel_stays_bit_exact(case):
    """The specialised element-wise kernel normally takes the aligned cases; the generic one must agree."""
    os.environ["VOYAGER_B200_GENERIC_EW"] = "1"
    try:
        outs, expected = run_case(case, torch.ops.quantized_ops, device="cuda")
        for o, e in zip(outs, expected):
            ok, msg = same_bits(o, e)
            assert ok, f"{case['name']}: {msg}"
    finally:
        del os.environ["VOYAGER_B200_GENERIC_EW"]


MX_CASES = [c for c in ELEMENTWISE if c["op"] == "quantize_mx"]


@pytest.mark.parametrize("case", MX_CASES, ids=[c["name"] for c in MX_CASES])
def test_generic_mx_kernels_stay_bit_exact(case):
    """The specialised fused kernel normally takes these; the generic kernels must agree too."""
    os.environ["VOYAGER_B200_GENERIC_MX"] = "1"
    try:
        outs, expected = run_case(case, torch.ops.quantized_ops, device="cuda")
        for o, e in zip(outs, expected):
            ok, msg = same_bits(o, e)
            assert ok, f"{case['name']}: {msg}"
    finally:
        del os.environ["VOYAGER_B200_GENERIC_MX"]


@pytest.mark.parametrize("case", GEMMS, ids=[c["name"] for c in GEMMS])
def test_gemm_fixture_within_tolerance(case):
    outs, expected = run_case(case, torch.ops.quantized_ops, device="cuda")
    o, e = outs[0].float().cpu().double(), expected[0].float().double()
    assert outs[0].dtype == expected[0].dtype and o.shape == e.shape
    rel = (o - e).norm() / e.norm()
    assert rel <= 1e-2, rel            # tolerance for the fp32-accumulate GEMM


def test_outputs_do_not_alias_inputs_and_are_deterministic():
    from golden_util import golden_table
    x = torch.randn(64, 128, device="cuda")
    keep = x.clone()
    q = golden_table("int8").cuda()
    a = torch.ops.quantized_ops.quantize_mx(x, q, (-1,), 32, 127.0, True)
    b = torch.ops.quantized_ops.quantize_mx(x, q, (-1,), 32, 127.0, True)
    assert torch.equal(x, keep)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert a[1].data_ptr() != x.data_ptr()


def test_empty_inputs():
    from golden_util import golden_table
    q = golden_table("int8").cuda()
    x = torch.empty(0, 32, device="cuda")
    s, c = torch.ops.quantized_ops.quantize_mx(x, q, (-1,), 32, 127.0, True)
    assert s.shape == (0, 1) and c.shape == (0, 32)
    assert torch.ops.quantized_ops.vmap(x, q).shape == (0, 32)
    assert torch.ops.quantized_ops.quantize(x, torch.ones(1, device="cuda"), None, None, None, q).shape == (0, 32)


def test_float16_vmap_and_unsupported_dtype():
    from golden_util import golden_table
    q = golden_table("int8")
    x = (torch.randn(1000) * 40).half()
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
    import voyager_oracle as vo
    want = vo.lut_map(x, q)
    got = torch.ops.quantized_ops.vmap(x.cuda(), q.cuda())
    assert same_bits(got.float(), want.float())[0] and got.dtype == torch.float16
    with pytest.raises(NotImplementedError):
        torch.ops.quantized_ops.vmap(x.double().cuda(), q.cuda())
