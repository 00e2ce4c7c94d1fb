"""Drop-in behaviour next to the real upstream package (runs only where a checkout is present)."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("VOYAGER_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "src", "voyager_compiler")),
                                reason="upstream checkout not available")


def _run(code):
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, os.path.join(ROOT, "tests", "golden")]))
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(code)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_impl_mode_keeps_upstream_cpu_kernels_and_op_identity():
    out = _run("""
        import torch
        from _reference_import import import_reference
        ref = import_reference()
        op_before = torch.ops.quantized_ops.quantize_mx.default
        import voyager_compiler_b200 as vb
        assert vb.REGISTERED_AS == "impl", vb.REGISTERED_AS
        assert torch.ops.quantized_ops.quantize_mx.default is op_before
        q = ref["fake_quantize"].get_quantization_map("int8")
        x = torch.randn(4, 64)
        s, c = torch.ops.quantized_ops.quantize_mx(x, q, (-1,), 32, 127.0, True)     # CPU: upstream composite
        s2, c2 = ref["ops"].quantize_mx(x, q, (-1,), 32, 127.0, True)
        assert torch.equal(s, s2) and torch.equal(c, c2)
        m = torch.empty(8, 64, device="meta")
        sm, cm = torch.ops.quantized_ops.quantize_mx(m, q.to("meta"), (-1,), 32, 127.0, True)
        assert sm.shape == (8, 2) and cm.shape == (8, 64)
        print("ok")
    """)
    assert "ok" in out


def test_patch_reference_rebinds_direct_imports_and_unpatches():
    out = _run("""
        import torch
        from _reference_import import import_reference
        ref = import_reference()
        import voyager_compiler_b200 as vb
        from voyager_compiler_b200 import compat
        fq = ref["fake_quantize"]
        orig = fq.vmap
        done = compat.patch_reference()
        assert "voyager_compiler.quantization.fake_quantize.vmap" in done, done
        assert fq.vmap is not orig and fq.vmap.__wrapped_original__ is orig
        q = fq.get_quantization_map("int8")
        x = torch.randn(100) * 30
        assert torch.equal(fq.vmap(x, q), orig(x, q))            # CPU tensors still use the original
        # the autograd functions: CPU tensors keep upstream's forward, module output unchanged
        assert "voyager_compiler.quantization.fake_quantize.FakeQuantizeFunction.forward" in done, done
        assert "voyager_compiler.quantization.fake_quantize.GroupWiseAffineFakeQuantFunction.forward" in done, done
        ga = fq.FusedAmaxObsFakeQuantize("int8", qscheme=ref["qspec"].QScheme.GROUP_WISE_AFFINE, quant_min=0.0, quant_max=15.0,
                                         ch_axis=-1, block_size=8)
        assert ga(torch.randn(3, 16)).shape == (3, 16) and ga.scale.shape == (3, 2)     # CPU: upstream's own forward
        m = fq.FusedAmaxObsFakeQuantize("int8", qscheme=ref["qspec"].QScheme.PER_TENSOR_SYMMETRIC, quant_max=127.0,
                                        amax_history_len=2)
        xs = [torch.randn(4, 16) for _ in range(3)]
        got = [m(v).clone() for v in xs]
        compat.unpatch_reference()
        assert fq.vmap is orig
        assert not hasattr(fq.FakeQuantizeFunction.forward, "__wrapped_original__")
        m2 = fq.FusedAmaxObsFakeQuantize("int8", qscheme=ref["qspec"].QScheme.PER_TENSOR_SYMMETRIC, quant_max=127.0,
                                         amax_history_len=2)
        assert all(torch.equal(a, m2(v)) for a, v in zip(got, xs))
        print("ok")
    """)
    assert "ok" in out


def test_patch_reference_rebinds_gptq_compensation():
    out = _run("""
        import types
        import torch
        import transformers                      # before the torchao stand-in of the import helper
        from transformers import PreTrainedModel
        from _reference_import import import_reference
        ref = import_reference()
        import importlib
        g = importlib.import_module("voyager_compiler.quantization.gptq")
        import voyager_compiler_b200 as vb
        from voyager_compiler_b200 import compat
        orig = g.compensate_weight
        done = compat.patch_reference()
        assert "voyager_compiler.quantization.gptq.compensate_weight" in done, done
        assert g.compensate_weight.__wrapped_original__ is orig
        torch.manual_seed(0)
        w = torch.randn(8, 64) * 0.1
        x = torch.randn(200, 64)
        fake = types.SimpleNamespace(qmap=ref["fake_quantize"].get_quantization_map("int4"), scale_qmap=None, quant_max=7.0,
                                     block_size=32, ch_axis=-1)
        a = g.compensate_weight(w, x.t() @ x, 200, fake, 0.01)            # CPU tensors: upstream's own walk
        b = orig(w, x.t() @ x, 200, fake, 0.01)
        assert torch.equal(a, b)
        compat.unpatch_reference()
        assert g.compensate_weight is orig
        print("ok")
    """)
    assert "ok" in out


def test_patch_reference_rebinds_lcq_accumulation():
    out = _run("""
        import types
        import torch
        import transformers                      # before the torchao stand-in of the import helper
        from transformers import PreTrainedModel
        from _reference_import import import_reference
        import_reference()
        import importlib
        lcq = importlib.import_module("voyager_compiler.quantization.lcq")
        import voyager_compiler_b200 as vb
        from voyager_compiler_b200 import compat
        orig = lcq._accumulate
        done = compat.patch_reference()
        assert "voyager_compiler.quantization.lcq._accumulate" in done, done
        module = types.SimpleNamespace(ch_axis=-1, block_size=32, quant_max=7.0)
        x = torch.randn(6, 64)
        a, b = lcq.Histogram(-7.0, 7.0), lcq.Histogram(-7.0, 7.0)
        lcq._accumulate(x, module, None, a)                 # CPU tensors: upstream's own pass
        orig(x, module, None, b)
        assert torch.equal(a.weight, b.weight) and torch.equal(a.square, b.square)
        compat.unpatch_reference()
        assert lcq._accumulate is orig
        print("ok")
    """)
    assert "ok" in out
