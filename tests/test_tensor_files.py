"""Tensor files: upstream's raw float32 dump (bufferize/emit.py:143-175) and the packed form next to it."""
import json
import os

import numpy as np
import pytest
import torch

from voyager_compiler_b200 import tensor_files as tf
from voyager_compiler_b200.model_quant import PackedMX


def test_float32_file_like_upstream(tmp_path):
    x = torch.randn(5, 7).bfloat16()
    tf.save_tensor(x, str(tmp_path / "w.bin"))
    tf.flush_tensor_files()
    back = np.fromfile(tmp_path / "w.bin", dtype=np.float32).reshape(5, 7)
    assert np.array_equal(back, x.float().numpy())


def test_packed_round_trip_on_host(tmp_path):
    g = torch.Generator().manual_seed(0)
    codes = torch.randint(0, 256, (6, 64), dtype=torch.uint8, generator=g)          # 4-bit codes of a [6, 128] tensor
    scale = torch.rand(6, 2, generator=g)
    levels = torch.linspace(-1, 1, 16)
    p = PackedMX(codes=codes, scale=scale, shape=(6, 128), block=64, code_bits=4, levels=levels)
    base = str(tmp_path / "layer0_w")
    tf.save_packed(p, base)
    tf.flush_tensor_files()
    assert os.path.getsize(base + ".codes.bin") == 6 * 64
    meta = json.load(open(base + ".json"))
    assert meta["shape"] == [6, 128] and meta["block"] == 64 and meta["code_bits"] == 4
    q = tf.load_packed(base)
    assert torch.equal(q.codes, codes) and torch.equal(q.scale, scale) and torch.equal(q.levels, levels)
    assert q.shape == (6, 128) and q.block == 64 and q.code_bits == 4
    with open(base + ".codes.bin", "ab") as f:
        f.write(b"x")
    with pytest.raises(ValueError):
        tf.load_packed(base)


def test_failed_write_is_reported(tmp_path):
    tf.save_tensor(torch.zeros(3), str(tmp_path / "missing_dir" / "w.bin"))
    with pytest.raises(OSError):
        tf.flush_tensor_files()


@pytest.mark.gpu
def test_packed_file_decodes_to_the_quantized_weight(tmp_path):
    from voyager_compiler_b200 import model_quant as mq
    w = (torch.randn(256, 512, device="cuda") * 0.02).bfloat16()
    (p,) = mq.quantize_tensors_mx([w], "nf4", 64, 1.0, False, code_bits=4)
    base = str(tmp_path / "w")
    tf.save_packed(p, base)
    tf.save_tensor(mq.dequantize_packed(p, torch.float32), base + ".bin")
    tf.flush_tensor_files()
    q = tf.load_packed(base, device="cuda")
    back = mq.dequantize_packed(q, torch.float32).cpu().numpy()
    assert np.array_equal(back, np.fromfile(base + ".bin", dtype=np.float32).reshape(256, 512))
    packed_bytes = sum(os.path.getsize(base + ext) for ext in (".codes.bin", ".scales.bin", ".levels.bin", ".json"))
    assert packed_bytes < os.path.getsize(base + ".bin") / 6          # 4.5 bits per element against 32
