"""Persisted quantized lm_head (vllm_quant_kernels/_checkpoint.py): the file holds the reference's
storage layouts, a round trip returns the same bits, and a file made from another weight, mode or
shape is refused.  The CPU part uses stand-in tensors; the GPU part goes through `_init_int8`."""

import os

import numpy as np
import pytest
import torch

from vllm_quant_kernels import _checkpoint as CK


def _fake(mode, V=64, H=128, seed=0):
    g = torch.Generator().manual_seed(seed)
    qd, sd = CK._DTYPES[mode]
    qs, ss = CK.expected_shapes(mode, V, H)
    q = torch.randint(0, 127, qs, generator=g).to(qd)
    s = (torch.rand(ss, generator=g) + 0.5).to(sd) if sd.is_floating_point else torch.randint(100, 140, ss, generator=g).to(sd)
    return q, s


@pytest.mark.parametrize("mode", ["int8", "w8a8", "fp8", "mxfp8", "mxfp4"])
def test_round_trip_and_layouts(tmp_path, mode):
    V, H = 64, 128
    q, s = _fake(mode, V, H)
    w = torch.randn(V, H).half()
    fp = CK.weight_fingerprint(w)
    path = CK.cache_path(str(tmp_path), mode, fp)
    CK.save(path, mode, q, s, H, w.dtype, fp)
    got = CK.load(path, mode, V, H, fp, "cpu")
    assert got is not None and torch.equal(got[0], q) and torch.equal(got[1], s)
    assert got[0].dtype == q.dtype and got[1].dtype == s.dtype
    # refused: another mode, another shape, another weight
    other = "int8" if mode != "int8" else "fp8"
    assert CK.load(path, other, V, H, fp, "cpu") is None
    assert CK.load(path, mode, V + 1, H, fp, "cpu") is None
    assert CK.load(path, mode, V, H, CK.weight_fingerprint(w + 1), "cpu") is None
    assert CK.load(str(tmp_path / "missing.safetensors"), mode, V, H, fp, "cpu") is None
    with pytest.raises(ValueError):
        CK.save(path, mode, q[:, :-1], s, H, w.dtype, fp)


def test_fingerprint_sees_shape_dtype_and_content():
    w = torch.randn(300, 64).half()
    a = CK.weight_fingerprint(w)
    assert a == CK.weight_fingerprint(w.clone())
    w2 = w.clone()
    w2[0, 0] += 1
    assert CK.weight_fingerprint(w2) != a
    assert CK.weight_fingerprint(w.bfloat16()) != a
    assert CK.weight_fingerprint(w[:299]) != a


def test_quantize_or_load_uses_the_cache(tmp_path, monkeypatch):
    calls = []

    def quantize(mode, w):
        calls.append(mode)
        return _fake(mode, w.shape[0], w.shape[1], seed=1)
    w = torch.randn(64, 128).half()
    monkeypatch.delenv("VLLM_QUANT_LMHEAD_CACHE", raising=False)
    assert CK.quantize_or_load("int8", w, quantize)[2] == "quantized"
    monkeypatch.setenv("VLLM_QUANT_LMHEAD_CACHE", str(tmp_path))
    q1, s1, how = CK.quantize_or_load("int8", w, quantize)
    assert how == "quantized+saved" and len(os.listdir(tmp_path)) == 1
    q2, s2, how = CK.quantize_or_load("int8", w, quantize)
    assert how == "loaded" and torch.equal(q1, q2) and torch.equal(s1, s2) and calls == ["int8", "int8"]
    assert CK.quantize_or_load("mxfp4", w, quantize)[2] == "quantized+saved"      # its own file
    assert CK.quantize_or_load("int8", w * 2, quantize)[2] == "quantized+saved"   # another weight


@pytest.mark.gpu
def test_init_reads_back_what_it_wrote(tmp_path, monkeypatch):
    from types import SimpleNamespace
    from tests.util import make_act, make_weight, t2n
    from vllm_quant_kernels._quant import QuantizedLogitsProcessor

    class FakeWeight:
        def __init__(self, t):
            self.data, self.dtype, self.shape, self.device = t, t.dtype, t.shape, t.device
    V, H = 100_016, 256
    w = make_weight(V, H, seed=4)
    x = make_act(3, H, seed=5)
    monkeypatch.setenv("VLLM_QUANT_LMHEAD_CACHE", str(tmp_path))
    for e in ("VLLM_USE_W8A8_LMHEAD", "VLLM_USE_FP8_LMHEAD", "VLLM_USE_MXFP8_LMHEAD"):
        monkeypatch.delenv(e, raising=False)
    monkeypatch.setenv("VLLM_USE_MXFP4_LMHEAD", "1")
    outs = []
    for rep in range(2):
        lm = SimpleNamespace(weight=FakeWeight(w))
        proc = QuantizedLogitsProcessor.__new__(QuantizedLogitsProcessor)
        proc._init_int8(lm)
        outs.append((t2n(lm._mxfp4_w), t2n(lm._mxfp4_w_scales), t2n(proc._quantized_forward(x, lm, None))))
    assert len(os.listdir(tmp_path)) == 1
    for a, b in zip(outs[0], outs[1]):
        assert (a.view(np.uint8) == b.view(np.uint8)).all()
