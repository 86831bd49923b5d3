"""C-ABI checks that need no GPU: the library loads, exports every declared symbol,
rejects bad arguments before touching the device, and the host-side mirror of the
reference's registration logic behaves like the reference's."""

import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from vllm_quant_kernels import _ffi
    hdr = open(os.path.join(ROOT, "include", "vqk.h")).read()
    declared = set(re.findall(r"\b(vqk_[a-z0-9_]+)\s*\(", hdr))
    assert declared == set(_ffi.SYMBOLS), declared ^ set(_ffi.SYMBOLS)
    L = _ffi.lib()
    for s in declared:
        assert hasattr(L, s), s
    assert L.vqk_version() == 100
    assert b"sm_100" in L.vqk_strerror(-5)


def test_bad_arguments_are_rejected_without_a_device():
    from vllm_quant_kernels import _ffi
    L = _ffi.lib()
    h = ctypes.c_void_p()
    # null pointers, bad mode, bad shapes, misaligned base
    assert L.vqk_lm_head_create(0, None, None, 16, 64, ctypes.byref(h)) == -1
    assert L.vqk_lm_head_create(9, 256, 256, 16, 64, ctypes.byref(h)) == -1
    assert L.vqk_lm_head_create(0, 256, 256, 16, 40, ctypes.byref(h)) == -2      # H % 16
    assert L.vqk_lm_head_create(3, 256, 256, 16, 48, ctypes.byref(h)) == -2      # MX needs H % 32
    assert L.vqk_lm_head_create(0, 260, 256, 16, 64, ctypes.byref(h)) == -1      # 16-byte alignment
    assert L.vqk_lm_head_create(0, 256, 256, 16, 64, ctypes.byref(h)) == 0 and h.value
    assert L.vqk_lm_head_forward(h, None, 0, 1, 64, None, None, 0, None, None, None, None, None, 0, None) == -1
    assert L.vqk_lm_head_forward(h, 256, 2, 1, 64, None, 256, 16, None, None, None, None, None, 0, None) == -1  # fp32 x
    assert L.vqk_lm_head_forward(h, 256, 0, 1, 32, None, 256, 16, None, None, None, None, None, 0, None) == -1  # ldx < H
    assert L.vqk_lm_head_destroy(h) == 0
    assert L.vqk_quantize_weight(0, None, 0, 1, 16, 16, None, None, None) == -1
    assert L.vqk_quantize_act(0, 256, 0, 1, 16, 8, 256, None, None) == -1
    assert L.vqk_sample(None, 2, 1, 10, 10, None, None, None, None, None, 0, None) == -1
    sp = _ffi.SampleParams(None, None, None, None, None, 0, 10)
    assert L.vqk_sample(256, 7, 1, 10, 10, ctypes.byref(sp), 256, None, None, None, 0, None) == -1  # dtype
    assert L.vqk_sample(256, 2, 1, 10, 5, ctypes.byref(sp), 256, None, None, None, 0, None) == -1   # ld < V
    assert L.vqk_sample_finalize(256, 9, 1, ctypes.byref(sp), 256, None, None) == -1                # G > 8
    assert L.vqk_topk_threshold(None, 2, 1, 10, 10, None, None, None) == -1
    assert L.vqk_sample_workspace_bytes(4, 248320) > 0
    assert L.vqk_comm_create(None, 0, 1, ctypes.byref(h)) == -1


def test_peer_exchange_rejects_bad_arguments_without_a_device():
    """vqk_peer_*: argument errors come back before any CUDA call; destroying nothing is fine."""
    from vllm_quant_kernels import _ffi
    L = _ffi.lib()
    h = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(_ffi.PEER_HANDLE_BYTES)
    assert L.vqk_peer_create(1, 1, 16, ctypes.byref(h), handle) == -1          # rank >= nranks
    assert L.vqk_peer_create(0, 9, 16, ctypes.byref(h), handle) == -1          # more than 8 ranks
    assert L.vqk_peer_create(0, 2, 0, ctypes.byref(h), handle) == -1           # no rows
    assert L.vqk_peer_create(0, 2, 16, ctypes.byref(h), None) == -1            # nowhere to put the handle
    assert L.vqk_peer_connect(None, handle) == -1
    sp = _ffi.SampleParams()
    assert L.vqk_peer_exchange_finalize(None, 256, 1, ctypes.byref(sp), 256, None, None) == -1
    assert L.vqk_peer_destroy(None) == 0
    assert _ffi.PEER_HANDLE_BYTES == 64 and _ffi.PEER_MAX_RANKS == 8


def test_missing_library_is_a_loud_error(monkeypatch):
    from vllm_quant_kernels import _ffi
    monkeypatch.setattr(_ffi, "_lib", None)
    monkeypatch.setattr(_ffi, "LIB_PATH", "/nonexistent/libvqk.so")
    with pytest.raises(RuntimeError, match="no Triton, torch or CPU fallback"):
        _ffi.lib()


def test_cpu_tensors_are_refused():
    import torch
    from vllm_quant_kernels import _lmhead
    with pytest.raises(RuntimeError, match="no CPU path"):
        _lmhead.quantize_weight("int8", torch.zeros(4, 64, dtype=torch.float16))
    with pytest.raises(RuntimeError, match="no CPU path"):
        _lmhead.sample_logits(torch.zeros(1, 64), _lmhead.SamplingArgs())


def test_env_priority_and_truthiness(monkeypatch):
    from vllm_quant_kernels import _registration as R
    for v in R._ALL_ENVS:
        monkeypatch.delenv(v, raising=False)
    assert R.selected_mode() is None
    monkeypatch.setenv("VLLM_USE_INT8_LMHEAD", "1")
    assert R.selected_mode() == "int8"
    monkeypatch.setenv("VLLM_USE_W8A8_LMHEAD", "true")
    assert R.selected_mode() == "w8a8"
    monkeypatch.setenv("VLLM_USE_FP8_LMHEAD", "YES")
    assert R.selected_mode() == "fp8"
    monkeypatch.setenv("VLLM_USE_MXFP8_LMHEAD", "On")
    assert R.selected_mode() == "mxfp8"
    monkeypatch.setenv("VLLM_USE_MXFP4_LMHEAD", "1")
    assert R.selected_mode() == "mxfp4"
    monkeypatch.setenv("VLLM_USE_MXFP4_LMHEAD", "0")
    assert R.selected_mode() == "mxfp8"
    monkeypatch.setenv("VLLM_USE_MXFP8_LMHEAD", "2")          # not in the truthy set
    assert R.selected_mode() == "fp8"
    assert R._env_bool("VLLM_USE_FUSED_SAMPLER") is False


def test_shard_bounds_cover_the_vocabulary():
    from vllm_quant_kernels._dist import shard_bounds
    for V in (248320, 152064, 1000, 17):
        for G in (1, 2, 4, 8):
            edges = [shard_bounds(V, G, r) for r in range(G)]
            assert edges[0][0] == 0 and edges[-1][1] == V
            for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(s % 16 == 0 for s, e in edges if e > s)
    assert [shard_bounds(248320, 8, r)[1] - shard_bounds(248320, 8, r)[0] for r in range(8)] == [31040] * 8


def test_record_pack_unpack_roundtrip():
    from vllm_quant_kernels._dist import pack_record, unpack_record
    r = unpack_record(pack_record(1.5, 42))
    assert r["score"] == 1.5 and r["token"] == 42 and r["n"] == 0
    c = [(float(i) / 3, 1000 + i) for i in range(126)]
    r = unpack_record(pack_record(cands=c))
    assert r["n"] == 126 and r["cands"][5][1] == 1005 and abs(r["cands"][5][0] - np.float32(5 / 3)) < 1e-7
    with pytest.raises(ValueError):
        pack_record(cands=c + [(0.0, 0)])
