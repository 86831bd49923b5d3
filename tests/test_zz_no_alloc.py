"""The sampler entry point that allocates nothing (`vqk_sample_static`).

Some callers cannot allocate where they sample: a serving engine that sized its KV cache
from a one-off memory measurement has no spare bytes to ask for later, and nothing may be
allocated between the begin and end of a stream capture.  For them the library keeps the
sampler's scratch in a fixed device array of its own.  This test calls that entry point
through the C ABI twice in a row and holds it to the workspace-based `vqk_sample`: the
same token ids and the same winning scores, bit for bit.

The file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test.  It passes alone in a fresh process as well as after the rest.
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import sampler as OS

pytestmark = pytest.mark.gpu


def _params(ffi, B, V, arrays):
    return ffi.SampleParams(arrays["T"].data_ptr(), arrays["seeds"].data_ptr(), arrays["k"].data_ptr(),
                            arrays["p"].data_ptr(), None, 0, V)


def _case(B, V, seed, dtype, dev):
    rng = np.random.default_rng(seed)
    logits = torch.from_numpy(OS.synth_logits(B, V, seed=seed)).to(dev).to(dtype)
    T = rng.uniform(0.5, 1.5, B).astype(np.float32)
    T[0] = 0.0                                   # a greedy row
    k = np.full(B, 50, np.int32)
    k[-1] = 0                                    # a row without top-k ...
    p = np.full(B, 0.9, np.float32)
    p[-1] = 1.0                                  # ... and without top-p: noise on every column
    if B > 2:
        k[1] = 0                                 # top-p only: the full-row pass
    arrays = dict(T=torch.from_numpy(T).to(dev), seeds=torch.from_numpy(rng.integers(0, 2**31 - 1, B).astype(np.int32)).to(dev),
                  k=torch.from_numpy(k).to(dev), p=torch.from_numpy(p).to(dev))
    return logits, arrays


def test_static_scratch_sampler_matches_workspace_sampler_twice():
    from vllm_quant_kernels import _ffi
    L = _ffi.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row, different shapes and dtypes, so the second one runs over whatever
    # the first left in the shared scratch
    for B, V, seed, dtype, code in ((8, 248320, 11, torch.float32, _ffi.F32), (5, 50000, 12, torch.bfloat16, _ffi.BF16)):
        logits, a = _case(B, V, seed, dtype, dev)
        sp = _params(_ffi, B, V, a)
        n = L.vqk_sample_workspace_bytes(B, V)
        ws = torch.empty(n, dtype=torch.uint8, device=dev)
        tok_ref = torch.full((B,), -7, dtype=torch.int64, device=dev)
        sc_ref = torch.zeros(B, dtype=torch.float32, device=dev)
        rc = L.vqk_sample(logits.data_ptr(), code, B, V, logits.stride(0), ctypes.byref(sp), tok_ref.data_ptr(),
                          sc_ref.data_ptr(), None, ws.data_ptr(), n, stream)
        assert rc == 0
        tok = torch.full((B,), -9, dtype=torch.int64, device=dev)
        sc = torch.zeros(B, dtype=torch.float32, device=dev)
        rc = L.vqk_sample_static(logits.data_ptr(), code, B, V, logits.stride(0), ctypes.byref(sp), tok.data_ptr(),
                                 sc.data_ptr(), stream)
        assert rc == 0, L.vqk_strerror(rc)
        torch.cuda.synchronize()
        assert torch.equal(tok, tok_ref), (tok.tolist(), tok_ref.tolist())
        assert torch.equal(sc, sc_ref)
        assert int(tok.min()) >= 0 and int(tok.max()) < V
        # ... and to the CPU oracle on the same logits, so the check does not lean on vqk_sample alone
        want = OS.sample(logits.float().cpu().numpy(), a["T"].cpu().numpy(), a["seeds"].cpu().numpy(),
                         top_k=a["k"].cpu().numpy(), top_p=a["p"].cpu().numpy())
        decided = (want["margin"] > 1e-4) & (want["p_margin"] > 2e-6)
        assert decided.mean() >= 0.5
        assert (tok.cpu().numpy()[decided] == want["tokens"][decided]).all()


def test_static_scratch_sampler_rejects_sizes_beyond_its_maximum():
    from vllm_quant_kernels import _ffi
    L = _ffi.lib()
    sp = _ffi.SampleParams(None, None, None, None, None, 0, 1000)
    # 65 rows, then a vocabulary above 262144: refused before anything is launched
    assert L.vqk_sample_static(256, _ffi.F32, _ffi.STATIC_MAX_ROWS + 1, 1000, 1000, ctypes.byref(sp), 256, None, None) == -7
    sp = _ffi.SampleParams(None, None, None, None, None, 0, _ffi.STATIC_MAX_VOCAB + 1)
    assert L.vqk_sample_static(256, _ffi.F32, 1, _ffi.STATIC_MAX_VOCAB + 1, _ffi.STATIC_MAX_VOCAB + 1,
                               ctypes.byref(sp), 256, None, None) == -7
    assert b"vqk_sample_static" in L.vqk_strerror(-7)


def test_static_scratch_sampler_inside_a_cuda_graph():
    """The use the entry point is made for: after one warm-up call it is captured into a CUDA
    graph (nothing may be allocated between the begin and end of a capture) with caller-owned
    outputs, and every replay gives what the workspace-based sampler gives."""
    from vllm_quant_kernels import _ffi
    L = _ffi.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, V = 6, 151936
    logits, a = _case(B, V, 21, torch.bfloat16, dev)
    sp = _params(_ffi, B, V, a)
    n = L.vqk_sample_workspace_bytes(B, V)
    ws = torch.empty(n, dtype=torch.uint8, device=dev)
    tok_ref = torch.empty(B, dtype=torch.int64, device=dev)
    sc_ref = torch.empty(B, dtype=torch.float32, device=dev)
    assert L.vqk_sample(logits.data_ptr(), _ffi.BF16, B, V, logits.stride(0), ctypes.byref(sp), tok_ref.data_ptr(),
                        sc_ref.data_ptr(), None, ws.data_ptr(), n, torch.cuda.current_stream().cuda_stream) == 0
    tok = torch.full((B,), -9, dtype=torch.int64, device=dev)
    sc = torch.zeros(B, dtype=torch.float32, device=dev)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        assert L.vqk_sample_static(logits.data_ptr(), _ffi.BF16, B, V, logits.stride(0), ctypes.byref(sp), tok.data_ptr(),
                                   sc.data_ptr(), side.cuda_stream) == 0          # warm-up: looks the scratch up
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            rc = L.vqk_sample_static(logits.data_ptr(), _ffi.BF16, B, V, logits.stride(0), ctypes.byref(sp),
                                     tok.data_ptr(), sc.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        for _ in range(2):
            tok.fill_(-9)
            sc.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(tok, tok_ref) and torch.equal(sc, sc_ref)
    torch.cuda.current_stream().wait_stream(side)
