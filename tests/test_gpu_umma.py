"""GPU parity of the tcgen05 tensor-core lm_head kernel (FP8 and W8A8, larger batches)
against the CPU oracle and against the register-streaming kernel."""

import numpy as np
import pytest
import torch

from oracle import lm_head as OLM, sampler as OS
from tests.util import assert_tokens_match, make_act, make_weight, sample_args, t2n

pytestmark = pytest.mark.gpu
REL_L2 = 1e-3
DEV = "cuda"


def L():
    from vllm_quant_kernels import _lmhead
    return _lmhead


def _oracle(mode, x, w, bias=None):
    wq, ws = OLM.quantize_weight(mode, t2n(w))
    return OLM.logits(mode, t2n(x), wq, ws, bias=None if bias is None else t2n(bias))


@pytest.mark.parametrize("mode", ["fp8", "w8a8"])
@pytest.mark.parametrize("B,H", [(1, 1024), (16, 3072), (17, 1024), (33, 3072), (64, 1024), (100, 2048),
                                 (256, 1024), (300, 1024)])
def test_umma_logits_vs_oracle(mode, B, H, monkeypatch):
    """Vocab not a multiple of the 128-row tile (TMA zero-fills the ragged tile), batches on both
    sides of every padded N, more than 256 columns (two launches)."""
    from vllm_quant_kernels import _ffi
    V = 16 * 333
    w = make_weight(V, H, seed=H + B)
    x = make_act(B, H, seed=B)
    bias = make_act(1, V, seed=7)[0]
    q, s = L().quantize_weight(mode, w)
    shard = L().LMHeadShard(mode, q, s)
    monkeypatch.setenv("VQK_LM_HEAD_KERNEL", "umma")
    got = t2n(shard.logits(x, bias))
    monkeypatch.setenv("VQK_LM_HEAD_KERNEL", "stream")
    got_stream = t2n(shard.logits(x, bias))
    monkeypatch.delenv("VQK_LM_HEAD_KERNEL", raising=False)
    assert _ffi.lib().vqk_device_error() == 0
    ref = _oracle(mode, x, w, bias)
    assert OLM.rel_l2(got, ref) <= REL_L2, (mode, B, H, OLM.rel_l2(got, ref))
    if mode == "w8a8":      # int32 accumulation is exact in both kernels
        assert (got.view(np.int16) == got_stream.view(np.int16)).all()
    else:
        assert OLM.rel_l2(got, got_stream) <= REL_L2


@pytest.mark.parametrize("mode", ["fp8", "w8a8"])
@pytest.mark.parametrize("B", [24, 64, 130])
def test_umma_fused_sampling(mode, B, monkeypatch):
    """Default dispatch (batch > 8 -> tensor-core kernel): fused tokens equal the sampler run on
    the logits the kernel materialises, and the oracle sampler where its margin allows."""
    V, H = 128 * 391 + 48, 1024
    w = make_weight(V, H, seed=5) * 4.0
    x = make_act(B, H, seed=B)
    q, s = L().quantize_weight(mode, w)
    shard = L().LMHeadShard(mode, q, s)
    rng = np.random.default_rng(B)
    T = rng.uniform(0.5, 1.5, B).astype(np.float32)
    T[3] = 0.0
    seeds = rng.integers(0, 2**31 - 1, B).astype(np.int32)
    monkeypatch.delenv("VQK_LM_HEAD_KERNEL", raising=False)
    for kw in (dict(), dict(top_k=np.full(B, 50, np.int32), top_p=np.full(B, 0.9, np.float32))):
        sp = sample_args(B, DEV, T, seeds, **kw)
        tok, sc, logits = shard.sample(x, sp, return_logits=True)
        tok2, sc2 = L().sample_logits(logits, sp)
        assert torch.equal(tok, tok2) and torch.equal(sc, sc2), (mode, B, list(kw))
        ref = OS.sample(t2n(logits).astype(np.float32), T, seeds, **kw)
        assert_tokens_match(tok, ref, what=f"umma fused {mode} {list(kw)}")
        tok3, _ = shard.sample(x, sp)
        assert torch.equal(tok, tok3)
    ref_logits = _oracle(mode, x, w)
    assert OLM.rel_l2(t2n(logits), ref_logits) <= REL_L2


@pytest.mark.parametrize("mode", ["mxfp8", "mxfp4"])
@pytest.mark.parametrize("B,H", [(1, 1024), (16, 3072), (33, 1024), (100, 2048), (128, 1024), (200, 1024)])
def test_umma_block_scaled_logits_vs_oracle(mode, B, H, monkeypatch):
    """Block-scaled tensor-core kernel (scale factors through TMEM, packed E2M1 expanded by the
    TMA unit) against the oracle and against the register-streaming kernel."""
    from vllm_quant_kernels import _ffi
    V = 16 * 333
    w = make_weight(V, H, seed=H + B)
    x = make_act(B, H, seed=B)
    q, s = L().quantize_weight(mode, w)
    shard = L().LMHeadShard(mode, q, s)
    monkeypatch.setenv("VQK_LM_HEAD_KERNEL", "umma")
    got = t2n(shard.logits(x))
    monkeypatch.setenv("VQK_LM_HEAD_KERNEL", "stream")
    got_stream = t2n(shard.logits(x))
    monkeypatch.delenv("VQK_LM_HEAD_KERNEL", raising=False)
    assert _ffi.lib().vqk_device_error() == 0
    ref = _oracle(mode, x, w)
    assert OLM.rel_l2(got_stream, ref) <= REL_L2
    assert OLM.rel_l2(got, ref) <= REL_L2, (mode, B, H, OLM.rel_l2(got, ref))


@pytest.mark.parametrize("mode", ["mxfp8", "mxfp4"])
@pytest.mark.parametrize("B,H", [(4, 1024), (40, 512), (20, 384)])
def test_umma_block_scaled_many_tiles(mode, B, H, monkeypatch):
    """More 128-row tiles than SMs, so every CTA walks several tiles (scale hand-over between
    tiles, accumulator double buffering), a ragged last tile, and a K with an odd number of
    128-element blocks (H = 384: the one-block-per-stage variant)."""
    from vllm_quant_kernels import _ffi
    V = 128 * 450 + 40
    w = make_weight(V, H, seed=H)
    x = make_act(B, H, seed=B)
    q, s = L().quantize_weight(mode, w)
    shard = L().LMHeadShard(mode, q, s)
    monkeypatch.setenv("VQK_LM_HEAD_KERNEL", "umma")
    got = t2n(shard.logits(x))
    monkeypatch.setenv("VQK_LM_HEAD_KERNEL", "stream")
    got_stream = t2n(shard.logits(x))
    monkeypatch.delenv("VQK_LM_HEAD_KERNEL", raising=False)
    assert _ffi.lib().vqk_device_error() == 0
    assert OLM.rel_l2(got, got_stream) <= REL_L2, (mode, B, H, OLM.rel_l2(got, got_stream))
    ref = _oracle(mode, x[:2], w[:4096])
    assert OLM.rel_l2(got[:2, :4096], ref) <= REL_L2


@pytest.mark.parametrize("mode", ["mxfp8", "mxfp4"])
@pytest.mark.parametrize("B", [1, 5, 8, 9, 16, 24])
def test_umma_block_scaled_fused_sampling(mode, B, monkeypatch):
    """Default dispatch of the block-scaled modes (tensor-core kernel at every batch size, three
    MMA pipelines per CTA for narrow batches): fused tokens equal the sampler run on the logits
    the kernel materialises, with and without a logits buffer, a bias, and a vocab that ends
    inside a tile."""
    V, H = 256 * 300 + 72, 1024
    w = make_weight(V, H, seed=11) * 4.0
    x = make_act(B, H, seed=B)
    bias = make_act(1, V, seed=3)[0]
    q, s = L().quantize_weight(mode, w)
    shard = L().LMHeadShard(mode, q, s)
    rng = np.random.default_rng(B)
    T = rng.uniform(0.5, 1.5, B).astype(np.float32)
    T[B // 2] = 0.0
    seeds = rng.integers(0, 2**31 - 1, B).astype(np.int32)
    monkeypatch.delenv("VQK_LM_HEAD_KERNEL", raising=False)
    for kw in (dict(), dict(top_k=np.full(B, 50, np.int32), top_p=np.full(B, 0.9, np.float32))):
        sp = sample_args(B, DEV, T, seeds, **kw)
        tok, sc, logits = shard.sample(x, sp, return_logits=True)
        tok2, sc2 = L().sample_logits(logits, sp)
        assert torch.equal(tok, tok2) and torch.equal(sc, sc2), (mode, B, list(kw))
        ref = OS.sample(t2n(logits).astype(np.float32), T, seeds, **kw)
        assert_tokens_match(tok, ref, what=f"block-scaled fused {mode} {list(kw)}")
        tok3, _ = shard.sample(x, sp)
        assert torch.equal(tok, tok3)
    ref_logits = _oracle(mode, x, w)
    assert OLM.rel_l2(t2n(logits), ref_logits) <= REL_L2
    got_b = t2n(shard.logits(x, bias))
    assert OLM.rel_l2(got_b, _oracle(mode, x, w, bias)) <= REL_L2
    monkeypatch.setenv("VQK_LM_HEAD_KERNEL", "stream")
    got_s = t2n(shard.logits(x, bias))
    monkeypatch.delenv("VQK_LM_HEAD_KERNEL", raising=False)
    assert OLM.rel_l2(got_b, got_s) <= REL_L2


@pytest.mark.parametrize("mode", ["fp8", "mxfp8", "mxfp4"])
def test_umma_small_vocab_sampling(mode, monkeypatch):
    """Fewer tiles than SMs: the CTAs without a tile still have to write their (empty) slice
    records, or the sampler would read stale scratch."""
    B, V, H = 6, 16 * 333, 1024
    w = make_weight(V, H, seed=2) * 4.0
    x = make_act(B, H, seed=1)
    q, s = L().quantize_weight(mode, w)
    shard = L().LMHeadShard(mode, q, s)
    T = np.full(B, 0.8, np.float32)
    T[0] = 0.0
    seeds = np.arange(B, dtype=np.int32) + 5
    monkeypatch.setenv("VQK_LM_HEAD_KERNEL", "umma")
    for kw in (dict(), dict(top_k=np.full(B, 20, np.int32))):
        sp = sample_args(B, DEV, T, seeds, **kw)
        tok, sc, logits = shard.sample(x, sp, return_logits=True)
        tok2, sc2 = L().sample_logits(logits, sp)
        assert torch.equal(tok, tok2) and torch.equal(sc, sc2)
        tok3, _ = shard.sample(x, sp)
        assert torch.equal(tok, tok3)
    monkeypatch.delenv("VQK_LM_HEAD_KERNEL", raising=False)
