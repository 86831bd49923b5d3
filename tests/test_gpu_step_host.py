"""vqk_lm_head_step_host: the decode step from host buffers gives the tokens (and scores) of the
device-tensor call, for the streaming and the tensor-core kernels, growing batches, and rows the
sampler tail hands to the full-row kernel."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

V, H = 4096 + 160, 512


def _shard(mode, seed=0):
    from vllm_quant_kernels import _lmhead as LH
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(V, H, generator=g) * 0.05).half().cuda()
    q, s = LH.quantize_weight(mode, w)
    return LH, LH.LMHeadShard(mode, q, s)


def _host_args(LH, B, seed, top_k=50, top_p=0.9):
    rng = np.random.default_rng(seed)
    return LH.SamplingArgs(
        temperature=torch.from_numpy(rng.uniform(0.5, 1.5, B).astype(np.float32)),
        seeds=torch.from_numpy(rng.integers(0, 2**31 - 1, B).astype(np.int32)),
        top_k=torch.full((B,), top_k, dtype=torch.int32), top_p=torch.full((B,), top_p, dtype=torch.float32),
        vocab_offset=0, vocab_total=V)


def _to_dev(LH, a):
    return LH.SamplingArgs(temperature=a.temperature.cuda(), seeds=a.seeds.cuda(), top_k=a.top_k.cuda(),
                           top_p=a.top_p.cuda(), vocab_offset=0, vocab_total=V)


@pytest.mark.parametrize("mode", ["int8", "fp8", "w8a8", "mxfp8", "mxfp4"])
def test_step_host_matches_the_device_call(mode):
    LH, shard = _shard(mode)
    for B in (1, 3, 8, 20, 2):      # growing, then shrinking: the staging buffers are reallocated, then reused
        x = torch.randn(B, H, generator=torch.Generator().manual_seed(B)).half()
        sp = _host_args(LH, B, seed=B)
        want, want_s = shard.sample(x.cuda(), _to_dev(LH, sp))
        got = shard.step_host(x, sp, torch.empty(B, dtype=torch.int64))
        assert got.tolist() == want.cpu().tolist(), (mode, B)
        out = torch.empty(B, dtype=torch.int64)
        run = shard.host_stepper(x, sp, out)                  # bound form: refill the host tensors, call again
        assert run().tolist() == want.cpu().tolist()
        x.copy_(torch.randn(B, H, generator=torch.Generator().manual_seed(100 + B)).half())
        want2, _ = shard.sample(x.cuda(), _to_dev(LH, sp))
        assert run().tolist() == want2.cpu().tolist()
        want, want_s = shard.sample(x.cuda(), _to_dev(LH, sp))
        sc = torch.empty(B, dtype=torch.float32)
        got2 = shard.step_host(x, sp, torch.empty(B, dtype=torch.int64), scores_host=sc)
        assert got2.tolist() == want.cpu().tolist()
        assert torch.equal(sc, want_s.cpu())


def test_step_host_rows_for_the_full_row_kernel_and_greedy_rows():
    LH, shard = _shard("int8", seed=3)
    B = 4
    x = torch.randn(B, H, generator=torch.Generator().manual_seed(9)).half()
    sp = _host_args(LH, B, seed=5)
    sp.top_k = torch.tensor([0, 50, 0, 4000], dtype=torch.int32)       # top-p only, top-k, none, k beyond the lists
    sp.top_p = torch.tensor([0.8, 1.0, 1.0, 0.95], dtype=torch.float32)
    want, _ = shard.sample(x.cuda(), _to_dev(LH, sp))
    got = shard.step_host(x, sp, torch.empty(B, dtype=torch.int64))
    assert got.tolist() == want.cpu().tolist()
    greedy = LH.SamplingArgs(vocab_offset=0, vocab_total=V)                # no temperature: argmax for every row
    got = shard.step_host(x, greedy, torch.empty(B, dtype=torch.int64))
    logits = shard.logits(x.cuda()).float()
    assert got.tolist() == logits.argmax(dim=1).cpu().tolist()
