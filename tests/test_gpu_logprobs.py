"""The raw log-probability of the sampled token from the stand-alone sampler (vqk_sample with
vqk_sample_params.logprobs): equal to log_softmax of the given logits at the sampled token, for every
logits dtype and row kind, without changing the tokens."""

import numpy as np
import pytest
import torch

from oracle import sampler as OS

pytestmark = pytest.mark.gpu


def _args(LH, B, V, seed, **kw):
    rng = np.random.default_rng(seed)
    t = lambda a, dt: None if a is None else torch.from_numpy(np.asarray(a)).to(dt).cuda()
    return LH.SamplingArgs(t(rng.uniform(0.5, 1.5, B).astype(np.float32), torch.float32),
                           t(rng.integers(0, 2**31 - 1, B).astype(np.int32), torch.int32),
                           t(kw.get("top_k"), torch.int32), t(kw.get("top_p"), torch.float32), None, 0, V)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,V", [(1, 248320), (8, 151936), (64, 32000), (3, 1000)])
def test_logprob_of_sampled_token(dtype, B, V):
    from vllm_quant_kernels import _lmhead as LH
    logits = torch.from_numpy(OS.synth_logits(B, V, seed=B + V)).to(dtype).cuda()
    for kw in (dict(), dict(top_k=np.full(B, 50, np.int32), top_p=np.full(B, 0.9, np.float32)),
               dict(top_p=np.full(B, 0.8, np.float32))):
        sp = _args(LH, B, V, seed=7, **kw)
        tok0, sc0 = LH.sample_logits(logits, sp)
        tok, sc, lp = LH.sample_logits(logits, sp, return_logprobs=True)
        assert torch.equal(tok, tok0) and torch.equal(sc, sc0)
        want = OS.raw_logprob(logits.float().cpu().numpy(), tok.cpu().numpy())
        ref = torch.log_softmax(logits.float(), dim=-1).gather(1, tok.view(-1, 1)).view(-1).cpu().numpy()
        got = lp.cpu().numpy()
        assert np.abs(got - want).max() <= 2e-4, (dtype, B, V, list(kw), np.abs(got - want).max())   # fp32 sums against float64
        assert np.abs(got - ref).max() <= 2e-4


def test_logprob_greedy_rows_and_rejections():
    from vllm_quant_kernels import _lmhead as LH, _ffi
    B, V = 4, 5000
    logits = torch.from_numpy(OS.synth_logits(B, V, seed=3)).cuda()
    greedy = LH.SamplingArgs(vocab_offset=0, vocab_total=V)
    tok, _, lp = LH.sample_logits(logits, greedy, return_logprobs=True)
    assert tok.tolist() == logits.argmax(dim=1).tolist()
    assert np.abs(lp.cpu().numpy() - OS.raw_logprob(logits.cpu().numpy(), tok.cpu().numpy())).max() <= 2e-4
    with pytest.raises(ValueError):
        LH.sample_logits(logits, greedy, records=True, return_logprobs=True)
    # the allocation-free entry point has no room for the per-slice sums
    sp = _args(LH, B, V, seed=1)
    spc = sp.to_c(B, V)
    out = torch.empty(B, dtype=torch.float32, device="cuda")
    spc.logprobs = out.data_ptr()
    tokens = torch.empty(B, dtype=torch.int64, device="cuda")
    import ctypes
    rc = _ffi.lib().vqk_sample_static(logits.data_ptr(), 2, B, V, logits.stride(0), ctypes.byref(spc), tokens.data_ptr(), None,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == -2          # VQK_ERR_UNSUPPORTED
