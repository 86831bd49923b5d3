"""Shared helpers for the GPU parity tests."""

import numpy as np
import torch

from oracle import lm_head as OLM, quant as OQ, sampler as OS

MODES = ("int8", "w8a8", "fp8", "mxfp8", "mxfp4")


def t2n(t: torch.Tensor) -> np.ndarray:
    """torch -> numpy keeping the bits (bf16 goes through fp32, which is exact)."""
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.float().numpy()
    return t.numpy()


def make_weight(V, H, seed=0, dtype=torch.float16, device="cuda"):
    """Row-spread synthetic weight (per-row std log-uniform over 6x, clipped to 0.19)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    std = torch.exp(torch.empty(V).uniform_(np.log(0.0072), np.log(0.0432), generator=g))
    w = torch.randn(V, H, generator=g) * std[:, None]
    return w.clamp_(-0.19, 0.19).to(dtype).to(device)


def make_act(B, H, seed=0xC0DE, dtype=torch.float16, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(B, H, generator=g).to(dtype).to(device)


def oracle_quant(mode, w_np):
    return OLM.quantize_weight(mode, w_np)


def check_codes(mode, w_np, q_gpu, s_gpu):
    """Bit-exact codes and scales, except MX groups whose ceil(log2) is
    implementation-defined (ratio within a few ulp above a power of two)."""
    q_ref, s_ref = oracle_quant(mode, w_np)
    q = t2n(q_gpu)
    s = t2n(s_gpu)
    if mode in ("int8", "fp8"):
        assert (s.view(np.int16) == s_ref.view(np.int16)).all(), f"{mode}: scale bits differ"
        assert (q.view(np.int8) == q_ref.view(np.int8)).all(), f"{mode}: codes differ"
    elif mode == "w8a8":
        assert (s == s_ref).all() and (q == q_ref).all()
    else:
        amb = OQ.mx_scale_ambiguous(w_np, 448.0 if mode == "mxfp8" else 6.0)
        ok = ~amb
        assert (s[ok] == s_ref[ok]).all(), f"{mode}: scale bytes differ"
        per = 32 if mode == "mxfp8" else 16
        okq = np.repeat(ok, per, axis=1)
        assert (q.view(np.uint8)[okq] == q_ref.view(np.uint8)[okq]).all(), f"{mode}: codes differ"
        assert amb.mean() < 1e-3


def sample_args(B, device, temperature=None, seeds=None, top_k=None, top_p=None, thr=None,
                vocab_offset=0, vocab_total=None):
    from vllm_quant_kernels._lmhead import SamplingArgs

    def dev(a, dt):
        return None if a is None else torch.as_tensor(np.asarray(a), dtype=dt).to(device).contiguous()
    return SamplingArgs(dev(temperature, torch.float32), dev(seeds, torch.int32), dev(top_k, torch.int32),
                        dev(top_p, torch.float32), dev(thr, torch.float32), vocab_offset, vocab_total)


def assert_tokens_match(tok_gpu, ref, min_margin=1e-4, min_p_margin=2e-6, what=""):
    """Token ids equal wherever the oracle's top-2 perturbed-score margin and top-p
    boundary margin are not razor thin."""
    tok = t2n(tok_gpu)
    strict = (ref["margin"] > min_margin) & (ref["p_margin"] > min_p_margin)
    bad = (tok != ref["tokens"]) & strict
    assert not bad.any(), f"{what}: rows {np.nonzero(bad)[0][:8]} got {tok[bad][:8]} want {ref['tokens'][bad][:8]}"
    # the gate must actually bite: most rows have to be decided, not excused
    assert strict.mean() >= 0.5, f"{what}: too few rows with a usable margin ({strict.mean():.2f})"
