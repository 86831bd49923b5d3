"""oracle.sampler.raw_logprob against torch.log_softmax (CPU)."""

import numpy as np
import torch

from oracle import sampler as OS


def test_raw_logprob_is_log_softmax_at_the_token():
    logits = OS.synth_logits(5, 4096, seed=11)
    tokens = np.array([0, 17, 4095, 2048, 1], dtype=np.int64)
    want = torch.log_softmax(torch.from_numpy(logits).double(), dim=-1)[torch.arange(5), torch.from_numpy(tokens)].numpy()
    assert np.abs(OS.raw_logprob(logits, tokens) - want).max() <= 1e-6
    shifted = OS.raw_logprob(logits + 100.0, tokens)      # shift invariance: the row maximum is taken out first
    assert np.abs(shifted - want).max() <= 1e-4
