"""Fused Gumbel-argmax sampling entry point (CUDA, libvqk.so).

Same name and contract as the reference's src/vllm_quant_kernels/_sampler_kernels.py
`fused_gumbel_sample`; the Triton kernel and the two torch reductions behind it
are one C-ABI call here.
"""

from __future__ import annotations

import torch

from ._lmhead import SamplingArgs, sample_logits


def fused_gumbel_sample(
    logits: torch.Tensor,                 # [B, V] fp32 (bf16 / fp16 also accepted)
    temperature: "torch.Tensor | None",   # [B] fp32 (None => plain argmax)
    seeds: torch.Tensor,                  # [B] int32
    topk_threshold: "torch.Tensor | None" = None,  # [B] fp32 raw-logit threshold or None
    block_size: int = 1024,               # accepted for signature compatibility; unused
) -> torch.Tensor:
    """Returns `[B]` int64 sampled token ids.

    `temperature[i] < 1e-5` makes row i greedy; `topk_threshold[i]` keeps only
    logits >= it (raw, pre-temperature space, as the reference kernel applies it).
    """
    B, V = logits.shape
    assert logits.dtype in (torch.float32, torch.bfloat16, torch.float16), (
        f"Fused sampler requires floating logits, got {logits.dtype}"
    )
    assert seeds.shape == (B,) and seeds.dtype == torch.int32
    if temperature is not None:
        assert temperature.shape == (B,) and temperature.dtype == torch.float32
    if topk_threshold is not None:
        assert topk_threshold.shape == (B,) and topk_threshold.dtype == torch.float32
    sp = SamplingArgs(
        temperature=None if temperature is None else temperature.contiguous(),
        seeds=seeds.contiguous(),
        topk_threshold=None if topk_threshold is None else topk_threshold.contiguous(),
    )
    tokens, _ = sample_logits(logits, sp)
    return tokens
