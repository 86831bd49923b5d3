"""Fused sampling replacement for vLLM's V1 Sampler, B200 build.

Overrides only `Sampler.sample()`, like the reference's
src/vllm_quant_kernels/_sampler.py.  Differences, all on the device side:
top-k is computed per row inside the CUDA sampler (no `torch.topk`, no
`.item()` host sync), and top-p is on the fast path (the reference fell back
to upstream for it).  Activation: `VLLM_USE_FUSED_SAMPLER=1`.
"""

from __future__ import annotations

import os
import sys
from typing import TYPE_CHECKING

import torch

from ._lmhead import SamplingArgs, sample_logits, topk_threshold
from ._sampler_kernels import fused_gumbel_sample  # noqa: F401  (re-exported like the reference)

if TYPE_CHECKING:
    from vllm.config.model import LogprobsMode
    from vllm.v1.sample.metadata import SamplingMetadata


_SAMPLING_EPS = 1e-5


def _fast_path_ok(sampling_metadata: "SamplingMetadata") -> bool:
    """Are all features outside the fused path inactive?  (reference: _sampler.py:28-59)

    Handled: per-row temperature incl. mixed greedy/random, top-k, top-p.
    Falls back for: allowed_token_ids_mask, bad_words, any logits processor,
    thinking-budget tracking, per-request generators.
    """
    sm = sampling_metadata
    if sm.allowed_token_ids_mask is not None:
        return False
    if sm.bad_words_token_ids:
        return False
    if sm.logitsprocs.argmax_invariant or sm.logitsprocs.non_argmax_invariant:
        return False
    holder = getattr(sm, "thinking_budget_state_holder", None)
    if holder is not None and holder.has_tracked_requests():
        return False
    if sm.generators:
        return False
    return True


def _compute_topk_threshold(logits: torch.Tensor, top_k: torch.Tensor, vocab_size: int) -> "torch.Tensor | None":
    """Per-row k-th largest raw logit (reference: _sampler.py:62-93), computed by a
    CUDA radix select without a host sync.  Rows with top_k >= vocab_size (vLLM's
    "disabled") get -inf, i.e. no mask for that row only; the reference disabled
    top-k for the WHOLE batch when any row had it disabled."""
    return topk_threshold(logits, top_k)


def _make_seeds(batch_size: int, device: torch.device) -> torch.Tensor:
    """One int32 seed per row from the default CUDA generator (reference: _sampler.py:96-116)."""
    return torch.randint(low=0, high=2**31 - 1, size=(batch_size,), dtype=torch.int32, device=device)


def try_fused_step(logits_processor, lm_head, hidden_states: torch.Tensor, sampling_metadata: "SamplingMetadata",
                   embedding_bias: "torch.Tensor | None" = None, seeds: "torch.Tensor | None" = None,
                   logprobs_mode: str = "raw_logprobs") -> "torch.Tensor | None":
    """The whole decode tail in one call: lm_head and sampler fused, logits never materialised.

    vLLM's runner calls `model.compute_logits(hidden)` and `sampler(logits, metadata)` one after the
    other; the two plugin hooks can only speed each up.  A runner that owns both calls can ask this
    function first: it returns the sampled token ids (int64 [B]) when the batch is on the fused
    path, or None, in which case the runner goes on with compute_logits + sampler as before.

    On the fused path: the quantized lm_head of `logits_processor` (a QuantizedLogitsProcessor),
    the fast-path predicate of the sampler hook, no logprobs of any kind (they need the logits), no
    penalties and no speculative tokens.  Soft cap, scale, bias and the vocabulary-padding trim are
    applied like upstream does before sampling."""
    sm = sampling_metadata
    if not hidden_states.is_cuda or not hasattr(logits_processor, "sample_fused"):
        return None
    if not _fast_path_ok(sm):
        return None
    if sm.max_num_logprobs is not None or sm.logprob_token_ids:
        return None
    if not getattr(sm, "no_penalties", True) or getattr(sm, "spec_token_ids", None):
        return None
    if getattr(lm_head, "_vqk_shard", None) is None and hasattr(logits_processor, "_int8_initialized"):
        return None                                   # this lm_head is not quantized: upstream path
    B = hidden_states.reshape(-1, hidden_states.shape[-1]).shape[0]
    if sm.all_greedy:
        sp = SamplingArgs()
    else:
        assert sm.temperature is not None
        sp = SamplingArgs(
            temperature=sm.temperature.to(torch.float32).contiguous(),
            seeds=_make_seeds(B, hidden_states.device) if seeds is None else seeds,
            top_k=None if sm.top_k is None else sm.top_k.to(torch.int32).contiguous(),
            top_p=None if sm.top_p is None else sm.top_p.to(torch.float32).contiguous(),
        )
    try:
        tokens, _ = logits_processor.sample_fused(hidden_states, lm_head, sp, embedding_bias)
    except RuntimeError:
        return None                                   # not quantized / tensor parallel: upstream path
    return tokens


def install_fused_sampler() -> None:
    """Monkey-patch vllm.v1.sample.sampler.Sampler with the fused variant.  Must run
    before `vllm.v1.worker.gpu_model_runner` imports Sampler by name
    (reference: _sampler.py:119-214)."""
    import vllm.v1.sample.sampler as upstream_module

    upstream_sampler = upstream_module.Sampler

    class FusedSampler(upstream_sampler):
        """Drop-in Sampler: temperature + top-k + top-p + Gumbel argmax in CUDA."""

        def sample(
            self,
            logits: torch.Tensor,
            sampling_metadata: "SamplingMetadata",
            logprobs_mode_override: "LogprobsMode | None" = None,
        ) -> "tuple[torch.Tensor, torch.Tensor | None]":
            if not logits.is_cuda or not _fast_path_ok(sampling_metadata):
                return super().sample(logits, sampling_metadata, logprobs_mode_override)

            logprobs_mode = logprobs_mode_override or self.logprobs_mode
            wants_processed_logprobs = (
                (sampling_metadata.max_num_logprobs is not None or sampling_metadata.logprob_token_ids)
                and logprobs_mode in ("processed_logits", "processed_logprobs")
            )
            if wants_processed_logprobs:
                return super().sample(logits, sampling_metadata, logprobs_mode_override)

            if sampling_metadata.all_greedy:
                return logits.argmax(dim=-1).view(-1), None

            assert sampling_metadata.temperature is not None
            B, V = logits.shape
            top_k = sampling_metadata.top_k
            top_p = sampling_metadata.top_p
            sp = SamplingArgs(
                temperature=sampling_metadata.temperature.to(torch.float32).contiguous(),
                seeds=_make_seeds(B, logits.device),
                top_k=None if top_k is None else top_k.to(torch.int32).contiguous(),
                top_p=None if top_p is None else top_p.to(torch.float32).contiguous(),
            )
            sampled, _ = sample_logits(logits, sp)
            return sampled, None

    upstream_module.Sampler = FusedSampler
    print(
        "[vllm-quant-kernels] FusedSampler installed "
        "(vllm.v1.sample.sampler.Sampler patched).",
        file=sys.stderr,
        flush=True,
    )


def env_bool(name: str, default: bool = False) -> bool:
    val = os.environ.get(name, "")
    if val == "":
        return default
    return val.lower() in ("1", "true", "yes", "on")
