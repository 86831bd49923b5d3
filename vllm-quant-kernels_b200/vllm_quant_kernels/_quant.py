"""Quantized LogitsProcessor for vLLM, B200 build.

Same class, method and attribute names as the reference plugin's
src/vllm_quant_kernels/_quant.py, so code and tests written against it keep
working: lazy one-time quantisation of `lm_head.weight` on the first call, state
stashed on the `lm_head` module (`_int8_w/_int8_scales`, `_w8a8_w/_w8a8_scales`,
`_fp8_w/_fp8_scales`, `_mxfp8_w/_mxfp8_w_scales`, `_mxfp4_w/_mxfp4_w_scales/_mxfp4_K`),
mode chosen by the `VLLM_USE_*_LMHEAD` variables in MXFP4 > MXFP8 > FP8 > W8A8 > INT8
order, fp16 logits out.  Every kernel is CUDA in libvqk.so; there is no Triton and
no non-sm_100 path: on another GPU the layer leaves the weight alone and defers to
upstream vLLM.
"""

import os
import sys
from typing import Optional

import torch

from vllm.model_executor.custom_op import PluggableLayer
from vllm.model_executor.layers.logits_processor import LogitsProcessor
from vllm.model_executor.layers.vocab_parallel_embedding import (
    VocabParallelEmbedding,
)

from . import _checkpoint, _lmhead
from ._kernels import MXFP4_GROUP_SIZE, MXFP8_GROUP_SIZE

_QUANT_ATTRS = ("_mxfp4_w", "_mxfp8_w", "_fp8_w", "_w8a8_w", "_int8_w")


def _quantize_to_mxfp8(t: torch.Tensor, group_size: int = MXFP8_GROUP_SIZE):
    """(R, K) fp32/fp16/bf16 -> (uint8 e4m3 view (R, K), uint8 E8M0 scales (R, K // 32)).
    Reference: _quant.py:34-61, bit-exact."""
    R, K = t.shape
    assert group_size == MXFP8_GROUP_SIZE, "only the OCP MX group size 32 is implemented"
    assert K % group_size == 0, f"K={K} must be divisible by group_size={group_size}"
    return _lmhead.quantize_weight("mxfp8", t)


def _quantize_to_mxfp4(t: torch.Tensor, group_size: int = MXFP4_GROUP_SIZE):
    """(R, K) -> (uint8 (R, K // 2) two E2M1 nibbles per byte, even index in the low
    nibble; uint8 E8M0 scales (R, K // 32)).  Reference: _quant.py:64-105, bit-exact."""
    R, K = t.shape
    assert group_size == MXFP4_GROUP_SIZE, "only the OCP MX group size 32 is implemented"
    assert K % group_size == 0, f"K={K} must be divisible by group_size={group_size}"
    assert K % 2 == 0, f"K={K} must be even (FP4 packing)"
    return _lmhead.quantize_weight("mxfp4", t.detach())


def _tp_world_size() -> int:
    try:
        from vllm.distributed import get_tensor_model_parallel_world_size
        return get_tensor_model_parallel_world_size()
    except Exception:
        return 1


@PluggableLayer.register_oot(name="LogitsProcessor")
class QuantizedLogitsProcessor(LogitsProcessor):
    """vLLM LogitsProcessor with a quantized lm_head matmul (reference: _quant.py:108-643)."""

    _VOCAB_THRESHOLD = 100_000

    def forward(self, lm_head, hidden_states, embedding_bias=None):
        """Upstream's forward (vllm logits_processor.py:54-73) with its post-ops - soft cap and scale,
        three to four extra passes over [B, V] there - folded into the lm_head epilogue when the
        quantized path runs.  Same values: the epilogue rounds to fp16 where upstream's tensor ops do."""
        if getattr(self, "logits_as_input", False):
            return super().forward(lm_head, hidden_states, embedding_bias)
        if not hasattr(self, "_int8_initialized"):
            self._int8_initialized = True
            self._init_int8(lm_head)
        shard = getattr(lm_head, "_vqk_shard", None)
        soft_cap, scale = getattr(self, "soft_cap", None), getattr(self, "scale", 1.0)
        if shard is None or (soft_cap is None and scale == 1.0):
            return super().forward(lm_head, hidden_states, embedding_bias)
        shard.set_post_ops(soft_cap, scale)
        try:
            return self._get_logits(hidden_states, lm_head, embedding_bias)
        finally:
            shard.set_post_ops(None, 1.0)   # direct _quantized_forward calls keep returning raw logits

    def _get_logits(
        self,
        hidden_states: torch.Tensor,
        lm_head: VocabParallelEmbedding,
        embedding_bias: Optional[torch.Tensor],
        *args,
        **kwargs,
    ) -> Optional[torch.Tensor]:
        # vLLM 0.22 passes three arguments, the reference declared a fourth
        # (`skip_gather`); whatever was given is forwarded to upstream unchanged.
        if not hasattr(self, "_int8_initialized"):
            self._int8_initialized = True
            self._init_int8(lm_head)

        if not any(hasattr(lm_head, a) for a in _QUANT_ATTRS):
            return super()._get_logits(hidden_states, lm_head, embedding_bias, *args, **kwargs)

        logits = self._quantized_forward(hidden_states, lm_head, embedding_bias)
        # Upstream gathers the vocab shards and trims vocabulary padding after the
        # matmul (vllm logits_processor.py:96-104); the reference skipped both.
        if _tp_world_size() > 1 and not kwargs.get("skip_gather", False):
            logits = self._gather_logits(logits)
        org = getattr(self, "org_vocab_size", None)
        if logits is not None and org is not None and org < logits.shape[-1]:
            logits = logits[..., :org]
        return logits

    # ------------------------------------------------------------------ init
    def _init_int8(self, lm_head: VocabParallelEmbedding) -> None:
        """Quantize lm_head.weight if applicable (reference: _quant.py:143-243)."""
        w = lm_head.weight.data
        if w.dtype not in (torch.bfloat16, torch.float16):
            return
        if w.shape[0] <= self._VOCAB_THRESHOLD:
            return

        cap = torch.cuda.get_device_capability(w.device)
        is_b200 = cap[0] == 10

        def _env_bool(name):
            return os.environ.get(name, "").lower() in ("1", "true", "yes", "on")

        def _say(msg):
            print(f"[vllm-quant-kernels] {msg}", file=sys.stderr, flush=True)

        if not is_b200:
            _say(f"quantized lm_head requires an sm_100 GPU (B200), found sm_{cap[0]}{cap[1]}; "
                 "leaving lm_head unquantized (upstream path)")
            return

        K = w.shape[1]
        if _env_bool("VLLM_USE_MXFP4_LMHEAD"):
            if K % MXFP4_GROUP_SIZE != 0:
                _say(f"VLLM_USE_MXFP4_LMHEAD requires K divisible by {MXFP4_GROUP_SIZE} (got K={K}), "
                     "falling back to int8")
            elif K % 2 != 0:
                _say(f"VLLM_USE_MXFP4_LMHEAD requires even K (got K={K}), falling back to int8")
            else:
                self._init_mxfp4(lm_head, w, sys)
                return
        if _env_bool("VLLM_USE_MXFP8_LMHEAD"):
            if K % MXFP8_GROUP_SIZE != 0:
                _say(f"VLLM_USE_MXFP8_LMHEAD requires K divisible by {MXFP8_GROUP_SIZE} (got K={K}), "
                     "falling back to int8")
            else:
                self._init_mxfp8(lm_head, w, sys)
                return
        if K % 16 != 0:
            _say(f"quantized lm_head requires K divisible by 16 (got K={K}); leaving lm_head unquantized")
            return
        if _env_bool("VLLM_USE_FP8_LMHEAD"):
            self._init_fp8(lm_head, w, sys)
            return
        if _env_bool("VLLM_USE_W8A8_LMHEAD"):
            self._init_w8a8(lm_head, w, sys)
            return
        self._init_int8_weights(lm_head, w, sys, True)

    @staticmethod
    def _banner(_sys, text):
        print(f"[vllm-quant-kernels] lm_head quantized: {text}", file=_sys.stderr, flush=True)

    @staticmethod
    def _quantize(mode, w):
        """Quantized codes and scales of `w`: computed, or read back from the directory
        `VLLM_QUANT_LMHEAD_CACHE` names when it holds them for this very weight (_checkpoint.py)."""
        q, s, how = _checkpoint.quantize_or_load(mode, w, _lmhead.quantize_weight)
        if how != "quantized":
            print(f"[vllm-quant-kernels] lm_head {mode}: {how} ({os.environ.get('VLLM_QUANT_LMHEAD_CACHE')})",
                  file=sys.stderr, flush=True)
        return q, s

    def _init_int8_weights(self, lm_head, w, _sys, is_thor: bool = True) -> None:
        """Per-row INT8 + fp16 scale (reference: _quant.py:245-273).  The original weight
        is kept: with tied embeddings it is the embedding table."""
        lm_head._int8_use_thor = True
        lm_head._int8_w, lm_head._int8_scales = self._quantize("int8", w)
        lm_head._vqk_shard = _lmhead.LMHeadShard("int8", lm_head._int8_w, lm_head._int8_scales)
        saved_mb = w.numel() * w.element_size() // 1024 // 1024
        self._banner(_sys, f"fp16 {w.shape[0]}×{w.shape[1]} → int8 (saved {saved_mb} MB, kernel=b200/int8)")

    def _init_w8a8(self, lm_head, w, _sys) -> None:
        """Per-row INT8 + fp32 scale; activations per-tensor INT8 at run time (reference: _quant.py:278-304)."""
        lm_head._w8a8_w, lm_head._w8a8_scales = self._quantize("w8a8", w)
        lm_head._vqk_shard = _lmhead.LMHeadShard("w8a8", lm_head._w8a8_w, lm_head._w8a8_scales)
        saved_mb = w.numel() * w.element_size() // 1024 // 1024
        self._banner(_sys, f"fp16 {w.shape[0]}×{w.shape[1]} → int8 w8a8 (saved {saved_mb} MB, kernel=b200/w8a8)")

    def _init_fp8(self, lm_head, w, _sys) -> None:
        """Per-row FP8 e4m3 stored as an int8 view + fp16 scale (reference: _quant.py:306-327)."""
        lm_head._fp8_w, lm_head._fp8_scales = self._quantize("fp8", w)
        lm_head._vqk_shard = _lmhead.LMHeadShard("fp8", lm_head._fp8_w, lm_head._fp8_scales)
        saved_mb = w.numel() * w.element_size() // 1024 // 1024
        self._banner(_sys, f"fp16 {w.shape[0]}×{w.shape[1]} → fp8e4m3 (saved {saved_mb} MB, kernel=b200/fp8)")

    def _init_mxfp8(self, lm_head, w, _sys) -> None:
        """e4m3 + E8M0 per 32 (reference: _quant.py:329-352)."""
        lm_head._mxfp8_w, lm_head._mxfp8_w_scales = self._quantize("mxfp8", w)
        lm_head._vqk_shard = _lmhead.LMHeadShard("mxfp8", lm_head._mxfp8_w, lm_head._mxfp8_w_scales)
        saved_mb = w.numel() * w.element_size() // 1024 // 1024
        scale_mb = lm_head._mxfp8_w_scales.numel() // 1024 // 1024
        self._banner(_sys, f"fp16 {w.shape[0]}×{w.shape[1]} → mxfp8 e4m3 "
                           f"(saved {saved_mb} MB, scales {scale_mb} MB, kernel=b200/mxfp8)")

    def _init_mxfp4(self, lm_head, w, _sys) -> None:
        """E2M1 packed two per byte + E8M0 per 32; W4A8 at run time (reference: _quant.py:354-380)."""
        lm_head._mxfp4_w, lm_head._mxfp4_w_scales = self._quantize("mxfp4", w.detach())
        lm_head._mxfp4_K = int(w.shape[1])
        lm_head._vqk_shard = _lmhead.LMHeadShard("mxfp4", lm_head._mxfp4_w, lm_head._mxfp4_w_scales, lm_head._mxfp4_K)
        orig_mb = w.numel() * w.element_size() // 1024 // 1024
        new_mb = (lm_head._mxfp4_w.numel() + lm_head._mxfp4_w_scales.numel()) // 1024 // 1024
        self._banner(_sys, f"fp16 {w.shape[0]}×{w.shape[1]} → mxfp4 e2m1 ({orig_mb} MB → {new_mb} MB, kernel=b200/mxfp4)")

    # --------------------------------------------------------------- forward
    @staticmethod
    def _shard(lm_head, mode, w_attr, s_attr, K=None):
        """The descriptor made at init, or one built on the fly for callers that set the
        quantized tensors on `lm_head` themselves (as the reference's tests do)."""
        sh = getattr(lm_head, "_vqk_shard", None)
        w = getattr(lm_head, w_attr)
        if sh is None or sh.mode != mode or sh.q.data_ptr() != w.data_ptr():
            sh = _lmhead.LMHeadShard(mode, w, getattr(lm_head, s_attr), K)
            lm_head._vqk_shard = sh
        return sh

    def _run(self, shard, hidden_states, embedding_bias):
        out = shard.logits(hidden_states, embedding_bias)
        return out.view(hidden_states.shape[:-1] + (shard.V,))

    def _quantized_forward(self, hidden_states, lm_head, embedding_bias) -> torch.Tensor:
        """Dispatch in priority order (reference: _quant.py:382-397)."""
        if hasattr(lm_head, "_mxfp4_w"):
            return self._mxfp4_forward(hidden_states, lm_head, embedding_bias)
        if hasattr(lm_head, "_mxfp8_w"):
            return self._mxfp8_forward(hidden_states, lm_head, embedding_bias)
        if hasattr(lm_head, "_fp8_w"):
            return self._fp8_forward(hidden_states, lm_head, embedding_bias)
        if hasattr(lm_head, "_w8a8_w"):
            return self._w8a8_forward(hidden_states, lm_head, embedding_bias)
        return self._int8_forward(hidden_states, lm_head, embedding_bias)

    def _fp8_forward(self, hidden_states, lm_head, embedding_bias) -> torch.Tensor:
        return self._run(self._shard(lm_head, "fp8", "_fp8_w", "_fp8_scales"), hidden_states, embedding_bias)

    def _mxfp8_forward(self, hidden_states, lm_head, embedding_bias) -> torch.Tensor:
        return self._run(self._shard(lm_head, "mxfp8", "_mxfp8_w", "_mxfp8_w_scales"), hidden_states, embedding_bias)

    def _mxfp4_forward(self, hidden_states, lm_head, embedding_bias=None) -> torch.Tensor:
        return self._run(self._shard(lm_head, "mxfp4", "_mxfp4_w", "_mxfp4_w_scales", lm_head._mxfp4_K),
                         hidden_states, embedding_bias)

    def _w8a8_forward(self, hidden_states, lm_head, embedding_bias) -> torch.Tensor:
        return self._run(self._shard(lm_head, "w8a8", "_w8a8_w", "_w8a8_scales"), hidden_states, embedding_bias)

    def _int8_forward(self, hidden_states, lm_head, embedding_bias) -> torch.Tensor:
        return self._run(self._shard(lm_head, "int8", "_int8_w", "_int8_scales"), hidden_states, embedding_bias)

    # ------------------------------------------------------- fused extension
    def sample_fused(self, hidden_states, lm_head, sampling_args: "_lmhead.SamplingArgs", embedding_bias=None):
        """lm_head and sampler in one pass: (tokens int64 [B], scores fp32 [B]); the
        logits are never written to memory unless a row needs top-k / top-p.  Not part
        of the reference's surface; vLLM's runner reaches it only if it is patched to.

        Samples over the first `org_vocab_size` rows only (vLLM pads the vocabulary; a padding
        row quantizes to zero and could otherwise win when the real logits are negative).
        Single shard: with tensor parallelism the vocab shards of the ranks have to be merged,
        which is `_dist.VocabShardedLMHead`'s job, so TP > 1 raises here."""
        if not hasattr(self, "_int8_initialized"):
            self._int8_initialized = True
            self._init_int8(lm_head)
        sh = getattr(lm_head, "_vqk_shard", None)
        if sh is None:
            raise RuntimeError("lm_head is not quantized (see the eligibility rules of _init_int8)")
        if _tp_world_size() > 1:
            raise RuntimeError("sample_fused samples one vocab shard; with tensor parallelism use "
                               "vllm_quant_kernels._dist.VocabShardedLMHead with this rank's vocab_start")
        org = getattr(self, "org_vocab_size", None)
        if org is not None and 0 < org < sh.V:
            fs = getattr(lm_head, "_vqk_fused_shard", None)
            if fs is None or fs.V != org or fs.q.data_ptr() != sh.q.data_ptr():
                fs = _lmhead.LMHeadShard(sh.mode, sh.q[:org], sh.scales[:org], sh.H)
                lm_head._vqk_fused_shard = fs
            sh = fs
        if embedding_bias is not None and embedding_bias.shape[-1] > sh.V:
            embedding_bias = embedding_bias[..., :sh.V]
        # the distribution vLLM samples from is the one after its post-ops (soft cap, scale)
        sh.set_post_ops(getattr(self, "soft_cap", None), getattr(self, "scale", 1.0))
        try:
            return sh.sample(hidden_states, sampling_args, embedding_bias)
        finally:
            sh.set_post_ops(None, 1.0)
