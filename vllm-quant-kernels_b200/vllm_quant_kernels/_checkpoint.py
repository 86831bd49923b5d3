"""Persisted quantized lm_head: save the quantized tensors once, load them at the next start.

The reference re-quantizes `lm_head.weight` at every start (src/vllm_quant_kernels/_quant.py:245-380:
a 3 GB fp32 temporary and a pass over the whole weight per start).  Here the result can be
written to a safetensors file in the reference's own storage layouts and read back:

    mode     "q"                                  "scales"
    int8     int8  [V, H]                         fp16 [V]
    w8a8     int8  [V, H]                         fp32 [V]
    fp8      int8  [V, H]  (view of e4m3 bytes)   fp16 [V]
    mxfp8    uint8 [V, H]  (e4m3 bytes)           uint8 [V, H/32]  (E8M0)
    mxfp4    uint8 [V, H/2] (E2M1, even index in  uint8 [V, H/32]  (E8M0)
                             the low nibble)

Metadata carries the mode, V, H, the source dtype and a fingerprint of the source weight (its
bytes sampled on a fixed row grid), so a file made from another weight, another mode or another
shape is refused rather than used.  Switched on by `VLLM_QUANT_LMHEAD_CACHE=<directory>`.
"""

from __future__ import annotations

import hashlib
import os
from typing import Optional, Tuple

import torch

FORMAT = "vqk-lm-head-1"
_DTYPES = {"int8": (torch.int8, torch.float16), "w8a8": (torch.int8, torch.float32), "fp8": (torch.int8, torch.float16),
           "mxfp8": (torch.uint8, torch.uint8), "mxfp4": (torch.uint8, torch.uint8)}


def expected_shapes(mode: str, V: int, H: int) -> Tuple[tuple, tuple]:
    q = (V, H // 2) if mode == "mxfp4" else (V, H)
    s = (V, H // 32) if mode in ("mxfp8", "mxfp4") else (V,)
    return q, s


def weight_fingerprint(w: torch.Tensor, rows: int = 64) -> str:
    """SHA-256 over the shape, dtype and the bytes of `rows` rows on an even grid (first and last
    included).  Cheap (a few hundred KB off the device) and enough to tell two checkpoints apart."""
    V = w.shape[0]
    idx = torch.unique(torch.linspace(0, V - 1, steps=min(rows, V)).round().long())
    sample = w[idx.to(w.device)].contiguous().view(torch.uint8).cpu().numpy().tobytes()
    h = hashlib.sha256()
    h.update(f"{tuple(w.shape)}|{w.dtype}".encode())
    h.update(sample)
    return h.hexdigest()


def cache_path(directory: str, mode: str, fingerprint: str) -> str:
    return os.path.join(directory, f"lm_head_{mode}_{fingerprint[:16]}.safetensors")


def save(path: str, mode: str, q: torch.Tensor, scales: torch.Tensor, H: int, src_dtype: torch.dtype,
         fingerprint: str) -> None:
    from safetensors.torch import save_file
    V = q.shape[0]
    qs, ss = expected_shapes(mode, V, H)
    if tuple(q.shape) != qs or tuple(scales.shape) != ss or (q.dtype, scales.dtype) != _DTYPES[mode]:
        raise ValueError(f"{mode}: tensors do not have the storage layout of this mode")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + f".tmp{os.getpid()}"
    save_file({"q": q.contiguous().cpu(), "scales": scales.contiguous().cpu()}, tmp,
              metadata={"format": FORMAT, "mode": mode, "V": str(V), "H": str(H), "src_dtype": str(src_dtype),
                        "fingerprint": fingerprint})
    os.replace(tmp, path)   # readers never see a half-written file


def load(path: str, mode: str, V: int, H: int, fingerprint: Optional[str], device) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
    """The quantized tensors on `device`, or None when the file is missing or was made from
    something else (mode, shape, weight)."""
    if not os.path.exists(path):
        return None
    from safetensors import safe_open
    try:
        with safe_open(path, framework="pt", device="cpu") as f:
            meta = f.metadata() or {}
            if meta.get("format") != FORMAT or meta.get("mode") != mode:
                return None
            if int(meta.get("V", -1)) != V or int(meta.get("H", -1)) != H:
                return None
            if fingerprint is not None and meta.get("fingerprint") != fingerprint:
                return None
            q, s = f.get_tensor("q"), f.get_tensor("scales")
    except Exception:
        return None
    qs, ss = expected_shapes(mode, V, H)
    if tuple(q.shape) != qs or tuple(s.shape) != ss or (q.dtype, s.dtype) != _DTYPES[mode]:
        return None
    return q.to(device), s.to(device)


def quantize_or_load(mode: str, w: torch.Tensor, quantize):
    """`quantize(mode, w)` unless `VLLM_QUANT_LMHEAD_CACHE` names a directory that already holds
    the result for this weight; a fresh result is written there.  Returns (q, scales, how) with
    how in {"quantized", "loaded", "quantized+saved"}."""
    directory = os.environ.get("VLLM_QUANT_LMHEAD_CACHE", "")
    if not directory:
        q, s = quantize(mode, w)
        return q, s, "quantized"
    V, H = int(w.shape[0]), int(w.shape[1])
    fp = weight_fingerprint(w)
    path = cache_path(directory, mode, fp)
    got = load(path, mode, V, H, fp, w.device)
    if got is not None:
        return got[0], got[1], "loaded"
    q, s = quantize(mode, w)
    try:
        save(path, mode, q, s, H, w.dtype, fp)
        return q, s, "quantized+saved"
    except OSError:
        return q, s, "quantized"
