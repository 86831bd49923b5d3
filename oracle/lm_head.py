"""Oracle: quantized lm_head logits, dequantise-then-fp32-matmul.

Test infrastructure only (see ``oracle/__init__.py``).

``logits[b, v] = sum_k X[b, k] * Wq[v, k]`` with each mode's epilogue, output
rounded to fp16 as every reference launcher does
(src/vllm_quant_kernels/_quant.py:409,445,492,533,570).  The accumulation
order over K is implementation-defined in the reference (Triton ``tl.dot`` /
``tl.sum``); the parity gate on logits is therefore rel-L2 <= 1e-3, and fp16
output rounding alone contributes about 2e-4.
"""

from __future__ import annotations

import numpy as np

from . import quant as Q

F32 = np.float32
MODES = ("int8", "w8a8", "fp8", "mxfp8", "mxfp4")


def quantize_weight(mode: str, w):
    """Offline weight quantisation in the reference's storage layout for ``mode``.
    Returns (codes, scales)."""
    if mode == "int8":
        return Q.quantize_int8_rows(w, np.float16)      # _quant.py:248-255
    if mode == "w8a8":
        return Q.quantize_int8_rows(w, np.float32)      # _quant.py:285-292
    if mode == "fp8":
        return Q.quantize_fp8_rows(w)                   # _quant.py:306-314
    if mode == "mxfp8":
        return Q.quantize_mxfp8(w)                      # _quant.py:326-328
    if mode == "mxfp4":
        return Q.quantize_mxfp4(w)                      # _quant.py:356-359
    raise ValueError(mode)


def _to_f16_act(x):
    """Activations are used as fp16 (bf16 inputs are converted first,
    _quant.py:579 ``x.to(torch.float16)``; _kernels.py:236)."""
    return np.asarray(x).astype(np.float16)


def quantize_act(mode: str, x):
    """Runtime activation quantisation for ``mode``; returns (xq, xs) where xs is
    None (int8/fp8), a float32 scalar (w8a8) or E8M0 bytes (mx modes)."""
    if mode == "int8":
        return _to_f16_act(x), None
    if mode == "fp8":
        return Q.act_quant_fp8(x), None                 # _quant.py:413
    if mode == "w8a8":
        return Q.act_quant_int8_tensor(x)               # _quant.py:536-540
    if mode in ("mxfp8", "mxfp4"):
        return Q.act_quant_mxfp8(x)                     # _quant.py:448,495
    raise ValueError(mode)


def _matmul(a, b_t, acc):
    """a [B,K] times b_t[V,K]^T, accumulating in ``acc`` dtype, result fp32."""
    return (a.astype(acc) @ b_t.astype(acc).T).astype(F32)


def logits_fp32(mode: str, x, wq, ws, acc=np.float32, row_chunk: int = 16384):
    """fp32 logits BEFORE the final fp16 rounding (for error analysis)."""
    xq, xs = quantize_act(mode, x)
    V = wq.shape[0]
    B = xq.shape[0]
    out = np.empty((B, V), dtype=F32)
    if mode == "int8":
        xa = xq.astype(F32)
    elif mode == "fp8":
        xa = Q.e4m3_decode(xq)
    elif mode == "w8a8":
        xa = xq.astype(np.float64)
    else:
        xa = Q.dequant_mxfp8(xq, xs)
    for r0 in range(0, V, row_chunk):
        r1 = min(V, r0 + row_chunk)
        w = wq[r0:r1]
        s = ws[r0:r1]
        if mode == "int8":
            # _kernels.py:77-78 / 241-247: fp32 acc times fp32(fp16 scale)
            a = _matmul(xa, w.astype(F32), acc)
            out[:, r0:r1] = a * s.astype(F32)[None, :]
        elif mode == "fp8":
            # _kernels.py:351-357
            a = _matmul(xa, Q.e4m3_decode(w.view(np.uint8)), acc)
            out[:, r0:r1] = a * s.astype(F32)[None, :]
        elif mode == "w8a8":
            # _kernels.py:470-471: int32 exact, then fp32(acc) * ws * xs, left to right
            a = (xa @ w.astype(np.float64).T)
            a = a.astype(F32)
            out[:, r0:r1] = (a * s.astype(F32)[None, :]).astype(F32) * F32(xs)
        elif mode == "mxfp8":
            # _kernels.py:616-631
            out[:, r0:r1] = _matmul(xa, Q.dequant_mxfp8(w, s), acc)
        elif mode == "mxfp4":
            # _kernels.py:786-801; tests/test_mxfp4_kernel.py:57-77
            out[:, r0:r1] = _matmul(xa, Q.dequant_mxfp4(w, s), acc)
        else:
            raise ValueError(mode)
    return out


def logits(mode: str, x, wq, ws, bias=None, acc=np.float32):
    """fp16 logits as the reference launchers return them, bias added in fp16
    (_quant.py:428-429)."""
    out = logits_fp32(mode, x, wq, ws, acc=acc).astype(np.float16)
    if bias is not None:
        out = (out.astype(F32) + np.asarray(bias).astype(np.float16).astype(F32)[None, :]).astype(np.float16)
    return out


def rel_l2(a, b) -> float:
    """||a - b|| / ||b|| over the entries finite in both; returns inf if the
    non-finite patterns (inf sign, NaN positions) differ."""
    a = np.asarray(a).astype(np.float64)
    b = np.asarray(b).astype(np.float64)
    fa, fb = np.isfinite(a), np.isfinite(b)
    if (fa != fb).any():
        return float("inf")
    bad = ~fa
    if bad.any() and not ((np.isnan(a[bad]) == np.isnan(b[bad])).all()
                          and (a[bad][~np.isnan(a[bad])] == b[bad][~np.isnan(b[bad])]).all()):
        return float("inf")
    return float(np.linalg.norm(a[fa] - b[fa]) / max(np.linalg.norm(b[fa]), 1e-30))


# --------------------------------------------------------------------------
# Synthetic inputs standing in for the Qwen3.5-122B lm_head tensor the
# reference measured on (README.md:58: row absmax varies about 6x, abs max 0.19,
# p99.9 about 0.057)
# --------------------------------------------------------------------------

SPREAD_STD_LO = 0.0072   # fitted so the pooled p99.9(|w|) is about 0.057


def synth_weight_rows(r0: int, r1: int, H: int, seed: int = 0) -> np.ndarray:
    """Rows [r0, r1) of the synthetic weight: per-row std log-uniform in
    [a, 6a], N(0, std), clipped to +-0.19, fp16.  Row-addressable so any shard
    or chunk is reproducible without generating the whole matrix."""
    out = np.empty((r1 - r0, H), dtype=np.float16)
    CH = 4096
    for c0 in range((r0 // CH) * CH, r1, CH):
        rng = np.random.default_rng([seed, c0 // CH])
        std = np.exp(rng.uniform(np.log(SPREAD_STD_LO), np.log(6 * SPREAD_STD_LO), size=CH)).astype(F32)
        blk = rng.standard_normal((CH, H), dtype=F32) * std[:, None]
        np.clip(blk, -0.19, 0.19, out=blk)
        lo = max(r0, c0)
        hi = min(r1, c0 + CH)
        out[lo - r0:hi - r0] = blk[lo - c0:hi - c0].astype(np.float16)
    return out


def synth_act(B: int, H: int, seed: int = 0xC0DE) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.standard_normal((B, H), dtype=F32).astype(np.float16)
