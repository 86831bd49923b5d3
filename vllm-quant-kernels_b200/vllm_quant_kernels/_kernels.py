"""Kernel-level entry points under the reference's names.

The reference's src/vllm_quant_kernels/_kernels.py holds six Triton kernels; here
each name is a plain function over torch tensors that runs the CUDA path in
libvqk.so.  Arguments keep the reference's meaning: `w` quantized rows (M, K),
`x` activations (N, K), `out` fp16 (N, M).
"""

from __future__ import annotations

import torch

from ._lmhead import LMHeadShard

MXFP8_GROUP_SIZE = 32
MXFP4_GROUP_SIZE = 32


def _n_bucket(n: int) -> int:
    """Batch bucket of the reference's autotune key (_kernels.py:87-98); kept for
    callers that pass it along.  The CUDA kernels do not autotune."""
    if n < 4:
        return 0
    if n < 8:
        return 1
    if n < 32:
        return 2
    return 3


def _run(mode, out, w, x, s, K=None):
    shard = LMHeadShard(mode, w, s, K)
    res = shard.logits(x)
    if out is not None:
        out.copy_(res)
        return out
    return res


def int8_gmv(out, w, x, s):
    """W8A16 GEMV/GEMM: out[b, m] = fp16(sum_k w[m,k] x[b,k] * s[m]) (reference _kernels.py:21-84)."""
    return _run("int8", out, w, x, s)


int8_gemm = int8_gmv  # reference _kernels.py:189-248: same math for any batch


def fp8_gemm(out, w, x, s):
    """Per-row FP8: `w` is the int8 view of e4m3 codes, `x` fp16/bf16 activations, cast
    to e4m3 inside (reference _kernels.py:299-358 with the cast of _quant.py:413)."""
    return _run("fp8", out, w, x, s)


def int8_w8a8_gemm(out, w, x, ws):
    """W8A8: per-tensor int8 activation quantisation inside, int32 accumulate
    (reference _kernels.py:412-477, _quant.py:536-540)."""
    return _run("w8a8", out, w, x, ws)


def mxfp8_gemm(out, w, x, ws):
    """MXFP8 block-scaled (reference _kernels.py:534-632); `x` is fp16/bf16 and is
    quantised to e4m3 + E8M0 inside."""
    return _run("mxfp8", out, w, x, ws)


def mxfp4_gemm(out, w, x, ws, K=None):
    """MXFP4 W4A8 (reference _kernels.py:701-802); `w` packed two E2M1 per byte."""
    return _run("mxfp4", out, w, x, ws, K)


def _make_thor_gemm_kernel():
    return int8_gemm, _n_bucket


def _make_thor_fp8_gemm_kernel():
    return fp8_gemm, _n_bucket


def _make_thor_w8a8_gemm_kernel():
    return int8_w8a8_gemm, _n_bucket


def _make_thor_mxfp8_gemm_kernel():
    return mxfp8_gemm, _n_bucket


def _make_thor_mxfp4_gemm_kernel():
    return mxfp4_gemm, _n_bucket
