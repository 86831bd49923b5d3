"""CPU baseline: the reference plugin's torch arithmetic on the host cores.

Test / benchmark infrastructure only (see ``oracle/__init__.py``); never a
fallback.  One "step" is what the reference does per decode step if its device
were the CPU: quantize the activations with the reference formulas, dequantize
the stored weight codes, fp32 matmul, fp16 round, then the UNFUSED sampler
chain the reference replaces (vLLM ``Sampler.sample``:
vllm/v1/sample/sampler.py:238-297 and
vllm/v1/sample/ops/topk_topp_sampler.py:328-416 -- temperature, sort, top-k
mask, softmax/cumsum top-p mask, scatter, softmax, exponential race, argmax).
Weight quantization (one-off in the reference, _quant.py:245-380) is timed
separately.  Uses every host thread torch will give it.
"""

from __future__ import annotations

import os
import time

import torch

GROUP = 32
_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_MID = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def threads() -> int:
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


def _q_mxfp8(t):
    """_quant.py:34-61"""
    R, K = t.shape
    g = t.float().view(R, K // GROUP, GROUP)
    gm = g.abs().amax(-1).clamp(min=1e-30)
    k = torch.ceil(torch.log2(gm / 448.0)).clamp(-127.0, 127.0)
    q = (g / torch.pow(2.0, k).unsqueeze(-1)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(R, K)
    return q, (k + 127.0).to(torch.uint8)


def _q_mxfp4(t):
    """_quant.py:64-105"""
    R, K = t.shape
    g = t.float().view(R, K // GROUP, GROUP)
    gm = g.abs().amax(-1).clamp(min=1e-30)
    k = torch.ceil(torch.log2(gm / 6.0)).clamp(-127.0, 127.0)
    sc = (g / torch.pow(2.0, k).unsqueeze(-1)).view(R, K)
    nib = ((sc < 0).to(torch.uint8) << 3) | torch.bucketize(sc.abs().clamp(max=6.0), _MID).to(torch.uint8)
    return ((nib[:, 1::2] << 4) | nib[:, 0::2]).contiguous(), (k + 127.0).to(torch.uint8)


def quantize_weight(mode: str, w: torch.Tensor):
    """The reference's `_init_*` arithmetic (_quant.py:245-380) on a CPU tensor."""
    if mode in ("int8", "w8a8"):
        s = (w.float().abs().amax(1) / 127.0).clamp(min=1e-12)
        q = (w.float() / s.unsqueeze(1)).round().clamp(-127, 127).to(torch.int8)
        return q, (s.half() if mode == "int8" else s)
    if mode == "fp8":
        s = (w.float().abs().amax(1) / 448.0).clamp(min=1e-12)
        return (w.float() / s.unsqueeze(1)).clamp(-448, 448).to(torch.float8_e4m3fn), s.half()
    if mode == "mxfp8":
        return _q_mxfp8(w)
    if mode == "mxfp4":
        return _q_mxfp4(w)
    raise ValueError(mode)


def _deq_mx8(q, s):
    R, K = q.shape
    return (q.float().view(R, K // GROUP, GROUP) * torch.pow(2.0, s.float() - 127.0).unsqueeze(-1)).view(R, K)


def _deq_mx4(p, s):
    """tests/test_mxfp4_accuracy.py:39-69"""
    R, Kh = p.shape
    nib = torch.stack([p & 0xF, (p >> 4) & 0xF], -1).view(R, Kh * 2)
    mag = _E2M1[(nib & 7).long()]
    v = torch.where(((nib >> 3) & 1).bool(), -mag, mag)
    return (v.view(R, Kh * 2 // GROUP, GROUP) * torch.pow(2.0, s.float() - 127.0).unsqueeze(-1)).view(R, Kh * 2)


def lm_head_step(mode: str, x: torch.Tensor, q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """Activation quantize + dequantize + fp32 matmul + fp16 round (the "dequant matmul"
    reference path; formulas of _quant.py:413,448,495,536-540 and the kernel epilogues
    _kernels.py:77-78,351-357,470-476,627-631,797-801)."""
    x = x.half()
    if mode == "int8":
        out = (x.float() @ q.float().t()) * s.float()[None, :]
    elif mode == "fp8":
        out = (x.to(torch.float8_e4m3fn).float() @ q.float().t()) * s.float()[None, :]
    elif mode == "w8a8":
        xs = (x.float().abs().amax() / 127.0).clamp(min=1e-12)
        xq = (x.float() / xs).round().clamp(-127, 127)
        out = (xq @ q.float().t()) * s[None, :] * xs
    elif mode == "mxfp8":
        xq, xs = _q_mxfp8(x)
        out = _deq_mx8(xq, xs) @ _deq_mx8(q, s).t()
    elif mode == "mxfp4":
        xq, xs = _q_mxfp8(x)
        out = _deq_mx8(xq, xs) @ _deq_mx4(q, s).t()
    else:
        raise ValueError(mode)
    return out.half()


def unfused_sampler_chain(logits_f16, temperature, top_k, top_p):
    """vLLM's chain on CPU: fp32 cast, temperature, sort-based top-k/top-p, softmax,
    exponential race, argmax."""
    l = logits_f16.float()
    V = l.shape[1]
    l = l.div_(temperature.unsqueeze(1))
    ls, li = l.sort(dim=-1, descending=False)
    if top_k is not None:
        kth = ls.gather(1, (V - top_k.long()).unsqueeze(1))
        ls.masked_fill_(ls < kth, -float("inf"))
    if top_p is not None:
        ps = ls.softmax(-1)
        cs = torch.cumsum(ps, -1)
        m = cs <= (1 - top_p.unsqueeze(1))
        m[:, -1] = False
        ls.masked_fill_(m, -float("inf"))
    l = l.scatter_(-1, li, ls)
    p = l.softmax(-1, dtype=torch.float32)
    q = torch.empty_like(p).exponential_()
    return p.div_(q).argmax(-1)


def time_steps(mode, x, q, s, temperature, top_k, top_p, steps: int, warmup: int = 1):
    """Median seconds of one lm_head + unfused-sampler step, and the last tokens."""
    ts = []
    tok = None
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        tok = unfused_sampler_chain(lm_head_step(mode, x, q, s), temperature, top_k, top_p)
        t1 = time.perf_counter()
        if i >= warmup:
            ts.append(t1 - t0)
    ts.sort()
    return ts[len(ts) // 2], tok
