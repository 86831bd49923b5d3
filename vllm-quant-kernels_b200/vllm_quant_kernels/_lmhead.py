"""Host side of the quantized lm_head + fused sampler, free of any vLLM import.

Thin: shape checks, output allocation through torch, and one C-ABI call per
operation on the current CUDA stream.  `_quant.py` / `_sampler.py` wrap these in
the reference plugin's vLLM classes.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _ffi

MODES = {"int8": _ffi.MODE_W8A16, "w8a8": _ffi.MODE_W8A8, "fp8": _ffi.MODE_FP8,
         "mxfp8": _ffi.MODE_MXFP8, "mxfp4": _ffi.MODE_MXFP4}
GROUP = 32

_DT = {torch.float16: _ffi.F16, torch.bfloat16: _ffi.BF16, torch.float32: _ffi.F32}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: these operators have no CPU path")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# --------------------------------------------------------------------------
# quantizers
# --------------------------------------------------------------------------

def quantize_weight(mode: str, w: torch.Tensor):
    """Offline weight quantisation in the reference's storage layouts
    (reference: _quant.py:245-380).  Returns (codes, scales):
    int8 -> int8 [V,H] + fp16 [V]; w8a8 -> int8 + fp32; fp8 -> int8 view of e4m3
    + fp16; mxfp8 -> uint8 [V,H] + uint8 [V,H/32]; mxfp4 -> uint8 [V,H/2] + uint8 [V,H/32]."""
    _require_cuda(w, "weight")
    assert w.dim() == 2 and w.dtype in _DT
    if w.stride(1) != 1:
        w = w.contiguous()
    V, H = w.shape
    m = MODES[mode]
    dev = w.device
    if mode in ("mxfp8", "mxfp4"):
        assert H % GROUP == 0, f"K={H} must be divisible by group_size={GROUP}"
    if mode == "mxfp4":
        q = torch.empty(V, H // 2, dtype=torch.uint8, device=dev)
    elif mode == "mxfp8":
        q = torch.empty(V, H, dtype=torch.uint8, device=dev)
    else:
        q = torch.empty(V, H, dtype=torch.int8, device=dev)
    if mode in ("int8", "fp8"):
        s = torch.empty(V, dtype=torch.float16, device=dev)
    elif mode == "w8a8":
        s = torch.empty(V, dtype=torch.float32, device=dev)
    else:
        s = torch.empty(V, H // GROUP, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _ffi.check(_ffi.lib().vqk_quantize_weight(m, w.data_ptr(), _DT[w.dtype], V, H, w.stride(0),
                                                  q.data_ptr(), s.data_ptr(), _stream(w)))
    return q, s


def quantize_act(mode: str, x: torch.Tensor):
    """Runtime activation quantisation (reference: _quant.py:413,448,495,536-540).
    Returns (xq, xs); xs is None (int8, fp8), a 1-element fp32 device tensor (w8a8,
    no host sync) or uint8 [B, H/32] (mx modes)."""
    _require_cuda(x, "activations")
    assert x.dim() == 2 and x.dtype in _DT
    if x.stride(1) != 1:
        x = x.contiguous()
    B, H = x.shape
    dev = x.device
    xs_ret = None
    if mode == "int8":
        xq = torch.empty(B, H, dtype=torch.float16, device=dev)
        xs = None
    elif mode == "fp8":
        xq = torch.empty(B, H, dtype=torch.uint8, device=dev)
        xs = None
    elif mode == "w8a8":
        xq = torch.empty(B, H, dtype=torch.int8, device=dev)
        xs = torch.empty(2, dtype=torch.float32, device=dev)
        xs_ret = xs[:1]
    else:
        xq = torch.empty(B, H, dtype=torch.uint8, device=dev)
        xs = torch.empty(B, H // GROUP, dtype=torch.uint8, device=dev)
        xs_ret = xs
    with torch.cuda.device(dev):
        _ffi.check(_ffi.lib().vqk_quantize_act(MODES[mode], x.data_ptr(), _DT[x.dtype], B, H, x.stride(0),
                                               xq.data_ptr(), _ptr(xs), _stream(x)))
    return xq, xs_ret


# --------------------------------------------------------------------------
# sampling arguments
# --------------------------------------------------------------------------

@dataclass
class SamplingArgs:
    """Per-row sampling controls, all device tensors of length B (or None).
    Semantics: include/vqk.h `vqk_sample_params`."""
    temperature: Optional[torch.Tensor] = None      # fp32; None -> argmax for every row
    seeds: Optional[torch.Tensor] = None            # int32
    top_k: Optional[torch.Tensor] = None            # int32; <=0 or >=vocab disables
    top_p: Optional[torch.Tensor] = None            # fp32; >=1 disables
    topk_threshold: Optional[torch.Tensor] = None   # fp32 raw-logit threshold (reference style)
    vocab_offset: int = 0
    vocab_total: Optional[int] = None

    def to_c(self, B: int, V_local: int) -> _ffi.SampleParams:
        def chk(t, dt, name):
            if t is None:
                return None
            if t.dtype != dt or t.shape != (B,) or not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous CUDA {dt} tensor of shape ({B},)")
            return t.data_ptr()
        total = V_local if self.vocab_total is None else int(self.vocab_total)
        return _ffi.SampleParams(
            chk(self.temperature, torch.float32, "temperature"), chk(self.seeds, torch.int32, "seeds"),
            chk(self.top_k, torch.int32, "top_k"), chk(self.top_p, torch.float32, "top_p"),
            chk(self.topk_threshold, torch.float32, "topk_threshold"), int(self.vocab_offset), total)


class _Workspace:
    """Scratch buffers per device (one instance per lm_head shard, one for the stand-alone
    sampler entry points).  A buffer that was
    handed out is never freed or replaced (a CUDA graph captured earlier keeps its raw pointer):
    a larger request adds a buffer, a smaller one reuses the smallest that fits.  Calls that share
    a buffer must run on one stream."""

    def __init__(self):
        self._bufs = {}

    def get(self, dev: torch.device, nbytes: int) -> torch.Tensor:
        key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
        bufs = self._bufs.setdefault(key, [])
        fit = [b for b in bufs if b.numel() >= nbytes]
        if fit:
            return min(fit, key=lambda b: b.numel())
        # grow geometrically: a run of ever larger requests then holds at most twice the largest
        largest = max((b.numel() for b in bufs), default=0)
        b = torch.empty(max(nbytes, 2 * largest, 1), dtype=torch.uint8, device=dev)
        bufs.append(b)
        return b


_WS = _Workspace()


# --------------------------------------------------------------------------
# lm_head shard
# --------------------------------------------------------------------------

class LMHeadShard:
    """Quantized rows [V, H] of one vocab shard plus the vqk_lm_head descriptor.
    Keeps the tensors alive; holds no other device memory."""

    def __init__(self, mode: str, q: torch.Tensor, scales: torch.Tensor, K: Optional[int] = None):
        _require_cuda(q, "quantized weight")
        assert q.is_contiguous() and scales.is_contiguous()
        self.mode = mode
        self.q = q
        self.scales = scales
        self.V = q.shape[0]
        self.H = int(K) if K is not None else (q.shape[1] * 2 if mode == "mxfp4" else q.shape[1])
        self.device = q.device
        self._dev_index = q.device.index if q.device.index is not None else torch.cuda.current_device()
        self._ws_bytes = {}
        self._wsp = _Workspace()  # this shard's own scratch, kept for the shard's lifetime
        h = ctypes.c_void_p()
        _ffi.check(_ffi.lib().vqk_lm_head_create(MODES[mode], q.data_ptr(), scales.data_ptr(), self.V, self.H,
                                                 ctypes.byref(h)))
        self._h = h

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _ffi.lib().vqk_lm_head_destroy(h)
            except Exception:
                pass
            self._h = None

    def set_kernel_events(self, start: Optional["torch.cuda.Event"], stop: Optional["torch.cuda.Event"]) -> None:
        """Measurement aid: record these CUDA events around the weight-streaming kernel of
        every following call (None, None switches it off).  The events must have been
        recorded once so that torch has created their handles."""
        a = None if start is None else start.cuda_event
        b = None if stop is None else stop.cuda_event
        _ffi.check(_ffi.lib().vqk_lm_head_set_kernel_events(self._h, a, b))

    def set_post_ops(self, soft_cap: Optional[float] = None, scale: float = 1.0) -> None:
        """vLLM's logits post-ops (soft cap, then scale) applied in the lm_head epilogue of every
        following call on this shard, with upstream's fp16 roundings; (None, 1.0) switches them off."""
        _ffi.check(_ffi.lib().vqk_lm_head_set_post_ops(self._h, float(soft_cap) if soft_cap else 0.0, float(scale)))

    def _x2d(self, x: torch.Tensor) -> torch.Tensor:
        _require_cuda(x, "hidden_states")
        x = x.reshape(-1, self.H)
        if x.dtype not in (torch.float16, torch.bfloat16):
            x = x.to(torch.float16)
        if x.stride(1) != 1:
            x = x.contiguous()
        return x

    def _ws(self, B: int, sample: bool):
        """Scratch of this shard for batch B.  Every shard owns its buffers and never frees one
        it handed out, so a step captured in a CUDA graph never sees its scratch replaced by a
        later, larger call, and two shards never share scratch.  Calls on ONE shard share
        buffers: keep them on one stream."""
        key = (B, sample)
        n = self._ws_bytes.get(key)
        if n is None:  # the size depends on (B, sample) only: ask the library once
            with torch.cuda.device(self.device):
                n = int(_ffi.lib().vqk_lm_head_workspace_bytes(self._h, B, 1 if sample else 0))
            if n < 0:
                _ffi.check(n)
            self._ws_bytes[key] = n
        return self._wsp.get(self.device, n), n

    def _forward(self, x, bias, logits, sp, tokens, scores, records):
        B = x.shape[0]
        ws, n = self._ws(B, sp is not None)
        spc = sp.to_c(B, self.V) if sp is not None else None

        def call():
            _ffi.check(_ffi.lib().vqk_lm_head_forward(
                self._h, x.data_ptr(), _DT[x.dtype], B, x.stride(0), _ptr(bias),
                _ptr(logits), logits.stride(0) if logits is not None else 0,
                ctypes.byref(spc) if spc is not None else None,
                _ptr(tokens), _ptr(scores), _ptr(records), ws.data_ptr(), n, _stream(x)))

        if torch.cuda.current_device() == self._dev_index:  # decode loop: no device switch to pay for
            call()
        else:
            with torch.cuda.device(self.device):
                call()

    def logits(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp16 logits [B, V] (reference: every `_*_forward` launcher, _quant.py:399-643)."""
        x2 = self._x2d(x)
        out = torch.empty(x2.shape[0], self.V, dtype=torch.float16, device=self.device)
        if bias is not None:
            bias = bias.to(torch.float16).contiguous()
        if x2.shape[0]:
            self._forward(x2, bias, out, None, None, None, None)
        return out

    def sample(self, x: torch.Tensor, sp: SamplingArgs, bias: Optional[torch.Tensor] = None,
               return_logits: bool = False):
        """lm_head + sampler in one pass: int64 tokens [B], fp32 winning scores [B]
        (and the fp16 logits if asked).  Single shard only."""
        x2 = self._x2d(x)
        B = x2.shape[0]
        tokens = torch.empty(B, dtype=torch.int64, device=self.device)
        scores = torch.empty(B, dtype=torch.float32, device=self.device)
        out = torch.empty(B, self.V, dtype=torch.float16, device=self.device) if return_logits else None
        if bias is not None:
            bias = bias.to(torch.float16).contiguous()
        if B:
            self._forward(x2, bias, out, sp, tokens, scores, None)
        return (tokens, scores, out) if return_logits else (tokens, scores)

    def step_sharded(self, x: torch.Tensor, sp: SamplingArgs, peer_handle, bias: Optional[torch.Tensor] = None):
        """This rank's part of a vocab-sharded step in ONE library call: lm_head shard, local
        sampling stage, record exchange over peer memory and merge (`vqk_lm_head_step_sharded`).
        `sp` carries this rank's vocab_offset and the global vocab_total; `peer_handle` is a
        connected vqk_peer.  Returns the merged (tokens, scores), identical on every rank."""
        x2 = self._x2d(x)
        B = x2.shape[0]
        tokens = torch.empty(B, dtype=torch.int64, device=self.device)
        scores = torch.empty(B, dtype=torch.float32, device=self.device)
        if bias is not None:
            bias = bias.to(torch.float16).contiguous()
        if not B:
            return tokens, scores
        L = _ffi.lib()
        key = ("sharded", B)
        n = self._ws_bytes.get(key)
        if n is None:
            with torch.cuda.device(self.device):
                n = int(L.vqk_lm_head_step_sharded_workspace_bytes(self._h, B))
            if n < 0:
                _ffi.check(n)
            self._ws_bytes[key] = n
        ws = self._wsp.get(self.device, n)
        spc = sp.to_c(B, self.V)
        with torch.cuda.device(self.device):
            _ffi.check(L.vqk_lm_head_step_sharded(self._h, peer_handle, x2.data_ptr(), _DT[x2.dtype], B, x2.stride(0),
                                                  _ptr(bias), ctypes.byref(spc), tokens.data_ptr(), scores.data_ptr(),
                                                  ws.data_ptr(), n, _stream(x2)))
        return tokens, scores

    def _host_step_args(self, x_host, sp_host, tokens_host, scores_host, peer_handle, bias, stream):
        assert x_host.dim() == 2 and x_host.shape[1] == self.H and x_host.dtype in (torch.float16, torch.bfloat16)
        assert not x_host.is_cuda and x_host.is_contiguous()
        B = x_host.shape[0]
        assert tokens_host.dtype == torch.int64 and tokens_host.shape == (B,) and not tokens_host.is_cuda
        if scores_host is not None:
            assert scores_host.dtype == torch.float32 and scores_host.shape == (B,) and not scores_host.is_cuda

        def hp(t, dt, name):
            if t is None:
                return None
            if t.is_cuda or t.dtype != dt or t.shape != (B,) or not t.is_contiguous():
                raise ValueError(f"{name} must be a contiguous CPU {dt} tensor of shape ({B},)")
            return t.data_ptr()
        total = self.V if sp_host.vocab_total is None else int(sp_host.vocab_total)
        spc = _ffi.SampleParams(
            hp(sp_host.temperature, torch.float32, "temperature"), hp(sp_host.seeds, torch.int32, "seeds"),
            hp(sp_host.top_k, torch.int32, "top_k"), hp(sp_host.top_p, torch.float32, "top_p"),
            hp(sp_host.topk_threshold, torch.float32, "topk_threshold"), int(sp_host.vocab_offset), total)
        if bias is not None:
            bias = bias.to(torch.float16).contiguous()
        L = _ffi.lib()
        key = ("host", B)
        n = self._ws_bytes.get(key)
        if n is None:
            with torch.cuda.device(self.device):
                n = int(L.vqk_lm_head_step_host_workspace_bytes(self._h, B))
            if n < 0:
                _ffi.check(n)
            self._ws_bytes[key] = n
        ws = self._wsp.get(self.device, n)
        st = (stream or torch.cuda.current_stream(self.device)).cuda_stream
        args = (self._h, peer_handle, x_host.data_ptr(), _DT[x_host.dtype], B, _ptr(bias), ctypes.byref(spc),
                tokens_host.data_ptr(), _ptr(scores_host), ws.data_ptr(), n, st)
        keep = (x_host, sp_host, tokens_host, scores_host, bias, ws, spc)  # what the raw pointers refer to
        return args, keep

    def step_host(self, x_host: torch.Tensor, sp_host: "SamplingArgs", tokens_host: torch.Tensor,
                  scores_host: Optional[torch.Tensor] = None, peer_handle=None, bias: Optional[torch.Tensor] = None,
                  stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """One decode step from HOST tensors in ONE library call (`vqk_lm_head_step_host`):
        `x_host` [B, H] fp16 / bf16 and the arrays of `sp_host` are CPU tensors (any memory; the
        library stages them through a pinned buffer of its own), `tokens_host` is a CPU int64
        tensor [B] that receives the tokens.  Returns `tokens_host` when the tokens are in it.
        Without `scores_host` the kernels write the tokens straight into mapped host memory and
        the call watches them arrive; with it (CPU fp32 [B]) both come back by a copy and a
        stream synchronise.  `peer_handle`: a connected vqk_peer for a vocab-sharded step."""
        args, _keep = self._host_step_args(x_host, sp_host, tokens_host, scores_host, peer_handle, bias, stream)
        with torch.cuda.device(self.device):
            _ffi.check(_ffi.lib().vqk_lm_head_step_host(*args))
        return tokens_host

    def host_stepper(self, x_host: torch.Tensor, sp_host: "SamplingArgs", tokens_host: torch.Tensor,
                     scores_host: Optional[torch.Tensor] = None, peer_handle=None,
                     bias: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None):
        """`step_host` bound to fixed host tensors: a decode loop that refills `x_host` and the
        sampling arrays in place calls the returned function once per step and reads
        `tokens_host`; the argument checks and the workspace lookup are done once, here.  The
        caller keeps this device current (`torch.cuda.set_device`)."""
        args, keep = self._host_step_args(x_host, sp_host, tokens_host, scores_host, peer_handle, bias, stream)
        fn, check = _ffi.lib().vqk_lm_head_step_host, _ffi.check

        def run(_keep=keep):
            rc = fn(*args)
            if rc:
                check(rc)
            return tokens_host
        return run

    def shard_records(self, x: torch.Tensor, sp: SamplingArgs, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """lm_head + local sampling stage of a vocab-sharded step: uint8 [B, 1024]
        exchange records to be all-gathered and passed to `finalize_records`."""
        x2 = self._x2d(x)
        B = x2.shape[0]
        rec = torch.empty(B, _ffi.RECORD_BYTES, dtype=torch.uint8, device=self.device)
        if bias is not None:
            bias = bias.to(torch.float16).contiguous()
        if B:
            self._forward(x2, bias, None, sp, None, None, rec)
        return rec


# --------------------------------------------------------------------------
# stand-alone sampler entry points
# --------------------------------------------------------------------------

def sample_logits(logits: torch.Tensor, sp: SamplingArgs, records: bool = False, return_logprobs: bool = False):
    """Sampler on materialised logits [B, V] (fp32 / bf16 / fp16).  Returns
    (tokens int64, scores fp32), or the uint8 [B, 1024] shard records if `records`.
    `return_logprobs`: also the fp32 raw log-softmax of every sampled token (of the logits as
    given, before temperature / top-k / top-p: vLLM's default "raw_logprobs"), computed from the
    first pass's per-slice maxima and sums of exponentials; single shard only."""
    _require_cuda(logits, "logits")
    assert logits.dim() == 2 and logits.dtype in _DT
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    B, V = logits.shape
    dev = logits.device
    L = _ffi.lib()
    n = int(L.vqk_sample_workspace_bytes(B, V))
    if n < 0:
        _ffi.check(n)
    ws = _WS.get(dev, n)
    spc = sp.to_c(B, V)
    tokens = scores = rec = lps = None
    if records:
        if return_logprobs:
            raise ValueError("log-probabilities belong to the merged token: not with shard records")
        rec = torch.empty(B, _ffi.RECORD_BYTES, dtype=torch.uint8, device=dev)
    else:
        tokens = torch.empty(B, dtype=torch.int64, device=dev)
        scores = torch.empty(B, dtype=torch.float32, device=dev)
    if return_logprobs:
        lps = torch.empty(B, dtype=torch.float32, device=dev)
        spc.logprobs = lps.data_ptr()
    if B:
        with torch.cuda.device(dev):
            _ffi.check(L.vqk_sample(logits.data_ptr(), _DT[logits.dtype], B, V, logits.stride(0), ctypes.byref(spc),
                                    _ptr(tokens), _ptr(scores), _ptr(rec), ws.data_ptr(), n, _stream(logits)))
    if records:
        return rec
    return (tokens, scores, lps) if return_logprobs else (tokens, scores)


def finalize_records(gathered: torch.Tensor, sp: SamplingArgs):
    """Merge all-gathered shard records [G, B, 1024] into (tokens, scores); every
    rank gets the same answer.  Rows that overflowed a record get token -1."""
    _require_cuda(gathered, "records")
    assert gathered.dtype == torch.uint8 and gathered.dim() == 3 and gathered.shape[2] == _ffi.RECORD_BYTES
    gathered = gathered.contiguous()
    G, B, _ = gathered.shape
    dev = gathered.device
    tokens = torch.empty(B, dtype=torch.int64, device=dev)
    scores = torch.empty(B, dtype=torch.float32, device=dev)
    total = sp.vocab_total if sp.vocab_total is not None else 0
    spc = sp.to_c(B, total)
    if B:
        with torch.cuda.device(dev):
            _ffi.check(_ffi.lib().vqk_sample_finalize(gathered.data_ptr(), G, B, ctypes.byref(spc), tokens.data_ptr(),
                                                      scores.data_ptr(), _stream(gathered)))
    return tokens, scores


def topk_threshold(logits: torch.Tensor, top_k: torch.Tensor) -> torch.Tensor:
    """Per-row k-th largest raw logit on the device, no host sync
    (reference: _sampler.py:62-93).  Rows with k <= 0 or k >= V get -inf."""
    _require_cuda(logits, "logits")
    if logits.stride(1) != 1:
        logits = logits.contiguous()
    B, V = logits.shape
    k = top_k.to(torch.int32).contiguous()
    thr = torch.empty(B, dtype=torch.float32, device=logits.device)
    if B:
        with torch.cuda.device(logits.device):
            _ffi.check(_ffi.lib().vqk_topk_threshold(logits.data_ptr(), _DT[logits.dtype], B, V, logits.stride(0),
                                                     k.data_ptr(), thr.data_ptr(), _stream(logits)))
    return thr


def sample_logits_static(logits: torch.Tensor, sp: SamplingArgs):
    """`sample_logits` for callers that must not allocate device memory inside the call:
    the library keeps the sampler's scratch in a fixed array of its own, so no workspace is
    requested from torch (or anyone).  The two output tensors are still the caller's; pass
    `out=(tokens, scores)`-style pre-allocated tensors through `sample_logits_static_into`
    to avoid even those.  Limits: at most 64 rows of at most 262144 columns, single shard.
    Calls share the scratch, so do not overlap two of them on different streams; make the
    first call on a device before any CUDA-graph capture starts there."""
    B = logits.shape[0]
    tokens = torch.empty(B, dtype=torch.int64, device=logits.device)
    scores = torch.empty(B, dtype=torch.float32, device=logits.device)
    sample_logits_static_into(logits, sp, tokens, scores)
    return tokens, scores


def sample_logits_static_into(logits: torch.Tensor, sp: SamplingArgs, tokens: torch.Tensor,
                              scores: Optional[torch.Tensor] = None) -> None:
    """Allocation-free form: every buffer, outputs included, comes from the caller."""
    _require_cuda(logits, "logits")
    assert logits.dim() == 2 and logits.dtype in _DT and logits.stride(1) == 1
    B, V = logits.shape
    assert tokens.dtype == torch.int64 and tokens.shape == (B,) and tokens.is_contiguous()
    if scores is not None:
        assert scores.dtype == torch.float32 and scores.shape == (B,) and scores.is_contiguous()
    spc = sp.to_c(B, V)
    with torch.cuda.device(logits.device):
        _ffi.check(_ffi.lib().vqk_sample_static(logits.data_ptr(), _DT[logits.dtype], B, V, logits.stride(0),
                                                ctypes.byref(spc), tokens.data_ptr(), _ptr(scores), _stream(logits)))
