"""Oracle: fused Gumbel-argmax sampler, top-k threshold, top-p mask, shard merge.

Test infrastructure only (see ``oracle/__init__.py``).

The reference sampler is src/vllm_quant_kernels/_sampler_kernels.py:38-182 with
its host wrapper src/vllm_quant_kernels/_sampler.py:62-206.  Its noise comes
from Triton's ``tl.rand`` (third-party: ``triton>=3.0`` per the reference's
pyproject.toml:14; the algorithm restated here is triton 3.6.0
``triton/language/random.py``: Philox-4x32 with 10 rounds, counter
``(offset, 0, 0, 0)``, key ``(seed_lo, seed_hi)``, output word 0).

top-p is NOT on the reference's fast path (_sampler.py:43-44 falls back to
vLLM); the mask restated here follows vLLM 0.22.0
``vllm/v1/sample/ops/topk_topp_sampler.py:328-369`` (ascending sort, softmax,
cumsum, drop while cumsum <= 1 - p, always keep the largest), applied after
temperature and after top-k.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32
GREEDY_EPS = F32(1e-5)            # _sampler_kernels.py:35
FP32_TINY = F32(2.0 ** -126)      # _sampler_kernels.py:32
UNIFORM_SCALE = F32(4.6566127342e-10)   # triton/language/random.py:138

_M32 = np.uint64(0xFFFFFFFF)


def philox_word0(seed, offset) -> np.ndarray:
    """Word 0 of Philox-4x32-10 for counter (offset, 0, 0, 0) and key
    (seed & 0xffffffff, (seed >> 32) & 0xffffffff) where ``seed`` is first
    widened to 64 bits the way ``tl.rand`` does (int32 sign-extends).
    triton/language/random.py:13-42,46-69,89-110."""
    seed64 = np.asarray(seed, dtype=np.int64).astype(np.uint64)
    off = np.asarray(offset)
    c0 = off.astype(np.int64).astype(np.uint64) & _M32
    shape = np.broadcast(seed64, c0).shape
    c0 = np.broadcast_to(c0, shape).copy()
    c1 = np.zeros(shape, np.uint64)
    c2 = np.zeros(shape, np.uint64)
    c3 = np.zeros(shape, np.uint64)
    k0 = np.broadcast_to(seed64 & _M32, shape).copy()
    k1 = np.broadcast_to((seed64 >> np.uint64(32)) & _M32, shape).copy()
    A = np.uint64(0xD2511F53)
    B = np.uint64(0xCD9E8D57)
    for _ in range(10):
        pa = A * c0
        pb = B * c2
        n0 = ((pb >> np.uint64(32)) ^ c1 ^ k0) & _M32
        n2 = ((pa >> np.uint64(32)) ^ c3 ^ k1) & _M32
        c1 = pb & _M32
        c3 = pa & _M32
        c0, c2 = n0, n2
        k0 = (k0 + np.uint64(0x9E3779B9)) & _M32
        k1 = (k1 + np.uint64(0xBB67AE85)) & _M32
    return c0.astype(np.uint32)


def uniform(seed, offset) -> np.ndarray:
    """``tl.rand``: word 0 as int32, negative values mirrored (``-x - 1``), times
    4.6566127342e-10 in fp32.  triton/language/random.py:127-156."""
    x = philox_word0(seed, offset).view(np.int32).astype(np.int64)
    x = np.where(x < 0, -x - 1, x)
    return (x.astype(F32) * UNIFORM_SCALE).astype(F32)


def gumbel(seed, offset) -> np.ndarray:
    """-log(-log(max(u, 2^-126))) in fp32.  _sampler_kernels.py:104-106."""
    u = np.maximum(uniform(seed, offset), FP32_TINY)
    with np.errstate(divide="ignore"):
        return (-np.log(-np.log(u).astype(F32))).astype(F32)


def topk_threshold(logits, top_k, vocab_size=None):
    """Per-row k-th largest RAW logit, or None when max(top_k) >= vocab (the
    reference then disables top-k for every row).  _sampler.py:62-93."""
    logits = np.asarray(logits, dtype=F32)
    top_k = np.asarray(top_k).astype(np.int64)
    V = logits.shape[1] if vocab_size is None else vocab_size
    max_k = int(top_k.max())
    if max_k >= V:
        return None
    srt = -np.sort(-logits, axis=1)[:, :max_k]          # descending top max_k
    idx = np.clip(np.clip(top_k, None, max_k) - 1, 0, None)
    return srt[np.arange(logits.shape[0]), idx].astype(F32)


def topk_threshold_per_row(logits, top_k):
    """Per-row variant used by the new build: row i gets the k_i-th largest raw
    logit; k_i <= 0 or k_i >= V disables top-k for that row only (-inf).  This
    is vLLM's per-row meaning (topk_topp_sampler.py:382-392) and equals the
    reference's for uniform k."""
    logits = np.asarray(logits, dtype=F32)
    B, V = logits.shape
    thr = np.full(B, -np.inf, dtype=F32)
    srt = -np.sort(-logits, axis=1)
    for i, k in enumerate(np.asarray(top_k).astype(np.int64)):
        if 0 < k < V:
            thr[i] = srt[i, k - 1]
    return thr


def top_p_keep(y_kept, p):
    """Upstream top-p on the surviving scaled logits of ONE row.

    y_kept : fp32 values (any order).  Returns (keep mask in the same order,
    boundary margin = min |cumsum - (1 - p)| over the elements).

    Upstream orders EQUAL values arbitrarily (torch.sort is not stable), so which
    members of a tie group straddling the nucleus boundary survive is unpinned
    there.  This build's rule, restated here: every value equal to the smallest
    surviving value survives too ("ties at the boundary are all kept")."""
    y = np.asarray(y_kept, dtype=F32)
    order = np.argsort(y, kind="stable")
    ys = y[order]
    e = np.exp((ys - ys[-1]).astype(F32)).astype(F32)
    probs = (e / e.sum(dtype=F32)).astype(F32)
    c = np.cumsum(probs, dtype=F32)
    lim = F32(1.0) - F32(p)
    drop = c <= lim
    drop[-1] = False
    keep = np.empty_like(drop)
    keep[order] = ~drop
    keep |= (y == ys[~drop].min())
    margin = float(np.min(np.abs(c[:-1].astype(np.float64) - float(lim)))) if len(c) > 1 else 1.0
    return keep, margin


def sample(logits, temperature, seeds, top_k=None, top_p=None, topk_thr=None,
           vocab_offset: int = 0):
    """Full sampler semantics of the new build on logits [B, V] (any float
    dtype, read as fp32 like vllm/v1/sample/sampler.py:91).

    Reference part (_sampler_kernels.py:62-120): raw-logit top-k mask with
    ``>=``, greedy iff T < 1e-5, else y = l / T + gumbel(seed, GLOBAL index),
    masked -> -inf, max with ties to the lowest index.
    Extension: per-row top_k (<=0 or >=V disables) and top_p (>=1 disables).

    Returns dict(tokens int64 [B] (global ids), scores fp32 [B], margin fp64 [B]
    = winner score minus runner-up, p_margin [B] = top-p boundary margin).
    """
    L = np.asarray(logits).astype(F32)
    B, V = L.shape
    tokens = np.zeros(B, np.int64)
    scores = np.zeros(B, F32)
    margin = np.full(B, np.inf)
    p_margin = np.full(B, 1.0)
    for i in range(B):
        l = L[i]
        keep = np.ones(V, bool)
        if topk_thr is not None:
            keep &= l >= F32(topk_thr[i])
        elif top_k is not None and 0 < int(top_k[i]) < V:
            kth = np.partition(l, V - int(top_k[i]))[V - int(top_k[i])]
            keep &= l >= kth
        T = None if temperature is None else F32(temperature[i])
        greedy = (T is None) or (T < GREEDY_EPS)
        if greedy:
            s = l.copy()
        else:
            y = (l / T).astype(F32)
            if top_p is not None and float(top_p[i]) < 1.0:
                idx = np.nonzero(keep)[0]
                k2, p_margin[i] = top_p_keep(y[idx], top_p[i])
                keep2 = np.zeros(V, bool)
                keep2[idx[k2]] = True
                keep = keep2
            idx = np.nonzero(keep)[0]
            s = np.full(V, -np.inf, dtype=F32)
            s[idx] = (y[idx] + gumbel(int(seeds[i]), idx + vocab_offset)).astype(F32)
        s = np.where(keep, s, F32(-np.inf))
        w = int(np.argmax(s))                       # first occurrence = lowest index
        tokens[i] = w + vocab_offset
        scores[i] = s[w]
        if V > 1:
            s2 = s.copy()
            s2[w] = -np.inf
            r = s2.max()
            margin[i] = float(s[w]) - float(r) if np.isfinite(r) else np.inf
    return dict(tokens=tokens, scores=scores, margin=margin, p_margin=p_margin)


def fused_gumbel_sample(logits, temperature, seeds, topk_threshold=None):
    """The reference entry point's contract, _sampler_kernels.py:123-182."""
    return sample(logits, temperature, seeds, topk_thr=topk_threshold)["tokens"]


def merge_winners(scores, tokens):
    """Cross-shard merge of per-rank winners: scores/tokens [G, B].  Higher score
    wins; equal scores -> lower token id (reproduces first-occurrence argmax,
    _sampler_kernels.py:116-120,180-181)."""
    scores = np.asarray(scores, dtype=F32)
    tokens = np.asarray(tokens, dtype=np.int64)
    G, B = scores.shape
    out_t = np.zeros(B, np.int64)
    out_s = np.zeros(B, F32)
    for b in range(B):
        best = 0
        for g in range(1, G):
            if scores[g, b] > scores[best, b] or (
                    scores[g, b] == scores[best, b] and tokens[g, b] < tokens[best, b]):
                best = g
        out_t[b] = tokens[best, b]
        out_s[b] = scores[best, b]
    return out_t, out_s


def synth_logits(B: int, V: int, seed: int = 0, dtype=np.float32):
    """Sampler workload: N(0, 3) logits with 5 distinct columns per row at +12."""
    rng = np.random.default_rng(seed)
    L = (rng.standard_normal((B, V), dtype=F32) * F32(3.0)).astype(F32)
    for i in range(B):
        cols = rng.choice(V, size=min(5, V), replace=False)
        L[i, cols] = 12.0
    return L.astype(dtype)


def resolve_candidates(values, tokens, T, seed, top_k=0, top_p=1.0):
    """Final choice among a candidate set that is known to contain every logit >= the
    k-th largest (the union of the shards' records).  Same semantics as :func:`sample`
    restricted to those candidates; noise by GLOBAL token id.  Returns (token, score)."""
    v = np.asarray(values, dtype=F32)
    t = np.asarray(tokens, dtype=np.int64)
    keep = np.ones(len(v), bool)
    if top_k and top_k > 0:
        kth = np.sort(v)[::-1][min(top_k, len(v)) - 1]
        keep &= v >= kth
    y = (v / F32(T)).astype(F32)
    if top_p < 1.0:
        idx = np.nonzero(keep)[0]
        k2, _ = top_p_keep(y[idx], top_p)
        keep2 = np.zeros(len(v), bool)
        keep2[idx[k2]] = True
        keep = keep2
    s = np.where(keep, (y + gumbel(int(seed), t)).astype(F32), F32(-np.inf))
    order = np.lexsort((t, -s.astype(np.float64)))     # highest score, then lowest token
    return int(t[order[0]]), F32(s[order[0]])


def raw_logprob(logits, tokens):
    """log-softmax of the given tokens over the logits as given (no temperature, no top-k / top-p):
    what vLLM reports as the sampled token's log-probability by default
    (vllm/v1/sample/sampler.py: `compute_logprobs` = log_softmax of the raw fp32 logits; the
    reference's FusedSampler sends every batch that wants it back to vLLM,
    src/vllm_quant_kernels/_sampler.py:158-169).  float64 arithmetic."""
    l = np.asarray(logits, dtype=np.float64)
    t = np.asarray(tokens, dtype=np.int64)
    m = l.max(axis=1, keepdims=True)
    lse = m[:, 0] + np.log(np.exp(l - m).sum(axis=1))
    return (l[np.arange(l.shape[0]), t] - lse).astype(np.float32)
