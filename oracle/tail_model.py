"""Oracle: the argument by which the lm_head kernels' sampler tail decides a top-k row from
per-slice lists of the largest logits, restated in numpy.

Test infrastructure only (see ``oracle/__init__.py``).  It has no counterpart in the reference,
whose sampler re-reads the whole logits row (src/vllm_quant_kernels/_sampler.py:62-93 computes the
k-th largest with ``torch.topk``).  The CUDA tail (csrc/tail.cuh) keeps, per slice of a row, the
``M`` largest logits with their tokens plus a witness (the ``M+1``-th largest), and resolves the
row from those alone when they PROVE to contain every logit >= the k-th largest of the row:

  tau0 = k-th largest slice maximum          (k slices hold a value >= it, so t_k >= tau0)
  candidates = list entries >= tau0 of the slices whose maximum is >= tau0
  t_k = k-th largest candidate
  proof: every witness of those slices is < t_k   (slices that were skipped have maximum < tau0 <= t_k)

The streaming kernel applies the argument at two levels: every warp group keeps such a list for
its slice (M = 4), and at its end every CTA merges the lists of its four groups into ONE record per
row (``cta_records``: the 8 largest listed values with their tokens, and a witness that bounds
every logit of the CTA that is not in the record); the tail then runs the argument above with
"slice" = CTA and M = 8.

This module computes the same thing with sorts, so a test can check (a) that whenever the proof
holds the candidate set >= t_k IS the exact top-k set with ties, and (b) that the proof fails
where it must (more than M of the top k in one slice).
"""

from __future__ import annotations

import numpy as np

F32 = np.float32


def slice_of_rows(V: int, nslices: int, tile: int = 16) -> np.ndarray:
    """Slice index of every vocab row under the streaming kernel's schedule: 16-row tiles dealt
    round-robin to the ``nslices`` warp groups of the grid."""
    return (np.arange(V) // tile) % nslices


def slice_lists(row: np.ndarray, slices: np.ndarray, nslices: int, M: int = 4):
    """Per slice: the M+1 largest values (descending, -inf padded) and the tokens of the first M."""
    vals = np.full((nslices, M + 1), -np.inf, dtype=F32)
    toks = np.full((nslices, M), -1, dtype=np.int64)
    order = np.lexsort((np.arange(row.size), -row.astype(np.float64), slices))   # by slice, then value desc
    srt_slices = slices[order]
    starts = np.searchsorted(srt_slices, np.arange(nslices), side="left")
    ends = np.searchsorted(srt_slices, np.arange(nslices), side="right")
    for s in range(nslices):
        idx = order[starts[s]:min(ends[s], starts[s] + M + 1)]
        vals[s, :idx.size] = row[idx]
        toks[s, :min(idx.size, M)] = idx[:M]
    return vals, toks


def resolve_from_lists(vals: np.ndarray, toks: np.ndarray, k: int):
    """Returns (proved, tokens, values): the top-k set with ties when the lists prove it."""
    M = toks.shape[1]
    heads = vals[:, 0]
    finite = np.isfinite(heads)
    tau0 = -np.inf
    if finite.sum() >= k:
        tau0 = np.sort(heads[finite])[::-1][k - 1]
    sel = finite & (heads >= tau0)
    cand_v = vals[sel, :M].ravel()
    cand_t = toks[sel].ravel()
    keep = cand_v >= tau0
    keep &= np.isfinite(cand_v)
    cand_v, cand_t = cand_v[keep], cand_t[keep]
    t_k = np.sort(cand_v)[::-1][k - 1] if cand_v.size >= k else -np.inf
    witness = vals[sel, M].max() if sel.any() else -np.inf
    proved = bool(witness < t_k) or (not np.isfinite(witness) and not np.isfinite(t_k))
    surv = cand_v >= t_k
    return proved, cand_t[surv], cand_v[surv]


def cta_records(vals: np.ndarray, toks: np.ndarray, groups: int = 4, M2: int = 8):
    """Merge of the warp groups' lists (slices ``c * groups .. c * groups + groups - 1`` belong to CTA
    c) into per-CTA records, as the streaming kernel's last step does: the M2 largest listed values
    of the CTA with their tokens, and the witness = max(the groups' witnesses, the listed values that
    did not fit).  Same shapes as ``slice_lists`` returns, so ``resolve_from_lists`` takes them."""
    nsl, M = toks.shape
    ncta = nsl // groups
    out_v = np.full((ncta, M2 + 1), -np.inf, dtype=F32)
    out_t = np.full((ncta, M2), -1, dtype=np.int64)
    for c in range(ncta):
        v = vals[c * groups:(c + 1) * groups, :M].ravel()
        t = toks[c * groups:(c + 1) * groups].ravel()
        order = np.lexsort((np.arange(v.size), -v.astype(np.float64)))
        keep, rest = order[:M2], order[M2:]
        out_v[c, :keep.size] = v[keep]
        out_t[c, :keep.size] = t[keep]
        w = vals[c * groups:(c + 1) * groups, M].max()
        if rest.size:
            w = max(w, v[rest].max())
        out_v[c, M2] = w
    return out_v, out_t
