"""The proof by which the sampler tail resolves a top-k row from per-slice lists (oracle/tail_model.py,
the numpy restatement of csrc/tail.cuh): sound whenever it claims success, and failing where it must."""

import numpy as np

from oracle import sampler as OS, tail_model as TM


def _exact_topk(row, k):
    kth = np.sort(row)[::-1][k - 1]
    return set(np.nonzero(row >= kth)[0].tolist())


def test_lists_give_the_exact_topk_set_whenever_the_proof_holds():
    V, nsl = 248320, 592
    slices = TM.slice_of_rows(V, nsl)
    proved = 0
    for seed in range(12):
        row = OS.synth_logits(1, V, seed=seed)[0].astype(np.float16).astype(np.float32)   # fp16 logits, ties included
        vals, toks = TM.slice_lists(row, slices, nsl)
        for k in (1, 50, 126):
            ok, t, v = TM.resolve_from_lists(vals, toks, k)
            if ok:
                proved += 1
                assert set(t.tolist()) == _exact_topk(row, k), (seed, k)
                assert (row[t] == v).all()
    assert proved >= 30          # i.i.d. logits: the lists decide nearly every row


def test_proof_fails_when_one_slice_holds_more_than_it_can_list():
    V, nsl = 16 * 592 * 4, 592
    slices = TM.slice_of_rows(V, nsl)
    rng = np.random.default_rng(0)
    row = rng.standard_normal(V).astype(np.float32)
    rows_of_slice7 = np.nonzero(slices == 7)[0]
    row[rows_of_slice7[:6]] = 20.0 + np.arange(6)          # six of the top ten sit in one slice
    vals, toks = TM.slice_lists(row, slices, nsl)
    ok, _, _ = TM.resolve_from_lists(vals, toks, 10)
    assert not ok
    ok, t, _ = TM.resolve_from_lists(vals, toks, 4)        # the top four are all listed: decidable
    assert ok and set(t.tolist()) == _exact_topk(row, 4)


def test_ties_at_the_threshold_are_kept_or_refused_never_dropped():
    V, nsl = 16 * 592 * 2, 592
    slices = TM.slice_of_rows(V, nsl)
    row = np.zeros(V, np.float32)
    row[::97] = 1.0                                        # hundreds of equal maxima
    vals, toks = TM.slice_lists(row, slices, nsl)
    ok, t, _ = TM.resolve_from_lists(vals, toks, 5)
    if ok:
        assert set(t.tolist()) == _exact_topk(row, 5)
    short = np.full(V, -np.inf, np.float32)                # a shard with fewer finite logits than k
    short[np.arange(30) * 16] = np.arange(30)              # one per slice: nothing is hidden
    vals, toks = TM.slice_lists(short, slices, nsl)
    ok, t, _ = TM.resolve_from_lists(vals, toks, 50)
    assert ok and set(t.tolist()) == set((np.arange(30) * 16).tolist())
    short[:30] = np.arange(30)                             # sixteen in one slice: the witness is finite, no proof
    vals, toks = TM.slice_lists(short, slices, nsl)
    ok, _, _ = TM.resolve_from_lists(vals, toks, 50)
    assert not ok


def test_cta_records_bound_what_they_leave_out_and_decide_like_the_slice_lists():
    V, nsl = 248320, 592
    slices = TM.slice_of_rows(V, nsl)
    ctas = slices // 4
    for seed in range(6):
        row = OS.synth_logits(1, V, seed=100 + seed)[0].astype(np.float16).astype(np.float32)
        vals, toks = TM.slice_lists(row, slices, nsl)
        cv, ct = TM.cta_records(vals, toks)
        for c in (0, 17, 147):                              # the witness bounds every logit the record leaves out
            mine = np.nonzero(ctas == c)[0]
            listed = set(ct[c][ct[c] >= 0].tolist())
            left = np.array([i for i in mine.tolist() if i not in listed])
            assert row[left].max() <= cv[c, 8]
            assert (np.diff(cv[c, :8]) <= 0).all()
        for k in (1, 50, 126):
            ok, t, v = TM.resolve_from_lists(cv, ct, k)
            if ok:
                assert set(t.tolist()) == _exact_topk(row, k), (seed, k)
    # five of the top ten in one warp group: its list holds four, the CTA's witness must refuse the row
    rng = np.random.default_rng(1)
    row = rng.standard_normal(16 * 592 * 4).astype(np.float32)
    sl = TM.slice_of_rows(row.size, nsl)
    row[np.nonzero(sl == 9)[0][:5]] = 30.0 + np.arange(5)
    vals, toks = TM.slice_lists(row, sl, nsl)
    ok, _, _ = TM.resolve_from_lists(*TM.cta_records(vals, toks), 10)
    assert not ok
