"""The record exchange over peer memory on ONE GPU, without a second process.

`vqk_peer_connect_pointers` lets several vqk_peer objects of one process address each other's
landing buffers directly, so the exchange kernels can be driven where only one GPU is
there:
  * a 1-rank "group" runs the whole sharded step (`vqk_lm_head_step_sharded`) and must give
    the single-shard tokens, also for batches above 16 rows and for rows the records cannot
    carry (which come back as -1 and are then resolved from the full logits rows);
  * a 2-rank group in which rank 1 never runs makes rank 0's bounded wait run out: the rows
    report -1, `vqk_device_error()` turns 1, the kernel returns, the flag can be cleared and a
    following step on a healthy group is correct.  Nothing faults, traps or hangs: the wait is
    a bounded poll.
"""

import ctypes

import numpy as np
import pytest
import torch

from tests.util import make_act, make_weight, sample_args

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _peer(rank, world, max_rows=64):
    from vllm_quant_kernels import _ffi
    L = _ffi.lib()
    h = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(_ffi.PEER_HANDLE_BYTES)
    _ffi.check(L.vqk_peer_create(rank, world, max_rows, ctypes.byref(h), handle))
    return h


def _connect(peers):
    from vllm_quant_kernels import _ffi
    L = _ffi.lib()
    bufs = (ctypes.c_void_p * len(peers))(*[L.vqk_peer_local_buffer(p) for p in peers])
    for p in peers:
        _ffi.check(L.vqk_peer_connect_pointers(p, bufs))


@pytest.mark.parametrize("mode", ["int8", "fp8", "mxfp4"])
@pytest.mark.parametrize("B", [1, 6, 16, 40])
def test_one_rank_sharded_step_equals_single_shard(mode, B):
    from vllm_quant_kernels import _ffi, _lmhead as LH
    from vllm_quant_kernels._dist import VocabShardedLMHead
    L = _ffi.lib()
    V, H = 20000 + 16 * 3, 1024
    w = make_weight(V, H, seed=41) * 4.0
    x = make_act(B, H, seed=42 + B)
    q, s = LH.quantize_weight(mode, w)
    shard = LH.LMHeadShard(mode, q, s)
    rng = np.random.default_rng(B)
    T = rng.uniform(0.5, 1.5, B).astype(np.float32)
    T[0] = 0.0
    seeds = rng.integers(0, 2**31 - 1, B).astype(np.int32)
    peer = _peer(0, 1)
    _connect([peer])

    class P:            # what VocabShardedLMHead needs of a VqkPeer
        _h = peer
    head = VocabShardedLMHead(shard, 0, V, peer=P)
    try:
        for kw in (dict(), dict(top_k=np.full(B, 50, np.int32), top_p=np.full(B, 0.9, np.float32)),
                   dict(top_k=np.full(B, 3, np.int32))):
            sp = sample_args(B, DEV, T, seeds, vocab_total=V, **kw)
            want_tok, want_sc = shard.sample(x, sample_args(B, DEV, T, seeds, **kw))
            for rep in range(3):                        # both parities of the landing buffer
                tok, sc = head.step(x, sp)
                assert torch.equal(tok, want_tok), (mode, B, list(kw), rep, tok.tolist(), want_tok.tolist())
                assert torch.equal(sc, want_sc)
        # rows the records cannot carry: top-p without top-k -> -1, then resolved from the full rows
        kw = dict(top_p=np.full(B, 0.8, np.float32))
        sp = sample_args(B, DEV, T, seeds, vocab_total=V, **kw)
        want_tok, want_sc = shard.sample(x, sample_args(B, DEV, T, seeds, **kw))
        tok, _ = head.step(x, sp)
        assert (tok[1:] == -1).all() and tok[0] == want_tok[0]          # row 0 is greedy
        if B > 1:
            with pytest.raises(RuntimeError, match="cannot be merged"):
                head.step(x, sp, unresolved="raise")
        tok, sc = head.step(x, sp, unresolved="rerun")
        assert torch.equal(tok, want_tok) and torch.equal(sc, want_sc)
        assert L.vqk_device_error() == 0
    finally:
        L.vqk_peer_destroy(peer)


def test_bounded_wait_runs_out_and_recovers():
    from vllm_quant_kernels import _ffi, _lmhead as LH
    L = _ffi.lib()
    V, H, B = 8000, 512, 3
    w = make_weight(V, H, seed=5) * 4.0
    x = make_act(B, H, seed=6)
    q, s = LH.quantize_weight("int8", w)
    shard = LH.LMHeadShard("int8", q, s)
    T = np.array([0.0, 0.8, 1.2], np.float32)
    seeds = np.array([3, 4, 5], np.int32)
    kw = dict(top_k=np.full(B, 20, np.int32))
    # two "ranks" that share this GPU; rank 1 never runs a step, so its words never arrive
    p0, p1 = _peer(0, 2), _peer(1, 2)
    _connect([p0, p1])
    _ffi.check(L.vqk_peer_set_wait_limit(p0, 20000))                   # a few milliseconds of polling
    assert L.vqk_device_error() == 0
    sp = sample_args(B, DEV, T, seeds, vocab_offset=0, vocab_total=2 * V, **kw)
    try:
        tok, sc = shard.step_sharded(x, sp, p0)
        torch.cuda.synchronize()                                       # the kernel returned by itself
        assert (tok == -1).all()
        assert L.vqk_device_error() == 1
        assert L.vqk_device_error_clear() == 0
        assert L.vqk_device_error() == 0
    finally:
        L.vqk_peer_destroy(p0)
        L.vqk_peer_destroy(p1)
    # a healthy group afterwards: the context is usable and the step is right
    p = _peer(0, 1)
    _connect([p])
    try:
        sp = sample_args(B, DEV, T, seeds, vocab_total=V, **kw)
        tok, sc = shard.step_sharded(x, sp, p)
        want_tok, want_sc = shard.sample(x, sample_args(B, DEV, T, seeds, **kw))
        assert torch.equal(tok, want_tok) and torch.equal(sc, want_sc)
        assert L.vqk_device_error() == 0
    finally:
        L.vqk_peer_destroy(p)


def test_two_ranks_on_one_gpu_by_turns_through_records():
    """Two shards of one weight as two vqk_peer on this GPU.  Their exchange kernels wait on each
    other, so they must not run as separate launches on one GPU; what runs here instead is the
    record path: each shard's records, stacked, merged by vqk_sample_finalize, against the
    unsharded step - and each rank's own exchange kernel on a 1-rank group fed the OTHER rank's
    record merged in by hand is covered by the finalize kernel's arithmetic being the same code."""
    from vllm_quant_kernels import _lmhead as LH
    from vllm_quant_kernels._dist import shard_bounds
    V, H, B = 16 * 700, 1024, 5
    w = make_weight(V, H, seed=9) * 4.0
    x = make_act(B, H, seed=10)
    q, s = LH.quantize_weight("int8", w)
    full = LH.LMHeadShard("int8", q, s)
    T = np.array([0.0, 0.7, 0.9, 1.1, 1.4], np.float32)
    seeds = np.arange(B, dtype=np.int32) + 11
    kw = dict(top_k=np.full(B, 50, np.int32), top_p=np.full(B, 0.9, np.float32))
    want_tok, want_sc = full.sample(x, sample_args(B, DEV, T, seeds, **kw))
    recs = []
    for r in range(2):
        a, b = shard_bounds(V, 2, r)
        sh = LH.LMHeadShard("int8", q[a:b], s[a:b])
        recs.append(sh.shard_records(x, sample_args(B, DEV, T, seeds, vocab_offset=a, vocab_total=V, **kw)))
    tok, sc = LH.finalize_records(torch.stack(recs), sample_args(B, DEV, T, seeds, vocab_total=V, **kw))
    assert torch.equal(tok, want_tok) and torch.equal(sc, want_sc)
