"""World-size-2 gloo run of the vocab-sharded step's HOST plumbing on CPU: shard bounds,
record packing, the rank-major all-gather, and the merge rule.  The per-shard records are
produced by the oracle (the CUDA producers are covered by the -m gpu tests); what is under
test here is the product's `_dist` module."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs():
    from oracle import sampler as OS
    B, V = 5, 4000
    L = OS.synth_logits(B, V, seed=3)
    T = np.float32([0.0, 0.7, 1.0, 1.3, 0.9])
    seeds = np.int32([5, 6, 7, 8, 9])
    top_k = np.int32([0, 0, 50, 10, 50])
    top_p = np.float32([1.0, 1.0, 1.0, 0.9, 0.8])
    return L, T, seeds, top_k, top_p


def _local_records(L, T, seeds, top_k, top_p, a, b):
    """What a rank's CUDA stage emits for rows [a, b) of the vocabulary."""
    from oracle import sampler as OS
    from vllm_quant_kernels._dist import pack_record
    recs = []
    for i in range(L.shape[0]):
        l = L[i, a:b]
        if T[i] < 1e-5 or (top_k[i] == 0 and top_p[i] >= 1.0):
            r = OS.sample(l[None], T[i:i + 1], seeds[i:i + 1], vocab_offset=a)
            recs.append(pack_record(float(r["scores"][0]), int(r["tokens"][0])))
        else:
            k = int(top_k[i])
            kth = np.sort(l)[::-1][k - 1]
            idx = np.nonzero(l >= kth)[0]
            recs.append(pack_record(cands=[(float(l[j]), int(j + a)) for j in idx]))
    return torch.from_numpy(np.stack(recs))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "vllm-quant-kernels_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from vllm_quant_kernels._dist import exchange_records, shard_bounds
        L, T, seeds, top_k, top_p = _inputs()
        a, b = shard_bounds(L.shape[1], world, rank)
        rec = _local_records(L, T, seeds, top_k, top_p, a, b)
        gathered = exchange_records(rec)
        assert gathered.shape == (world, L.shape[0], 1024)
        assert torch.equal(gathered[rank], rec)
        if rank == 0:
            np.save(out, gathered.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_rank_record_exchange_and_merge(tmp_path):
    from oracle import sampler as OS
    from vllm_quant_kernels._dist import unpack_record
    out = str(tmp_path / "gathered.npy")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    gathered = np.load(out)
    L, T, seeds, top_k, top_p = _inputs()
    ref = OS.sample(L, T, seeds, top_k=top_k, top_p=top_p)
    for i in range(L.shape[0]):
        recs = [unpack_record(gathered[g, i]) for g in range(world)]
        if all(r["n"] == 0 for r in recs):
            tok, _ = OS.merge_winners(np.float32([[r["score"]] for r in recs]), np.int64([[r["token"]] for r in recs]))
            tok = int(tok[0])
        else:
            vals = [v for r in recs for v, _ in r["cands"]]
            toks = [t for r in recs for _, t in r["cands"]]
            tok, _ = OS.resolve_candidates(vals, toks, T[i], seeds[i], int(top_k[i]), float(top_p[i]))
        assert tok == ref["tokens"][i], (i, tok, ref["tokens"][i])


def _peer_worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "vllm-quant-kernels_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from vllm_quant_kernels._dist import VqkPeer
        msg = "no error"
        try:
            VqkPeer(rank, world, max_rows=4, device="cuda:0")
        except RuntimeError as exc:
            msg = str(exc)
        with open(f"{out}.{rank}", "w") as f:
            f.write(msg)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_peer_setup_fails_on_every_rank_together(tmp_path):
    """Without a GPU the landing buffer cannot be created.  Every rank must still walk through
    the same collectives and raise the same error: a rank failing on its own would leave its
    peers blocked in the handle exchange."""
    if torch.cuda.is_available():
        pytest.skip("the failure path under test needs a machine without a GPU")
    out = str(tmp_path / "peer")
    mp.spawn(_peer_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    msgs = [open(f"{out}.{r}").read() for r in range(2)]
    assert all(m.startswith("peer-memory exchange unavailable") for m in msgs), msgs
    assert "rank 0" in msgs[1] and "rank 1" in msgs[0]
