"""Worker of tests/test_gpu_multi.py (launched by torch.distributed.run, one rank per GPU).

Every rank builds the same seeded weights, keeps its vocab slice, and runs the sharded step
three times: exchanging records through libvqk's own NCCL communicator, through
torch.distributed, and through the fused peer-memory exchange (also replayed from a CUDA graph
several times, which exercises the step counters and the two landing-buffer parities).  Every
rank also runs the unsharded step; all results must be identical."""

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "vllm-quant-kernels_b200"))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    from vllm_quant_kernels import _lmhead as LH
    from vllm_quant_kernels import _ffi
    from vllm_quant_kernels._dist import VocabShardedLMHead, VqkComm, VqkPeer, shard_bounds
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    V, H, B = 16 * 8 * 97, 1024, 6
    g = torch.Generator().manual_seed(7)
    std = torch.exp(torch.empty(V).uniform_(np.log(0.03), np.log(0.18), generator=g))
    w = (torch.randn(V, H, generator=g) * std[:, None]).clamp_(-0.76, 0.76).half().to(dev)
    x = torch.randn(B, H, generator=g).half().to(dev)
    rng = np.random.default_rng(3)
    T = rng.uniform(0.5, 1.5, B).astype(np.float32)
    T[0] = 0.0
    seeds = rng.integers(0, 2**31 - 1, B).astype(np.int32)

    def args(**kw):
        t = lambda a, dt: None if a is None else torch.from_numpy(np.asarray(a)).to(dt).to(dev)
        return LH.SamplingArgs(t(T, torch.float32), t(seeds, torch.int32), t(kw.get("top_k"), torch.int32),
                               t(kw.get("top_p"), torch.float32), None, 0, V)

    comm = VqkComm(rank, world)
    peer = VqkPeer(rank, world, max_rows=32)
    a, b = shard_bounds(V, world, rank)
    for mode in ("int8", "mxfp4"):
        q, s = LH.quantize_weight(mode, w)
        full = LH.LMHeadShard(mode, q, s)
        mine = LH.LMHeadShard(mode, q[a:b].contiguous(), s[a:b].contiguous())
        for kw in (dict(), dict(top_k=np.full(B, 50, np.int32), top_p=np.full(B, 0.9, np.float32))):
            sp = args(**kw)
            ref_tok, ref_sc = full.sample(x, sp)
            for c in (comm, None):
                tok, sc = VocabShardedLMHead(mine, a, V, comm=c).step(x, sp)
                torch.cuda.synchronize()
                assert torch.equal(tok, ref_tok), (rank, mode, list(kw), tok.tolist(), ref_tok.tolist())
                assert torch.equal(sc, ref_sc)
            ph = VocabShardedLMHead(mine, a, V, peer=peer)
            for _ in range(3):  # both parities of the landing buffer; the whole step is one library call
                tok, sc = ph.step(x, sp)
                torch.cuda.synchronize()
                assert torch.equal(tok, ref_tok), ("peer", rank, mode, list(kw), tok.tolist(), ref_tok.tolist(),
                                                   "device_error", _ffi.lib().vqk_device_error())
                assert torch.equal(sc, ref_sc)
            # the exchange as a kernel of its own, fed the records of the separate lm_head call
            rec = mine.shard_records(x, ph.local_args(sp))
            tok, sc = peer.exchange_finalize(rec, ph.local_args(sp))
            torch.cuda.synchronize()
            assert torch.equal(tok, ref_tok) and torch.equal(sc, ref_sc), ("peer records", rank, mode, list(kw))
        # the same step from host tensors, one library call (vqk_lm_head_step_host with the peer handle)
        spk = args(top_k=np.full(B, 50, np.int32), top_p=np.full(B, 0.9, np.float32))
        ref_tok, _ = full.sample(x, spk)
        sp_cpu = LH.SamplingArgs(spk.temperature.cpu(), spk.seeds.cpu(), spk.top_k.cpu(), spk.top_p.cpu(), None, 0, V)
        th = torch.empty(B, dtype=torch.int64)
        run = VocabShardedLMHead(mine, a, V, peer=peer).host_stepper(x.cpu(), sp_cpu, th)
        for _ in range(3):
            assert run().tolist() == ref_tok.cpu().tolist(), ("host step", rank, mode, th.tolist(), ref_tok.tolist())
        torch.cuda.synchronize()
        # a batch above 16 rows: the full-row sampler kernel does the exchange
        xb = torch.randn(24, H, generator=torch.Generator().manual_seed(11)).half().to(dev)
        rngb = np.random.default_rng(5)
        Tb = torch.from_numpy(rngb.uniform(0.5, 1.5, 24).astype(np.float32)).to(dev)
        sb = torch.from_numpy(rngb.integers(0, 2**31 - 1, 24).astype(np.int32)).to(dev)
        kb = torch.full((24,), 40, dtype=torch.int32, device=dev)
        pb = torch.full((24,), 0.85, dtype=torch.float32, device=dev)
        spb = LH.SamplingArgs(Tb, sb, kb, pb, None, 0, V)
        ref_tok, ref_sc = full.sample(xb, spb)
        tok, sc = VocabShardedLMHead(mine, a, V, peer=peer).step(xb, spb)
        torch.cuda.synchronize()
        assert torch.equal(tok, ref_tok) and torch.equal(sc, ref_sc), ("peer batch 24", rank, mode)
        # rows the records cannot carry (top-p without top-k): -1 from the merge, exact after the rerun
        spp = args(top_p=np.full(B, 0.8, np.float32))
        ref_tok, ref_sc = full.sample(x, spp)
        for c, ph2 in ((comm, VocabShardedLMHead(mine, a, V, comm=comm)), (None, VocabShardedLMHead(mine, a, V, peer=peer))):
            tok, _ = ph2.step(x, spp)
            torch.cuda.synchronize()
            assert (tok[1:] == -1).all() and tok[0] == ref_tok[0], ("unresolved rows", rank, tok.tolist())
            tok, sc = ph2.step(x, spp, unresolved="rerun")
            torch.cuda.synchronize()
            assert torch.equal(tok, ref_tok) and torch.equal(sc, ref_sc), ("rerun", rank, mode, tok.tolist(), ref_tok.tolist())
    # the peer step inside a CUDA graph: the step number lives on the device, so replays stay in step
    sp = args()
    ph = VocabShardedLMHead(mine, a, V, peer=peer)
    ref_tok, _ = full.sample(x, sp)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ph.step(x, sp)  # warm-up outside the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            gtok, _ = ph.step(x, sp)
        for _ in range(5):
            graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(gtok, ref_tok), ("peer graph", rank, gtok.tolist(), ref_tok.tolist())
    assert _ffi.lib().vqk_device_error() == 0
    dist.barrier()
    peer.close()
    comm.close()
    if rank == 0:
        print("MULTI_GPU_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
