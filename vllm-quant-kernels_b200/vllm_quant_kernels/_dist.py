"""Vocab-sharded lm_head + sampler step across the GPUs of one node.

Rows of the lm_head weight are independent, so rank r owns a contiguous vocab
slice and computes its slice of the logits plus a small per-row *record*: its
Gumbel winner, or its top-k candidates when top-k / top-p is active.  One tiny
exchange of the records (1 KiB per row per rank) is the only communication: an
all-gather (NCCL) followed by a merge kernel, or, with `VqkPeer`, one kernel that
stores the records into every rank's buffer over NVLink peer mappings, waits for
the peers' records and merges.  Every rank resolves the same final token.  Philox noise is indexed by the GLOBAL
token id, so the answer does not depend on the number of shards.

The reference plugin is single-GPU; the merge has the shape of vLLM's
`LogitsProcessor.get_top_tokens` (vllm/model_executor/layers/logits_processor.py:106-156).
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import numpy as np
import torch

from . import _ffi
from ._lmhead import LMHeadShard, SamplingArgs, finalize_records, sample_logits

ROW_ALIGN = 16  # shard boundaries fall on the kernels' 16-row tiles


def shard_bounds(vocab: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows [start, end) of the global vocabulary owned by `rank`: equal contiguous
    slices rounded up to a multiple of 16 rows, the last ranks taking what is left."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    per = -(-vocab // world)
    per = -(-per // ROW_ALIGN) * ROW_ALIGN
    start = min(vocab, rank * per)
    return start, min(vocab, start + per)


class VqkComm:
    """NCCL communicator owned by libvqk (bound at run time to the NCCL PyTorch loaded),
    so the record all-gather is enqueued on the caller's stream with no extra
    event hand-off.  The unique id travels through torch.distributed's store."""

    def __init__(self, rank: int, world: int, group=None):
        import torch.distributed as dist
        L = _ffi.lib()
        buf = ctypes.create_string_buffer(_ffi.COMM_ID_BYTES)
        if rank == 0:
            _ffi.check(L.vqk_comm_unique_id(buf))
        obj = [buf.raw if rank == 0 else None]
        dist.broadcast_object_list(obj, src=0, group=group)
        h = ctypes.c_void_p()
        _ffi.check(L.vqk_comm_create(obj[0], rank, world, ctypes.byref(h)))
        self._h = h
        self.rank, self.world = rank, world

    def allgather(self, send: torch.Tensor) -> torch.Tensor:
        send = send.contiguous()
        out = torch.empty((self.world,) + tuple(send.shape), dtype=send.dtype, device=send.device)
        _ffi.check(_ffi.lib().vqk_comm_allgather(self._h, send.data_ptr(), out.data_ptr(),
                                                 send.numel() * send.element_size(),
                                                 torch.cuda.current_stream(send.device).cuda_stream))
        return out

    def close(self):
        if self._h:
            _ffi.lib().vqk_comm_destroy(self._h)
            self._h = None


class VqkPeer:
    """Record exchange over peer memory (CUDA IPC mappings, one process per GPU on one
    node), fused with the merge into ONE kernel: no NCCL call on the step.  The IPC
    handles travel through torch.distributed once, at construction."""

    def __init__(self, rank: int, world: int, max_rows: int = 256, group=None, device=None):
        import torch.distributed as dist
        if world > _ffi.PEER_MAX_RANKS:
            raise ValueError(f"at most {_ffi.PEER_MAX_RANKS} ranks")
        L = _ffi.lib()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        h = ctypes.c_void_p()
        mine = ctypes.create_string_buffer(_ffi.PEER_HANDLE_BYTES)
        # Every rank takes part in every collective below whatever happened locally, and all
        # ranks raise together: a rank that failed alone would leave the others waiting.
        err = None
        try:
            with torch.cuda.device(self.device):
                _ffi.check(L.vqk_peer_create(rank, world, max_rows, ctypes.byref(h), mine))
        except Exception as exc:  # noqa: BLE001
            err = f"rank {rank}: create: {exc}"
        self._h = h if err is None else None
        gathered = [None] * world
        dist.all_gather_object(gathered, (err, mine.raw), group=group)
        if err is None and all(e is None for e, _ in gathered):
            try:
                with torch.cuda.device(self.device):
                    _ffi.check(L.vqk_peer_connect(self._h, b"".join(hb for _, hb in gathered)))
            except Exception as exc:  # noqa: BLE001
                err = f"rank {rank}: connect: {exc}"
        errs = [None] * world
        dist.all_gather_object(errs, err if err is not None else next((e for e, _ in gathered if e), None), group=group)
        bad = [e for e in errs if e]
        if bad:
            self.close()
            raise RuntimeError("peer-memory exchange unavailable: " + "; ".join(sorted(set(bad))))
        dist.barrier(group=group)  # nobody pushes before every rank has mapped every buffer
        self.rank, self.world, self.max_rows = rank, world, max_rows

    def exchange_finalize(self, rec: torch.Tensor, sp: SamplingArgs):
        """This rank's records [B, 1024] in, (tokens, scores) of the merged step out;
        identical on every rank.  A peer that never shows up gives token -1."""
        assert rec.is_cuda and rec.dtype == torch.uint8 and rec.dim() == 2 and rec.shape[1] == _ffi.RECORD_BYTES
        rec = rec.contiguous()
        B = rec.shape[0]
        tokens = torch.empty(B, dtype=torch.int64, device=rec.device)
        scores = torch.empty(B, dtype=torch.float32, device=rec.device)
        spc = sp.to_c(B, sp.vocab_total if sp.vocab_total is not None else 0)
        if B:
            with torch.cuda.device(rec.device):
                _ffi.check(_ffi.lib().vqk_peer_exchange_finalize(
                    self._h, rec.data_ptr(), B, ctypes.byref(spc), tokens.data_ptr(), scores.data_ptr(),
                    torch.cuda.current_stream(rec.device).cuda_stream))
        return tokens, scores

    def set_wait_limit(self, polls: int) -> None:
        """Bound of every wait for a peer's words, in polls (the default is about a second).  A
        wait that runs out gives the row token -1 and raises `vqk_device_error`."""
        _ffi.check(_ffi.lib().vqk_peer_set_wait_limit(self._h, int(polls)))

    def close(self):
        if self._h:
            _ffi.lib().vqk_peer_destroy(self._h)
            self._h = None


def exchange_records(rec: torch.Tensor, group=None, comm: Optional[VqkComm] = None) -> torch.Tensor:
    """All-gather per-rank records [B, 1024] into [G, B, 1024] (rank-major).  With a
    VqkComm the collective runs on the current CUDA stream; otherwise through
    torch.distributed (NCCL for CUDA tensors, gloo for CPU tensors)."""
    if comm is not None:
        return comm.allgather(rec)
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(rec.shape), dtype=rec.dtype, device=rec.device)
    if rec.is_cuda:
        dist.all_gather_into_tensor(out, rec.contiguous(), group=group)
    else:
        parts = [out[i] for i in range(world)]
        dist.all_gather(parts, rec.contiguous(), group=group)
    return out


class VocabShardedLMHead:
    """One rank's part of a vocab-sharded lm_head + sampler step."""

    def __init__(self, shard: LMHeadShard, vocab_start: int, vocab_total: int, group=None,
                 comm: Optional[VqkComm] = None, peer: Optional["VqkPeer"] = None):
        self.shard = shard
        self.vocab_start = int(vocab_start)
        self.vocab_total = int(vocab_total)
        self.group = group
        self.comm = comm
        self.peer = peer  # exchange over peer memory fused with the merge; else all-gather + finalize

    def local_args(self, sp: SamplingArgs) -> SamplingArgs:
        return SamplingArgs(sp.temperature, sp.seeds, sp.top_k, sp.top_p, sp.topk_threshold,
                            vocab_offset=self.vocab_start, vocab_total=self.vocab_total)

    def step_host(self, x_host: torch.Tensor, sp_host: SamplingArgs, tokens_host: torch.Tensor,
                  bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The sharded step from HOST tensors in one library call (`LMHeadShard.step_host` with this
        rank's vocab offset and the peer handle); peer-memory exchange only.  Rows the records
        cannot carry come back as -1, as with ``unresolved="leave"``."""
        if self.peer is None:
            raise RuntimeError("step_host needs the peer-memory exchange (VqkPeer)")
        return self.shard.step_host(x_host, self.local_args(sp_host), tokens_host, peer_handle=self.peer._h, bias=bias)

    def host_stepper(self, x_host: torch.Tensor, sp_host: SamplingArgs, tokens_host: torch.Tensor,
                     bias: Optional[torch.Tensor] = None):
        """`step_host` bound to fixed host tensors (`LMHeadShard.host_stepper`)."""
        if self.peer is None:
            raise RuntimeError("host_stepper needs the peer-memory exchange (VqkPeer)")
        return self.shard.host_stepper(x_host, self.local_args(sp_host), tokens_host, peer_handle=self.peer._h, bias=bias)

    def step(self, hidden_states: torch.Tensor, sp: SamplingArgs, bias: Optional[torch.Tensor] = None,
             unresolved: str = "leave"):
        """(tokens int64 [B], scores fp32 [B]), identical on every rank.

        The one-exchange merge decides a row from the ranks' 1 KiB records.  A row whose record
        cannot hold what the merge needs - top-p without top-k (vLLM also marks a disabled top-k
        as k = vocab size), or more than 126 top-k survivors on one shard - comes back as token
        -1.  `unresolved` says what to do about it:
          "leave"  return the -1 (no host synchronisation: safe inside a CUDA-graph capture);
          "raise"  synchronise, raise RuntimeError if any row is -1;
          "rerun"  synchronise, and resolve the -1 rows exactly: their fp16 shard logits are
                   all-gathered (torch.distributed, 0.5 MB per row at 248320 columns) and the
                   single-shard sampler runs on the full rows; every rank gets the same tokens.
        """
        if unresolved not in ("leave", "raise", "rerun"):
            raise ValueError("unresolved must be 'leave', 'raise' or 'rerun'")
        lsp = self.local_args(sp)
        if self.peer is not None:
            tokens, scores = self.shard.step_sharded(hidden_states, lsp, self.peer._h, bias)
        else:
            rec = self.shard.shard_records(hidden_states, lsp, bias)
            gathered = exchange_records(rec, self.group, self.comm)
            tokens, scores = finalize_records(gathered, lsp)
        if unresolved == "leave":
            return tokens, scores
        missing = torch.nonzero(tokens < 0).flatten()      # host synchronisation
        if missing.numel() == 0:
            return tokens, scores
        if unresolved == "raise":
            raise RuntimeError(f"rows {missing.tolist()} cannot be merged from the shard records "
                               "(top-p without top-k, or more than 126 top-k survivors on a shard)")
        t2, s2 = self.resolve_rows(hidden_states, sp, missing, bias)
        tokens = tokens.clone()
        scores = scores.clone()
        tokens[missing] = t2
        scores[missing] = s2
        return tokens, scores

    def resolve_rows(self, hidden_states: torch.Tensor, sp: SamplingArgs, rows: torch.Tensor,
                     bias: Optional[torch.Tensor] = None):
        """Exact sampling of the given batch rows from the FULL logits rows: every rank computes its
        fp16 logits slice of those rows, the slices are all-gathered (torch.distributed on
        `self.group`), and the single-shard sampler runs on the concatenation.  All ranks must
        call it with the same rows."""
        import torch.distributed as dist
        x = hidden_states.reshape(-1, self.shard.H)[rows]
        local = self.shard.logits(x, bias)                                   # [n, V_local]
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        per = shard_bounds(self.vocab_total, world, 0)[1]
        padded = torch.full((local.shape[0], per), float("-inf"), dtype=local.dtype, device=local.device)
        padded[:, :local.shape[1]] = local
        if world > 1:
            parts = torch.empty((world,) + tuple(padded.shape), dtype=padded.dtype, device=padded.device)
            dist.all_gather_into_tensor(parts, padded, group=self.group)
        else:
            parts = padded.unsqueeze(0)
        full = parts.permute(1, 0, 2).reshape(local.shape[0], world * per)[:, :self.vocab_total].contiguous()

        def pick(t):
            return None if t is None else t[rows].contiguous()
        rsp = SamplingArgs(pick(sp.temperature), pick(sp.seeds), pick(sp.top_k), pick(sp.top_p),
                           pick(sp.topk_threshold), 0, self.vocab_total)
        return sample_logits(full, rsp)


# ---- record layout helpers (host side; used by tools and tests) -----------------------

_HDR = np.dtype([("score", "<f4"), ("token", "<i4"), ("n", "<i4"), ("flags", "<i4")])
_CAND = np.dtype([("v", "<f4"), ("t", "<i4")])


def pack_record(score: float = float("-inf"), token: int = -1, cands=(), flags: int = 0) -> np.ndarray:
    """One 1 KiB record as uint8: the 16-byte header then up to 126 (raw logit, token) pairs."""
    if len(cands) > _ffi.RECORD_CAP:
        raise ValueError("too many candidates for one record")
    buf = np.zeros(_ffi.RECORD_BYTES, dtype=np.uint8)
    hdr = buf[:16].view(_HDR)
    hdr["score"], hdr["token"], hdr["n"], hdr["flags"] = score, token, len(cands), flags
    body = buf[16:16 + 8 * len(cands)].view(_CAND)
    for i, (v, t) in enumerate(cands):
        body[i] = (v, t)
    return buf


def unpack_record(buf) -> dict:
    buf = np.ascontiguousarray(np.asarray(buf, dtype=np.uint8))
    hdr = buf[:16].view(_HDR)[0]
    n = int(hdr["n"])
    body = buf[16:16 + 8 * n].view(_CAND)
    return dict(score=float(hdr["score"]), token=int(hdr["token"]), n=n, flags=int(hdr["flags"]),
                cands=[(float(c["v"]), int(c["t"])) for c in body])
