"""Data-parallel serving: independent engine replicas, one per GPU, no collective on the hot path.

The reference's only multi-GPU scaffold is tensor-parallel worker processes that are never given
sharded layers (engine/llm_engine.py:38-50, engine/model_runner.py:66-134).  This design shards
REQUESTS instead: request i goes to replica ``i mod N``; every replica owns its scheduler, block
pool and KV cache, so the token stream of a request is bit-identical to what a single-GPU run of
the same sub-list produces.  ``torch.distributed`` is used only off the hot path, to hand the
results and timing back to rank 0 (``gather_object``) — NCCL on GPUs, gloo on CPU ranks in tests.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field


def shard_requests(requests: list, world_size: int, rank: int) -> list:
    """The sub-list of ``requests`` served by ``rank`` (round-robin by arrival index)."""
    return requests[rank::world_size]


def merge_outputs(per_rank: list[list], total: int) -> list:
    """Inverse of ``shard_requests``: per-rank result lists back into arrival order."""
    world = len(per_rank)
    out = [None] * total
    for r, items in enumerate(per_rank):
        for j, item in enumerate(items):
            out[r + j * world] = item
    if any(x is None for x in out):
        raise ValueError("replica results do not cover every request")
    return out


@dataclass
class ReplicaReport:
    rank: int
    token_ids: list = field(default_factory=list)     # completions of this rank's shard, in shard order
    wall_s: float = 0.0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    steps: int = 0
    timing: dict = field(default_factory=dict)        # the engine's per-component wall times for this shard
    # online runs only, one entry per request of the shard (seconds from the start of the run): when it arrived,
    # when the step that produced its first token ended, when the step that finished it ended
    arrival_s: list = field(default_factory=list)
    first_token_s: list = field(default_factory=list)
    finish_s: list = field(default_factory=list)


def serve_shard(engine, shard: list, rank: int = 0, arrivals=None) -> ReplicaReport:
    """Runs one replica over its shard: ``shard`` is a list of (token_ids, SamplingParams).

    ``arrivals`` (seconds from the start, one per request, non-decreasing) turns the run into an online
    one: a request is handed to the scheduler only once the wall clock has passed its arrival time, and
    the replica sleeps when it is idle before the next arrival.  Without it every request is present
    at t = 0.
    """
    rep = ReplicaReport(rank=rank)
    before = dict(getattr(engine, "timing", {}))
    t0 = time.perf_counter()
    if arrivals is None:
        seqs = [engine.add_request(tok, sp) for tok, sp in shard]
        pending = 0
    else:
        seqs, pending = [], 0
        rep.arrival_s = [float(a) for a in arrivals[:len(shard)]]
        rep.first_token_s = [0.0] * len(shard)
        rep.finish_s = [0.0] * len(shard)
    index_of = {}             # seq_id -> position in the shard (online runs)
    unstarted = 0             # requests before this position have their first token (admission is first come, first served)
    while pending < (len(shard) if arrivals is not None else 0) or not engine.is_finished():
        if arrivals is not None:
            now = time.perf_counter() - t0
            while pending < len(shard) and arrivals[pending] <= now:
                seqs.append(engine.add_request(*shard[pending]))
                index_of[seqs[-1].seq_id] = pending
                pending += 1
            if engine.is_finished():
                if pending < len(shard):
                    time.sleep(max(0.0, arrivals[pending] - (time.perf_counter() - t0)))
                continue
        outputs, n, is_prefill = engine.step()
        if n == 0 and not outputs:
            raise RuntimeError("nothing schedulable: KV pool too small for the waiting request")
        rep.steps += 1
        if is_prefill:
            rep.prefill_tokens += n
        else:
            rep.decode_tokens += n
        if arrivals is not None:
            now = time.perf_counter() - t0
            if is_prefill:
                while unstarted < len(seqs) and seqs[unstarted].num_tokens > seqs[unstarted].num_prompt_tokens:
                    rep.first_token_s[unstarted] = now
                    unstarted += 1
            for seq_id, _ in outputs:
                rep.finish_s[index_of[seq_id]] = now
    rep.wall_s = time.perf_counter() - t0
    rep.timing = {k: v - before.get(k, 0) for k, v in getattr(engine, "timing", {}).items()}
    rep.token_ids = [s.completion_token_ids for s in seqs]
    return rep


def serve_sharded(make_engine, requests: list, arrivals=None):
    """Every rank of the initialised process group serves its shard; rank 0 gets
    ``(token_ids in arrival order, [ReplicaReport per rank])``, other ranks get ``(None, None)``.

    ``make_engine(rank)`` builds the replica's engine (on ``cuda:LOCAL_RANK`` for GPU runs).
    Without an initialised process group this is a single replica.
    """
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        rep = serve_shard(make_engine(0), requests, 0, arrivals)
        return rep.token_ids, [rep]
    rank, world = dist.get_rank(), dist.get_world_size()
    rep = serve_shard(make_engine(rank), shard_requests(requests, world, rank), rank,
                      None if arrivals is None else shard_requests(list(arrivals), world, rank))
    gathered = [None] * world if rank == 0 else None
    dist.gather_object(rep, gathered, dst=0)
    if rank != 0:
        return None, None
    return merge_outputs([r.token_ids for r in gathered], len(requests)), gathered
