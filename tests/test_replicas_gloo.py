"""Request sharding across engine replicas, exercised with two CPU ranks over gloo.

The replicas use the real scheduler / block manager / engine loop with a stand-in executor (a pure
function of sequence id and length), so the test covers exactly the multi-rank host logic: shard,
serve, gather, merge — and that the merged streams equal a single-replica run.
"""
import itertools
import os
import sys

import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class FakeRunner:
    num_kv_blocks = 512

    def run(self, seqs, is_prefill):
        # depends only on the request's own tokens, like a real model under greedy decoding
        return [(sum(s.token_ids[-3:]) * 31 + s.num_tokens * 7) % 1000 for s in seqs]

    def exit(self):
        pass


def _requests():
    import random
    from llm_from_scratch_b200.engine import SamplingParams
    rng = random.Random(3)
    return [([rng.randrange(1000) for _ in range(rng.randint(3, 70))],
             SamplingParams(temperature=0.0, max_tokens=rng.randint(2, 20), ignore_eos=True)) for _ in range(23)]


def _make_engine(rank):
    from llm_from_scratch_b200.engine import Sequence
    from llm_from_scratch_b200.engine.llm_engine import LLMEngine
    Sequence.counter = itertools.count()
    cfg = dict(block_size=16, max_num_sequences=4, max_num_batched_tokens=256, eos=-1)
    return LLMEngine(cfg, runner=FakeRunner())


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from llm_from_scratch_b200.engine.replicas import serve_sharded
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        tokens, reports = serve_sharded(_make_engine, _requests())
        if rank == 0:
            q.put((tokens, [(r.rank, r.decode_tokens, r.prefill_tokens, len(r.token_ids)) for r in reports]))
        else:
            assert tokens is None and reports is None
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_shard_and_merge_are_inverse():
    from llm_from_scratch_b200.engine.replicas import merge_outputs, shard_requests
    items = list(range(11))
    for world in (1, 2, 3, 4, 8):
        shards = [shard_requests(items, world, r) for r in range(world)]
        assert sorted(x for s in shards for x in s) == items
        assert merge_outputs(shards, len(items)) == items
    with pytest.raises(ValueError):
        merge_outputs([[0], []], 3)


@pytest.mark.timeout(180)
def test_two_replicas_over_gloo_match_one_replica():
    from llm_from_scratch_b200.engine.replicas import serve_sharded
    want, _ = serve_sharded(_make_engine, _requests())
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    tokens, summary = q.get(timeout=150)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert tokens == want
    assert [s[0] for s in summary] == [0, 1] and [s[3] for s in summary] == [12, 11]
    assert sum(s[1] for s in summary) > 0 and sum(s[2] for s in summary) > 0


def test_online_arrivals_give_the_same_streams_as_offline():
    """Requests handed over as their (Poisson) arrival times pass produce the same completions: a
    request's stream depends only on its own tokens."""
    from llm_from_scratch_b200.engine.replicas import serve_shard
    reqs = _requests()[:9]
    offline = serve_shard(_make_engine(0), reqs).token_ids
    arrivals = [0.0, 0.0, 0.002, 0.004, 0.004, 0.01, 0.03, 0.03, 0.05]
    online = serve_shard(_make_engine(0), reqs, arrivals=arrivals)
    assert online.token_ids == offline
    assert online.wall_s >= 0.05
    # per-request clock: arrival <= first token <= completion <= end of the run, one entry per request
    assert online.arrival_s == arrivals and len(online.first_token_s) == len(online.finish_s) == len(reqs)
    for a, f, d, toks in zip(online.arrival_s, online.first_token_s, online.finish_s, online.token_ids):
        assert a <= f <= d <= online.wall_s and f > 0.0
        assert len(toks) > 1 or f == d                     # a one-token request finishes in its prefill step
    from llm_from_scratch_b200.microbench import request_latencies
    lat = request_latencies([online])
    assert 0.0 <= lat["ttft_ms"]["p50"] <= lat["ttft_ms"]["p99"] <= 1e3 * online.wall_s
    assert lat["request_s"]["p99"] <= online.wall_s and lat["ms_per_output_token"]["mean"] > 0.0
