"""Default (non reference-exact) block pool and scheduler: invariants the reference's ref-count
arithmetic breaks, and agreement with the reference-exact mode wherever the reference is sound."""
import itertools
import random

import pytest
from hypothesis import given, settings, strategies as st

from llm_from_scratch_b200.engine import BlockManager, Scheduler, Sequence, SamplingParams
from llm_from_scratch_b200.engine import metadata


@pytest.fixture(autouse=True)
def _fresh():
    Sequence.block_size = 16
    Sequence.counter = itertools.count()
    Sequence.reference_exact = False
    yield
    Sequence.reference_exact = False


def check_pool(bm: BlockManager, live):
    free, used = set(bm.free_block_ids), set(bm.used_block_ids)
    assert not (free & used) and len(free) + len(used) == len(bm.blocks)
    refs = {}
    for s in live:
        for b in s.block_table:
            refs[b] = refs.get(b, 0) + 1
    assert set(refs) == used
    for b, n in refs.items():
        assert bm.blocks[b].ref_count == n


def test_blocks_return_to_the_pool_and_shared_blocks_outlive_their_first_user():
    bm = BlockManager(8, 16)
    a, b = Sequence(list(range(40))), Sequence(list(range(40)))
    bm.allocate(a)
    bm.allocate(b)
    assert a.block_table[:2] == b.block_table[:2] and a.block_table[2] != b.block_table[2]
    assert b.num_cached_tokens == 32
    check_pool(bm, [a, b])
    shared = list(a.block_table[:2])
    bm.deallocate(a)
    check_pool(bm, [b])
    assert all(x in bm.used_block_ids for x in shared)      # still referenced by b
    bm.deallocate(b)
    check_pool(bm, [])
    assert bm.num_free_blocks == 8
    # contents survive release: a third identical request revives the cached prefix
    c = Sequence(list(range(40)))
    bm.allocate(c)
    assert c.num_cached_tokens == 32 and c.block_table[:2] == shared


def test_exactly_full_prompt_gets_slots_for_every_token_and_decodes_into_a_new_block():
    bm = BlockManager(8, 16)
    s = Sequence(list(range(32)))
    bm.allocate(s)
    md = metadata.prepare_prefill([s], 16)
    assert md.slot_mapping.tolist() == [b * 16 + i for b in s.block_table for i in range(16)]
    s.append_token(5)
    assert bm.can_append(s)
    bm.append(s)
    assert len(s.block_table) == 3
    md = metadata.prepare_decode([s], 16)
    assert md.slot_mapping.tolist() == [s.block_table[2] * 16]
    for _ in range(15):
        s.append_token(1)
        bm.append(s)
    md = metadata.prepare_decode([s], 16)          # 48 tokens: last slot of the third block
    assert md.slot_mapping.tolist() == [s.block_table[2] * 16 + 15]
    assert bm.blocks[s.block_table[2]].hash == bm.compute_hash(s.token_ids[32:48], bm.blocks[s.block_table[1]].hash)


def _run(engine_cfg, requests, exact, steps=400):
    Sequence.counter = itertools.count()
    Sequence.block_size = engine_cfg["block_size"]
    Sequence.reference_exact = exact
    sched = Scheduler(**engine_cfg, reference_exact=exact)
    for toks, mt in requests:
        sched.add_sequence(Sequence(toks, SamplingParams(max_tokens=mt, ignore_eos=True)))
    trace = []
    for _ in range(steps):
        if sched.is_finished():
            break
        seqs, is_prefill = sched.schedule()
        if not seqs:
            break
        md = (metadata.prepare_prefill if is_prefill else metadata.prepare_decode)(seqs, engine_cfg["block_size"])
        trace.append((is_prefill, [s.seq_id for s in seqs], [list(s.block_table) for s in seqs],
                      [s.num_tokens for s in seqs], md.slot_mapping.tolist()))
        sched.postprocess(seqs, [(s.seq_id * 31 + s.num_tokens) % 1000 for s in seqs])
    return trace, sched


def test_default_mode_equals_reference_exact_mode_away_from_block_multiples():
    """Distinct prompts, ample pool, no batch-size truncation: the two modes may differ only on
    steps where some sequence length is an exact multiple of the block size."""
    rng = random.Random(5)
    reqs = [([rng.randrange(1000) for _ in range(rng.choice([5, 17, 30, 45, 61]))], rng.randint(3, 25)) for _ in range(6)]
    cfg = dict(max_num_sequences=8, max_num_batched_tokens=4096, max_cached_blocks=512, block_size=16, eos=-1)
    a, _ = _run(cfg, reqs, exact=False)
    b, _ = _run(cfg, reqs, exact=True)
    assert len(a) == len(b)
    for sa, sb in zip(a, b):
        assert sa[:4] == sb[:4]                       # same schedule, same tables, same lengths
        clean = [i for i, n in enumerate(sa[3]) if n % 16 != 0]
        if not sa[0]:
            assert [sa[4][i] for i in clean] == [sb[4][i] for i in clean]


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.integers(1, 70), st.integers(2, 40), st.integers(0, 3)), min_size=1, max_size=10),
       st.integers(6, 40))
def test_default_mode_invariants_under_pressure(reqs, num_blocks):
    """Random workloads on small pools (preemption happens): every scheduled token owns the slot
    block_table[pos // bs] * bs + pos % bs, no two live sequences share a partially filled block,
    the pool partition stays consistent, and every request that fits the pool finishes."""
    bs = 8
    Sequence.block_size = bs
    Sequence.counter = itertools.count()
    prefixes = [[7] * 16, [9] * 24, [], [3] * 8]
    sched = Scheduler(max_num_sequences=4, max_num_batched_tokens=128, max_cached_blocks=num_blocks,
                      block_size=bs, eos=-1)
    all_seqs = []
    for n, mt, p in reqs:
        toks = (prefixes[p] + list(range(100, 100 + n)))[:60]
        if -(-(len(toks) + mt) // bs) > num_blocks:
            continue
        s = Sequence(toks, SamplingParams(max_tokens=mt, ignore_eos=True))
        all_seqs.append(s)
        sched.add_sequence(s)
    for _ in range(3000):
        if sched.is_finished():
            break
        seqs, is_prefill = sched.schedule()
        assert seqs, "scheduler made no progress"
        md = (metadata.prepare_prefill if is_prefill else metadata.prepare_decode)(seqs, bs)
        assert len(md.slot_mapping) == len(md.input_ids)
        k = 0
        for s in seqs:
            span = range(s.num_cached_tokens, s.num_tokens) if is_prefill else [s.num_tokens - 1]
            for pos in span:
                assert md.slot_mapping[k] == s.block_table[pos // bs] * bs + pos % bs
                assert md.positions[k] == pos
                k += 1
        check_pool(sched.block_manager, list(sched.running))
        sched.postprocess(seqs, [1] * len(seqs))
    assert sched.is_finished()
    assert all(s.is_finished and s.num_completion_tokens == s.max_tokens - 1 for s in all_seqs)
    assert sched.block_manager.num_free_blocks == num_blocks


def test_a_fully_cached_prompt_still_has_a_token_to_run():
    """A repeated prompt whose length is a multiple of the block size hits on every block; the last block is
    recomputed into a fresh one so that the prefill step has a query token (and a logits row) for the request."""
    bm = BlockManager(8, 16)
    a, b = Sequence(list(range(32))), Sequence(list(range(32)))
    bm.allocate(a)
    bm.allocate(b)
    assert a.num_cached_tokens == 0 and b.num_cached_tokens == 16
    assert b.block_table[0] == a.block_table[0] and b.block_table[1] != a.block_table[1]
    check_pool(bm, [a, b])
    md = metadata.prepare_prefill([a, b], 16)
    assert md.cu_seqlens_q.tolist() == [0, 32, 48] and md.cu_seqlens_k.tolist() == [0, 32, 64]
    assert md.last_token_index.tolist() == [31, 47]
    assert md.slot_mapping[32:].tolist() == [b.block_table[1] * 16 + i for i in range(16)]
    # a single-block prompt repeated: nothing may be reused
    c, d = Sequence(list(range(100, 116))), Sequence(list(range(100, 116)))
    bm.allocate(c)
    bm.allocate(d)
    assert d.num_cached_tokens == 0 and d.block_table != c.block_table
    # a longer prompt sharing the same first two blocks reuses both
    e = Sequence(list(range(40)))
    bm.allocate(e)
    assert e.num_cached_tokens == 32
    for s in (a, b, c, d, e):
        bm.deallocate(s)
    check_pool(bm, [])
