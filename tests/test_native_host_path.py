"""The C++ host path (block pool and step metadata behind the C ABI) against the Python classes it replaces in the
engine's default mode: same block tables, prefix hits, free-list order, reference counts and hash entries on
random request traces, and the same metadata arrays."""
import itertools
import random

import numpy as np
import pytest

from llm_from_scratch_b200.engine import BlockManager, NativeBlockManager, Scheduler, Sequence, SamplingParams
from llm_from_scratch_b200.engine import metadata


@pytest.fixture(autouse=True)
def _fresh():
    Sequence.block_size = 16
    Sequence.counter = itertools.count()
    Sequence.reference_exact = False
    yield


def same_state(a: BlockManager, b: NativeBlockManager):
    assert list(a.free_block_ids) == b.free_block_ids
    assert set(a.used_block_ids) == b.used_block_ids
    va, vb = a.blocks, b.blocks
    assert [x.ref_count for x in va] == [x.ref_count for x in vb]
    # hashes of live or revivable blocks (a fresh block's hash is -1 in both)
    assert [x.hash for x in va] == [x.hash for x in vb]
    assert a.hash_to_block_id == b.hash_to_block_id


@pytest.mark.parametrize("seed", range(6))
def test_native_pool_follows_the_python_pool_on_random_traces(seed):
    """Requests with shared prefixes arrive, decode for a while and leave, in random order, against a pool small
    enough that blocks are recycled (and stale hash entries dropped) all the time."""
    rng = random.Random(seed)
    bs, blocks = 16, 48
    a, b = BlockManager(blocks, bs), NativeBlockManager(blocks, bs)
    prefixes = [[rng.randrange(100) for _ in range(rng.choice([16, 32, 48, 40]))] for _ in range(4)]
    live = []
    for step in range(400):
        op = rng.random()
        if op < 0.35 or not live:
            toks = list(rng.choice(prefixes)) if rng.random() < 0.7 else []
            toks += [rng.randrange(100) for _ in range(rng.randrange(0, 40))]
            toks = toks or [1]
            sa, sb = Sequence(toks), Sequence(toks)
            if a.can_allocate(sa):
                assert b.can_allocate(sb)
                a.allocate(sa)
                b.allocate(sb)
                assert sa.block_table == sb.block_table and sa.num_cached_tokens == sb.num_cached_tokens
                live.append((sa, sb))
        elif op < 0.85:
            sa, sb = rng.choice(live)
            for _ in range(rng.randrange(1, 20)):      # decode steps: append a token, then grow / seal
                tok = rng.randrange(100)
                sa.append_token(tok)
                sb.append_token(tok)
                if not a.can_append(sa):           # the scheduler would preempt: take the token back
                    assert not b.can_append(sb)
                    for s in (sa, sb):
                        s.token_ids.pop()
                        s.num_tokens -= 1
                        s.last_token = s.token_ids[-1]
                    break
                a.append(sa)
                b.append(sb)
                assert sa.block_table == sb.block_table
        else:
            sa, sb = live.pop(rng.randrange(len(live)))
            a.deallocate(sa)
            b.deallocate(sb)
        if step % 25 == 0:
            same_state(a, b)
    for sa, sb in live:
        a.deallocate(sa)
        b.deallocate(sb)
    same_state(a, b)
    assert b.num_free_blocks == blocks


def test_native_pool_runs_the_scheduler_like_the_python_pool():
    """Two schedulers, one per pool, over the same requests with preemptions (a pool too small for all of them):
    identical batches, tables and cached-token counts at every step."""
    rng = random.Random(3)
    reqs = [([rng.randrange(50) for _ in range(rng.randrange(1, 70))], rng.randrange(2, 60)) for _ in range(30)]
    runs = []
    for native in (False, True):
        Sequence.counter = itertools.count()
        sch = Scheduler(max_num_sequences=6, max_num_batched_tokens=128, max_cached_blocks=20, block_size=16, eos=-1,
                        native_pool=native)
        assert isinstance(sch.block_manager, NativeBlockManager) == native
        for toks, mx in reqs:
            sch.add_sequence(Sequence(toks, SamplingParams(temperature=0.0, max_tokens=mx, ignore_eos=True)))
        trace, tok_rng = [], random.Random(9)
        while not sch.is_finished():
            batch, is_prefill = sch.schedule()
            assert batch
            trace.append((is_prefill, [(s.seq_id, list(s.block_table), s.num_cached_tokens) for s in batch]))
            sch.postprocess(batch, [tok_rng.randrange(50) for _ in batch])
        runs.append(trace)
    assert runs[0] == runs[1]


def test_native_metadata_builders_equal_the_numpy_builders():
    rng = random.Random(5)
    bm = NativeBlockManager(200, 16)
    shared = [rng.randrange(100) for _ in range(48)]
    seqs = []
    for i in range(9):
        toks = (shared if i % 2 else []) + [rng.randrange(100) for _ in range(rng.randrange(1, 90))]
        s = Sequence(toks)
        bm.allocate(s)
        seqs.append(s)
    assert any(s.num_cached_tokens for s in seqs)
    got, want = metadata.prepare_prefill(seqs, 16), metadata.prepare_prefill_py(seqs, 16)
    for name in ("input_ids", "slot_mapping", "positions", "cu_seqlens_q", "cu_seqlens_k", "block_tables",
                 "last_token_index"):
        x, y = getattr(got, name), getattr(want, name)
        assert (x is None) == (y is None), name
        if x is not None:
            assert x.dtype == y.dtype and np.array_equal(x, y), name
    assert (got.max_seqlen_q, got.max_seqlen_k) == (want.max_seqlen_q, want.max_seqlen_k)
    for s in seqs:
        for _ in range(rng.randrange(1, 40)):
            s.append_token(rng.randrange(100))
            bm.append(s)
    got, want = metadata.prepare_decode(seqs, 16), metadata.prepare_decode_py(seqs, 16)
    for name in ("input_ids", "slot_mapping", "positions", "context_lens", "block_tables", "last_token_index"):
        x, y = getattr(got, name), getattr(want, name)
        assert x.dtype == y.dtype and np.array_equal(x, y), name
