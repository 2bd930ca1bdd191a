"""The interpreter-level fast paths of the host layer give exactly what the plain code gives:
scheduler decode rounds without queue surgery, and decode metadata from per-sequence table rows."""
import itertools
import random

import numpy as np
import pytest

from llm_from_scratch_b200.engine import SamplingParams, Sequence, metadata as md
from llm_from_scratch_b200.engine.llm_engine import LLMEngine
from llm_from_scratch_b200.engine.scheduler import Scheduler


class _Runner:
    """Stands in for the GPU: samples pseudo-random tokens, records what it was asked to run."""

    def __init__(self, blocks, block_size, check_builder=False):
        self.num_kv_blocks, self.block_size = blocks, block_size
        self.rng = random.Random(7)
        self.log = []
        self.builder = md.DecodeBatchBuilder(block_size, 64, rows=8) if check_builder else None
        # a second builder drives a stand-in for the device-resident table through patches only
        self.patcher = md.DecodeBatchBuilder(block_size, 64, rows=8, device_rows=16) if check_builder else None
        self.dev_tables = np.full((16, 64), -9, dtype=np.int32)
        self.patch_counts = []

    def run(self, seqs, is_prefill):
        self.log.append((is_prefill, [s.seq_id for s in seqs], [list(s.block_table) for s in seqs]))
        if self.builder is not None:
            if is_prefill:
                self.builder.invalidate(seqs)
                self.patcher.invalidate(seqs)
            else:
                want = md.prepare_decode(seqs, self.block_size)
                n = len(seqs)
                ids, slots, lens = (np.full(n + 3, -7, dtype=np.int64) for _ in range(3))
                tables = np.full((n + 3, 64), -7, dtype=np.int32)
                self.builder.build(seqs, ids, slots, lens, tables)
                assert np.array_equal(ids[:n], want.input_ids) and np.array_equal(slots[:n], want.slot_mapping)
                assert np.array_equal(lens[:n], want.context_lens)
                for i, s in enumerate(seqs):      # entries past a sequence's table are not part of the contract
                    k = len(s.block_table)
                    assert np.array_equal(tables[i, :k], want.block_tables[i, :k])
                assert (ids[n:] == -7).all() and (tables[n:] == -7).all()
                # incremental form: apply the patches (or the full upload when they do not fit) to the
                # persistent table; every sequence's entries must then be what the full rebuild gives
                patches = np.zeros((6, 3), dtype=np.int32)
                full = np.full((n, 64), -7, dtype=np.int32)
                ids2, slots2, lens2 = (np.zeros(n, dtype=np.int64) for _ in range(3))
                cnt = self.patcher.build(seqs, ids2, slots2, lens2, full, patches=patches)
                self.patch_counts.append(cnt)
                if cnt >= 0:
                    for r, c, v in patches[:cnt].tolist():
                        self.dev_tables[r, c] = v
                else:
                    for i, s in enumerate(seqs):
                        self.dev_tables[i, :len(s.block_table)] = full[i, :len(s.block_table)]
                assert np.array_equal(ids2, want.input_ids) and np.array_equal(slots2, want.slot_mapping)
                for i, s in enumerate(seqs):
                    k = len(s.block_table)
                    assert np.array_equal(self.dev_tables[i, :k], want.block_tables[i, :k]), (i, cnt)
        return [self.rng.randrange(50) for _ in seqs]

    def exit(self):
        pass


def _serve(blocks, general_only=False, check_builder=False, n_req=40, seed=3):
    Sequence.counter = itertools.count()
    rng = random.Random(seed)
    runner = _Runner(blocks, 4, check_builder)
    eng = LLMEngine(dict(block_size=4, max_num_sequences=6, max_num_batched_tokens=64, eos=-1), runner=runner)
    if general_only:
        sched = eng.scheduler
        limit = min(sched.max_num_sequences, sched.max_num_batched_tokens)
        sched._grow_running = lambda: Scheduler._grow_running_general(sched, limit)
    pending = [[rng.randrange(50) for _ in range(rng.randrange(1, 30))] for _ in range(n_req)]
    outs = {}
    while pending or not eng.is_finished():
        for _ in range(rng.randrange(0, 3)):          # requests trickle in while others decode
            if pending:
                eng.add_request(pending.pop(), SamplingParams(temperature=0.0, max_tokens=rng.randrange(2, 25),
                                                              ignore_eos=True))
        done, _n, _p = eng.step()
        outs.update(done)
    _serve.last_runner = runner
    return runner.log, outs


@pytest.mark.parametrize("blocks", [400, 24, 14])      # ample pool, and pools small enough to preempt
def test_decode_round_fast_path_equals_the_general_loop(blocks):
    fast_log, fast_out = _serve(blocks)
    slow_log, slow_out = _serve(blocks, general_only=True)
    assert fast_log == slow_log and fast_out == slow_out
    assert any(not p for p, _, _ in fast_log) and any(p for p, _, _ in fast_log)


@pytest.mark.parametrize("blocks", [400, 14])
def test_decode_batch_builder_equals_prepare_decode(blocks):
    """Rows are reused (8 rows at first, 6 running sequences, 40 requests), tables grow, and with the
    small pool sequences are preempted and prefilled again into different blocks."""
    log, _ = _serve(blocks, check_builder=True)
    assert sum(1 for p, _, _ in log if not p) > 20
    counts = _serve.last_runner.patch_counts
    # steady batches ship nothing or a block or two; a new composition falls back to the full table
    assert counts.count(0) > 5 and any(0 < c <= 6 for c in counts) and -1 in counts


def test_decode_batch_builder_rejects_rows_of_another_builder():
    Sequence.block_size = 4
    a, b = md.DecodeBatchBuilder(4, 8, rows=4), md.DecodeBatchBuilder(4, 8, rows=4)
    seqs = []
    for i in range(3):
        s = Sequence(list(range(5 + i)), SamplingParams())
        s.block_table = [10 * i, 10 * i + 1]
        seqs.append(s)
    outs = lambda: (np.zeros(3, np.int64), np.zeros(3, np.int64), np.zeros(3, np.int64), np.zeros((3, 8), np.int32))
    oa, ob = outs(), outs()
    a.build(seqs, *oa)
    b.build(list(reversed(seqs)), *ob)             # same sequences, rows assigned in another order
    want = md.prepare_decode(list(reversed(seqs)), 4)
    assert np.array_equal(ob[1], want.slot_mapping) and np.array_equal(ob[3][:, :2], want.block_tables)
    a.build(seqs, *oa)                              # a's rows are no longer the sequences' rows: reassigned
    want = md.prepare_decode(seqs, 4)
    assert np.array_equal(oa[1], want.slot_mapping) and np.array_equal(oa[3][:, :2], want.block_tables)


def test_block_hash_chain_equals_block_by_block_hashing():
    from llm_from_scratch_b200 import ops
    rng = random.Random(1)
    for n in (0, 1, 15, 16, 17, 100, 160):
        ids = [rng.randrange(32000) for _ in range(n)]
        h, want = -1, []
        for i in range(n // 16):
            h = ops.block_hash(ids[i * 16:(i + 1) * 16], h)
            want.append(h)
        assert ops.block_hash_chain(ids, 16) == want


class _WindowRunner:
    """Greedy stand-in whose token depends only on the request's own tokens.  ``run_window`` plays the
    device's part of a window: it carries each row's tokens forward itself and checks that the block the
    new position falls into was opened before the window started."""

    def __init__(self, blocks, block_size, max_len=512):
        self.num_kv_blocks, self.block_size, self.max_model_length = blocks, block_size, max_len
        self.windows = []

    @staticmethod
    def _token(tokens):
        return (sum(tokens[-3:]) * 31 + len(tokens) * 7) % 50

    def run(self, seqs, is_prefill):
        return [self._token(s.token_ids) for s in seqs]

    def can_run_window(self, seqs):
        return True

    def run_window(self, seqs, steps):
        self.windows.append(steps)
        rows = [list(s.token_ids) for s in seqs]
        tables = [list(s.block_table) for s in seqs]
        out = []
        for _ in range(steps):
            for r, t in zip(rows, tables):
                assert (len(r) - 1) // self.block_size < len(t), "position without a block"
            toks = [self._token(r) for r in rows]
            for r, tok in zip(rows, toks):
                r.append(tok)
            out.append(toks)
        return out

    def exit(self):
        pass


def _serve_windowed(window, blocks, eos, seed=5, n_req=30):
    Sequence.counter = itertools.count()
    rng = random.Random(seed)
    runner = _WindowRunner(blocks, 4)
    eng = LLMEngine(dict(block_size=4, max_num_sequences=5, max_num_batched_tokens=64, eos=eos,
                         decode_window=window), runner=runner)
    for _ in range(n_req):
        eng.add_request([rng.randrange(50) for _ in range(rng.randrange(1, 30))],
                        SamplingParams(temperature=0.0, max_tokens=rng.randrange(2, 40), ignore_eos=eos < 0))
    outs = {}
    while not eng.is_finished():
        done, _n, _p = eng.step()
        outs.update(done)
    bm = eng.scheduler.block_manager
    assert bm.num_free_blocks == blocks and not bm.used_block_ids
    return outs, set(bm.hash_to_block_id), runner.windows


@pytest.mark.parametrize("eos", [-1, 7])                # stops by max_tokens only, and by a sampled end token too
@pytest.mark.parametrize("blocks", [400, 40])
def test_decode_windows_give_the_step_by_step_tokens(blocks, eos):
    """Several decode steps per scheduling decision: the same tokens per request as one step at a time
    (a request's tokens depend on nothing but its own), every block sealed with the same hash, the pool
    whole again at the end; sequences that stop inside a window lose their surplus tokens."""
    want, want_hashes, _ = _serve_windowed(1, blocks, eos)
    got, got_hashes, windows = _serve_windowed(4, blocks, eos)
    assert got == want
    assert got_hashes == want_hashes
    assert windows and max(windows) == 4


def test_decode_window_planning_respects_length_and_pool_limits():
    """The window never runs past the block table's capacity, ends where the longest-lived sequence stops,
    opens exactly the blocks the extra steps write into, and collapses to 1 when the pool cannot cover them."""
    Sequence.counter = itertools.count()
    Sequence.block_size = 4
    sched = Scheduler(max_num_sequences=4, max_num_batched_tokens=64, max_cached_blocks=8, block_size=4, eos=-1)
    a = Sequence(list(range(6)), SamplingParams(temperature=0.0, max_tokens=50, ignore_eos=True))
    b = Sequence(list(range(3)), SamplingParams(temperature=0.0, max_tokens=50, ignore_eos=True))
    for s in (a, b):
        sched.add_sequence(s)
    seqs, is_prefill = sched.schedule()
    assert is_prefill and seqs == [a, b]
    sched.postprocess(seqs, [1, 2])                      # lengths 7 and 4
    seqs, is_prefill = sched.schedule()                  # decode round: b (4 = full block) is sealed
    assert not is_prefill
    tables = [list(s.block_table) for s in seqs]
    # 30 positions at most: a (7 tokens) could run 24 steps, the table bound cuts the window at 30 - 7 + 1
    assert sched.plan_decode_window(seqs, 4, 30) == 4
    # steps 2-4 write positions 7,8,9 of a (block 1, then block 2 opened ahead) and 4,5,6 of b (block 1 opened ahead)
    assert len(a.block_table) == len(tables[0]) + 1 and len(b.block_table) == len(tables[1]) + 1
    assert sched.plan_decode_window(seqs, 4, 8) == 2     # a has room for one more step only (8 - 7 + 1)
    a.max_tokens = b.max_tokens = 3                      # both stop after their next token
    assert sched.plan_decode_window(seqs, 4, 30) == 1
    a.max_tokens = b.max_tokens = 50
    free = sched.block_manager.num_free_blocks
    for _ in range(free):                                # drain the pool: nothing can be opened ahead
        sched.block_manager.open_block(a)
    a.num_tokens = 8                                     # next lengths 9.. would start a block
    assert sched.plan_decode_window(seqs, 4, 300) == 1
