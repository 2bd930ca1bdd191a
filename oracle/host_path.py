"""Integer-exact CPU restatement of the reference's host path (test oracle).

Restates, defects included, what these reference files compute:

* engine/sequence.py:14-114      -> ``OracleSeq``
* engine/block_manager.py:8-157  -> ``OraclePool``
* engine/scheduler.py:8-95       -> ``OracleScheduler``
* engine/model_runner.py:202-278 -> ``prepare_prefill`` / ``prepare_decode`` (metadata only)

The restatement is deliberately literal about behaviour, because bit-exact parity of block tables
and slot mappings depends on the reference's quirks:

* a block's ref-count starts at 0, so an unshared block drops to -1 on release and never returns
  to the free list, and a shared block is released by its first finisher (block_manager.py:23-26,
  116-127);
* ``last_block_num_tokens`` is 0 when the length is a multiple of the block size
  (sequence.py:66-69), which makes ``block(last)`` return the whole token list (sequence.py:76),
  drops the slots of a prompt's exactly-full last block (model_runner.py:229-230) and points the
  decode slot one before the last block's first slot (model_runner.py:261);
* ``max_tokens = N`` stops after N-1 generated tokens (scheduler.py:89).

It is checked step by step against recordings of the reference itself
(``tests/golden/host_path.json.gz``).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from itertools import count

from .xxh64 import block_hash

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class OracleParams:
    temperature: float = 1.0
    max_tokens: int = 256
    ignore_eos: bool = False
    max_model_length: int | None = None


class OracleSeq:
    """sequence.py:14-86."""
    ids = count()

    def __init__(self, token_ids, params: OracleParams, block_size: int):
        self.seq_id = next(OracleSeq.ids)
        self.bs = block_size
        self.status = WAITING
        self.tokens = list(token_ids)
        self.n_prompt = len(self.tokens)
        self.n_cached = 0
        self.table: list[int] = []
        self.params = params

    def __len__(self):
        return len(self.tokens)

    @property
    def n_blocks(self) -> int:            # sequence.py:62-64
        return -(-len(self.tokens) // self.bs)

    @property
    def n_cached_blocks(self) -> int:     # sequence.py:58-60
        return -(-self.n_cached // self.bs)

    @property
    def tail(self) -> int:                # sequence.py:66-69 (0 at exact multiples)
        return len(self.tokens) - (len(self.tokens) // self.bs) * self.bs

    def block(self, i: int):              # sequence.py:71-81
        assert 0 <= i < self.n_blocks
        if i == self.n_blocks - 1:
            return self.tokens[-self.tail:]   # [-0:] is the whole list
        return self.tokens[i * self.bs:(i + 1) * self.bs]

    @property
    def completion(self):
        return self.tokens[self.n_prompt:]


@dataclass
class _Blk:
    hash: int = -1
    refs: int = 0
    tokens: list = field(default_factory=list)


class OraclePool:
    """block_manager.py:28-157."""

    def __init__(self, num_blocks: int, block_size: int):
        self.bs = block_size
        self.blocks = [_Blk() for _ in range(num_blocks)]
        self.by_hash: dict[int, int] = {}
        self.free = deque(range(num_blocks))
        self.used: set[int] = set()

    def _take(self, bid: int) -> _Blk:    # :60-69
        b = self.blocks[bid]
        assert b.refs == 0
        b.hash, b.refs, b.tokens = -1, 0, []
        self.free.remove(bid)
        self.used.add(bid)
        return b

    def _give_back(self, bid: int):       # :71-78
        b = self.blocks[bid]
        assert b.refs == 0
        b.tokens = []
        self.used.remove(bid)
        self.free.append(bid)

    def can_allocate(self, s: OracleSeq) -> bool:   # :81-83
        return len(self.free) >= s.n_blocks

    def allocate(self, s: OracleSeq):               # :85-114
        h = -1
        for i in range(s.n_blocks):
            toks = s.block(i)
            h = block_hash(toks, h) if len(toks) == self.bs else -1
            bid = self.by_hash.get(h, -1)
            if bid == -1 or self.blocks[bid].tokens != toks:
                bid = self.free[0]
                b = self._take(bid)
                b.hash, b.tokens = h, toks
                if h != -1:
                    self.by_hash[h] = bid
            else:
                s.n_cached += self.bs
                if bid not in self.used:
                    self._take(bid)
                else:
                    bid = self.by_hash[h]
                    self.blocks[bid].refs += 1
            s.table.append(bid)

    def deallocate(self, s: OracleSeq):             # :116-127
        for bid in s.table:
            b = self.blocks[bid]
            b.refs -= 1
            if b.refs == 0:
                self._give_back(bid)
        s.table = []
        s.n_cached = 0

    def can_append(self, s: OracleSeq) -> bool:     # :130-134
        return len(self.free) > 0 if len(s) % self.bs == 0 else True

    def append(self, s: OracleSeq):                 # :136-157
        last = s.table[-1]
        if len(s) % self.bs == 0:
            prefix = -1 if len(s.table) == 1 else self.blocks[s.table[-2]].hash
            toks = s.block(s.n_blocks - 1)
            h = block_hash(toks, prefix)
            self.blocks[last].hash, self.blocks[last].tokens = h, toks
            self.by_hash[h] = last
        elif len(s) % self.bs == 1:
            assert self.blocks[last].hash != -1
            bid = self.free[0]
            self._take(bid)
            s.table.append(bid)
        else:
            assert last in self.used and self.blocks[last].hash == -1


class OracleScheduler:
    """scheduler.py:8-95."""

    def __init__(self, max_num_sequences, max_num_batched_tokens, max_cached_blocks, block_size, eos):
        self.pool = OraclePool(max_cached_blocks, block_size)
        self.max_seqs, self.max_tokens, self.eos = max_num_sequences, max_num_batched_tokens, eos
        self.waiting: deque[OracleSeq] = deque()
        self.running: deque[OracleSeq] = deque()

    def add(self, s: OracleSeq):
        self.waiting.append(s)

    def done(self) -> bool:
        return not self.waiting and not self.running

    def schedule(self):
        batch, budget = [], 0
        while self.waiting and len(batch) < self.max_seqs:            # :32-43
            s = self.waiting[0]
            if not (self.pool.can_allocate(s) and len(s) + budget <= self.max_tokens):
                break
            self.waiting.popleft()
            self.pool.allocate(s)
            s.status = RUNNING
            self.running.append(s)
            batch.append(s)
            budget += len(s)
        if batch:
            return batch, True                                        # :45-46
        while self.running:                                           # :49-64
            s = self.running.popleft()
            if not self.pool.can_append(s):
                if self.running:
                    self._preempt(self.running.pop())
                else:
                    self._preempt(s)
                    break
            else:
                if budget >= self.max_tokens or len(batch) >= self.max_seqs:
                    break
                self.pool.append(s)
                batch.append(s)
                budget += 1
        if batch:
            self.running.extendleft(reversed(batch))                  # :66-67
        return batch, False

    def _preempt(self, s: OracleSeq):                                 # :72-76
        self.pool.deallocate(s)
        s.status = WAITING
        self.waiting.appendleft(s)

    def postprocess(self, batch, token_ids):                          # :79-95
        for s, t in zip(batch, token_ids):
            s.tokens.append(t)
            p = s.params
            stop = (not p.ignore_eos and t == self.eos) \
                or 1 + (len(s) - s.n_prompt) >= p.max_tokens \
                or (p.max_model_length is not None and len(s) >= p.max_model_length)
            if stop:
                s.status = FINISHED
                self.pool.deallocate(s)
                self.running.remove(s)


def _pad_tables(batch):
    width = max(len(s.table) for s in batch)
    return [s.table + [-1] * (width - len(s.table)) for s in batch]


def prepare_prefill(batch, block_size: int) -> dict:
    """model_runner.py:202-249, as plain lists (dtypes there: input_ids/slot_mapping int64,
    cu_seqlens/block_tables int32)."""
    ids, slots, cu_q, cu_k, lens_q, lens_k = [], [], [0], [0], [], []
    for s in batch:
        ids += s.tokens[s.n_cached:]
        lens_q.append(len(s) - s.n_cached)
        lens_k.append(len(s))
        cu_q.append(cu_q[-1] + lens_q[-1])
        cu_k.append(cu_k[-1] + lens_k[-1])
        for j, bid in enumerate(s.table[s.n_cached_blocks:]):
            full = s.n_cached_blocks + j != s.n_blocks - 1
            slots += range(bid * block_size, bid * block_size + (block_size if full else s.tail))
    tables = _pad_tables(batch) if cu_q[-1] < cu_k[-1] else None
    return dict(input_ids=ids, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, max_seqlen_q=max(lens_q),
                max_seqlen_k=max(lens_k), slot_mapping=slots, context_lens=None, block_tables=tables)


def prepare_decode(batch, block_size: int) -> dict:
    """model_runner.py:253-278."""
    return dict(input_ids=[s.tokens[-1] for s in batch], cu_seqlens_q=None, cu_seqlens_k=None,
                max_seqlen_q=0, max_seqlen_k=0,
                slot_mapping=[s.table[-1] * block_size + s.tail - 1 for s in batch],
                context_lens=[len(s) for s in batch], block_tables=_pad_tables(batch))
