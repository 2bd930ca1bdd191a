"""Prefill-first continuous batching (reference: engine/scheduler.py:8-95).

``schedule()`` returns ``(sequences, is_prefill)``; batches are never mixed: as soon as at least
one waiting request was admitted the step is a prefill step, otherwise every running sequence gets
one decode token.  ``postprocess()`` appends the sampled tokens and retires finished sequences.

``reference_exact=True`` reproduces the reference decision for decision, including that a running
sequence that cannot grow is dropped from the step after a victim was preempted
(scheduler.py:52-57) and the ``1 + completions >= max_tokens`` stop rule (scheduler.py:89), which
ends a request after ``max_tokens - 1`` generated tokens.  The default differs only when the pool
runs dry: it preempts newest-first until the sequence at hand can grow, then keeps it.
The stop rule is the reference's in both modes.
"""
from __future__ import annotations

import itertools
from collections import deque

from .block_manager import BlockManager, NativeBlockManager
from .sequence import Sequence, SequenceStatus


class Scheduler:
    def __init__(self, max_num_sequences: int, max_num_batched_tokens: int, max_cached_blocks: int,
                 block_size: int, eos: int, reference_exact: bool = False, native_pool: bool = True):
        self.max_num_sequences = max_num_sequences
        self.max_num_batched_tokens = max_num_batched_tokens
        self.eos = eos
        self.reference_exact = reference_exact
        # the default mode keeps its block pool in the library (C++); the reference-exact mode, which reproduces
        # the reference's ref-count arithmetic for the parity recordings, is the Python class
        if reference_exact or not native_pool:
            self.block_manager = BlockManager(max_cached_blocks, block_size, reference_exact)
        else:
            self.block_manager = NativeBlockManager(max_cached_blocks, block_size)
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def add_sequence(self, sequence: Sequence) -> None:
        self.waiting.append(sequence)

    # ------------------------------------------------------------------ one step
    def schedule(self) -> tuple[list[Sequence], bool]:
        admitted = self._admit_waiting()
        if admitted:
            return admitted, True
        return self._grow_running(), False

    def _admit_waiting(self) -> list[Sequence]:
        bm, batch, tokens = self.block_manager, [], 0
        while self.waiting and len(batch) < self.max_num_sequences:
            seq = self.waiting[0]
            if tokens + len(seq) > self.max_num_batched_tokens or not bm.can_allocate(seq):
                break
            self.waiting.popleft()
            bm.allocate(seq)
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            batch.append(seq)
            tokens += len(seq)
        return batch

    def _grow_running(self) -> list[Sequence]:
        bm = self.block_manager
        block_size = bm.block_size
        limit = min(self.max_num_sequences, self.max_num_batched_tokens)
        if not self.reference_exact:
            # Common case, no queue surgery: the first `limit` running sequences decode, those at a
            # block boundary get their block opened (n % bs == 1) or sealed (== 0) in order, and
            # nobody has to be preempted because the free list covers every block to be opened.
            # Exactly what the general loop below does in that case.
            batch = list(itertools.islice(self.running, limit))
            edge = [s for s in batch if s.num_tokens % block_size <= 1]
            opening = sum(1 for s in edge if s.num_tokens % block_size == 1)
            if opening <= bm.num_free_blocks:
                for s in edge:
                    bm.append(s)
                return batch
        return self._grow_running_general(limit)

    def _grow_running_general(self, limit: int) -> list[Sequence]:
        bm, batch = self.block_manager, []
        block_size = bm.block_size
        while self.running:
            seq = self.running.popleft()
            if self.reference_exact:
                if not bm.can_append(seq):
                    if self.running:
                        self.preempt(self.running.pop())
                    else:
                        self.preempt(seq)
                        break
                    continue
            else:
                rem = seq.num_tokens % block_size
                if rem > 1:
                    # mid-block: no block is opened or sealed this step (BlockManager.append would
                    # only assert); the batch limits below still apply
                    if len(batch) >= limit:
                        self.running.appendleft(seq)
                        break
                    batch.append(seq)
                    continue
                evicted_self = False
                while not bm.can_append(seq):
                    if self.running:
                        self.preempt(self.running.pop())
                    else:
                        self.preempt(seq)
                        evicted_self = True
                        break
                if evicted_self:
                    break
            if len(batch) >= self.max_num_sequences or len(batch) >= self.max_num_batched_tokens:
                if not self.reference_exact:
                    self.running.appendleft(seq)
                break
            bm.append(seq)
            batch.append(seq)
        if batch:
            self.running.extendleft(reversed(batch))
        return batch

    # ------------------------------------------------------------------ several decode steps per schedule
    def plan_decode_window(self, seqs: list[Sequence], max_steps: int, max_positions: int) -> int:
        """How many decode steps the batch ``schedule()`` just returned may run back to back without the
        host (the sampled token of one step is the input of the next on the device), at most
        ``max_steps``; opens the blocks those steps write into.  The window ends where the longest-lived
        sequence stops, never passes ``max_positions`` tokens, and is 1 when the pool cannot cover the
        blocks to open.  Sequences that stop inside the window still occupy their row to its end (their
        extra tokens are dropped by ``postprocess_window``), and waiting requests are admitted after it."""
        bm = self.block_manager
        bs = bm.block_size
        if max_steps <= 1 or self.reference_exact:
            return 1
        k, longest = min(max_steps, bs), 0
        for s in seqs:
            n = s.num_tokens
            left = s.max_tokens - 1 - (n - s.num_prompt_tokens)        # appends until the stop rule fires
            if s.max_model_length is not None and s.max_model_length - n < left:
                left = s.max_model_length - n
            if left > longest:
                longest = left
            if max_positions - n + 1 < k:
                k = max_positions - n + 1
        k = min(k, longest)
        if k <= 1:
            return 1
        # lengths n+1 .. n+k-1 that start a block (n itself was handled by schedule())
        opening = [s for s in seqs if 1 <= (1 - s.num_tokens) % bs <= k - 1]
        if len(opening) > bm.num_free_blocks:
            return 1
        for s in opening:
            bm.open_block(s)
        return k

    def postprocess_window(self, seqs: list[Sequence], steps: list[list[int]]) -> int:
        """``postprocess`` for a window of decode steps: ``steps[j][i]`` is the token step j sampled for
        ``seqs[i]``.  Tokens after a sequence's stop are dropped; blocks that filled inside the window
        get their hash now.  Returns the number of tokens kept."""
        eos, bm = self.eos, self.block_manager
        bs, last = bm.block_size, len(steps) - 1
        kept = 0
        for i, seq in enumerate(seqs):
            for j, row in enumerate(steps):
                token_id = row[i]
                seq.token_ids.append(token_id)
                seq.last_token = token_id
                n = seq.num_tokens = seq.num_tokens + 1
                kept += 1
                hit_eos = token_id == eos and not seq.ignore_eos
                hit_max_tokens = 1 + n - seq.num_prompt_tokens >= seq.max_tokens
                hit_max_length = seq.max_model_length is not None and n >= seq.max_model_length
                if hit_eos or hit_max_tokens or hit_max_length:
                    seq.status = SequenceStatus.FINISHED
                    bm.deallocate(seq)
                    self.running.remove(seq)
                    break
                if j < last and n % bs == 0:
                    bm.seal_block(seq, n // bs - 1)
        return kept

    def preempt(self, seq: Sequence) -> None:
        self.block_manager.deallocate(seq)
        seq.status = SequenceStatus.WAITING
        self.waiting.appendleft(seq)

    # ------------------------------------------------------------------ after the model ran
    def postprocess(self, seqs: list[Sequence], token_ids: list[int]) -> None:
        eos = self.eos
        for seq, token_id in zip(seqs, token_ids):
            # Sequence.append_token, inlined (this loop runs once per generated token)
            seq.token_ids.append(token_id)
            seq.last_token = token_id
            n = seq.num_tokens = seq.num_tokens + 1
            hit_eos = token_id == eos and not seq.ignore_eos
            hit_max_tokens = 1 + n - seq.num_prompt_tokens >= seq.max_tokens
            hit_max_length = seq.max_model_length is not None and n >= seq.max_model_length
            if hit_eos or hit_max_tokens or hit_max_length:
                seq.status = SequenceStatus.FINISHED
                self.block_manager.deallocate(seq)
                self.running.remove(seq)
