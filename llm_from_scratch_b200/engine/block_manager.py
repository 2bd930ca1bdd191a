"""Paged KV-block pool with chained-hash prefix caching (reference: engine/block_manager.py:8-157).

Public surface is the reference's: ``BlockManager(num_blocks, block_size)``, ``compute_hash``,
``can_allocate`` / ``allocate`` / ``deallocate``, ``can_append`` / ``append`` and the attributes
``blocks``, ``hash_to_block_id``, ``free_block_ids``, ``used_block_ids``.

Differences in mechanism, not in results:

* block hashes come from the library's native XXH64 (``b200_block_hash``) instead of the xxhash
  package + a numpy round trip per block;
* the free list is an insertion-ordered dict used as an ordered set, so "take the oldest free
  block", "take this particular free block" and "return a block" are all O(1); the reference's
  ``deque.remove`` is O(num_blocks) per allocation (engine/block_manager.py:67).

Two behaviours are selectable with ``reference_exact``:

``reference_exact=True`` reproduces the reference's integer results bit for bit, including its
ref-count arithmetic: a block's count starts at 0 (block_manager.py:23-26), so an unshared block
falls to -1 when released and never returns to the free list, and a block shared by two sequences
returns to the free list when the first of them finishes.  The parity tests run in this mode on
workloads whose pool never runs dry (outside that the reference raises or drops requests).

The default keeps the same allocation order and hashing but counts references from 1, so blocks
are released exactly when their last user finishes, released blocks keep their contents and can be
revived by a later prefix hit, and ``can_append`` asks for a free block on the same step on which
``append`` takes one.  A prefix hit never covers the whole prompt: when every block of a prompt whose
length is a multiple of the block size is cached, the last block is recomputed, so that the prefill
step has at least one query token per sequence (the reference would emit none and sample the
request's first token from another sequence's logits).
"""
from __future__ import annotations

from collections import OrderedDict

from .sequence import Sequence
from .. import ops


class Block:
    __slots__ = ("block_id", "hash", "ref_count", "token_ids")

    def __init__(self, block_id: int):
        self.block_id = block_id
        self.hash = -1
        self.ref_count = 0
        self.token_ids: list[int] = []

    def update(self, h: int, token_ids) -> None:
        self.hash = h
        self.token_ids = token_ids

    def reset(self) -> None:
        self.hash = -1
        self.ref_count = 0
        self.token_ids = []


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int, reference_exact: bool = False):
        self.block_size = block_size
        self.reference_exact = reference_exact
        self.blocks = [Block(i) for i in range(num_blocks)]
        self.hash_to_block_id: dict[int, int] = {}
        # ordered set, oldest first.  OrderedDict, not dict: a plain dict whose oldest keys keep being
        # deleted makes next(iter(d)) scan the deleted slots, which is linear in the pool size
        self._free: OrderedDict[int, None] = OrderedDict.fromkeys(range(num_blocks))
        self.used_block_ids: set[int] = set()

    # ------------------------------------------------------------------ views
    @property
    def free_block_ids(self):
        """Free block ids, oldest first (supports len(), iteration and ``in``)."""
        return self._free.keys()

    @property
    def num_free_blocks(self) -> int:
        return len(self._free)

    # ------------------------------------------------------------------ hashing
    @staticmethod
    def compute_hash(token_ids, prefix_hash_value: int = -1) -> int:
        """XXH64 over [8-byte LE prefix hash unless -1] || int32-LE token ids (block_manager.py:45-57)."""
        return ops.block_hash(token_ids, prefix_hash_value)

    # ------------------------------------------------------------------ block moves
    def _oldest_free(self) -> int:
        try:
            return next(iter(self._free))
        except StopIteration:
            raise IndexError("KV block pool exhausted") from None

    def _allocate_block(self, block_id: int, keep_contents: bool = False) -> Block:
        block = self.blocks[block_id]
        if self.reference_exact:
            assert block.ref_count == 0, "block is already allocated"
            block.reset()
        else:
            if not keep_contents:
                if block.hash != -1 and self.hash_to_block_id.get(block.hash) == block_id:
                    del self.hash_to_block_id[block.hash]
                block.reset()
            block.ref_count = 1
        del self._free[block_id]
        self.used_block_ids.add(block_id)
        return block

    def _deallocate_block(self, block_id: int) -> None:
        block = self.blocks[block_id]
        assert block.ref_count == 0, "block is still in use"
        if self.reference_exact:
            block.token_ids = []
        self.used_block_ids.remove(block_id)
        self._free[block_id] = None

    # ------------------------------------------------------------------ prefill-time allocation
    def can_allocate(self, seq: Sequence) -> bool:
        return len(self._free) >= seq.num_blocks

    def allocate(self, seq: Sequence) -> None:
        """Give ``seq`` a block per ``block_size`` tokens, reusing blocks whose chained hash and
        token ids match (block_manager.py:85-114)."""
        if not self.reference_exact:
            return self._allocate_fast(seq)
        h = -1
        bs = self.block_size
        for i in range(seq.num_blocks):
            token_ids = seq.block(i)
            h = self.compute_hash(token_ids, h) if len(token_ids) == bs else -1
            block_id = self.hash_to_block_id.get(h, -1)
            hit = block_id != -1 and self.blocks[block_id].token_ids == token_ids
            if hit:
                seq.num_cached_tokens += bs
                if block_id in self.used_block_ids:
                    block = self.blocks[block_id]
                    block.ref_count += 1
                else:
                    block = self._allocate_block(block_id, keep_contents=True)
            else:
                block = self._allocate_block(self._oldest_free())
                block.update(h, token_ids)
                if h != -1:
                    self.hash_to_block_id[h] = block.block_id
            seq.block_table.append(block.block_id)

    def _allocate_fast(self, seq: Sequence) -> None:
        """``allocate`` of the default mode with the per-block calls folded into one loop: all full-block
        hashes of the prompt come from one native call (the same chain of values), and a miss takes the
        oldest free block, drops the stale hash entry that still points at it and fills it in place."""
        bs = self.block_size
        ids = seq.token_ids
        chain = ops.block_hash_chain(ids, bs)
        blocks, free, used, h2b = self.blocks, self._free, self.used_block_ids, self.hash_to_block_id
        table = seq.block_table
        cached = 0
        total = len(ids)
        for i in range(seq.num_blocks):
            token_ids = ids[i * bs:(i + 1) * bs]
            h = chain[i] if len(token_ids) == bs else -1
            block_id = h2b.get(h, -1)
            # a hit on the block that ends the prompt would leave no token to run through the model (the
            # step samples from the last prompt token's logits): that block is recomputed into a fresh one
            if block_id != -1 and blocks[block_id].token_ids == token_ids and cached + bs < total:
                cached += bs
                block = blocks[block_id]
                if block_id in used:
                    block.ref_count += 1
                else:                       # a free block whose contents are still what this prompt needs
                    block.ref_count = 1
                    del free[block_id]
                    used.add(block_id)
            else:
                try:
                    block_id = free.popitem(last=False)[0]
                except KeyError:
                    raise IndexError("KV block pool exhausted") from None
                block = blocks[block_id]
                old = block.hash
                if old != -1 and h2b.get(old) == block_id:
                    del h2b[old]
                block.hash, block.token_ids, block.ref_count = h, token_ids, 1
                used.add(block_id)
                if h != -1:
                    h2b[h] = block_id
            table.append(block_id)
        seq.num_cached_tokens += cached

    def deallocate(self, seq: Sequence) -> None:
        order = seq.block_table if self.reference_exact else reversed(seq.block_table)
        for block_id in order:
            block = self.blocks[block_id]
            block.ref_count -= 1
            if block.ref_count == 0:
                self._deallocate_block(block_id)
        seq.block_table = []
        seq.num_cached_tokens = 0

    # ------------------------------------------------------------------ decode-time growth
    def can_append(self, seq: Sequence) -> bool:
        trigger = 0 if self.reference_exact else 1   # block_manager.py:132 tests == 0
        return len(self._free) > 0 if len(seq) % self.block_size == trigger else True

    def append(self, seq: Sequence) -> None:
        """Called once per decode step before the step runs (block_manager.py:136-157): opens a new
        block when the previous one has just filled, seals the hash of a block that is now full."""
        table = seq.block_table
        last = self.blocks[table[-1]]
        rem = len(seq) % self.block_size
        if rem == 0:
            prefix = -1 if len(table) == 1 else self.blocks[table[-2]].hash
            token_ids = seq.block(seq.num_blocks - 1)
            h = self.compute_hash(token_ids, prefix)
            last.update(h, token_ids)
            self.hash_to_block_id[h] = last.block_id
        elif rem == 1:
            assert last.hash != -1, "previous block should have been sealed"
            table.append(self._allocate_block(self._oldest_free()).block_id)
        else:
            assert last.block_id in self.used_block_ids and last.hash == -1

    # ------------------------------------------------------------------ several decode steps per schedule
    def open_block(self, seq: Sequence) -> None:
        """Opens the next block of ``seq`` ahead of time: what ``append`` does at ``len % block_size == 1``,
        for a length the sequence reaches inside a window of decode steps (its tokens are not known yet,
        so the block before it is sealed afterwards, by ``seal_block``)."""
        seq.block_table.append(self._allocate_block(self._oldest_free()).block_id)

    def seal_block(self, seq: Sequence, index: int) -> None:
        """Gives block ``index`` of ``seq``, now full, its chained hash: what ``append`` does at
        ``len % block_size == 0``, for a length passed inside a window of decode steps."""
        table, bs = seq.block_table, self.block_size
        block = self.blocks[table[index]]
        prefix = -1 if index == 0 else self.blocks[table[index - 1]].hash
        token_ids = seq.token_ids[index * bs:(index + 1) * bs]
        h = self.compute_hash(token_ids, prefix)
        block.update(h, token_ids)
        self.hash_to_block_id[h] = block.block_id



class _BlockView:
    """Read-only snapshot of one block of a ``NativeBlockManager`` (inspection and tests)."""
    __slots__ = ("block_id", "hash", "ref_count")

    def __init__(self, block_id: int, h: int, ref_count: int):
        self.block_id, self.hash, self.ref_count = block_id, h, ref_count


class NativeBlockManager:
    """The default-mode pool with its inner loops in C++ (``b200_pool_*`` of the library): the hash chain, the
    lookup with token comparison, the O(1) free list and the reference counts live behind a handle, and a call
    per ``allocate`` / ``append`` / ``deallocate`` replaces a Python loop per block.  Same methods and the same
    results as ``BlockManager(reference_exact=False)`` — allocation order, prefix hits, what a released block
    keeps — which ``tests/test_native_host_path.py`` checks on random request traces.  The reference-exact mode
    (the reference's ref-count arithmetic, reproduced for the parity recordings) stays in Python."""

    reference_exact = False

    def __init__(self, num_blocks: int, block_size: int):
        import ctypes
        import numpy as np
        from .._lib import lib
        self._np, self._ct, self._lib = np, ctypes, lib
        self.block_size = block_size
        self.num_blocks = num_blocks
        self._h = lib.b200_pool_create(num_blocks, block_size)
        if not self._h:
            raise MemoryError("could not create the native block pool")
        self._cached = ctypes.c_int64(0)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.b200_pool_destroy(h)

    # ------------------------------------------------------------------ views (inspection; not on the hot path)
    def _snapshot(self):
        np = self._np
        order = np.empty(self.num_blocks, dtype=np.int32)
        refs = np.empty(self.num_blocks, dtype=np.int32)
        sealed = np.empty(self.num_blocks, dtype=np.uint8)
        hashes = np.empty(self.num_blocks, dtype=np.uint64)
        n = self._lib.b200_pool_snapshot(self._h, order.ctypes.data, refs.ctypes.data, sealed.ctypes.data,
                                         hashes.ctypes.data)
        return order[:n], refs, sealed, hashes

    @property
    def free_block_ids(self):
        return self._snapshot()[0].tolist()

    @property
    def num_free_blocks(self) -> int:
        return self._lib.b200_pool_num_free(self._h)

    @property
    def used_block_ids(self) -> set:
        return set(self._np.nonzero(self._snapshot()[1] > 0)[0].tolist())

    @property
    def blocks(self):
        _, refs, sealed, hashes = self._snapshot()
        return [_BlockView(i, int(hashes[i]) if sealed[i] else -1, int(refs[i])) for i in range(self.num_blocks)]

    @property
    def hash_to_block_id(self) -> dict:
        _, _refs, sealed, hashes = self._snapshot()
        out = {}
        for h in set(hashes[sealed > 0].tolist()):
            b = self._lib.b200_pool_lookup(self._h, h)
            if b >= 0:
                out[h] = b
        return out

    compute_hash = staticmethod(BlockManager.compute_hash)

    # ------------------------------------------------------------------ prefill-time allocation
    def can_allocate(self, seq: Sequence) -> bool:
        return self.num_free_blocks >= seq.num_blocks

    def allocate(self, seq: Sequence) -> None:
        np = self._np
        ids = np.asarray(seq.token_ids, dtype=np.int32)
        table = np.empty(seq.num_blocks, dtype=np.int32)
        n = self._lib.b200_pool_allocate(self._h, ids.ctypes.data, ids.size, table.ctypes.data,
                                         self._ct.addressof(self._cached))
        if n < 0:
            raise IndexError("KV block pool exhausted")
        seq.block_table.extend(table.tolist())
        seq.num_cached_tokens += self._cached.value

    def deallocate(self, seq: Sequence) -> None:
        table = self._np.asarray(seq.block_table, dtype=self._np.int32)
        if self._lib.b200_pool_deallocate(self._h, table.ctypes.data, table.size) != 0:
            raise RuntimeError("deallocate: a block of the table is not in use")
        seq.block_table = []
        seq.num_cached_tokens = 0

    # ------------------------------------------------------------------ decode-time growth
    def can_append(self, seq: Sequence) -> bool:
        return self.num_free_blocks > 0 if len(seq) % self.block_size == 1 else True

    def _tokens(self, token_ids):
        return (self._ct.c_int32 * self.block_size)(*token_ids)

    def append(self, seq: Sequence) -> None:
        n = len(seq)
        rem = n % self.block_size
        if rem > 1:
            return
        table = seq.block_table
        toks = self._tokens(seq.token_ids[-self.block_size:]) if rem == 0 else None
        b = self._lib.b200_pool_append(self._h, table[-1], table[-2] if len(table) > 1 else -1, n, toks)
        if b >= 0:
            table.append(b)
        elif b < -1:
            raise IndexError("KV block pool exhausted")

    def open_block(self, seq: Sequence) -> None:
        b = self._lib.b200_pool_open_block(self._h)
        if b < 0:
            raise IndexError("KV block pool exhausted")
        seq.block_table.append(b)

    def seal_block(self, seq: Sequence, index: int) -> None:
        table, bs = seq.block_table, self.block_size
        toks = self._tokens(seq.token_ids[index * bs:(index + 1) * bs])
        if self._lib.b200_pool_seal_block(self._h, table[index], table[index - 1] if index > 0 else -1, toks) != 0:
            raise RuntimeError("seal_block: bad block")
