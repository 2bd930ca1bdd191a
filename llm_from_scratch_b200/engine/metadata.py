"""Host-side builders of the per-step attention metadata (reference:
ModelRunner.prepare_prefill / prepare_decode, engine/model_runner.py:202-278).

They return numpy arrays with the reference's dtypes (input_ids, slot_mapping, context_lens int64;
cu_seqlens, block_tables int32) so that the model runner can copy them to the device in one go and
the parity tests can compare them on the CPU.  Slots are computed per block with ``numpy.arange``
rather than per token in Python.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from .sequence import Sequence


@dataclass
class StepMetadata:
    is_prefill: bool
    input_ids: np.ndarray                       # int64 [T]
    slot_mapping: np.ndarray                    # int64 [T]
    positions: np.ndarray                       # int64 [T]  RoPE position of every input token
    cu_seqlens_q: Optional[np.ndarray] = None   # int32 [n+1]
    cu_seqlens_k: Optional[np.ndarray] = None   # int32 [n+1]
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    context_lens: Optional[np.ndarray] = None   # int64 [n]
    block_tables: Optional[np.ndarray] = None   # int32 [n, maxb]
    last_token_index: Optional[np.ndarray] = None  # int64 [n]  row of each sequence's last token


def block_table_array(s: Sequence) -> np.ndarray:
    """int32 copy of ``s.block_table`` kept on the sequence between steps.  The block manager only ever
    appends to the list or replaces it by a new list (deallocate), so the copy is extended by the new
    entries when the list object is the same and rebuilt when it is not."""
    bt = s.block_table
    n = len(bt)
    c = s._bt_cache
    if c is not None and c[0] is bt and c[2] <= n <= c[1].size:
        if c[2] < n:
            c[1][c[2]:n] = bt[c[2]:]
            c[2] = n
        return c[1][:n]
    buf = np.empty(max(64, 2 * n), dtype=np.int32)
    buf[:n] = bt
    s._bt_cache = [bt, buf, n]
    return buf[:n]


def pad_block_tables(seqs: list[Sequence], out: np.ndarray | None = None) -> np.ndarray:
    """[n, width] int32, -1 beyond every sequence's table (``out``: write into rows [:n] of a wider
    preallocated array instead, leaving its other entries as they are)."""
    arrays = [block_table_array(s) for s in seqs]
    if out is None:
        width = max(a.size for a in arrays)
        out = np.full((len(seqs), max(width, 1)), -1, dtype=np.int32)
    for i, a in enumerate(arrays):
        out[i, :a.size] = a
    return out


def _flat_tables(seqs: list[Sequence]):
    """(offsets int64 [n + 1], flat int32 block ids) of the sequences' block tables."""
    arrays = [block_table_array(s) for s in seqs]
    offsets = np.zeros(len(seqs) + 1, dtype=np.int64)
    np.cumsum([a.size for a in arrays], out=offsets[1:])
    flat = np.concatenate(arrays) if arrays else np.zeros(0, dtype=np.int32)
    return offsets, np.ascontiguousarray(flat, dtype=np.int32)


def prepare_prefill(seqs: list[Sequence], block_size: int) -> StepMetadata:
    """Packs the non-cached suffix of every sequence (model_runner.py:202-249): cu_seqlens, positions and the slot
    mapping come from the library's native builder (``b200_prepare_prefill``); ``prepare_prefill_py`` is the
    same thing in numpy, kept as the definition and for the reference-exact mode."""
    if Sequence.reference_exact or any(not s.block_table for s in seqs):
        return prepare_prefill_py(seqs, block_size)
    from .._lib import lib
    n = len(seqs)
    num_tokens = np.fromiter((s.num_tokens for s in seqs), dtype=np.int64, count=n)
    cached = np.fromiter((s.num_cached_tokens for s in seqs), dtype=np.int64, count=n)
    offsets, flat = _flat_tables(seqs)
    total = int((num_tokens - cached).sum())
    cu_q, cu_k = np.empty(n + 1, dtype=np.int32), np.empty(n + 1, dtype=np.int32)
    positions, slots = np.empty(total, dtype=np.int64), np.empty(total, dtype=np.int64)
    mx = np.zeros(2, dtype=np.int32)
    got = lib.b200_prepare_prefill(n, num_tokens.ctypes.data, cached.ctypes.data, offsets.ctypes.data, flat.ctypes.data,
                                   block_size, cu_q.ctypes.data, cu_k.ctypes.data, positions.ctypes.data,
                                   slots.ctypes.data, total, mx.ctypes.data)
    if got != total:
        raise RuntimeError(f"prepare_prefill: the native builder returned {got} for {total} tokens")
    ids = [np.asarray(s.token_ids[s.num_cached_tokens:], dtype=np.int64) for s in seqs]
    return StepMetadata(
        is_prefill=True, input_ids=np.concatenate(ids) if ids else np.zeros(0, dtype=np.int64),
        slot_mapping=slots, positions=positions, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k,
        max_seqlen_q=int(mx[0]), max_seqlen_k=int(mx[1]),
        block_tables=pad_block_tables(seqs) if cu_q[-1] < cu_k[-1] else None,
        last_token_index=(cu_q[1:] - 1).astype(np.int64))


def prepare_prefill_py(seqs: list[Sequence], block_size: int) -> StepMetadata:
    """Packs the non-cached suffix of every sequence (model_runner.py:202-249).

    The reference produces no positions tensor; the RoPE position of packed token j of a sequence
    is ``num_cached_tokens + j``.
    """
    ids, slots, pos = [], [], []
    q_lens, k_lens = [], []
    in_block = np.arange(block_size, dtype=np.int64)
    for s in seqs:
        cached = s.num_cached_tokens
        ids.append(np.asarray(s.token_ids[cached:], dtype=np.int64))
        q_lens.append(s.num_tokens - cached)
        k_lens.append(s.num_tokens)
        pos.append(np.arange(cached, s.num_tokens, dtype=np.int64))
        if not s.block_table:
            continue
        # slots of blocks [num_cached_blocks, end of the table): whole blocks, the sequence's last one ragged
        first, last = s.num_cached_blocks, s.num_blocks - 1
        bt = np.asarray(s.block_table[first:], dtype=np.int64)
        if bt.size:
            n = bt.size * block_size
            if first + bt.size - 1 == last:
                n -= block_size - s.last_block_num_tokens
            slots.append((bt[:, None] * block_size + in_block).reshape(-1)[:n])
    cu_q = np.zeros(len(seqs) + 1, dtype=np.int32)
    cu_k = np.zeros(len(seqs) + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu_q[1:])
    np.cumsum(k_lens, out=cu_k[1:])
    empty = np.zeros(0, dtype=np.int64)
    return StepMetadata(
        is_prefill=True,
        input_ids=np.concatenate(ids) if ids else empty,
        slot_mapping=np.concatenate(slots) if slots else empty,
        positions=np.concatenate(pos) if pos else empty,
        cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, max_seqlen_q=max(q_lens), max_seqlen_k=max(k_lens),
        block_tables=pad_block_tables(seqs) if cu_q[-1] < cu_k[-1] else None,
        last_token_index=(cu_q[1:] - 1).astype(np.int64))


def prepare_decode(seqs: list[Sequence], block_size: int, tables_out: np.ndarray | None = None) -> StepMetadata:
    """One token per running sequence (model_runner.py:253-278): context lengths, slots and the padded block tables
    come from the library's native builder (``b200_prepare_decode``); ``prepare_decode_py`` is the numpy form."""
    if Sequence.reference_exact or tables_out is not None or not seqs:
        return prepare_decode_py(seqs, block_size, tables_out)
    from .._lib import lib
    n = len(seqs)
    num_tokens = np.fromiter((s.num_tokens for s in seqs), dtype=np.int64, count=n)
    offsets, flat = _flat_tables(seqs)
    width = max(int((offsets[1:] - offsets[:-1]).max()), 1)
    lens, slots = np.empty(n, dtype=np.int64), np.empty(n, dtype=np.int64)
    tables = np.empty((n, width), dtype=np.int32)
    rc = lib.b200_prepare_decode(n, num_tokens.ctypes.data, offsets.ctypes.data, flat.ctypes.data, block_size,
                                 lens.ctypes.data, slots.ctypes.data, tables.ctypes.data, width)
    if rc != 0:
        raise RuntimeError(f"prepare_decode: the native builder returned {rc}")
    return StepMetadata(
        is_prefill=False, input_ids=np.fromiter((s.last_token for s in seqs), dtype=np.int64, count=n),
        slot_mapping=slots, positions=lens - 1, context_lens=lens, block_tables=tables,
        last_token_index=np.arange(n, dtype=np.int64))


def prepare_decode_py(seqs: list[Sequence], block_size: int, tables_out: np.ndarray | None = None) -> StepMetadata:
    """One token per running sequence (model_runner.py:253-278).  With ``tables_out`` (a preallocated
    [>= n, >= widest table] int32 array) the block tables are written into its first n rows, entries
    beyond a sequence's table keep their old values, and ``block_tables`` is that row range."""
    n = len(seqs)
    lens = np.fromiter((s.num_tokens for s in seqs), dtype=np.int64, count=n)
    slots = np.fromiter((s.block_table[-1] * block_size + s.last_block_num_tokens - 1 for s in seqs),
                        dtype=np.int64, count=n)
    return StepMetadata(
        is_prefill=False,
        input_ids=np.fromiter((s.last_token for s in seqs), dtype=np.int64, count=n),
        slot_mapping=slots, positions=lens - 1, context_lens=lens,
        block_tables=pad_block_tables(seqs) if tables_out is None else pad_block_tables(seqs, tables_out)[:n],
        last_token_index=np.arange(n, dtype=np.int64))


class DecodeBatchBuilder:
    """Decode-step metadata without a per-sequence rebuild: every sequence owns a row of a host table that
    mirrors its block table and is only touched when the table changes (a block is appended once in
    ``block_size`` steps; a prefill rewrites it), so a step costs four passes over the batch in the
    interpreter plus a few numpy gathers.  ``build`` writes exactly what ``prepare_decode`` returns
    (input_ids, slot_mapping, context_lens, block_tables) into caller-owned arrays.

    The owner must call ``invalidate`` for every sequence that goes through a prefill (its block table
    may have been replaced by one of the same length after a preemption).

    With ``device_rows`` > 0 the builder also mirrors what the device-resident table holds at every batch
    position (which sequence row, at which epoch, how many entries), and ``build(..., patches=)`` emits only
    the (position, column, block id) triples the device lacks: block tables are append-only between two
    prefills of a sequence, so a steady batch costs one triple per sequence every ``block_size`` steps
    instead of a ``batch x max_blocks`` upload (the reference re-uploads the table, model_runner.py:263-268)."""

    def __init__(self, block_size: int, max_blocks: int, rows: int = 1024, device_rows: int = 0):
        self.block_size = block_size
        self.tables = np.zeros((rows, max_blocks), dtype=np.int32)
        self.row_blocks = np.full(rows, -1, dtype=np.int64)     # valid entries per row, -1 = rebuild
        self.row_seq: list = [None] * rows
        self.row_owner = np.zeros(rows, dtype=np.int64)         # id() of the owning sequence, 0 = none
        self.row_epoch = np.zeros(rows, dtype=np.int64)         # bumped whenever the row's table may have been replaced
        self.free = list(range(rows - 1, -1, -1))
        self.dev_row = np.full(device_rows, -1, dtype=np.int64)      # builder row mirrored at each batch position
        self.dev_epoch = np.zeros(device_rows, dtype=np.int64)
        self.dev_blocks = np.zeros(device_rows, dtype=np.int64)      # entries of that row present on the device

    def invalidate(self, seqs) -> None:
        for s in seqs:
            if s._row is not None and self.row_seq[s._row] is s:
                self.row_blocks[s._row] = -1
                self.row_epoch[s._row] += 1

    def _assign(self, s) -> int:
        if not self.free:
            # reclaim rows of sequences that are finished or were handed another row; else grow
            for r, owner in enumerate(self.row_seq):
                if owner is not None and (owner.is_finished or owner._row != r):
                    self.row_seq[r] = None
                    self.row_owner[r] = 0
                    self.free.append(r)
            if not self.free:
                old = self.tables.shape[0]
                self.tables = np.concatenate([self.tables, np.zeros_like(self.tables)])
                self.row_blocks = np.concatenate([self.row_blocks, np.full(old, -1, dtype=np.int64)])
                self.row_owner = np.concatenate([self.row_owner, np.zeros(old, dtype=np.int64)])
                self.row_epoch = np.concatenate([self.row_epoch, np.zeros(old, dtype=np.int64)])
                self.row_seq.extend([None] * old)
                self.free = list(range(2 * old - 1, old - 1, -1))
        r = self.free.pop()
        self.row_seq[r] = s
        self.row_owner[r] = id(s)
        self.row_blocks[r] = -1
        self.row_epoch[r] += 1
        s._row = r
        return r

    def build(self, seqs, out_ids: np.ndarray, out_slots: np.ndarray, out_lens: np.ndarray,
              out_tables: np.ndarray, patches: np.ndarray | None = None) -> int:
        """Writes the step's metadata.  Without ``patches`` the block tables go to ``out_tables`` and the
        result is -1.  With ``patches`` (int32 [capacity, 3]) the entries the device table lacks are written
        there as (position, column, block id) and their number is returned; when they exceed the capacity
        (a new batch composition) the whole tables go to ``out_tables`` instead and the result is -1."""
        n, bs = len(seqs), self.block_size
        rows_l = [s._row for s in seqs]
        ids = np.array([id(s) for s in seqs], dtype=np.int64)
        # a row is this sequence's only if the table says so (rows are reclaimed; a sequence may come
        # from another builder): one vectorised check, the slow path only for the newcomers
        if None in rows_l or not np.array_equal(self.row_owner[np.array(rows_l, dtype=np.int64)], ids):
            row_seq = self.row_seq
            rows_l = [s._row if s._row is not None and s._row < len(row_seq) and row_seq[s._row] is s
                      else self._assign(s) for s in seqs]
        rows = np.array(rows_l, dtype=np.int64)
        lens = np.array([s.num_tokens for s in seqs], dtype=np.int64)
        nblk = np.array([len(s.block_table) for s in seqs], dtype=np.int64)
        have = self.row_blocks[rows]
        for i in np.nonzero(have != nblk)[0].tolist():
            r, bt = rows_l[i], seqs[i].block_table
            k = int(have[i])
            if k < 0 or k > len(bt):
                k = 0
            self.tables[r, k:len(bt)] = bt[k:]
            self.row_blocks[r] = len(bt)
        count = -1
        if patches is not None:
            same = (self.dev_row[:n] == rows) & (self.dev_epoch[:n] == self.row_epoch[rows])
            start = np.where(same, np.minimum(self.dev_blocks[:n], nblk), 0)
            cnt = nblk - start
            total = int(cnt.sum())
            if total <= patches.shape[0]:
                count = total
                if total:
                    pos = np.repeat(np.arange(n, dtype=np.int64), cnt)
                    col = np.arange(total, dtype=np.int64) - np.repeat(np.cumsum(cnt) - cnt, cnt) + np.repeat(start, cnt)
                    patches[:total, 0] = pos
                    patches[:total, 1] = col
                    patches[:total, 2] = self.tables[rows[pos], col]
            self.dev_row[:n] = rows
            self.dev_epoch[:n] = self.row_epoch[rows]
            self.dev_blocks[:n] = nblk
        if count < 0:
            width = int(nblk.max())
            out_tables[:n, :width] = self.tables[rows, :width]
        out_ids[:n] = [s.last_token for s in seqs]
        out_lens[:n] = lens
        # the block the new token falls into: the last one, unless blocks were opened ahead for later steps
        out_slots[:n] = self.tables[rows, (lens - 1) // bs].astype(np.int64) * bs + (lens - 1) % bs
        return count
