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


def pad_block_tables(seqs: list[Sequence]) -> np.ndarray:
    width = max(len(s.block_table) for s in seqs)
    out = np.full((len(seqs), max(width, 1)), -1, dtype=np.int32)
    for i, s in enumerate(seqs):
        out[i, :len(s.block_table)] = s.block_table
    return out


def prepare_prefill(seqs: list[Sequence], block_size: int) -> StepMetadata:
    """Packs the non-cached suffix of every sequence (model_runner.py:202-249).

    The reference produces no positions tensor; the RoPE position of packed token j of a sequence
    is ``num_cached_tokens + j``.
    """
    ids, slots, pos = [], [], []
    q_lens, k_lens = [], []
    for s in seqs:
        cached = s.num_cached_tokens
        ids.append(np.asarray(s.token_ids[cached:], dtype=np.int64))
        q_lens.append(s.num_tokens - cached)
        k_lens.append(s.num_tokens)
        pos.append(np.arange(cached, s.num_tokens, dtype=np.int64))
        if not s.block_table:
            continue
        first, last = s.num_cached_blocks, s.num_blocks - 1
        for j in range(first, len(s.block_table)):
            n = block_size if j != last else s.last_block_num_tokens
            base = s.block_table[j] * block_size
            slots.append(np.arange(base, base + n, dtype=np.int64))
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


def prepare_decode(seqs: list[Sequence], block_size: int) -> StepMetadata:
    """One token per running sequence (model_runner.py:253-278)."""
    n = len(seqs)
    lens = np.fromiter((s.num_tokens for s in seqs), dtype=np.int64, count=n)
    slots = np.fromiter((s.block_table[-1] * block_size + s.last_block_num_tokens - 1 for s in seqs),
                        dtype=np.int64, count=n)
    return StepMetadata(
        is_prefill=False,
        input_ids=np.fromiter((s.last_token for s in seqs), dtype=np.int64, count=n),
        slot_mapping=slots, positions=lens - 1, context_lens=lens,
        block_tables=pad_block_tables(seqs), last_token_index=np.arange(n, dtype=np.int64))
