"""Process-global attention metadata handed from the model runner to the attention layers.

Same fields and accessors as the reference's utils/context.py:5-27, so a model written against the
reference's context reads this one unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class Context:
    is_prefill: bool = False
    cu_seqlens_q: Optional[torch.Tensor] = None   # int32 [num_seqs + 1]
    cu_seqlens_k: Optional[torch.Tensor] = None   # int32 [num_seqs + 1]
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    slot_mapping: Optional[torch.Tensor] = None   # int64 [num_tokens], -1 = skip
    context_lens: Optional[torch.Tensor] = None   # int64 [batch] (decode)
    block_tables: Optional[torch.Tensor] = None   # int32 [batch, max_blocks], -1 padded
    # not in the reference (its runner builds no positions although the model needs them for RoPE):
    positions: Optional[torch.Tensor] = None      # int64 [num_tokens]; None in decode = context_lens - 1
    prefill_plan: object = None                   # ops.PrefillPlan of this step's cu_seqlens_q, or None


_current = Context()


def get_context() -> Context:
    return _current


def set_context(is_prefill, cu_seqlens_q=None, cu_seqlens_k=None, max_seqlen_q=0, max_seqlen_k=0,
                slot_mapping=None, context_lens=None, block_tables=None, positions=None,
                prefill_plan=None) -> None:
    global _current
    _current = Context(is_prefill, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                       slot_mapping, context_lens, block_tables, positions, prefill_plan)


def reset_context() -> None:
    global _current
    _current = Context()
