"""Per-request state (reference: engine/sequence.py:14-114).

Attribute and property names follow the reference so that scheduler / block-manager / runner code
written against it works unchanged.

``Sequence.reference_exact`` (class attribute, default False) selects how a length that is an exact
multiple of the block size is treated.  The reference computes ``last_block_num_tokens`` as the
length of ``token_ids[full_blocks * block_size:]`` (engine/sequence.py:66-69), which is 0 — not
``block_size`` — at exact multiples; ``block(last)`` then slices ``token_ids[-0:]``, the whole
list.  With ``reference_exact = True`` both are reproduced bit for bit (the host-path parity tests
run that way); by default the last block of an exactly-full sequence holds ``block_size`` tokens,
which is what the slot arithmetic of the model runner needs to address the right cache row.
"""
from __future__ import annotations

from enum import Enum, auto
from itertools import count

from .sampling_params import SamplingParams


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


class Sequence:
    block_size = 256          # tokens per KV block; the engine sets it from its config
    counter = count()         # process-wide sequence ids
    reference_exact = False   # see module docstring

    __slots__ = ("seq_id", "status", "token_ids", "last_token", "num_tokens", "num_prompt_tokens",
                 "num_cached_tokens", "block_table", "temperature", "max_tokens", "ignore_eos",
                 "max_model_length", "_bt_cache", "_row")

    def __init__(self, token_ids, sampling_params: SamplingParams | None = None):
        sp = sampling_params if sampling_params is not None else SamplingParams()
        self.seq_id = next(Sequence.counter)
        self.status = SequenceStatus.WAITING
        self.token_ids = list(token_ids)
        self.last_token = self.token_ids[-1] if self.token_ids else None
        self.num_tokens = self.num_prompt_tokens = len(self.token_ids)
        self.num_cached_tokens = 0
        self.block_table: list[int] = []
        self._bt_cache = None     # [list object, int32 buffer, entries valid]: see metadata.block_table_array
        self._row = None          # row of this sequence in a metadata.DecodeBatchBuilder table
        self.temperature = sp.temperature
        self.max_tokens = sp.max_tokens
        self.ignore_eos = sp.ignore_eos
        self.max_model_length = sp.max_model_length

    def __len__(self) -> int:
        return self.num_tokens

    def __getitem__(self, idx):
        return self.token_ids[idx]

    # ---- derived counters ---------------------------------------------------------------
    @property
    def is_finished(self) -> bool:
        return self.status is SequenceStatus.FINISHED

    @property
    def num_completion_tokens(self) -> int:
        return self.num_tokens - self.num_prompt_tokens

    @property
    def prompt_token_ids(self):
        return self.token_ids[:self.num_prompt_tokens]

    @property
    def completion_token_ids(self):
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def num_blocks(self) -> int:
        return (self.num_tokens + self.block_size - 1) // self.block_size

    @property
    def num_cached_blocks(self) -> int:
        return (self.num_cached_tokens + self.block_size - 1) // self.block_size

    @property
    def last_block_num_tokens(self) -> int:
        rem = self.num_tokens % self.block_size
        if rem or self.reference_exact or self.num_tokens == 0:
            return rem
        return self.block_size

    def block(self, i: int):
        """Token ids of the i-th block."""
        if not 0 <= i < self.num_blocks:
            raise IndexError(f"block {i} out of range [0, {self.num_blocks})")
        if self.reference_exact and i == self.num_blocks - 1:
            return self.token_ids[-self.last_block_num_tokens:]
        lo = i * self.block_size
        return self.token_ids[lo:lo + self.block_size]

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(token_id)
        self.last_token = token_id
        self.num_tokens += 1

    # ---- compact pickling: a decode step only ships the last token (sequence.py:88-113) ----
    def __getstate__(self):
        payload = self.token_ids if self.num_completion_tokens == 0 else self.last_token
        return (self.num_tokens, self.num_prompt_tokens, self.num_cached_tokens, self.block_table, payload)

    def __setstate__(self, state):
        self.num_tokens, self.num_prompt_tokens, self.num_cached_tokens, self.block_table, payload = state
        self._bt_cache = None
        self._row = None
        self.token_ids = payload if self.num_tokens == self.num_prompt_tokens else [payload]
        self.last_token = self.token_ids[-1] if self.token_ids else None
