"""Seeded request scenarios for the host-path (scheduler / block manager / metadata) parity tests.

Shared by ``make_golden.py`` (which drives the REFERENCE classes with them and records every step)
and by the tests (which drive the oracle and the product host layer with the same inputs).  The
"model" is a pure function of (sequence id, sequence length), so token streams are reproducible
without any weights.
"""
from __future__ import annotations

import random

VOCAB = 10000
EOS = 7


def fake_next_token(seq_id: int, num_tokens: int, eos_every: int = 0) -> int:
    """Deterministic stand-in for model + sampler.  ``num_tokens`` is the length before appending."""
    if eos_every and (seq_id + num_tokens) % eos_every == 0:
        return EOS
    t = (seq_id * 7919 + num_tokens * 104729 + 13) % VOCAB
    return t if t != EOS else EOS + 1


def _rand_ids(rng: random.Random, n: int) -> list[int]:
    return [rng.randrange(VOCAB) for _ in range(n)]


def scenarios() -> dict:
    """name -> dict(engine=..., requests=[{arrival_step, token_ids, params}], eos_every=...)."""
    out = {}

    # 8 prompts with lengths in [16,128], 64 new tokens each (max_tokens 65: the reference stops one
    # token early), one prefill batch then pure decode.
    rng = random.Random(0)
    reqs = []
    for _ in range(8):
        n = rng.randint(16, 128)
        reqs.append(dict(arrival_step=0, token_ids=_rand_ids(rng, n),
                         params=dict(temperature=1.0, max_tokens=65, ignore_eos=True, max_model_length=None)))
    out["eight_prompts"] = dict(
        engine=dict(max_num_sequences=16, max_num_batched_tokens=1024, max_cached_blocks=256, block_size=16, eos=EOS),
        requests=reqs, eos_every=0)

    # shared prefixes: later arrivals hit blocks that are still in use -> cached prefill with block_tables
    rng = random.Random(1)
    base = _rand_ids(rng, 48)
    other = _rand_ids(rng, 33)
    dup = base + [1, 2, 3]
    reqs = [
        dict(arrival_step=0, token_ids=base + _rand_ids(rng, 10)),
        dict(arrival_step=0, token_ids=base + _rand_ids(rng, 21)),
        dict(arrival_step=2, token_ids=base[:32] + _rand_ids(rng, 9)),
        dict(arrival_step=2, token_ids=list(dup)),
        dict(arrival_step=4, token_ids=other),
        dict(arrival_step=5, token_ids=other + _rand_ids(rng, 14)),
        dict(arrival_step=9, token_ids=list(dup)),
        dict(arrival_step=30, token_ids=base[:16]),
        dict(arrival_step=31, token_ids=base + _rand_ids(rng, 40)),
    ]
    for i, r in enumerate(reqs):
        r["params"] = dict(temperature=1.0, max_tokens=12 + 3 * i, ignore_eos=True, max_model_length=None)
    out["shared_prefixes"] = dict(
        engine=dict(max_num_sequences=8, max_num_batched_tokens=512, max_cached_blocks=512, block_size=16, eos=EOS),
        requests=reqs, eos_every=0)

    # admission limits, EOS stops, max_model_length stops, staggered arrivals, small blocks
    rng = random.Random(2)
    reqs = []
    for i in range(14):
        n = rng.randint(3, 90)
        if n % 8 == 0 and n > 8:
            n += 1  # the reference asserts on multi-block prompts that fill their last block
        reqs.append(dict(
            arrival_step=rng.choice([0, 0, 0, 1, 3, 8, 20]),
            token_ids=_rand_ids(rng, n),
            params=dict(temperature=1.0, max_tokens=rng.randint(2, 40), ignore_eos=(i % 3 == 0),
                        max_model_length=(n + 7 if i % 4 == 1 else None))))
    reqs.sort(key=lambda r: r["arrival_step"])
    out["limits_and_stops"] = dict(
        engine=dict(max_num_sequences=4, max_num_batched_tokens=120, max_cached_blocks=2048, block_size=8, eos=EOS),
        requests=reqs, eos_every=11)

    # block-boundary lengths with block size 16 (a multi-block prompt that exactly fills its last
    # block makes the reference raise, so 32 and 48 are left out; 16 runs but loses its slots)
    reqs = [dict(arrival_step=0, token_ids=_rand_ids(rng, n),
                 params=dict(temperature=1.0, max_tokens=36, ignore_eos=True, max_model_length=None))
            for n in (1, 15, 16, 17, 31, 33, 47)]
    out["block_boundaries"] = dict(
        engine=dict(max_num_sequences=16, max_num_batched_tokens=4096, max_cached_blocks=128, block_size=16, eos=EOS),
        requests=reqs, eos_every=0)
    return out
