"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

No public dataset is involved: token ids are uniform over the vocabulary, q/K/V are N(0,1), and
lengths follow the distribution each configuration names.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch


@dataclass
class PagedDecodeCase:
    """Metadata of a paged-decode batch (host side, numpy)."""
    context_lens: np.ndarray   # [B] int64
    block_tables: np.ndarray   # [B, maxb] int32, -1 padded
    slot_mapping: np.ndarray   # [B] int64: slot of the last token of every sequence
    num_blocks: int
    block_size: int

    @property
    def batch(self) -> int:
        return int(self.context_lens.shape[0])

    @property
    def total_tokens(self) -> int:
        return int(self.context_lens.sum())


def deal_blocks(context_lens, block_size: int, rng: np.random.Generator, pad_blocks: int = 0,
                pad_value: int = -1) -> PagedDecodeCase:
    """Physical pool = random permutation of block ids, dealt to the sequences in order."""
    lens = np.asarray(context_lens, dtype=np.int64)
    nblk = (lens + block_size - 1) // block_size
    total = int(nblk.sum()) + pad_blocks
    perm = rng.permutation(total).astype(np.int32)
    maxb = max(1, int(nblk.max()) if len(nblk) else 1)
    tables = np.full((len(lens), maxb), pad_value, dtype=np.int32)
    slots = np.full(len(lens), -1, dtype=np.int64)
    pos = 0
    for i, n in enumerate(nblk):
        n = int(n)
        tables[i, :n] = perm[pos:pos + n]
        pos += n
        if lens[i] > 0:
            last = int(lens[i]) - 1
            slots[i] = int(tables[i, last // block_size]) * block_size + last % block_size
    return PagedDecodeCase(lens, tables, slots, max(total, 1), block_size)


def c2_decode_case(batch: int = 256, lo: int = 128, hi: int = 8192, block_size: int = 16,
                   seed: int = 1) -> PagedDecodeCase:
    """Paged GQA decode microbenchmark metadata: context lengths log-uniform in [lo, hi]."""
    rng = np.random.default_rng(seed)
    lens = np.rint(np.exp(rng.uniform(math.log(lo), math.log(hi), size=batch))).astype(np.int64)
    lens = np.clip(lens, lo, hi)
    return deal_blocks(lens, block_size, rng, pad_blocks=8)


def decode_algorithmic_bytes(case: PagedDecodeCase, num_q_heads: int, num_kv_heads: int,
                             head_dim: int, itemsize: int) -> int:
    """Bytes one paged-decode call must move: every K and V row of every live context once, the
    block-table entries and context lengths it walks, q in and out."""
    lens = case.context_lens
    kv = int(lens.sum()) * 2 * num_kv_heads * head_dim * itemsize
    meta = int(((lens + case.block_size - 1) // case.block_size).sum()) * 4 + 8 * case.batch
    qo = case.batch * 2 * num_q_heads * head_dim * itemsize
    return kv + meta + qo


def randn_bf16_pool(shape, seed: int, device) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)


def c5_prefill_lengths(num_seqs: int = 64, total: int = 262144, lo: int = 1, hi: int = 16384,
                       alpha: float = 1.2, seed: int = 5) -> np.ndarray:
    """Ragged prefill stress lengths: Zipf(alpha) truncated to [lo, hi] by inverse CDF, rescaled so
    that the lengths sum to ``total`` (remainder goes to the longest sequence that still has room)."""
    rng = np.random.default_rng(seed)
    ks = np.arange(lo, hi + 1, dtype=np.float64)
    cdf = np.cumsum(ks ** -alpha)
    cdf /= cdf[-1]
    lens = ks[np.searchsorted(cdf, rng.uniform(size=num_seqs))]
    lens = np.clip(np.rint(lens * (total / lens.sum())), lo, hi).astype(np.int64)
    for _ in range(64):
        diff = total - int(lens.sum())
        if diff == 0:
            break
        order = np.argsort(-lens)
        for i in order:
            room = (hi - lens[i]) if diff > 0 else (lens[i] - lo)
            step = int(np.sign(diff)) * min(abs(diff), int(room))
            lens[i] += step
            diff -= step
            if diff == 0:
                break
    return lens


def prefill_flops(lens, num_q_heads: int, head_dim_qk: int, head_dim_v: int) -> float:
    """Causal attention FLOPs: every (query, visible key) pair costs 2*Dqk (scores) + 2*Dv (values)."""
    lens = np.asarray(lens, dtype=np.float64)
    pairs = (lens * (lens + 1) / 2).sum()
    return float(pairs * num_q_heads * 2 * (head_dim_qk + head_dim_v))


def c4_decode_case(batch: int = 240, lo: int = 512, hi: int = 16384, block_size: int = 16,
                   seed: int = 4) -> PagedDecodeCase:
    """MLA decode part of the mixed MLA workload: contexts uniform in [lo, hi]."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, size=batch).astype(np.int64)
    return deal_blocks(lens, block_size, rng, pad_blocks=8)


def c3_requests(num_requests: int = 2048, vocab: int = 32000, seed: int = 3, prompt_lo: int = 64,
                prompt_hi: int = 1024, mean_out: int = 256, max_out: int = 1024, rate: float | None = None):
    """Continuous-batching request stream: prompt lengths uniform in [lo, hi], output lengths
    geometric with the given mean capped at ``max_out``, token ids uniform; arrivals Poisson with
    ``rate`` requests/s (``None`` = all present at t = 0).  Returns (prompts, out_lens, arrivals)."""
    rng = np.random.default_rng(seed)
    plens = rng.integers(prompt_lo, prompt_hi + 1, size=num_requests)
    outs = np.minimum(rng.geometric(1.0 / mean_out, size=num_requests), max_out).astype(np.int64)
    prompts = [rng.integers(0, vocab, size=int(n)).tolist() for n in plens]
    arrivals = np.zeros(num_requests) if rate is None else np.cumsum(rng.exponential(1.0 / rate, size=num_requests))
    return prompts, outs, arrivals
