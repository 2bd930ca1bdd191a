"""Timed runs of the secondary kernels on their benchmark shapes (used by ``bench.py --workload``).

Each function builds the seeded synthetic inputs on the current CUDA device, times the op with CUDA
events after warm-up and returns a dict with the time per call, the algorithmic bytes / FLOPs of a
call and the achieved rate.  Inputs are larger than the 126 MB L2, so no flush is needed.
"""
from __future__ import annotations

import numpy as np
import torch

from . import ops
from .workloads import c4_decode_case, c5_prefill_lengths, prefill_flops


def _time(fn, steps: int, warmup: int) -> float:
    for _ in range(max(warmup, 1)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def mla_decode(steps: int = 50, warmup: int = 5, batch: int = 240) -> dict:
    """MLA latent decode: ``batch`` sequences, contexts uniform in [512,16384], 16 heads, 512+64."""
    case = c4_decode_case(batch)
    H, r, dr = 16, 512, 64
    g = torch.Generator(device="cuda").manual_seed(4)
    lat = torch.randn(case.num_blocks, 16, r + dr, generator=g, device="cuda", dtype=torch.bfloat16)
    qa = (torch.randn(case.batch, H, r, generator=g, device="cuda") * 0.2).to(torch.bfloat16)
    qr = torch.randn(case.batch, H, dr, generator=g, device="cuda", dtype=torch.bfloat16)
    bt, cl = torch.from_numpy(case.block_tables).cuda(), torch.from_numpy(case.context_lens).cuda()
    out = torch.empty_like(qa)
    ms = _time(lambda: ops.mla_decode(qa, qr, lat, bt, cl, 192 ** -0.5, out=out), steps, warmup)
    ops.check_status()
    tok = case.total_tokens
    nbytes = tok * (r + dr) * 2 + case.batch * H * (2 * r + dr) * 2 + 4 * int(((case.context_lens + 15) // 16).sum())
    flops = tok * H * 2 * (2 * r + dr)
    return dict(workload=f"MLA latent decode: {case.batch} seqs, ctx uniform [512,16384], 16 heads, r=512, dr=64, bf16",
                ms=ms, context_tokens=tok, algorithmic_bytes=nbytes, flops=flops, gbs=nbytes / ms / 1e6,
                tflops=flops / ms / 1e9, launches_per_call=2)


def prefill(steps: int = 5, warmup: int = 2, total: int = 262144) -> dict:
    """Ragged causal prefill: 64 sequences, Zipf(1.2) lengths in [1,16384], 32/8 heads, head_dim 128,
    together with the store_kvcache scatter of the same tokens into a block-16 pool through a shuffled
    slot mapping (seed 2).  One call = tile list + (scatter, attention) through one entry point; the attention
    alone is also timed."""
    lens = c5_prefill_lengths(total=total)
    T, Hq, Hkv, D = int(lens.sum()), 32, 8, 128
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(T, Hq, D, generator=g, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(T, Hkv, D, generator=g, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(T, Hkv, D, generator=g, device="cuda", dtype=torch.bfloat16)
    cu = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).cuda()
    out = torch.empty_like(q)
    mx = int(lens.max())
    rows = ops.prefill_tile_rows(Hq, Hkv, D, D, torch.bfloat16)

    bs = 16
    nblk = (T + bs - 1) // bs
    perm = torch.randperm(nblk, generator=g, device="cuda")
    slots = (perm.repeat_interleave(bs) * bs + torch.arange(bs, device="cuda").repeat(nblk))[:T].to(torch.int64)
    kc = torch.zeros(nblk, bs, Hkv, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)

    def attention():   # the tile list is per-step work (shared by the layers of a model): timed with the attention
        plan = ops.prefill_plan(cu, T, mx, rows)
        ops.prefill_varlen(q, k, v, cu, cu, mx, mx, D ** -0.5, out=out, plan=plan)

    def call():        # the scatter rides in the attention call (slot_mapping argument of b200_prefill_varlen)
        plan = ops.prefill_plan(cu, T, mx, rows)
        ops.prefill_varlen(q, k, v, cu, cu, mx, mx, D ** -0.5, out=out, plan=plan, k_cache=kc, v_cache=vc,
                           slot_mapping=slots)

    ms_att = _time(attention, steps, warmup)
    ms = _time(call, steps, warmup)
    ops.check_status()
    flops = prefill_flops(lens, Hq, D, D)
    return dict(workload=f"ragged causal prefill: 64 seqs, Zipf(1.2) lengths in [1,16384], {T} tokens, 32/8 heads, "
                         "head_dim 128, bf16", ms=ms, tokens=T, lengths=sorted(lens.tolist(), reverse=True),
                flops=flops, tflops=flops / ms / 1e9, attention_only_ms=ms_att, attention_only_tflops=flops / ms_att / 1e9,
                scatter_bytes=T * (2 * Hkv * D * 2 * 2 + 8), launches_per_call=3)


def mla_prefill(steps: int = 10, warmup: int = 3, seqs: int = 16) -> dict:
    """Prefill attention of the MLA+MoE decoder's benchmark step: ``seqs`` prompts with lengths uniform
    [256,4096] (seed 4), 16 heads, keys = 128 per-head columns (a strided view of the fused up-projection
    output, like the values) + 64 rotary columns shared by all heads (a view of the latent rows), values
    128 wide; one call = the step's tile list + the attention of one layer."""
    rng = np.random.default_rng(4)
    lens = rng.integers(256, 4097, size=seqs)
    T, H, hd, dr, r = int(lens.sum()), 16, 128, 64, 512
    g = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn(T, H, hd + dr, generator=g, device="cuda", dtype=torch.bfloat16)
    kv = torch.randn(T, 2 * H * hd, generator=g, device="cuda", dtype=torch.bfloat16)
    rows = torch.randn(T, r + dr, generator=g, device="cuda", dtype=torch.bfloat16)
    k_head, v, tail = kv[:, :H * hd].view(T, H, hd), kv[:, H * hd:].view(T, H, hd), rows[:, r:]
    cu = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).cuda()
    out = torch.empty(T, H, hd, device="cuda", dtype=torch.bfloat16)
    mx = int(lens.max())
    tile_rows = ops.prefill_tile_rows(H, H, hd + dr, hd, torch.bfloat16)

    def call():
        plan = ops.prefill_plan(cu, T, mx, tile_rows)
        ops.prefill_varlen_shared_tail(q, k_head, tail, v, cu, cu, mx, (hd + dr) ** -0.5, out=out, plan=plan)

    ms = _time(call, steps, warmup)
    ops.check_status()
    flops = prefill_flops(lens, H, hd + dr, hd)
    return dict(workload=f"MLA prefill attention: {seqs} seqs U[256,4096], {T} tokens, 16 heads, 192/128 head dims "
                         "(128 + shared 64-wide rotary tail), bf16", ms=ms, tokens=T, flops=flops,
                tflops=flops / ms / 1e9, tile_rows=tile_rows, launches_per_call=2)


def prefill64(steps: int = 20, warmup: int = 3, seqs: int = 120) -> dict:
    """Prefill attention at the GQA+MoE decoder's shape (16 query heads / 4 KV heads, head_dim 64) on a batch of
    the continuous-batching workload's prompts: ``seqs`` sequences with lengths uniform [64,1024] (seed 3), packed;
    one call = the step's tile list + the attention of one layer (tcgen05, four heads of a KV head per CTA)."""
    rng = np.random.default_rng(3)
    lens = rng.integers(64, 1025, size=seqs)
    T, Hq, Hkv, D = int(lens.sum()), 16, 4, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, generator=g, device="cuda", dtype=torch.bfloat16)   # fused projection output
    q = qkv[:, :Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D:].view(T, Hkv, D)
    cu = torch.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).cuda()
    out = torch.empty(T, Hq, D, device="cuda", dtype=torch.bfloat16)
    mx = int(lens.max())
    rows = ops.prefill_tile_rows(Hq, Hkv, D, D, torch.bfloat16)

    def call():
        plan = ops.prefill_plan(cu, T, mx, rows)
        ops.prefill_varlen(q, k, v, cu, cu, mx, mx, D ** -0.5, out=out, plan=plan)

    ms = _time(call, steps, warmup)
    ops.check_status()
    flops = prefill_flops(lens, Hq, D, D)
    return dict(workload=f"prefill attention, head_dim 64: {seqs} seqs U[64,1024], {T} tokens, 16/4 heads, bf16",
                ms=ms, tokens=T, flops=flops, tflops=flops / ms / 1e9, tile_rows=rows, launches_per_call=2)


def lm_head(steps: int = 50, warmup: int = 5, rows: int = 64) -> dict:
    """Greedy head of the GQA+MoE decoder: ``rows`` hidden states x the [32000, 1024] head matrix (+ bias), argmax
    per row, fused (the logits are never written); 64 rows is the largest batch for which the engine uses the fused
    head (above it the library GEMM + the argmax kernel are faster).  Eight distinct head matrices are used in turn so that the
    65.5 MB matrix is streamed from HBM on every call, as in a decode step (the other weights of a step evict it
    from the 126 MB L2)."""
    V, d = 32000, 1024
    g = torch.Generator(device="cuda").manual_seed(7)
    ws = [(torch.randn(V, d, generator=g, device="cuda") * d ** -0.5).bfloat16() for _ in range(8)]
    b = (torch.randn(V, generator=g, device="cuda") * 0.1).bfloat16()
    h = torch.randn(rows, d, generator=g, device="cuda").bfloat16()
    out = torch.empty(rows, dtype=torch.int64, device="cuda")
    state = {"i": 0}

    def call():
        ops.lm_head_argmax(h, ws[state["i"] % 8], b, out)
        state["i"] += 1

    ms = _time(call, steps, warmup)
    ops.check_status()
    nbytes = V * d * 2 + V * 2 + rows * d * 2 + rows * 8
    return dict(workload=f"greedy head: {rows} rows x [32000, 1024] + bias -> argmax, bf16, fused",
                ms=ms, algorithmic_bytes=nbytes, gbs=nbytes / ms / 1e6, launches_per_call=2)


def store(steps: int = 50, warmup: int = 5, tokens: int = 262144) -> dict:
    """store_kvcache of the prefill stress batch: shuffled slot mapping (seed 2), 8 x 128 bf16 rows."""
    Hkv, D, bs = 8, 128, 16
    g = torch.Generator(device="cuda").manual_seed(2)
    k = torch.randn(tokens, Hkv, D, generator=g, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(tokens, Hkv, D, generator=g, device="cuda", dtype=torch.bfloat16)
    nblk = tokens // bs
    perm = torch.randperm(nblk, generator=g, device="cuda")
    slots = (perm.repeat_interleave(bs) * bs + torch.arange(bs, device="cuda").repeat(nblk)).to(torch.int64)
    kc = torch.zeros(nblk, bs, Hkv, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    ms = _time(lambda: ops.store_kvcache(k, v, kc, vc, slots), steps, warmup)
    ops.check_status()
    nbytes = tokens * (2 * Hkv * D * 2 * 2 + 8)
    return dict(workload=f"store_kvcache: {tokens} tokens, 8 kv heads x 128, bf16, block-contiguous shuffled slots",
                ms=ms, tokens=tokens, algorithmic_bytes=nbytes, gbs=nbytes / ms / 1e6, launches_per_call=1)


def moe_experts(steps: int = 20, warmup: int = 3, tokens: int = 256, layers: int = 12) -> dict:
    """Expert GEMMs of the GQA+MoE decoder at decode size: ``tokens`` tokens routed top-2 over 16 experts
    (d_model 1024, d_ff 704, bf16); per layer the grouped up-projection + SwiGLU and the grouped
    down-projection stream 69 MB of expert weights.  ``layers`` distinct weight sets (0.83 GB) are run
    back to back from one CUDA graph, so no weight stays in L2 between uses, as in the model."""
    E, d, dff, K = 16, 1024, 704, 2
    g = torch.Generator(device="cuda").manual_seed(6)
    w13 = [(torch.randn(E, 2 * dff, d, generator=g, device="cuda") * d ** -0.5).bfloat16() for _ in range(layers)]
    w2 = [(torch.randn(E, d, dff, generator=g, device="cuda") * dff ** -0.5).bfloat16() for _ in range(layers)]
    b13 = torch.randn(E, 2 * dff, generator=g, device="cuda").bfloat16()
    logits = torch.randn(tokens, E, generator=g, device="cuda").bfloat16()
    _tok, _experts, _w, offs, _inv = ops.moe_route(logits, torch.zeros(E, device="cuda"), K)
    xs = torch.randn(tokens * K, d, generator=g, device="cuda").bfloat16()

    def all_layers():
        for i in range(layers):
            ops.moe_grouped_gemm(ops.moe_grouped_gemm(xs, w13[i], offs, b13, swiglu=True, early_launch=True), w2[i], offs,
                                 early_launch=True)

    all_layers()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        all_layers()
    ms = _time(graph.replay, steps, warmup) / layers
    ops.check_status()
    nbytes = (w13[0].numel() + w2[0].numel()) * 2 + tokens * K * (d + 2 * dff + d) * 2
    return dict(workload=f"MoE expert GEMMs, decode size: {tokens} tokens top-2 over 16 experts, d 1024, d_ff 704, "
                         f"bf16; {layers} layers from one CUDA graph", ms=ms, us_per_layer=ms * 1e3,
                algorithmic_bytes=nbytes, gbs=nbytes / ms / 1e6, launches_per_call=2)


C3_MODEL = dict(vocab_size=32000, context_length=2048, d_model=1024, num_layers=16, num_heads=16, num_kv_heads=4,
                d_ff=704, attention_type="GQA", use_moe=True, n_routed_experts=16, num_experts_per_tok=2,
                n_shared_experts=1)


def engine(steps: int = 0, warmup: int = 0, batch: int = 512, rate: float | None = None,
           pool_blocks: int = 110000, decode_window: int = 1) -> dict:
    """End-to-end continuous batching, GQA+MoE decoder (d_model 1024, 16 layers, 16/4 heads, head_dim 64,
    16 experts top-2 + shared, d_ff 704, vocab 32000), bf16, random init (seed 0): ``batch`` requests,
    prompts uniform [64,1024], outputs geometric(mean 256) capped at 1024, max 256 sequences and 8192
    batched tokens per step, KV block 16; arrivals Poisson with ``rate`` requests/s, or all at t = 0.
    The KV pool holds ``pool_blocks`` blocks of 256 KiB (110,000 = 27 GB: the cumulative demand of the
    2048 requests, so no request is preempted and re-prefilled; the scheduler admits waiting requests
    before it decodes, whatever the number already running, and fills any smaller pool).
    Under torchrun every rank is an independent replica serving requests rank, rank + N, ...; the
    aggregate is tokens of all replicas / the slowest replica's wall time.  ``steps``/``warmup`` unused.
    ``decode_window`` > 1: that many decode steps per scheduling decision (the engine's ``decode_window``)."""
    import itertools
    import os
    import time

    import torch.distributed as dist

    from .engine import SamplingParams, Sequence
    from .engine.llm_engine import LLMEngine
    from .engine.replicas import serve_sharded
    from .workloads import c3_requests
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    prompts, outs, arrivals = c3_requests(batch, rate=rate)
    built = {}

    def make_engine(rank):
        Sequence.counter = itertools.count()
        cfg = dict(model=C3_MODEL, dtype=torch.bfloat16, block_size=16, max_num_sequences=256,
                   max_num_batched_tokens=8192, max_cached_blocks=pool_blocks, eos=-1, device=f"cuda:{local_rank}",
                   max_model_length=2048, seed=0, decode_window=decode_window)
        t0 = time.perf_counter()
        built["engine"] = LLMEngine(cfg)
        built["build_s"] = time.perf_counter() - t0
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()        # replicas start serving together
        return built["engine"]

    requests = [(p, SamplingParams(temperature=0.0, max_tokens=int(n) + 1, ignore_eos=True))
                for p, n in zip(prompts, outs)]
    tokens, reports = serve_sharded(make_engine, requests, None if rate is None else arrivals.tolist())
    torch.cuda.synchronize()
    ops.check_status()
    eng = built["engine"]
    graphs, timing = bool(eng.model_runner.graphs), dict(eng.timing)
    eng.exit()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if tokens is None:            # not rank 0
        return {}
    gen = sum(len(t) for t in tokens)
    assert gen == int(outs.sum()), (gen, int(outs.sum()))
    wall = max(r.wall_s for r in reports)
    prompt_tokens = int(sum(len(p) for p in prompts))
    out = dict(workload=f"continuous batching GQA+MoE bf16: {batch} requests "
                        f"({'all at t=0' if rate is None else f'Poisson {rate}/s'}), prompts U[64,1024], outputs "
                        "geometric(256) cap 1024, max 256 seqs / 8192 tokens per step per replica",
               replicas=world, requests=batch, generated_tokens=gen, prompt_tokens=prompt_tokens, wall_s=wall,
               replica_wall_s=[r.wall_s for r in reports], steps=[r.steps for r in reports],
               output_tokens_per_s=gen / wall, total_tokens_per_s=(gen + prompt_tokens) / wall,
               engine_build_s=built["build_s"], cuda_graphs=graphs, kv_pool_blocks=pool_blocks,
               decode_window=decode_window, rank0_timing=timing)
    if rate is not None:
        out["latency"] = request_latencies(reports)
    return out


def request_latencies(reports) -> dict:
    """Per-request latencies of an online run over all replicas: time to the first token (arrival -> end of the
    step that produced it), time per output token after the first, and arrival -> completion."""
    ttft, tpot, e2e = [], [], []
    for r in reports:
        for a, f, d, toks in zip(r.arrival_s, r.first_token_s, r.finish_s, r.token_ids):
            ttft.append(f - a)
            e2e.append(d - a)
            if len(toks) > 1:
                tpot.append((d - f) / (len(toks) - 1))
    q = lambda v, p: float(np.percentile(v, p)) if v else None
    return dict(ttft_ms={"p50": q(ttft, 50) * 1e3, "p90": q(ttft, 90) * 1e3, "p99": q(ttft, 99) * 1e3},
                ms_per_output_token={"mean": float(np.mean(tpot)) * 1e3, "p50": q(tpot, 50) * 1e3, "p99": q(tpot, 99) * 1e3},
                request_s={"p50": q(e2e, 50), "p99": q(e2e, 99)})


def decode_step_bytes(model: dict, seq_steps: int, ctx_tokens: int, steps: int, itemsize: int = 2) -> float:
    """Bytes the decode steps of a GQA(+MoE) decoder must move, summed over ``steps`` steps that advanced
    ``seq_steps`` sequences in total over ``ctx_tokens`` context tokens in total:

    * per step, every weight the step touches, once: the attention projections, the MoE gate, the shared
      expert, the routed experts that at least one token selected (expected count for a step of the average
      batch size with uniform routing: E (1 - (1 - k/E)^batch)), and the lm_head matrix;
    * per context token, its K and V rows in every layer (read); per stepped sequence, the new K/V rows
      (written), its embedding row (fp32) and its logits row (written by the GEMM, read by the argmax).
    Activations between the layers' kernels are left out: they are a small fraction of this and mostly stay
    in the 126 MB L2."""
    d, L, H, Hkv = model["d_model"], model["num_layers"], model["num_heads"], model["num_kv_heads"]
    hd, dff, V = d // H, model["d_ff"], model["vocab_size"]
    E, K = model.get("n_routed_experts", 0), model.get("num_experts_per_tok", 0)
    attn = d * (H * hd + 2 * Hkv * hd) + (H * hd + 2 * Hkv * hd) + H * hd * d + d
    expert = 3 * d * dff + 2 * dff + d
    batch = seq_steps / max(steps, 1)
    if model.get("use_moe"):
        touched = E * (1.0 - (1.0 - K / E) ** batch)
        ffn = d * E + touched * expert + model.get("n_shared_experts", 0) * expert
    else:
        ffn = expert
    weights = (L * (attn + ffn) + V * d + V) * itemsize
    kv_row = L * 2 * Hkv * hd * itemsize
    return steps * weights + ctx_tokens * kv_row + seq_steps * (kv_row + d * 4 + 2 * V * itemsize)


def engine_jobs(pool_blocks: int = 110000, requests: int = 2048, decode_window: int = 8,
                hbm_peak_gbs: float = 6542.1, online_rate: float = 256.0) -> dict:
    """The continuous-batching benchmark through the engine (GQA+MoE decoder of ``C3_MODEL``, bf16, random init
    seed 0, KV block 16, at most 256 sequences and 8192 batched tokens per step, all requests present at
    t = 0), as the two jobs a multi-GPU run can mean.  Every rank of the process group is an independent
    replica with its own scheduler, block pool and KV cache; nothing is exchanged while a job runs.

    * ``fixed``: ``requests`` requests in total; replica r serves requests r, r + N, ...  (strong scaling)
    * ``weak``:  ``requests`` requests per replica, each replica its own seeded stream   (weak scaling)

    ``fixed`` runs twice: with one decode step per scheduling decision (the reference's loop) and, as
    ``fixed_window``, with ``decode_window`` decode graph replays per decision (same token streams; the sampled
    token of one step feeds the next on the device); ``weak`` runs with the window.
    With one replica fixed and weak are the same job.  Rates are tokens of all replicas over the
    slowest replica's wall time.

    * ``online``: the fixed job's requests arriving as a Poisson process of ``online_rate`` requests/s in total (the
      other arrival pattern of the configuration; 0 skips it), one decode step per scheduling decision: the load
      is below what the engine sustains, so the record is about latency — time to the first token, time per
      output token, arrival to completion — not throughput.

    Returns {} on ranks other than 0."""
    import itertools
    import os
    import time

    import torch.distributed as dist

    from .engine import SamplingParams, Sequence
    from .engine.llm_engine import LLMEngine
    from .engine.replicas import serve_shard, shard_requests
    from .workloads import c3_requests
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    distributed = world > 1 and dist.is_initialized()
    Sequence.counter = itertools.count()
    cfg = dict(model=C3_MODEL, dtype=torch.bfloat16, block_size=16, max_num_sequences=256,
               max_num_batched_tokens=8192, max_cached_blocks=pool_blocks, eos=-1, device=f"cuda:{local_rank}",
               max_model_length=2048, seed=0, decode_window=1)
    t0 = time.perf_counter()
    eng = LLMEngine(cfg)
    build_s = time.perf_counter() - t0

    def run(job: str, window: int, rate: float | None = None):
        eng.decode_window = window
        # a fresh block pool: a job must not find the previous job's prompts in the prefix cache
        bm = eng.scheduler.block_manager
        eng.scheduler.block_manager = type(bm)(eng.model_runner.num_kv_blocks, bm.block_size)
        arrivals = None
        if job == "fixed":
            prompts, outs, arr = c3_requests(requests, seed=3, rate=rate)
            shard = shard_requests(list(zip(prompts, outs)), world, rank)
            if rate is not None:
                arrivals = shard_requests(arr.tolist(), world, rank)
        else:
            prompts, outs, _ = c3_requests(requests, seed=1000 + rank)
            shard = list(zip(prompts, outs))
        reqs = [(p, SamplingParams(temperature=0.0, max_tokens=int(n) + 1, ignore_eos=True)) for p, n in shard]
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()                      # replicas start the job together
        rep = serve_shard(eng, reqs, rank, arrivals)
        torch.cuda.synchronize()
        ops.check_status()
        gen = sum(len(t) for t in rep.token_ids)
        assert gen == int(sum(n for _, n in shard)), (gen, job)
        t = rep.timing
        nbytes = decode_step_bytes(C3_MODEL, t["decode_seq_steps"], t["decode_ctx_tokens"], t["decode_steps"])
        mine = dict(wall_s=rep.wall_s, generated=gen, prompt=sum(len(p) for p, _ in shard), steps=rep.steps,
                    decode_steps=t["decode_steps"], prefill_steps=t["prefill_steps"], run_decode_s=t["run_decode_s"],
                    run_prefill_s=t["run_prefill_s"], schedule_s=t["schedule_s"], postprocess_s=t["postprocess_s"],
                    decode_seq_steps=t["decode_seq_steps"], decode_ctx_tokens=t["decode_ctx_tokens"],
                    decode_bytes=nbytes)
        if rate is not None:
            mine["report"] = rep
        rows = [mine]
        if distributed:
            rows = [None] * world if rank == 0 else None
            dist.gather_object(mine, rows, dst=0)
        if rank != 0:
            return None
        if rate is not None:
            lat = request_latencies([r["report"] for r in rows])
            wall = max(r["wall_s"] for r in rows)
            gen_all = sum(r["generated"] for r in rows)
            return dict(decode_window=window, requests=requests, replicas=world, arrivals=f"Poisson, {rate:g} requests/s "
                        "over all replicas (seed 3), request i to replica i mod N", wall_s=wall,
                        output_tokens_per_s=gen_all / wall, latency=lat,
                        mean_decode_batch=sum(r["decode_seq_steps"] for r in rows) / max(sum(r["decode_steps"] for r in rows), 1))
        wall = max(r["wall_s"] for r in rows)
        gen_all, prompt_all = sum(r["generated"] for r in rows), sum(r["prompt"] for r in rows)
        fracs = [r["decode_bytes"] / r["run_decode_s"] / 1e9 / hbm_peak_gbs for r in rows]
        return dict(
            decode_window=window,
            requests=requests * (world if job == "weak" else 1), replicas=world, generated_tokens=gen_all,
            prompt_tokens=prompt_all, wall_s=wall, replica_wall_s=[round(r["wall_s"], 4) for r in rows],
            output_tokens_per_s=gen_all / wall, total_tokens_per_s=(gen_all + prompt_all) / wall,
            decode_steps=[r["decode_steps"] for r in rows], prefill_steps=[r["prefill_steps"] for r in rows],
            decode_step_ms=max(1e3 * r["run_decode_s"] / max(r["decode_steps"], 1) for r in rows),
            mean_decode_batch=sum(r["decode_seq_steps"] for r in rows) / max(sum(r["decode_steps"] for r in rows), 1),
            mean_context_tokens_per_step=sum(r["decode_ctx_tokens"] for r in rows) / max(sum(r["decode_steps"] for r in rows), 1),
            # bytes the decode steps had to move (weights touched + KV of the live contexts + logits) over the wall
            # time of those steps (host share included), against the measured HBM copy peak
            decode_hbm_frac=min(fracs), decode_hbm_frac_by_replica=[round(f, 4) for f in fracs],
            decode_gbs=min(r["decode_bytes"] / r["run_decode_s"] / 1e9 for r in rows),
            host_s=dict(schedule=rows[0]["schedule_s"], postprocess=rows[0]["postprocess_s"]),
            prefill_tokens_per_s=rows[0]["prompt"] / max(rows[0]["run_prefill_s"], 1e-9))

    out = dict(model="GQA+MoE decoder: d_model 1024, 16 layers, 16/4 heads, head_dim 64, 16 experts top-2 + shared, "
                     "d_ff 704, vocab 32000, bf16, random init seed 0",
               workload=f"{requests} requests at t=0, prompts U[64,1024], outputs geometric(256) cap 1024, max 256 "
                        "seqs / 8192 tokens per step per replica, KV block 16",
               replicas=world, kv_pool_blocks=pool_blocks, engine_build_s=build_s,
               cuda_graphs=bool(eng.model_runner.graphs))
    fixed = run("fixed", 1)
    fixed_window = run("fixed", decode_window)
    weak = run("weak", decode_window) if world > 1 else None
    online = run("fixed", 1, rate=online_rate) if online_rate else None
    eng.exit()
    if rank != 0:
        return {}
    out["fixed"] = fixed
    out["fixed_window"] = fixed_window
    out["weak"] = weak if weak is not None else "one replica: the same job as fixed_window"
    if online is not None:
        out["online"] = online
    return out


def engine_step(steps: int = 0, warmup: int = 0, batch: int = 1024) -> dict:
    """Kernel shares of one decode step and one prefill step of the GQA+MoE engine at steady state
    (``batch`` requests of the continuous-batching workload, all at t = 0): the engine runs normally and
    the first decode step after engine step 300 and the first prefill step after engine step 40 are
    recorded with the CUPTI activity profiler.  Durations under the profiler are for shares, not rates."""
    import itertools

    from torch.profiler import ProfilerActivity, profile

    from .engine import SamplingParams, Sequence
    from .engine.llm_engine import LLMEngine
    from .workloads import c3_requests
    prompts, outs, _ = c3_requests(batch, rate=None)
    Sequence.counter = itertools.count()
    eng = LLMEngine(dict(model=C3_MODEL, dtype=torch.bfloat16, block_size=16, max_num_sequences=256,
                         max_num_batched_tokens=8192, max_cached_blocks=110000, eos=-1, device="cuda:0",
                         max_model_length=2048, seed=0))
    for p, n in zip(prompts, outs):
        eng.add_request(p, SamplingParams(temperature=0.0, max_tokens=int(n) + 1, ignore_eos=True))
    want = {"prefill": 40, "decode": 300}
    got, step = {}, 0
    while not eng.is_finished():
        due = [k for k, first in want.items() if k not in got and step >= first]
        if not due:
            eng.step()
            step += 1
            continue
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            _out, n, is_prefill = eng.step()
            torch.cuda.synchronize()
        step += 1
        kind = "prefill" if is_prefill else "decode"
        if kind in due:
            rows = [(e.key, e.self_device_time_total, e.count) for e in prof.key_averages()
                    if e.self_device_time_total > 0 and not e.key.startswith(("aten::", "cuda", "Memcpy", "Memset",
                                                                              "Activity", "Lazy"))]
            total = sum(r[1] for r in rows)
            rows.sort(key=lambda r: -r[1])
            got[kind] = dict(engine_step=step, tokens=n, kernel_us=total, kernels=[
                dict(name=k[:100], us=round(us, 1), share=round(us / total, 4), launches=c) for k, us, c in rows[:14]])
    ops.check_status()
    eng.exit()
    return dict(workload=f"GQA+MoE engine, {batch} requests at t=0: kernel shares of one decode and one prefill step "
                         "(CUPTI activity records)", **got)


C4_MODEL = dict(vocab_size=32000, context_length=16640, d_model=2048, num_layers=12, num_heads=16, d_ff=1024,
                attention_type="MLA", kv_lora_rank=512, q_lora_rank=1024, rope_dim=64, use_moe=True,
                n_routed_experts=32, num_experts_per_tok=4, n_shared_experts=1)


def engine_mla(steps: int = 10, warmup: int = 3, batch: int = 240, prefills: int = 16) -> dict:
    """Mixed ragged steps of the MLA+MoE decoder (d_model 2048, 12 layers, 16 heads, latent 512 + 64,
    q_lora 1024, 32 experts top-4 + shared, d_ff 1024, vocab 32000; bf16, random init seed 0) through the
    engine: every step is one prefill call of ``prefills`` new prompts (lengths uniform [256,4096]) and one
    decode call of ``batch`` running sequences (contexts uniform [512,16384]); the scheduler never mixes
    the two in one call.  The decode sequences enter with their blocks allocated and a latent cache of
    random rows (their contexts are not prefilled: 2 M tokens of set-up that the step does not contain)."""
    import itertools
    import time

    from .engine import SamplingParams, Sequence
    from .engine.llm_engine import LLMEngine
    from .engine.sequence import SequenceStatus
    steps = min(steps, 20)
    rng = np.random.default_rng(4)
    ctx = rng.integers(512, 16384 + 1, size=batch)
    plens = rng.integers(256, 4096 + 1, size=(steps + warmup, prefills))
    need = int(sum((int(c) + steps + warmup + 15) // 16 + 1 for c in ctx)) + prefills * 257 + 64
    Sequence.counter = itertools.count()
    cfg = dict(model=C4_MODEL, dtype=torch.bfloat16, block_size=16, max_num_sequences=256,
               max_num_batched_tokens=prefills * 4096, max_cached_blocks=need, eos=-1, device="cuda:0",
               max_model_length=16640, seed=0, prefill_graphs=False)
    t0 = time.perf_counter()
    eng = LLMEngine(cfg)
    build_s = time.perf_counter() - t0
    eng.model_runner.kv_cache.normal_(0.0, 0.3)
    sched = eng.scheduler
    for c in ctx:            # running sequences in the state a prefill leaves: c - 1 tokens cached, one sampled
        seq = Sequence(rng.integers(0, 32000, size=int(c) - 1).tolist(),
                       SamplingParams(temperature=0.0, max_tokens=1 << 20, ignore_eos=True))
        sched.block_manager.allocate(seq)
        seq.append_token(int(rng.integers(0, 32000)))
        seq.status = SequenceStatus.RUNNING
        sched.running.append(seq)
    times = dict(prefill=[], decode=[])
    tokens = dict(prefill=0, decode=0)
    for it in range(steps + warmup):
        for n in plens[it]:  # finish right after their first token, freeing their blocks
            eng.add_request(rng.integers(0, 32000, size=int(n)).tolist(),
                            SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
        for kind in ("prefill", "decode"):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            _out, n, is_prefill = eng.step()
            torch.cuda.synchronize()
            assert is_prefill == (kind == "prefill"), (kind, is_prefill)
            if it >= warmup:
                times[kind].append(time.perf_counter() - t0)
                tokens[kind] += n
    ops.check_status()
    graphs = bool(eng.model_runner.graphs)
    eng.exit()
    pre, dec = float(np.mean(times["prefill"])), float(np.mean(times["decode"]))
    return dict(workload=f"MLA+MoE decoder, mixed steps: {prefills} prefills U[256,4096] + {batch} decodes with "
                         "contexts U[512,16384] per step, bf16", ms=(pre + dec) * 1e3, prefill_ms=pre * 1e3,
                decode_ms=dec * 1e3, prefill_tokens_per_step=tokens["prefill"] / steps,
                decode_tokens_per_step=tokens["decode"] / steps,
                tokens_per_s=(tokens["prefill"] + tokens["decode"]) / steps / (pre + dec),
                decode_tokens_per_s=tokens["decode"] / steps / dec, prefill_tokens_per_s=tokens["prefill"] / steps / pre,
                context_tokens=int(ctx.sum()), engine_build_s=build_s, cuda_graphs=graphs)
