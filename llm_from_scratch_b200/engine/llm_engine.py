"""Engine facade (reference: engine/llm_engine.py:24-102): ``add_prompt`` / ``step`` / ``generate``.

One engine = one process = one GPU replica with its own scheduler, block pool and KV cache; the
reference's tensor-parallel worker processes are not part of this design.  ``step`` always
returns the 3-tuple ``(finished outputs, tokens processed, is_prefill)`` (the reference returns a
2-tuple when nothing is schedulable, which its own ``generate`` cannot unpack).  Prompts may be
strings (a tokenizer with ``encode`` / ``decode`` must then be supplied) or lists of token ids.
"""
from __future__ import annotations

import time

from .model_runner import ModelRunner, _cfg
from .sampling_params import SamplingParams
from .scheduler import Scheduler
from .sequence import Sequence


class LLMEngine:
    def __init__(self, config: dict, model=None, tokenizer=None, verbose: bool = False, runner=None):
        self.config = config
        block_size = _cfg(config, "block_size", default=256)
        Sequence.block_size = block_size
        # ``runner`` lets a caller supply its own executor (anything with ``run(seqs, is_prefill)``,
        # ``num_kv_blocks`` and ``exit()``); by default the GPU model runner is built here
        self.model_runner = runner if runner is not None else ModelRunner(config, model)
        self.scheduler = Scheduler(
            max_num_sequences=_cfg(config, "max_num_sequences", "max_num_seqs", default=16),
            max_num_batched_tokens=_cfg(config, "max_num_batched_tokens", "max_num_batch_tokens", default=1024),
            max_cached_blocks=self.model_runner.num_kv_blocks,
            block_size=block_size,
            eos=_cfg(config, "eos", default=50256),
        )
        # decode steps the engine may run per scheduling decision (1 = the reference's step-by-step loop);
        # larger values keep the GPU busy while the host schedules, at the price of admitting waiting
        # requests and retiring finished ones up to decode_window - 1 steps later
        self.decode_window = int(_cfg(config, "decode_window", default=1))
        self.tokenizer = tokenizer
        self.verbose = verbose
        self.stats = dict(prefill_tokens=0, decode_tokens=0, prefill_time=0.0, decode_time=0.0, steps=0)
        # wall time per step component: host scheduling, model run (incl. metadata upload and the
        # device-to-host read of the sampled tokens), host post-processing
        self.timing = dict(schedule_s=0.0, run_prefill_s=0.0, run_decode_s=0.0, postprocess_s=0.0,
                           prefill_steps=0, decode_steps=0, decode_seq_steps=0, decode_ctx_tokens=0)

    def exit(self) -> None:
        self.model_runner.exit()

    # ------------------------------------------------------------------ requests
    def add_request(self, token_ids, sampling_params: SamplingParams | None = None) -> Sequence:
        seq = Sequence(token_ids, sampling_params or SamplingParams())
        self.scheduler.add_sequence(seq)
        return seq

    def add_prompt(self, prompt, sampling_params: SamplingParams | None = None) -> Sequence:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a string prompt needs a tokenizer; pass token ids or LLMEngine(tokenizer=...)")
            prompt = self.tokenizer.encode(prompt)
        return self.add_request(prompt, sampling_params)

    # ------------------------------------------------------------------ one step
    def step(self):
        t0 = time.perf_counter()
        seqs, is_prefill = self.scheduler.schedule()
        t1 = time.perf_counter()
        self.timing["schedule_s"] += t1 - t0
        if not seqs:
            return [], 0, is_prefill
        runner = self.model_runner
        window = 1
        if not is_prefill and self.decode_window > 1 and getattr(runner, "can_run_window", None) \
                and runner.can_run_window(seqs):
            window = self.scheduler.plan_decode_window(seqs, self.decode_window, runner.max_model_length)
            t1 = time.perf_counter()
            self.timing["schedule_s"] += t1 - t0
        if window > 1:
            # several decode steps back to back: each step's sampled tokens feed the next on the device
            steps = runner.run_window(seqs, window)
            t2 = time.perf_counter()
            self.timing["run_decode_s"] += t2 - t1
            self.timing["decode_steps"] += window
            processed = self.scheduler.postprocess_window(seqs, steps)
        else:
            token_ids = runner.run(seqs, is_prefill)
            t2 = time.perf_counter()
            kind = "prefill" if is_prefill else "decode"
            self.timing[f"run_{kind}_s"] += t2 - t1
            self.timing[f"{kind}_steps"] += 1
            self.scheduler.postprocess(seqs, token_ids)
            processed = sum(len(s) for s in seqs) if is_prefill else len(seqs)
        self.timing["postprocess_s"] += time.perf_counter() - t2
        if not is_prefill:
            self.timing["decode_seq_steps"] = getattr(runner, "decode_seq_steps", 0)
            self.timing["decode_ctx_tokens"] = getattr(runner, "decode_ctx_tokens", 0)
        outputs = [(s.seq_id, s.completion_token_ids) for s in seqs if s.is_finished]
        return outputs, processed, is_prefill

    def is_finished(self) -> bool:
        return self.scheduler.is_finished()

    # ------------------------------------------------------------------ whole job
    def generate(self, prompts, sampling_params) -> dict:
        if isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params] * len(prompts)
        for prompt, sp in zip(prompts, sampling_params):
            self.add_prompt(prompt, sp)
        done: dict[int, list[int]] = {}
        while not self.scheduler.is_finished():
            t0 = time.perf_counter()
            outputs, n, is_prefill = self.step()
            dt = time.perf_counter() - t0
            if n == 0 and not outputs:
                raise RuntimeError("nothing schedulable: the KV pool is too small for the waiting request")
            kind = "prefill" if is_prefill else "decode"
            self.stats[kind + "_tokens"] += n
            self.stats[kind + "_time"] += dt
            self.stats["steps"] += 1
            if self.verbose:
                print(f"{n} tokens, {n / (dt + 1e-10):.0f} tokens/s during {kind}")
            done.update(outputs)
        token_ids = [done[k] for k in sorted(done)]
        text = [self.tokenizer.decode(t) for t in token_ids] if self.tokenizer is not None else None
        return {"text": text, "token_ids": token_ids}
