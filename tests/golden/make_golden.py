"""Generates the golden fixtures in this directory by running the REFERENCE's own code.

Needs a checkout of the reference project (the tests themselves never do); give its path:

    B200_REFERENCE=<reference checkout> python tests/golden/make_golden.py

Host path: the reference's Sequence / BlockManager / Scheduler (engine/*.py) are imported with a
seven-line ``sampling_parameters`` shim (the module they import is missing from the reference), and
ModelRunner.prepare_prefill / prepare_decode (engine/model_runner.py:202-278) are executed
unmodified with stand-ins for the modules the file cannot import (models.qwen3, myvllm.*) and a
``torch`` proxy that maps ``pin_memory=True`` / ``.cuda()`` to plain CPU tensors.  Every engine step
of every scenario in ``scenarios.py`` is recorded to ``host_path.json.gz``.

Float path: outputs of the reference's attention functions and modules on seeded inputs are
written to ``*.npz``; see the individual writers below.
"""
from __future__ import annotations

import gzip
import itertools
import json
import os
import sys
import tempfile
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REF = Path(os.environ["B200_REFERENCE"])
sys.path.insert(0, str(HERE))
import scenarios as sc  # noqa: E402


# --------------------------------------------------------------------------------------------
# importing the reference
# --------------------------------------------------------------------------------------------
def import_reference_engine():
    shim = Path(tempfile.mkdtemp(prefix="ref_shim_"))
    (shim / "sampling_parameters.py").write_text(
        "from dataclasses import dataclass\n"
        "@dataclass\n"
        "class SamplingParams:\n"
        "    temperature: float = 1.0\n"
        "    max_tokens: int = 256\n"
        "    ignore_eos: bool = False\n"
        "    max_model_length: int | None = None\n")
    for p in (str(REF), str(REF / "engine"), str(shim)):
        sys.path.insert(0, p)

    import importlib
    ctx = importlib.import_module("utils.context")
    # stand-ins for modules that the reference imports but does not ship
    for name in ("models", "models.qwen3", "myvllm", "myvllm.layers", "myvllm.layers.sampler", "myvllm.utils"):
        sys.modules[name] = types.ModuleType(name)
    sys.modules["models.qwen3"].Qwen3ForCausalLM = object
    sys.modules["myvllm.layers.sampler"].SamplerLayer = object
    mu = sys.modules["myvllm.utils"]
    mu.set_context, mu.get_context, mu.reset_context = ctx.set_context, ctx.get_context, ctx.reset_context
    mu.__all__ = ["set_context", "get_context", "reset_context"]

    seq_mod = importlib.import_module("engine.sequence")
    sched_mod = importlib.import_module("engine.scheduler")
    mr = importlib.import_module("engine.model_runner")
    sp_mod = importlib.import_module("sampling_parameters")

    class _CpuTensor(torch.Tensor):
        def cuda(self, *a, **k):
            return self.as_subclass(torch.Tensor)

    class _TorchProxy:
        def __getattr__(self, name):
            return getattr(torch, name)

        @staticmethod
        def tensor(data, dtype=None, pin_memory=False):
            return torch.tensor(data, dtype=dtype).as_subclass(_CpuTensor)

    mr.torch = _TorchProxy()
    return seq_mod, sched_mod, mr, ctx, sp_mod


def _tolist(t):
    return None if t is None else t.tolist()


def record_host_scenario(name, scn, seq_mod, sched_mod, mr, ctx, sp_mod):
    eng = scn["engine"]
    seq_mod.Sequence.block_size = eng["block_size"]
    seq_mod.Sequence.counter = itertools.count()
    sched = sched_mod.Scheduler(**eng)
    runner = types.SimpleNamespace(block_size=eng["block_size"])
    pending = sorted(enumerate(scn["requests"]), key=lambda x: x[1]["arrival_step"])
    steps, finished, step_no, pi = [], {}, 0, 0
    seqs_all = []
    while pi < len(pending) or not sched.is_finished():
        while pi < len(pending) and pending[pi][1]["arrival_step"] <= step_no:
            r = pending[pi][1]
            s = seq_mod.Sequence(r["token_ids"], sp_mod.SamplingParams(**r["params"]))
            seqs_all.append(s)
            sched.add_sequence(s)
            pi += 1
        seqs, is_prefill = sched.schedule()
        rec = dict(step=step_no, is_prefill=bool(is_prefill), seq_ids=[s.seq_id for s in seqs])
        if seqs:
            if is_prefill:
                ids = mr.ModelRunner.prepare_prefill(runner, seqs)
            else:
                ids = mr.ModelRunner.prepare_decode(runner, seqs)
            c = ctx.get_context()
            rec.update(input_ids=ids.tolist(), cu_seqlens_q=_tolist(c.cu_seqlens_q),
                       cu_seqlens_k=_tolist(c.cu_seqlens_k), max_seqlen_q=int(c.max_seqlen_q),
                       max_seqlen_k=int(c.max_seqlen_k), slot_mapping=_tolist(c.slot_mapping),
                       context_lens=_tolist(c.context_lens), block_tables=_tolist(c.block_tables),
                       num_cached_tokens=[s.num_cached_tokens for s in seqs])
            ctx.reset_context()
            toks = [sc.fake_next_token(s.seq_id, s.num_tokens, scn["eos_every"]) for s in seqs]
            sched.postprocess(seqs, toks)
            rec["sampled"] = toks
            rec["finished"] = [s.seq_id for s in seqs if s.is_finished]
            for s in seqs:
                if s.is_finished:
                    finished[s.seq_id] = list(s.completion_token_ids)
        bm = sched.block_manager
        rec["free_head"] = list(itertools.islice(bm.free_block_ids, 0, 6))
        rec["num_free"] = len(bm.free_block_ids)
        rec["num_used"] = len(bm.used_block_ids)
        steps.append(rec)
        step_no += 1
        assert step_no < 5000, "scenario does not terminate"
    return dict(scenario=scn, steps=steps, outputs={str(k): v for k, v in sorted(finished.items())})


def write_host_golden(ref):
    seq_mod, sched_mod, mr, ctx, sp_mod = ref
    out = {name: record_host_scenario(name, scn, *ref) for name, scn in sc.scenarios().items()}
    # compute_hash known answers straight from the reference BlockManager
    bm_mod = sys.modules["engine.block_manager"]
    bm = bm_mod.BlockManager(1, 16)
    h0 = bm.compute_hash(list(range(16)), -1)
    out["_hash_kat"] = [
        dict(token_ids=list(range(16)), prefix=-1, hash=h0),
        dict(token_ids=list(range(16, 32)), prefix=h0, hash=bm.compute_hash(list(range(16, 32)), h0)),
        dict(token_ids=[0] * 16, prefix=-1, hash=bm.compute_hash([0] * 16, -1)),
        dict(token_ids=[9999, 1, 2], prefix=-1, hash=bm.compute_hash([9999, 1, 2], -1)),
        dict(token_ids=list(range(100, 108)), prefix=2 ** 63 + 5, hash=bm.compute_hash(list(range(100, 108)), 2 ** 63 + 5)),
    ]
    with gzip.open(HERE / "host_path.json.gz", "wt") as f:
        json.dump(out, f, separators=(",", ":"))
    n = sum(len(v["steps"]) for k, v in out.items() if not k.startswith("_"))
    print(f"host_path.json.gz: {len(out) - 1} scenarios, {n} steps")


if __name__ == "__main__":
    torch.manual_seed(0)
    ref = import_reference_engine()
    write_host_golden(ref)
    import make_golden_float  # noqa: E402
    make_golden_float.write_all(REF)
