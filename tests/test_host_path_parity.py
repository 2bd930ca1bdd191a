"""Host path (scheduler, block pool, prefix hashing, step metadata) against recordings of the
reference's own classes (tests/golden/host_path.json.gz, written by tests/golden/make_golden.py).

Both the oracle restatement and the product host layer (in reference-exact mode) must reproduce
every recorded step bit for bit: schedule decisions, block tables, slot mappings, cu_seqlens,
context lengths, free-list state and the final token streams.
"""
import gzip
import itertools
import json
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import scenarios as sc  # noqa: E402

with gzip.open(os.path.join(HERE, "golden", "host_path.json.gz"), "rt") as _f:
    GOLDEN = json.load(_f)
NAMES = [k for k in GOLDEN if not k.startswith("_")]


def _norm(x):
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        return x.tolist()
    return x


class OracleDriver:
    def __init__(self, eng):
        from oracle import host_path as hp
        self.hp, self.bs = hp, eng["block_size"]
        hp.OracleSeq.ids = itertools.count()
        self.sched = hp.OracleScheduler(**eng)

    def add(self, token_ids, params):
        self.sched.add(self.hp.OracleSeq(token_ids, self.hp.OracleParams(**params), self.bs))

    def done(self):
        return self.sched.done()

    def schedule(self):
        return self.sched.schedule()

    def metadata(self, seqs, is_prefill):
        f = self.hp.prepare_prefill if is_prefill else self.hp.prepare_decode
        return f(seqs, self.bs)

    def view(self, s):
        return dict(seq_id=s.seq_id, n=len(s), cached=s.n_cached, finished=s.status == self.hp.FINISHED,
                    completion=s.completion)

    def postprocess(self, seqs, toks):
        self.sched.postprocess(seqs, toks)

    def pool(self):
        p = self.sched.pool
        return list(itertools.islice(p.free, 0, 6)), len(p.free), len(p.used)


class ProductDriver:
    def __init__(self, eng, exact=True):
        from llm_from_scratch_b200.engine import Scheduler, Sequence, SamplingParams
        from llm_from_scratch_b200.engine import metadata
        self.Sequence, self.SamplingParams, self.md = Sequence, SamplingParams, metadata
        self.bs = eng["block_size"]
        Sequence.block_size = self.bs
        Sequence.counter = itertools.count()
        Sequence.reference_exact = exact
        self.sched = Scheduler(**eng, reference_exact=exact)

    def add(self, token_ids, params):
        self.sched.add_sequence(self.Sequence(token_ids, self.SamplingParams(**params)))

    def done(self):
        return self.sched.is_finished()

    def schedule(self):
        return self.sched.schedule()

    def metadata(self, seqs, is_prefill):
        m = (self.md.prepare_prefill if is_prefill else self.md.prepare_decode)(seqs, self.bs)
        return {k: _norm(getattr(m, k)) for k in ("input_ids", "cu_seqlens_q", "cu_seqlens_k", "max_seqlen_q",
                                                   "max_seqlen_k", "slot_mapping", "context_lens", "block_tables")}

    def view(self, s):
        return dict(seq_id=s.seq_id, n=s.num_tokens, cached=s.num_cached_tokens, finished=s.is_finished,
                    completion=s.completion_token_ids)

    def postprocess(self, seqs, toks):
        self.sched.postprocess(seqs, toks)

    def pool(self):
        bm = self.sched.block_manager
        return list(itertools.islice(bm.free_block_ids, 0, 6)), len(bm.free_block_ids), len(bm.used_block_ids)


def replay(name, make_driver):
    g = GOLDEN[name]
    scn = g["scenario"]
    drv = make_driver(scn["engine"])
    pending = sorted(scn["requests"], key=lambda r: r["arrival_step"])
    pi, finished = 0, {}
    for rec in g["steps"]:
        while pi < len(pending) and pending[pi]["arrival_step"] <= rec["step"]:
            drv.add(pending[pi]["token_ids"], pending[pi]["params"])
            pi += 1
        seqs, is_prefill = drv.schedule()
        views = [drv.view(s) for s in seqs]
        where = f"{name} step {rec['step']}"
        assert bool(is_prefill) == rec["is_prefill"], where
        assert [v["seq_id"] for v in views] == rec["seq_ids"], where
        if seqs:
            md = drv.metadata(seqs, is_prefill)
            for key in ("input_ids", "cu_seqlens_q", "cu_seqlens_k", "max_seqlen_q", "max_seqlen_k",
                        "slot_mapping", "context_lens", "block_tables"):
                assert _norm(md[key]) == rec[key], f"{where}: {key}"
            assert [v["cached"] for v in views] == rec["num_cached_tokens"], where
            toks = [sc.fake_next_token(v["seq_id"], v["n"], scn["eos_every"]) for v in views]
            assert toks == rec["sampled"], where
            drv.postprocess(seqs, toks)
            after = [drv.view(s) for s in seqs]
            assert [v["seq_id"] for v in after if v["finished"]] == rec["finished"], where
            for v in after:
                if v["finished"]:
                    finished[str(v["seq_id"])] = list(v["completion"])
        head, nfree, nused = drv.pool()
        assert (head, nfree, nused) == (rec["free_head"], rec["num_free"], rec["num_used"]), where
    assert drv.done()
    assert finished == g["outputs"]


@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_reference_recording(name):
    replay(name, OracleDriver)


@pytest.mark.parametrize("name", NAMES)
def test_product_host_layer_reproduces_reference_recording(name):
    try:
        replay(name, lambda eng: ProductDriver(eng, exact=True))
    finally:
        from llm_from_scratch_b200.engine import Sequence
        Sequence.reference_exact = False


def test_block_hash_known_answers_from_reference():
    from oracle.xxh64 import block_hash
    from llm_from_scratch_b200.engine import BlockManager
    for kat in GOLDEN["_hash_kat"]:
        assert block_hash(kat["token_ids"], kat["prefix"]) == kat["hash"]
        assert BlockManager.compute_hash(kat["token_ids"], kat["prefix"]) == kat["hash"]


def test_recordings_cover_the_interesting_cases():
    """The fixtures must actually exercise cached prefills, block growth and the boundary quirk."""
    steps = [r for n in NAMES for r in GOLDEN[n]["steps"]]
    assert any(r["is_prefill"] and r.get("block_tables") for r in steps), "no cached prefill recorded"
    assert any((not r["is_prefill"]) and r["seq_ids"] for r in steps)
    assert any(sum(r.get("num_cached_tokens") or [0]) > 0 for r in steps)
    bb = GOLDEN["block_boundaries"]["steps"][1]
    # a 16-token context decodes into "slot -1 of its block" in the reference (sequence.py:66-69)
    assert bb["context_lens"][1] == 16 and bb["slot_mapping"][1] == bb["block_tables"][1][0] * 16 - 1
