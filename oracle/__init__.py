"""CPU oracle for the continuous-batching prefill/decode path.  TEST INFRASTRUCTURE ONLY.

Nothing in ``llm_from_scratch_b200`` imports this package.  It restates, on the CPU, what the
reference (ZenoAFfectionate/LLM_from_Scratch) computes on this path, so that the CUDA kernels and
the host layer can be compared with it:

* ``host_path``  — Sequence / BlockManager / Scheduler / prepare_prefill / prepare_decode
                   (engine/sequence.py, engine/block_manager.py, engine/scheduler.py,
                   engine/model_runner.py:202-278), integer-exact;
* ``xxh64``      — the XXH64 hash (third-party ``xxhash`` package, unpinned by the reference;
                   frozen public algorithm) used by BlockManager.compute_hash;
* ``attention``  — softmax / scaled_dot_product_attention / RoPE (model/attention/utils.py:8-63),
                   the GQA cache branch (model/attention/GQA.py:99-130) and the absorbed MLA
                   branch (model/attention/MLA.py:136-178) applied to a paged pool gathered
                   through block tables, all in fp32;
* ``model``      — the layer arithmetic of TransformerLM (model/transformer.py, model/utils.py,
                   model/architecture/mlp.py, model/architecture/moe.py) driven one request at a
                   time with dense caches.

Pinning: the reference has no test for the engine path, so the oracle is pinned against outputs
of the reference's own code run in the build container (``tests/golden/make_golden.py`` imports
the reference and writes the fixtures under ``tests/golden/``) and against the reference's
scaled-dot-product-attention snapshot.  Only ``tests/``, ``__graft_entry__.smoke`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import this package.
"""
