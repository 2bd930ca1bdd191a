"""bf16 layer-level parity on the GPU at the benchmark layer shapes, against the reference's own modules
run under CPU autocast (fixtures of tests/golden/make_golden_layers.py; weights and inputs are drawn
again from the fixture's seeds and checked against its checksums).

Tolerances (bf16 against the bf16 reference): max-abs <= 2e-2 of the output scale (the largest reference
magnitude) and mean relative error <= 1e-2.  Rows whose expert choice differs from the reference's — a
near-tie of two gate logits that bf16 rounding resolves differently — are counted, bounded, and left out
of the output comparison: they are a different (equally valid) routing, not an arithmetic error."""
import numpy as np
import pytest
import torch

from layer_fixtures import (MLA_LAYER, MOE_LAYER, checked_input, from_bf16_bits, layer_weights, load, rel_errors)

pytestmark = pytest.mark.gpu


def _model(cfg, weights):
    from llm_from_scratch_b200.model import EngineTransformerLM, ModelConfig
    return EngineTransformerLM(ModelConfig.from_dict(cfg), weights, torch.device("cuda"), torch.bfloat16)


@pytest.fixture(scope="module")
def moe_layer():
    z = load("moe_layer_c3.npz")
    model = _model(MOE_LAYER, layer_weights(MOE_LAYER, z, "layers.0.ffn."))
    return z, model.layers[0].ffn


@pytest.mark.parametrize("tag,own_gemm", [("decode", True), ("decode", False), ("prefill", False), ("prefill", True)])
def test_moe_layer_of_the_gqa_moe_decoder(moe_layer, tag, own_gemm):
    """d_model 1024, 16 experts top-2 + shared, d_ff 704: 256 rows (decode size) and 2048 rows (prefill size),
    each through the weight-streaming tcgen05 grouped GEMM and through the large-batch grouped path."""
    from llm_from_scratch_b200 import ops
    z, moe = moe_layer
    rows = int(z[f"{tag}_rows"])
    x = checked_input(z, f"{tag}_input_seed", f"{tag}_input_sum", rows, 1024).cuda()
    # routing first: the kernel's expert choice against the reference's Gate.forward
    _tok, experts, _w, _offs, inv = ops.moe_route((x @ moe.gate_w.t()).contiguous(), moe.gate_bias, moe.K)
    sel = experts[inv.long().reshape(-1)].view(rows, moe.K).cpu().numpy()
    same = (np.sort(sel, axis=1) == z[f"{tag}_experts"]).all(axis=1)
    assert same.mean() >= 0.99, f"expert choice differs on {(~same).sum()} of {rows} rows"
    moe.own_gemm_max_rows_per_expert = 1 << 30 if own_gemm else 0
    try:
        y = moe(x)
        ops.check_status()
    finally:
        del moe.own_gemm_max_rows_per_expert          # back to the class default
    kept = z[f"{tag}_kept"]
    want = from_bf16_bits(z[f"{tag}_out"])
    ok = torch.from_numpy(same[kept])
    got = y[torch.from_numpy(kept).cuda()].cpu()
    max_abs, mean_rel = rel_errors(got[ok], want[ok])
    scale = want.float().abs().max().item()
    print(f"moe layer {tag} own_gemm={own_gemm}: max-abs {max_abs:.3e} (scale {scale:.3f}), mean-rel {mean_rel:.3e}, "
          f"routing differs on {(~same).sum()} rows")
    assert max_abs <= 2e-2 * scale and mean_rel <= 1e-2


def _paged_single_sequence(total, block_size, num_blocks, seed):
    perm = np.random.default_rng(seed).permutation(num_blocks).astype(np.int32)
    table = perm[:(total + block_size - 1) // block_size]
    pos = np.arange(total)
    slots = table[pos // block_size].astype(np.int64) * block_size + pos % block_size
    return table, slots


@pytest.mark.parametrize("neighbour", [0, 77])
def test_latent_attention_layer_of_the_mla_moe_decoder(neighbour):
    """16 heads, kv_lora_rank 512, q_lora_rank 1024, rope_dim 64, d_model 2048: a 300-token prefill (pre-attention
    kernel -> expanded-key tcgen05 prefill) and three decode steps (pre-attention kernel -> absorbed W_UK ->
    MLA decode kernel over the paged latent pool -> W_UV), against MultiHeadLatentAttention.forward's cache
    branch.  ``neighbour`` > 0 packs a second, unrelated sequence into the prefill and decode batches."""
    from llm_from_scratch_b200 import ops
    from llm_from_scratch_b200.utils.context import get_context, reset_context, set_context
    z = load("mla_layer_c4.npz")
    model = _model(MLA_LAYER, layer_weights(MLA_LAYER, z, "layers.0.att."))
    att = model.layers[0].att
    P, Dn, bs, nblk = int(z["prefill"]), int(z["decode"]), 16, 64
    total = P + Dn
    x = checked_input(z, "input_seed", "input_sum", total, 2048).cuda()
    want = from_bf16_bits(z["out"])
    pool = torch.zeros(nblk, bs, 512 + 64, dtype=torch.bfloat16, device="cuda")
    att.latent_cache = pool
    table, slots = _paged_single_sequence(total, bs, 24, seed=7)
    dev = torch.device("cuda")
    # an unrelated sequence in other blocks of the same pool
    ntab = np.arange(24, 24 + (neighbour + Dn + bs - 1) // bs, dtype=np.int32)
    npos = np.arange(neighbour + Dn)
    nslots = ntab[npos // bs].astype(np.int64) * bs + npos % bs if neighbour else np.zeros(0, dtype=np.int64)
    xn = torch.randn(neighbour + Dn, 2048, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    tile_rows = ops.prefill_tile_rows(16, 16, 192, 128, torch.bfloat16)

    # ---- prefill
    lens = [P] + ([neighbour] if neighbour else [])
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
    xs = torch.cat([x[:P], xn[:neighbour]])
    positions = torch.cat([torch.arange(P), torch.arange(neighbour)]).to(dev)
    slot_t = torch.from_numpy(np.concatenate([slots[:P], nslots[:neighbour]])).to(dev)
    plan = ops.prefill_plan(cu, xs.shape[0], max(lens), tile_rows) if tile_rows else None
    set_context(True, cu, cu, max(lens), max(lens), slot_t, None, None, positions, plan)
    with torch.inference_mode():
        y0 = att(xs, get_context(), positions)[:P].cpu()
    ops.check_status()
    # the latent rows written into the paged pool are the rows the reference caches
    flat = pool.view(-1, 576)[torch.from_numpy(slots[:P]).to(dev)].cpu()
    lat_abs, lat_rel = rel_errors(flat[:, :512], from_bf16_bits(z["latent"])[:P])
    pe_abs, pe_rel = rel_errors(flat[:, 512:], from_bf16_bits(z["pe"])[:P])
    assert lat_rel <= 1e-2 and pe_rel <= 1e-2, (lat_abs, lat_rel, pe_abs, pe_rel)
    scale = want.float().abs().max().item()
    max_abs, mean_rel = rel_errors(y0, want[:P])
    print(f"mla layer prefill (+{neighbour}): max-abs {max_abs:.3e} (scale {scale:.3f}), mean-rel {mean_rel:.3e}")
    assert max_abs <= 2e-2 * scale and mean_rel <= 1e-2

    # ---- three decode steps
    width = max(len(table), len(ntab))
    bt = np.full((2 if neighbour else 1, width), -1, dtype=np.int32)
    bt[0, :len(table)] = table
    if neighbour:
        bt[1, :len(ntab)] = ntab
    bt = torch.from_numpy(bt).to(dev)
    for i in range(Dn):
        rows = [x[P + i:P + i + 1]] + ([xn[neighbour + i:neighbour + i + 1]] if neighbour else [])
        lens_now = [P + i + 1] + ([neighbour + i + 1] if neighbour else [])
        sl = [slots[P + i]] + ([nslots[neighbour + i]] if neighbour else [])
        cl = torch.tensor(lens_now, dtype=torch.int64, device=dev)
        set_context(False, slot_mapping=torch.tensor(sl, dtype=torch.int64, device=dev), context_lens=cl,
                    block_tables=bt)
        with torch.inference_mode():
            y = att(torch.cat(rows), get_context(), cl - 1)[:1].cpu()
        ops.check_status()
        max_abs, mean_rel = rel_errors(y, want[P + i:P + i + 1])
        print(f"mla layer decode step {i} (+{neighbour}): max-abs {max_abs:.3e}, mean-rel {mean_rel:.3e}")
        assert max_abs <= 2e-2 * scale and mean_rel <= 1e-2
    reset_context()


def test_small_mla_decoder_bf16_tracks_reference_autocast():
    """The small MLA+MoE decoder in bf16 through the engine against the reference's greedy streams under CPU
    autocast: the first token of every stream (pure prefill) and the fraction of matching later tokens."""
    from test_gpu_engine import greedy_run, make_engine, prompts_of, weights_of
    z = load("mla_model.npz")
    cfg = dict(vocab_size=512, context_length=128, d_model=128, num_layers=2, num_heads=8, d_ff=96, use_moe=True,
               n_routed_experts=4, num_experts_per_tok=2, n_shared_experts=1, attention_type="MLA", rope_dim=8,
               q_lora_rank=48, kv_lora_rank=64)
    eng = make_engine(cfg, weights_of(z), dtype=torch.bfloat16)
    streams, _last = greedy_run(eng, prompts_of(z), 12)
    want = z["streams_bf16"].tolist()
    match = np.mean([a == b for s, w in zip(streams, want) for a, b in zip(s, w)])
    first = np.mean([s[0] == w[0] for s, w in zip(streams, want)])
    print(f"small MLA decoder bf16: first-token match {first:.2f}, all-token match {match:.2f}")
    assert first == 1.0, "first greedy token (pure prefill) differs"
    assert match >= 0.7, match
