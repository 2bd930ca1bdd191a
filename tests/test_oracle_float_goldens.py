"""The float-path oracle against fixtures written by the reference's own code
(tests/golden/make_golden_float.py): attention primitives, attention modules with their dense
caches, and whole-model greedy streams."""
import os

import numpy as np
import pytest
import torch

from oracle import attention as A
from oracle.model import OracleModel

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(G, name))


def weights_of(z, strip=""):
    return {k[3:][len(strip):]: torch.from_numpy(z[k]) for k in z.files if k.startswith("w::")}


def test_sdpa_matches_reference_snapshots():
    z = load("attn_kat.npz")
    q, k, v = (torch.from_numpy(z[n]) for n in ("sdpa_q", "sdpa_k", "sdpa_v"))
    mask = torch.from_numpy(z["sdpa_mask"])
    np.testing.assert_allclose(A.sdpa(q, k, v, mask).numpy(), z["sdpa_out3"], atol=1e-6)
    q4, k4, v4 = (x.view(2, 2, *x.shape[1:]) for x in (q, k, v))
    np.testing.assert_allclose(A.sdpa(q4, k4, v4, mask.view(2, 2, 12, 16)).numpy(), z["sdpa_out4"], atol=1e-6)


def test_softmax_rope_rmsnorm_known_answers():
    z = load("attn_kat.npz")
    x = torch.from_numpy(z["softmax_in"])
    np.testing.assert_allclose(A.softmax(x, -1).numpy(), z["softmax_out"], atol=1e-7)
    np.testing.assert_allclose(A.softmax(x, 1).numpy(), z["softmax_out_dim1"], atol=1e-7)
    table = A.rope_table(float(z["rope_theta"]), int(z["rope_dk"]), int(z["rope_maxlen"]))
    pos = torch.from_numpy(z["rope_pos"])
    np.testing.assert_allclose(A.apply_rope(torch.from_numpy(z["rope_x"]), pos, table).numpy(), z["rope_out"], atol=1e-6)
    # d_x smaller than the table width: the reference's slice holds cosines only; norms are not preserved
    xt = torch.from_numpy(z["rope_trunc_x"])
    yt = A.apply_rope(xt, pos, table)
    np.testing.assert_allclose(yt.numpy(), z["rope_trunc_out"], atol=1e-6)
    assert not torch.allclose(yt.norm(dim=-1), xt.norm(dim=-1), atol=1e-3)
    w, xn, rn = (torch.from_numpy(z[n]) for n in ("rms_w", "rms_x", "rms_res"))
    np.testing.assert_allclose(A.rms_norm(xn, w, float(z["rms_eps"])).numpy(), z["rms_plain"], atol=1e-6)
    y, r = A.rms_norm(xn, w, float(z["rms_eps"]), rn)
    np.testing.assert_allclose(y.numpy(), z["rms_fused"], atol=1e-6)
    np.testing.assert_allclose(r.numpy(), z["rms_fused_res"], atol=1e-6)


@pytest.mark.parametrize("kind", ["gqa", "mla"])
def test_attention_module_with_dense_cache(kind):
    z = load(f"{kind}_module.npz")
    w = {"layers.0.att." + k: v for k, v in weights_of(z).items()}
    if kind == "gqa":
        cfg = dict(d_model=128, num_heads=8, num_kv_heads=2, attention_type="GQA", context_length=64, num_layers=1)
    else:
        cfg = dict(d_model=256, num_heads=4, attention_type="MLA", rope_dim=16, q_lora_rank=48, kv_lora_rank=64,
                   context_length=64, num_layers=1)
    m = OracleModel(cfg, w)
    cache = m.new_cache(64)[0]
    x = torch.from_numpy(z["x"])
    att = m._gqa if kind == "gqa" else m._mla
    outs = [att(x[:20], "layers.0.att", 0, torch.tril(torch.ones(20, 20, dtype=torch.bool)), cache)]
    for i in range(3):
        outs.append(att(x[20 + i:21 + i], "layers.0.att", 20 + i, None, cache))
    np.testing.assert_allclose(torch.cat(outs).numpy(), z["out"], atol=2e-5)


@pytest.mark.parametrize("name,att", [("moe_model.npz", "GQA"), ("mla_model.npz", "MLA")])
def test_small_moe_models_greedy_streams(name, att):
    z = load(name)
    cfg = dict(vocab_size=512, context_length=128, d_model=128, num_layers=2, num_heads=8, d_ff=96, use_moe=True,
               n_routed_experts=4, num_experts_per_tok=2, n_shared_experts=1, attention_type=att)
    cfg.update(dict(num_kv_heads=2) if att == "GQA" else dict(rope_dim=8, q_lora_rank=48, kv_lora_rank=64))
    m = OracleModel(cfg, weights_of(z))
    lens = z["prompt_lens"]
    prompts = np.split(z["prompts"], np.cumsum(lens)[:-1])
    for i, p in enumerate(prompts):
        toks, last = m.greedy(p.tolist(), 12)
        assert toks == z["streams"][i].tolist()
        np.testing.assert_allclose(last.numpy(), z["last_logits"][i], atol=1e-4)
    if "streams_bf16" in z.files:   # same operators under CPU autocast: identical rounding points
        toks, last = m.greedy(prompts[1].tolist(), 12, autocast=True)
        assert toks == z["streams_bf16"][1].tolist()
        np.testing.assert_allclose(last.numpy(), z["last_logits_bf16"][1], atol=5e-2)


def test_first_benchmark_configuration_seed0_streams():
    """fp32 GQA+SwiGLU decoder, d_model 512, 4 layers, 16/4 heads, vocab 10000: weights drawn in the
    reference's order from seed 0 give the reference's greedy streams."""
    from llm_from_scratch_b200.model import ModelConfig, init_reference_order
    z = load("c1_model.npz")
    mc = ModelConfig(vocab_size=10000, context_length=512, d_model=512, num_layers=4, num_heads=16, num_kv_heads=4,
                     d_ff=1344)
    w = init_reference_order(mc, 0)
    for k in z.files:
        if k.startswith("sum::"):
            assert w[k[5:]].double().sum().item() == float(z[k]), k
    m = OracleModel(mc.to_dict(), w)
    lens = z["prompt_lens"]
    prompts = np.split(z["prompts"], np.cumsum(lens)[:-1])
    for i in (0, 6):   # the two shortest prompts keep the CPU suite quick
        toks, last = m.greedy(prompts[i].tolist(), 64)
        assert toks == z["streams"][i].tolist()
        np.testing.assert_allclose(last.numpy(), z["last_logits"][i], atol=1e-4)
