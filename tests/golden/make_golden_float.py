"""Float-path golden fixtures, produced by running the REFERENCE's modules on the CPU in fp32.

Called from make_golden.py (build container only).  Writes:

  attn_kat.npz     softmax / scaled_dot_product_attention / RoPE / RMSNorm known answers; the sdpa
                   inputs are the reference's own test fixtures (tests/conftest.py:253-280) and the
                   outputs are checked against its snapshots (tests/_snapshots/*.npz) on the spot
  gqa_module.npz   GroupedQueryAttention with its dense cache: prefill of 20 tokens + 3 decode steps
  mla_module.npz   MultiHeadLatentAttention (absorbed cache branch): the same
  c1_model.npz     the fp32 GQA+SwiGLU decoder of the first benchmark configuration, seed 0:
                   8 prompts, 64 greedy tokens each, last-step logits, parameter checksums
  moe_model.npz    a small GQA+MoE decoder (fp32 and CPU-autocast bf16 logits)
  mla_model.npz    a small MLA+MoE decoder (the same)
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _np(t):
    return t.detach().float().numpy()


def _state(module):
    return {f"w::{k}": _np(v) for k, v in module.state_dict().items()}


# ------------------------------------------------------------------------------------------------
def write_attn_kat(ref: Path):
    from model.attention.utils import RotaryPositionalEmbedding, scaled_dot_product_attention, softmax
    from model.utils import RMSNorm
    out = {}
    torch.manual_seed(1); q = torch.randn(4, 12, 64)
    torch.manual_seed(2); k = torch.randn(4, 16, 64)
    torch.manual_seed(3); v = torch.randn(4, 16, 64)
    torch.manual_seed(5); mask = torch.randn(4, 12, 16) > 0.5
    o3 = scaled_dot_product_attention(q, k, v, mask)
    q4, k4, v4 = (x.view(2, 2, *x.shape[1:]) for x in (q, k, v))
    m4 = mask.view(2, 2, 12, 16)
    o4 = scaled_dot_product_attention(q4, k4, v4, m4)
    snap3 = np.load(ref / "tests/_snapshots/test_scaled_dot_product_attention.npz")["array"]
    snap4 = np.load(ref / "tests/_snapshots/test_4d_scaled_dot_product_attention.npz")["array"]
    assert np.allclose(_np(o3), snap3, atol=1e-6) and np.allclose(_np(o4), snap4, atol=1e-6), \
        "reference sdpa no longer matches its own snapshot"
    out.update(sdpa_q=_np(q), sdpa_k=_np(k), sdpa_v=_np(v), sdpa_mask=mask.numpy(), sdpa_out3=snap3, sdpa_out4=snap4)
    torch.manual_seed(7)
    x = torch.randn(3, 5, 33) * 4
    out.update(softmax_in=_np(x), softmax_out=_np(softmax(x, dim=-1)), softmax_out_dim1=_np(softmax(x, dim=1)))
    rope = RotaryPositionalEmbedding(10000.0, 32, 64)
    torch.manual_seed(8)
    xr = torch.randn(2, 4, 10, 32)
    pos = torch.tensor([0, 1, 2, 3, 7, 8, 20, 33, 62, 63])
    out.update(rope_theta=np.float64(10000.0), rope_dk=np.int64(32), rope_maxlen=np.int64(64), rope_x=_np(xr),
               rope_pos=pos.numpy(), rope_out=_np(rope(xr, pos)))
    xt = torch.randn(2, 1, 10, 16)      # d_x < d_k: the table slice holds cosines only
    out.update(rope_trunc_x=_np(xt), rope_trunc_out=_np(rope(xt, pos)))
    norm = RMSNorm(48)
    with torch.no_grad():
        norm.weight.copy_(torch.randn(48))
    xn, rn = torch.randn(6, 48), torch.randn(6, 48)
    y1 = norm(xn.clone())
    y2, r2 = norm(xn.clone(), rn.clone())   # the fused path adds in place when the input is fp32
    out.update(rms_w=_np(norm.weight), rms_x=_np(xn), rms_res=_np(rn), rms_plain=_np(y1), rms_fused=_np(y2),
               rms_fused_res=_np(r2), rms_eps=np.float64(norm.eps))
    np.savez_compressed(HERE / "attn_kat.npz", **out)
    print("attn_kat.npz (sdpa outputs equal the reference's snapshots)")


# ------------------------------------------------------------------------------------------------
def _enable_dense_cache(model, ctx_len):
    """The shipped Block never switches the modules' caches on (model/transformer.py:40-43)."""
    for layer in model.layers:
        att = layer.att
        att.cache_enabled = True
        if hasattr(att, "kv_lora_rank"):
            att.register_buffer("kv_cache", torch.zeros(1, ctx_len, att.kv_lora_rank), persistent=False)
            att.register_buffer("pe_cache", torch.zeros(1, ctx_len, att.rope_dim), persistent=False)
            att.register_buffer("cache_seqlens", torch.zeros(1, dtype=torch.long), persistent=False)
        else:
            att.register_buffer("k_cache", torch.zeros(1, att.num_kv_heads, ctx_len, att.head_dim), persistent=False)
            att.register_buffer("v_cache", torch.zeros(1, att.num_kv_heads, ctx_len, att.head_dim), persistent=False)


@torch.no_grad()
def _greedy(model, prompt, n_new, autocast=False):
    """Batch-1 prefill + incremental decode with argmax (generate.py:55-66 semantics)."""
    toks, logits_last = [], None
    ids = torch.tensor(prompt).unsqueeze(0)
    start = 0
    for _ in range(n_new):
        with torch.autocast("cpu", dtype=torch.bfloat16, enabled=autocast):
            logits = model(ids, start_pos=start)
        logits_last = logits[0, -1].float()
        nxt = int(logits_last.argmax())
        toks.append(nxt)
        start += ids.shape[1]
        ids = torch.tensor([[nxt]])
    return toks, logits_last


def c1_prompts():
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(16, 129, (8,), generator=g)
    return [torch.randint(0, 10000, (int(n),), generator=g).tolist() for n in lens]


def write_c1_model():
    from model.config import Config
    from model.transformer import TransformerLM
    torch.manual_seed(0)
    cfg = Config(vocab_size=10000, context_length=512, d_model=512, num_layers=4, num_heads=16, num_kv_heads=4,
                 d_ff=1344, attention_type="GQA", use_moe=False, dropout=0.0, rope_theta=10000.0)
    model = TransformerLM(cfg).eval()
    _enable_dense_cache(model, 512)
    prompts = c1_prompts()
    streams, last = [], []
    for p in prompts:
        t, lg = _greedy(model, p, 64)
        streams.append(t)
        last.append(_np(lg))
    sums = {f"sum::{k}": np.float64(v.double().sum().item()) for k, v in model.state_dict().items()}
    np.savez_compressed(HERE / "c1_model.npz", prompt_lens=np.array([len(p) for p in prompts]),
                        prompts=np.concatenate([np.array(p) for p in prompts]), streams=np.array(streams),
                        last_logits=np.stack(last).astype(np.float32), **sums)
    print("c1_model.npz", [len(p) for p in prompts], streams[0][:8])


def _small_model(att, use_moe, seed):
    from model.config import Config
    from model.transformer import TransformerLM
    torch.manual_seed(seed)
    kw = dict(vocab_size=512, context_length=128, d_model=128, num_layers=2, num_heads=8, d_ff=96, dropout=0.0,
              rope_theta=10000.0, use_moe=use_moe, n_routed_experts=4, num_experts_per_tok=2, n_shared_experts=1)
    if att == "GQA":
        kw.update(attention_type="GQA", num_kv_heads=2)
    else:
        kw.update(attention_type="MLA", rope_dim=8, q_lora_rank=48, kv_lora_rank=64)
    cfg = Config(**kw)
    model = TransformerLM(cfg).eval()
    _enable_dense_cache(model, 128)
    return cfg, model


def write_small_model(name, att):
    cfg, model = _small_model(att, True, 11)
    # make the routing bias non-trivial so that topk runs on logits + bias (moe.py:56-63)
    with torch.no_grad():
        for layer in model.layers:
            layer.ffn.gate.expert_bias.copy_(torch.tensor([0.02, -0.01, 0.0, 0.015]))
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (5, 16, 23, 40)]
    streams, last, streams_bf, last_bf = [], [], [], []
    for p in prompts:
        t, lg = _greedy(model, p, 12)
        streams.append(t)
        last.append(_np(lg))
        tb, lb = _greedy(model, p, 12, autocast=True)
        streams_bf.append(tb)
        last_bf.append(_np(lb))
    extra = {}
    if streams_bf:
        extra = dict(streams_bf16=np.array(streams_bf), last_logits_bf16=np.stack(last_bf))
    np.savez_compressed(HERE / name, prompt_lens=np.array([len(p) for p in prompts]),
                        prompts=np.concatenate([np.array(p) for p in prompts]), streams=np.array(streams),
                        last_logits=np.stack(last), **_state(model), **extra)
    print(name, streams[0])


@torch.no_grad()
def write_attention_module(name, att):
    from model.attention.utils import RotaryPositionalEmbedding
    torch.manual_seed(3)
    if att == "GQA":
        from model.attention.GQA import GroupedQueryAttention
        rope = RotaryPositionalEmbedding(10000.0, 16, 64)
        m = GroupedQueryAttention(128, 8, 2, rope, use_gate=False, cache_enabled=True, max_batch_size=1, max_seq_len=64)
        d = 128
    else:
        from model.attention.MLA import MultiHeadLatentAttention
        rope = RotaryPositionalEmbedding(10000.0, 64, 64)
        m = MultiHeadLatentAttention(256, 4, rope, rope_dim=16, q_lora_rank=48, kv_lora_rank=64, use_gate=False,
                                     cache_enabled=True, max_batch_size=1, max_seq_len=64)
        d = 256
    m.eval()
    x0 = torch.randn(1, 20, d)
    mask = torch.tril(torch.ones(20, 20, dtype=torch.bool))
    outs = [m(x0, 0, mask)]
    xs = [x0]
    for i in range(3):
        xi = torch.randn(1, 1, d)
        xs.append(xi)
        outs.append(m(xi, 20 + i, None))
    np.savez_compressed(HERE / name, x=_np(torch.cat(xs, dim=1)[0]), out=_np(torch.cat(outs, dim=1)[0]), **_state(m))
    print(name)


def write_all(ref: Path):
    sys.path.insert(0, str(ref))
    write_attn_kat(ref)
    write_attention_module("gqa_module.npz", "GQA")
    write_attention_module("mla_module.npz", "MLA")
    write_small_model("moe_model.npz", "GQA")
    write_small_model("mla_model.npz", "MLA")
    write_c1_model()
