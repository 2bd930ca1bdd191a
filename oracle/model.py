"""CPU restatement of the reference decoder's layer arithmetic, one request at a time with dense
caches (test oracle).

Follows, with the same torch operators so that CPU autocast rounds at the same places:

* TransformerLM.forward / Block.forward  model/transformer.py:90-118,162-183 (residual stream with
  fused add + RMSNorm, causal mask only when more than one token is fed)
* RMSNorm                                 model/utils.py:54-67 (fp32 math, returns the input dtype)
* GroupedQueryAttention.forward           model/attention/GQA.py:65-139 (cache branch; q/k RMSNorm
  over the whole projected vector with eps=None, half-split RoPE, K cached after norm+RoPE)
* MultiHeadLatentAttention.forward        model/attention/MLA.py:105-208 (absorbed cache branch;
  kv_up_proj_fused biases unused)
* MLP / Gate / MOE.moe_infer              model/architecture/mlp.py:61-67, moe.py:45-90,288-341

Weights come in under the reference's state_dict names.  ``greedy`` mirrors the incremental loop
of generate.py:55-66 (prefill, then one token at a time, argmax).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .attention import apply_rope, rope_table


class OracleModel:
    def __init__(self, cfg: dict, weights: dict):
        self.cfg = dict(cfg)
        self.w = {k: torch.as_tensor(v) for k, v in weights.items()}
        c = self.cfg
        self.d = c["d_model"]
        self.H = c["num_heads"]
        self.hd = self.d // self.H
        self.att = c.get("attention_type", "GQA")
        self.Hkv = c.get("num_kv_heads") or self.H
        self.table = rope_table(c.get("rope_theta", 10000.0), self.hd, c["context_length"])
        self.moe_layers = c.get("moe_layers")

    # ------------------------------------------------------------------ pieces
    def _lin(self, x, name):
        return F.linear(x, self.w[name + ".weight"], self.w.get(name + ".bias"))

    def _rms(self, x, name, residual=None, eps=1e-5):
        """model/utils.py:54-67."""
        w = self.w[name + ".weight"]
        dt = x.dtype
        if residual is None:
            xf = x.float()
            return (w * xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dt)
        xf = x.float() + residual.float()
        return (w * xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dt), xf.to(dt)

    def _nn_rms(self, x, name):
        """torch.nn.RMSNorm with eps=None (GQA.py:39-40, MLA.py:71-72): the operator the reference calls, so
        whatever epsilon and rounding torch applies (for a bf16 input with an fp32 weight: fp32 arithmetic,
        fp32 machine epsilon, one rounding at the end) is applied here too."""
        w = self.w[name + ".weight"]
        return F.rms_norm(x, (x.shape[-1],), w, None)

    def _mlp(self, x, p):
        return self._lin(F.silu(self._lin(x, p + ".w1")) * self._lin(x, p + ".w3"), p + ".w2")

    def _moe(self, x, p):
        """Gate.forward (moe.py:45-90) + MOE.moe_infer (moe.py:288-341) + shared expert (:272-273)."""
        c = self.cfg
        E, K = c["n_routed_experts"], c["num_experts_per_tok"]
        flat = x.reshape(-1, x.shape[-1])
        logits = flat @ self.w[p + ".gate.weight"].t()
        scores = torch.sigmoid(logits)
        biased = logits + self.w[p + ".gate.expert_bias"].to(logits.dtype).unsqueeze(0)
        _, idx = torch.topk(biased, k=K, dim=-1, sorted=False)
        wts = torch.gather(scores, -1, idx)
        if K > 1:
            wts = wts / (wts.sum(-1, keepdim=True) + 1e-10)
        flat_idx, flat_w = idx.reshape(-1), wts.reshape(-1, 1).to(flat.dtype)
        out = torch.zeros_like(flat)
        order = flat_idx.argsort()
        counts = flat_idx.bincount(minlength=E).tolist()
        tok = order // K
        lo = 0
        for e in range(E):
            hi = lo + counts[e]
            if hi > lo:
                t = tok[lo:hi]
                y = self._mlp(flat[t], f"{p}.experts.{e}") * flat_w[order[lo:hi]]
                out.scatter_add_(0, t.unsqueeze(1).expand(-1, flat.shape[-1]), y)
            lo = hi
        y = out.view_as(x)
        if c.get("n_shared_experts", 0) > 0:
            y = y + self._mlp(x, p + ".shared_expert")
        return y

    # ------------------------------------------------------------------ attention
    def _gqa(self, x, p, start, mask, cache):
        L = x.shape[0]
        pos = torch.arange(start, start + L)
        q = self._nn_rms(self._lin(x, p + ".q_proj"), p + ".q_norm")
        k = self._nn_rms(self._lin(x, p + ".k_proj"), p + ".k_norm")
        v = self._lin(x, p + ".v_proj")
        q = q.view(L, self.H, self.hd).transpose(0, 1)
        k = k.view(L, self.Hkv, self.hd).transpose(0, 1)
        v = v.view(L, self.Hkv, self.hd).transpose(0, 1)
        q, k = apply_rope(q, pos, self.table), apply_rope(k, pos, self.table)
        cache["k"][:, start:start + L] = k
        cache["v"][:, start:start + L] = v
        total = start + L
        kk, vv = cache["k"][:, :total], cache["v"][:, :total]
        if mask is not None:
            full = torch.ones(L, total, dtype=torch.bool)
            full[:, :L] = mask       # GQA.py:108-113 (only ever used with start == 0)
            mask = full
        g = self.H // self.Hkv
        if g > 1:
            kk = kk.unsqueeze(1).expand(self.Hkv, g, total, self.hd).reshape(self.H, total, self.hd)
            vv = vv.unsqueeze(1).expand(self.Hkv, g, total, self.hd).reshape(self.H, total, self.hd)
        o = F.scaled_dot_product_attention(q.unsqueeze(0), kk.unsqueeze(0), vv.unsqueeze(0), attn_mask=mask)[0]
        return self._lin(o.transpose(0, 1).contiguous().view(L, self.d), p + ".output_proj")

    def _mla(self, x, p, start, mask, cache):
        c = self.cfg
        L, H, hd, dr, r = x.shape[0], self.H, self.hd, c["rope_dim"], c["kv_lora_rank"]
        pos = torch.arange(start, start + L)
        qf = self._lin(self._nn_rms(self._lin(x, p + ".q_down_proj"), p + ".q_norm"), p + ".q_up_proj_fused")
        q_nope = qf[..., :self.d].view(L, H, hd)
        q_rope = qf[..., self.d:].view(L, H, dr).transpose(0, 1)
        q_rope = apply_rope(q_rope, pos, self.table).transpose(0, 1)
        kv = self._nn_rms(self._lin(x, p + ".kv_down_proj"), p + ".kv_norm")
        k_rope = apply_rope(self._lin(x, p + ".k_rope_proj").unsqueeze(0), pos, self.table).squeeze(0)
        cache["kv"][start:start + L] = kv
        cache["pe"][start:start + L] = k_rope
        total = start + L
        ckv, cpe = cache["kv"][:total], cache["pe"][:total]
        W = self.w[p + ".kv_up_proj_fused.weight"]
        w_uk = W[:self.d].view(H, hd, r)
        w_uv = W[self.d:].view(H, hd, r)
        # the reference's einsums carry a batch axis (MLA.py:153-178); it is kept (size 1) because the CPU
        # bf16 kernels behind einsum pick their blocking by operand shape, and outputs are compared bit for bit
        q_abs = torch.einsum("bqhd,hdk->bqhk", q_nope.unsqueeze(0), w_uk)
        score = torch.einsum("bqhk,btk->bhqt", q_abs, ckv.unsqueeze(0)) + \
            torch.einsum("bqhd,btd->bhqt", q_rope.unsqueeze(0), cpe.unsqueeze(0))
        score = score / (hd + dr) ** 0.5
        if mask is not None:
            full = torch.ones(L, total, dtype=torch.bool)
            full[:, :L] = mask
            score = score.masked_fill(~full.view(1, 1, L, total), float("-inf"))
        lat = torch.einsum("bhqt,btk->bhqk", F.softmax(score, dim=-1), ckv.unsqueeze(0))
        o = torch.einsum("bhqk,hdk->bqhd", lat, w_uv)[0]
        return self._lin(o.contiguous().view(L, -1), p + ".output_proj")

    # ------------------------------------------------------------------ model
    def new_cache(self, ctx_len: int | None = None, dtype=torch.float32):
        n = ctx_len or self.cfg["context_length"]
        if self.att == "MLA":
            return [dict(kv=torch.zeros(n, self.cfg["kv_lora_rank"], dtype=dtype),
                         pe=torch.zeros(n, self.cfg["rope_dim"], dtype=dtype)) for _ in range(self.cfg["num_layers"])]
        return [dict(k=torch.zeros(self.Hkv, n, self.hd, dtype=dtype), v=torch.zeros(self.Hkv, n, self.hd, dtype=dtype))
                for _ in range(self.cfg["num_layers"])]

    def forward(self, ids, start: int, cache) -> torch.Tensor:
        """ids [L] at positions start..start+L-1 -> logits [L, vocab]."""
        ids = torch.as_tensor(ids, dtype=torch.long)
        L = ids.shape[0]
        x = self.w["token_embeddings.weight"][ids]
        mask = torch.tril(torch.ones(L, L, dtype=torch.bool)) if L > 1 else None
        residual = None
        for i in range(self.cfg["num_layers"]):
            p = f"layers.{i}"
            if residual is None:
                x, residual = self._rms(x, p + ".att_norm"), x
            else:
                x, residual = self._rms(x, p + ".att_norm", residual)
            att = self._mla if self.att == "MLA" else self._gqa
            x = att(x, p + ".att", start, mask, cache[i])
            x, residual = self._rms(x, p + ".ffn_norm", residual)
            moe_here = self.cfg.get("use_moe") and (self.moe_layers is None or i in self.moe_layers)
            x = self._moe(x, p + ".ffn") if moe_here else self._mlp(x, p + ".ffn")
        x, _ = self._rms(x, "final_norm", residual)
        return self._lin(x, "lm_head")

    @torch.no_grad()
    def greedy(self, prompt, n_new: int, autocast: bool = False):
        cache = self.new_cache()
        toks, ids, start, last = [], list(prompt), 0, None
        for _ in range(n_new):
            with torch.autocast("cpu", dtype=torch.bfloat16, enabled=autocast):
                logits = self.forward(ids, start, cache)
            last = logits[-1].float()
            nxt = int(last.argmax())
            toks.append(nxt)
            start += len(ids)
            ids = [nxt]
        return toks, last
