"""Engine-mode decoder over flat ragged token batches and paged caches.

The reference's engine expects a model that takes flat 1-D ``input_ids`` and reads the global
attention ``Context`` (engine/model_runner.py:288-293); it does not ship one.  This module supplies
it, with the layer arithmetic of the reference's dense-batch model:

* residual stream with fused add + RMSNorm          model/transformer.py:90-118, model/utils.py:54-67
* GQA: biased q/k/v projections, RMSNorm over the whole projected q / k vector with
  the fp32 machine epsilon (eps=None), half-split RoPE, K cached after norm + RoPE, V raw   model/attention/GQA.py:79-130
* MLA: absorbed form, one latent row [kv_norm(kv_down(x)) | rope(k_rope(x))] cached per token,
  kv_up_proj_fused biases unused                     model/attention/MLA.py:114-178
* SwiGLU MLP with biases, sigmoid-score top-k MoE with renormalised weights, experts applied in
  ascending order, shared expert added last          mlp.py:61-67, moe.py:45-90,272-341

Attention itself is not computed here: q/k/v go to the CUDA kernels behind ``ops`` (store_kvcache,
varlen prefill, paged decode, MLA decode).  The projections are plain torch GEMMs.

Precision: ``dtype=float32`` computes everything in fp32.  ``dtype=bfloat16`` reproduces the
rounding points of the reference's mixed-precision mode (fp32 parameters under bf16 autocast):
linear layers, attention and caches in bf16; RMSNorm arithmetic and RoPE in fp32; the embedding
lookup stays fp32 so the first norm sees fp32, as under autocast.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..utils.context import get_context
from .config import ModelConfig


def _rope_table(theta: float, d_k: int, max_len: int) -> torch.Tensor:
    """[max_len, d_k] rows cat(cos, sin) (model/attention/utils.py:25-32); built on the CPU."""
    inv = 1.0 / (theta ** (torch.arange(0, d_k, 2).float() / d_k))
    ang = torch.einsum("i,j->ij", torch.arange(max_len).float(), inv)
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=-1)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x [T, H, d_x] rotated at positions [T]; the table is sliced to d_x columns exactly as the
    reference does (utils.py:38), including when d_x is smaller than the table width."""
    d_x = x.shape[-1]
    cs = table[positions, :d_x].unsqueeze(1)
    cos, sin = torch.chunk(cs, 2, dim=-1)
    x1, x2 = torch.chunk(x, 2, dim=-1)
    y1 = torch.addcmul(x1 * cos, x2, sin, value=-1)
    y2 = torch.addcmul(x2 * cos, x1, sin, value=1)
    return torch.cat((y1, y2), dim=-1)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """fp32 RMSNorm returning the input dtype; with ``residual`` also returns the new residual.
    One fused kernel on the GPU; the tensor-op form below is its definition."""
    if x.is_cuda and x.dim() == 2 and x.is_contiguous() and (residual is None or residual.is_contiguous()):
        return ops.add_rmsnorm(x, weight, eps, residual)
    dt = x.dtype
    xf = x.float()
    if residual is not None:
        xf = xf + residual.float()
    y = (weight * xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dt)
    return y if residual is None else (y, xf.to(dt))


def _vector_norm(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """nn.RMSNorm(eps=None) over the last dim as the reference's mode evaluates it (fp32 weight): fp32
    arithmetic with the fp32 machine epsilon, one rounding to x.dtype at the end."""
    eps = ops.VECTOR_NORM_EPS
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight).to(x.dtype)


class _Params:
    """Moves reference-named weights to the device in the compute dtype."""

    def __init__(self, weights: dict, device, dtype):
        self.w, self.device, self.dtype = weights, device, dtype

    def lin(self, *names):
        """Concatenated [sum(out), in] weight and bias of one or more Linear layers."""
        W = torch.cat([self.w[n + ".weight"] for n in names], dim=0).to(self.device, self.dtype).contiguous()
        b = torch.cat([self.w[n + ".bias"] for n in names], dim=0).to(self.device, self.dtype).contiguous()
        return W, b

    def f32(self, name):
        return self.w[name].to(self.device, torch.float32).contiguous()


class MLP(nn.Module):
    def __init__(self, p: _Params, prefix: str):
        super().__init__()
        self.w13, self.b13 = p.lin(prefix + ".w1", prefix + ".w3")
        self.w2, self.b2 = p.lin(prefix + ".w2")
        self.d_ff = self.w2.shape[1]

    def forward(self, x):
        h = F.linear(x, self.w13, self.b13)
        if h.dtype == torch.bfloat16 and h.is_cuda and h.dim() == 2:
            return F.linear(ops.swiglu(h), self.w2, self.b2)     # silu(h1) * h3 in one kernel
        return F.linear(F.silu(h[..., :self.d_ff]) * h[..., self.d_ff:], self.w2, self.b2)


class MoE(nn.Module):
    """Routing of Gate.forward (moe.py:45-90) and the expert mixture of MOE.moe_infer (moe.py:288-341).

    Two evaluation orders of the same sum  y[t] = sum_k w[t,k] * expert_{idx[t,k]}(x[t]) (+ shared):

    * ``forward_sorted`` — the reference's: tokens grouped by expert, experts visited in ascending
      order, each output scaled and accumulated in the activation dtype.  It reads the per-expert
      counts on the host (one sync per layer, as moe.py:307) and is used for large (prefill) batches.
    * ``forward_dense`` — for small (decode) batches: every expert is applied to every token with
      three batched GEMMs over the stacked expert weights and the routing weights select the two
      that count.  No host sync and a fixed launch sequence, so the decode step can be captured in
      a CUDA graph; at decode sizes the layer is bound by reading the expert weights either way.
    """

    dense_max_tokens = 512
    use_grouped = True     # bf16: grouped GEMMs over tokens sorted by expert (no host sync)
    # Average rows per expert up to which the grouped GEMMs of this package are used (weight-streaming kernel up to
    # 64, compute-bound kernel above); larger batches go to the library grouped GEMM, which on the 7,300-token
    # prefill steps of the benchmark engine is 11 % faster per step than the compute-bound kernel (both are bound by
    # L2-to-SM traffic; the library overlaps its epilogue with the next tile).  At 2,048 tokens the own kernels win
    # (122 against 163-195 us per layer, fewer launches: SwiGLU and the shared expert ride in the two GEMMs).
    own_gemm_max_rows_per_expert = 256
    # Gate projection + routing (+ gather) as one launch (ops.moe_gate_route).  Off: measured on B200 inside a
    # CUDA graph the one launch takes 10.0 / 11.7 / 12.1 us at 1 / 64 / 256 tokens against 9.6 / 8.9 / 10.3 us for
    # the library GEMM + routing kernel + gather it replaces — each of those is a single memory round trip behind
    # a ~2.3 us launch, while the fused kernel chains four (rows and gate matrix, bias, ticket, masks).
    fused_gate_route = False

    def __init__(self, p: _Params, prefix: str, cfg: ModelConfig):
        super().__init__()
        self.E, self.K = cfg.n_routed_experts, cfg.num_experts_per_tok
        self.gate_w = p.w[prefix + ".gate.weight"].to(p.device, p.dtype).contiguous()
        self.gate_bias = p.f32(prefix + ".gate.expert_bias")
        self.experts = nn.ModuleList([MLP(p, f"{prefix}.experts.{e}") for e in range(self.E)])
        # stacked copies share storage with the per-expert modules
        self.w13 = torch.stack([m.w13 for m in self.experts])      # [E, 2*d_ff, d]
        self.b13 = torch.stack([m.b13 for m in self.experts])      # [E, 2*d_ff]
        self.w2 = torch.stack([m.w2 for m in self.experts])        # [E, d, d_ff]
        self.b2 = torch.stack([m.b2 for m in self.experts])        # [E, d]
        for e, m in enumerate(self.experts):
            m.w13, m.b13, m.w2, m.b2 = self.w13[e], self.b13[e], self.w2[e], self.b2[e]
        self.d_ff = self.w2.shape[2]
        self.shared = MLP(p, prefix + ".shared_expert") if cfg.n_shared_experts > 0 else None
        if self.shared is not None and p.dtype == torch.bfloat16:
            # routed experts + the shared one as weight set E: one grouped launch covers both at decode sizes
            self.w13_all = torch.cat([self.w13, self.shared.w13.unsqueeze(0)]).contiguous()
            self.b13_all = torch.cat([self.b13, self.shared.b13.unsqueeze(0)]).contiguous()
            self.w2_all = torch.cat([self.w2, self.shared.w2.unsqueeze(0)]).contiguous()
            self.b2_all = torch.cat([self.b2, self.shared.b2.unsqueeze(0)]).contiguous()
        else:
            self.w13_all = None

    def route(self, x):
        logits = x @ self.gate_w.t()
        scores = torch.sigmoid(logits)
        biased = logits + self.gate_bias.to(logits.dtype).unsqueeze(0)
        _, idx = torch.topk(biased, k=self.K, dim=-1, sorted=False)
        wts = torch.gather(scores, -1, idx)
        if self.K > 1:
            wts = wts / (wts.sum(-1, keepdim=True) + 1e-10)
        return idx, wts

    def forward(self, x):
        if (x.dtype == torch.bfloat16 and self.use_grouped and self.E <= ops.MOE_ROUTE_MAX_EXPERTS
                and self.K <= ops.MOE_ROUTE_MAX_TOPK and x.shape[0] <= ops.MOE_ROUTE_MAX_TOKENS):
            return self.forward_routed(x)
        idx, wts = self.route(x)
        if x.dtype == torch.bfloat16 and self.use_grouped:
            out = self.forward_grouped(x, idx, wts)
        elif x.shape[0] <= self.dense_max_tokens:
            out = self.forward_dense(x, idx, wts)
        else:
            out = self.forward_sorted(x, idx, wts)
        if self.shared is not None:
            out = out + self.shared(x)
        return out

    def forward_sorted(self, x, idx, wts):
        flat_idx = idx.reshape(-1)
        flat_w = wts.reshape(-1, 1).to(x.dtype)
        out = torch.zeros_like(x)
        order = flat_idx.argsort()
        counts = flat_idx.bincount(minlength=self.E).tolist()
        tok = order // self.K
        lo = 0
        for e in range(self.E):
            hi = lo + counts[e]
            if hi > lo:
                t = tok[lo:hi]
                y = self.experts[e](x[t]) * flat_w[order[lo:hi]]
                out.index_add_(0, t, y)
            lo = hi
        return out

    def forward_routed(self, x):
        """bf16 fast path: routing kernel (top-k, weights, grouping by expert), two grouped GEMMs with
        the bias + SwiGLU between them, and one combine kernel that adds every token's K contributions
        in ascending expert order and then the shared expert.  Batches with few rows per expert
        (decode) are bound by streaming the expert weights and use the tcgen05 grouped GEMM of this
        package (SwiGLU in its epilogue); large prefill batches are compute-bound and go to the
        library grouped GEMM."""
        T = x.shape[0]
        small = (T * self.K <= self.own_gemm_max_rows_per_expert * self.E and x.shape[1] % 8 == 0
                 and self.d_ff % 8 == 0)
        fused_gate = (self.fused_gate_route and T <= ops.MOE_GATE_ROUTE_MAX_TOKENS and x.is_contiguous()
                      and x.shape[1] <= 2048
                      and self.gate_w.numel() * 2 <= ops.MOE_GATE_ROUTE_MAX_GATE_BYTES)
        in_kernel_gather = fused_gate and T <= ops.MOE_GATE_ROUTE_GATHER_MAX_TOKENS

        def route(identity_tail):
            """(sorted_token, experts, weights, offsets, slot_to_row, rows of x in sorted order)"""
            if fused_gate:     # gate projection + routing (+ the gather for small batches) in one launch
                tok, experts, w, offs, inv, xs = ops.moe_gate_route(x, self.gate_w, self.gate_bias, self.K,
                                                                    identity_tail=identity_tail, gather=in_kernel_gather)
            else:
                tok, experts, w, offs, inv = ops.moe_route((x @ self.gate_w.t()).contiguous(), self.gate_bias, self.K,
                                                           identity_tail=identity_tail)
                xs = None
            if xs is None:
                xs = x.index_select(0, tok)
            return tok, experts, w, offs, inv, xs

        # early launch of a grouped GEMM needs its offsets and weights complete before the kernel in front of it
        # started: true behind the separate gather, not when the routing launch itself is that kernel
        early_up = not in_kernel_gather
        if small and self.w13_all is not None:
            # decode sizes with a shared expert: its rows (every token, gathered through the identity tail of the
            # routing) ride in the same two launches as the routed rows, as one more weight set; biases are added
            # in the GEMM epilogues
            tok, experts, w, offs, inv, xs = route(True)           # [T*K routed rows | T shared rows]
            act = ops.moe_grouped_gemm(xs, self.w13_all, offs, self.b13_all, swiglu=True, dense_rows=T, early_launch=early_up)
            y = ops.moe_grouped_gemm(act, self.w2_all, offs, self.b2_all, dense_rows=T, early_launch=True)
            R = T * self.K
            return ops.moe_combine(y[:R], None, experts, w, inv, y[R:])
        tok, experts, w, offs, inv, xs = route(False)
        if small:
            act = ops.moe_grouped_gemm(xs, self.w13, offs, self.b13, swiglu=True, early_launch=early_up)
            y = ops.moe_grouped_gemm(act, self.w2, offs, early_launch=True)
        else:
            act = ops.swiglu(torch._grouped_mm(xs, self.w13.transpose(1, 2), offs=offs), self.b13, experts)
            y = torch._grouped_mm(act, self.w2.transpose(1, 2), offs=offs)
        shared = self.shared(x) if self.shared is not None else None
        return ops.moe_combine(y, self.b2, experts, w, inv, shared)

    def forward_grouped(self, x, idx, wts):
        """bf16: rows sorted by expert, two grouped GEMMs with device-side group offsets, then the
        K contributions of every token are added in ascending expert order in the activation dtype
        (the accumulation order of moe.py:312-339).  No host sync, no per-expert launch."""
        T, K, E = x.shape[0], self.K, self.E
        sidx, perm = idx.sort(dim=1)                       # ascending expert ids per token
        w_sorted = wts.gather(1, perm).to(x.dtype).reshape(-1)
        flat = sidx.reshape(-1)                            # expert of row t*K + k
        order = flat.argsort(stable=True)                  # rows grouped by expert
        experts = flat[order]
        xs = x[order // K]
        counts = torch.zeros(E, dtype=torch.int32, device=x.device).scatter_add_(
            0, flat, torch.ones_like(flat, dtype=torch.int32))     # bincount would sync the host
        offs = counts.cumsum(0).to(torch.int32)
        h = torch._grouped_mm(xs, self.w13.transpose(1, 2), offs=offs) + self.b13[experts]
        act = F.silu(h[:, :self.d_ff]) * h[:, self.d_ff:]
        y = torch._grouped_mm(act, self.w2.transpose(1, 2), offs=offs) + self.b2[experts]
        y = y * w_sorted[order].unsqueeze(1)
        yt = torch.empty_like(y)
        yt[order] = y
        yt = yt.view(T, K, -1)
        out = yt[:, 0]
        for k in range(1, K):
            out = out + yt[:, k]
        return out

    def forward_dense(self, x, idx, wts):
        T = x.shape[0]
        xe = x.unsqueeze(0).expand(self.E, T, x.shape[1])
        h = torch.baddbmm(self.b13.unsqueeze(1), xe, self.w13.transpose(1, 2))          # [E, T, 2*d_ff]
        act = F.silu(h[..., :self.d_ff]) * h[..., self.d_ff:]
        y = torch.baddbmm(self.b2.unsqueeze(1), act, self.w2.transpose(1, 2))           # [E, T, d]
        dense_w = torch.zeros(T, self.E, dtype=x.dtype, device=x.device).scatter_(1, idx, wts.to(x.dtype))
        return torch.einsum("etd,te->td", y, dense_w)


class GQAAttention(nn.Module):
    def __init__(self, p: _Params, prefix: str, cfg: ModelConfig, rope: torch.Tensor):
        super().__init__()
        self.H, self.Hkv, self.hd, self.d = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.d_model
        self.w_qkv, self.b_qkv = p.lin(prefix + ".q_proj", prefix + ".k_proj", prefix + ".v_proj")
        self.w_o, self.b_o = p.lin(prefix + ".output_proj")
        self.q_norm, self.k_norm = p.f32(prefix + ".q_norm.weight"), p.f32(prefix + ".k_norm.weight")
        self.rope = rope
        self.scale = self.hd ** -0.5
        self.dtype = p.dtype
        self.fused = True   # False: the same stage as separate tensor ops + store_kvcache
        # views into the pool; set by ModelRunner.allocate_kv_cache (model_runner.py:186-190)
        self.k_cache = self.v_cache = torch.empty(0)

    def forward(self, x, ctx, positions, out=None):
        T = x.shape[0]
        kvw = self.Hkv * self.hd
        qkv = F.linear(x.to(self.dtype), self.w_qkv, self.b_qkv)
        if self.fused:
            # q/k RMSNorm + RoPE + store_kvcache in one kernel
            q, k, v = ops.qk_norm_rope_store(qkv, self.q_norm, self.k_norm, self.rope, positions, self.H, self.Hkv,
                                             self.hd, self.k_cache, self.v_cache, ctx.slot_mapping)
        else:
            q = _vector_norm(qkv[:, :self.d], self.q_norm).view(T, self.H, self.hd)
            k = _vector_norm(qkv[:, self.d:self.d + kvw], self.k_norm).view(T, self.Hkv, self.hd)
            v = qkv[:, self.d + kvw:].view(T, self.Hkv, self.hd)
            q = apply_rope(q, positions, self.rope).to(self.dtype)
            k = apply_rope(k, positions, self.rope).to(self.dtype)
            if self.k_cache.numel():
                ops.store_kvcache(k, v, self.k_cache, self.v_cache, ctx.slot_mapping)
        if ctx.is_prefill:
            if ctx.block_tables is not None:   # part of the context is already cached
                o = ops.prefill_varlen(q, None, None, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.max_seqlen_q,
                                       ctx.max_seqlen_k, self.scale, self.k_cache, self.v_cache, ctx.block_tables,
                                       out=out, plan=ctx.prefill_plan)
            else:
                o = ops.prefill_varlen(q, k, v, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.max_seqlen_q,
                                       ctx.max_seqlen_k, self.scale, out=out, plan=ctx.prefill_plan)
        else:
            o = ops.paged_decode_gqa(q, self.k_cache, self.v_cache, ctx.block_tables, ctx.context_lens, self.scale)
        return F.linear(o.view(T, self.d), self.w_o, self.b_o)


class MLAAttention(nn.Module):
    def __init__(self, p: _Params, prefix: str, cfg: ModelConfig, rope: torch.Tensor):
        super().__init__()
        self.H, self.hd, self.d = cfg.num_heads, cfg.head_dim, cfg.d_model
        self.r, self.dr = cfg.kv_lora_rank, cfg.rope_dim
        self.w_qd, self.b_qd = p.lin(prefix + ".q_down_proj")
        self.w_qu, self.b_qu = p.lin(prefix + ".q_up_proj_fused")
        # kv_down_proj and k_rope_proj read the same input: one GEMM
        self.w_kv, self.b_kv = p.lin(prefix + ".kv_down_proj", prefix + ".k_rope_proj")
        up = p.w[prefix + ".kv_up_proj_fused.weight"].to(p.device, p.dtype)
        self.w_uk = up[:self.d].view(self.H, self.hd, self.r).contiguous()      # [H, hd, r]
        self.w_uv = up[self.d:].view(self.H, self.hd, self.r).contiguous()      # [H, hd, r]
        self.w_o, self.b_o = p.lin(prefix + ".output_proj")
        self.q_norm, self.kv_norm = p.f32(prefix + ".q_norm.weight"), p.f32(prefix + ".kv_norm.weight")
        self.rope = rope
        self.scale = (self.hd + self.dr) ** -0.5
        self.dtype = p.dtype
        self.w_ukv = up.contiguous()         # [2*H*hd, r]: W_UK of all heads, then W_UV, for the prefill expansion
        self.fused = True                    # False: the pre-attention stage as separate tensor ops
        self.latent_cache = torch.empty(0)   # [num_blocks, block_size, r + dr]; set by the runner

    def forward(self, x, ctx, positions, out=None):
        T, H, hd, r, dr = x.shape[0], self.H, self.hd, self.r, self.dr
        x = x.to(self.dtype)
        fused = self.fused and ops.mla_prologue_supported(hd, dr, r, self.dtype)
        qd = F.linear(x, self.w_qd, self.b_qd)
        qc = ops.add_rmsnorm(qd, self.q_norm, ops.VECTOR_NORM_EPS) if fused else _vector_norm(qd, self.q_norm)
        qf = F.linear(qc, self.w_qu, self.b_qu)
        kvp = F.linear(x, self.w_kv, self.b_kv)
        if fused:
            # q assembly + RoPE, latent RMSNorm + RoPE and the cache write in one kernel
            q, rows = ops.mla_prologue(qf, kvp, self.kv_norm, self.rope, positions, H, hd, dr, r,
                                       self.latent_cache, ctx.slot_mapping)
        else:
            q_rope = apply_rope(qf[:, self.d:].view(T, H, dr), positions, self.rope).to(self.dtype)
            q = torch.cat([qf[:, :self.d].view(T, H, hd), q_rope], dim=-1)
            c = _vector_norm(kvp[:, :r], self.kv_norm)
            pe = apply_rope(kvp[:, r:].unsqueeze(1), positions, self.rope).squeeze(1).to(self.dtype)
            rows = torch.cat([c, pe], dim=-1)                               # [T, r + dr]
            if self.latent_cache.numel():
                ops.store_rows(rows, self.latent_cache, ctx.slot_mapping)
        if ctx.is_prefill:
            o = self._prefill(q, rows, ctx, out)
        else:
            q_abs = torch.einsum("thd,hdk->thk", q[..., :hd], self.w_uk)     # absorb W_UK (MLA.py:153)
            lat = ops.mla_decode(q_abs.contiguous(), q[..., hd:].contiguous(), self.latent_cache, ctx.block_tables,
                                 ctx.context_lens, self.scale)
            o = torch.einsum("thk,hdk->thd", lat, self.w_uv)                 # absorb W_UV (MLA.py:178)
        return F.linear(o.reshape(T, H * hd), self.w_o, self.b_o)

    def _prefill(self, q, rows, ctx, out=None):
        """Causal attention of the packed new tokens over their contexts.

        Prefill expands the latent rows once per step instead of absorbing the up-projections into
        every query: K = [c W_UK^T | pe], V = c W_UV^T per head, without the kv_up_proj_fused biases.
        That is the same function as the absorbed form the reference evaluates (the q.b_k term is
        constant over keys and cancels in the softmax; b_v is absent from the reference's cache
        branch), at 320 instead of 1088 multiply-adds per (query, key, head).
        """
        r, H, hd, dr = self.r, self.H, self.hd, self.dr
        if ctx.block_tables is not None:
            rows = self._gather_context_rows(ctx)
        c, pe = rows[:, :r], rows[:, r:]
        Tk = rows.shape[0]
        # one GEMM for both expansions: [Tk, r] x [r, 2*H*hd] -> K_nope of all heads, then V of all heads
        kv = F.linear(c, self.w_ukv)
        k_nope, v = kv[:, :H * hd].view(Tk, H, hd), kv[:, H * hd:].view(Tk, H, hd)
        if rows.dtype == torch.bfloat16 and (hd, dr) == (128, 64):
            # the kernel reads the rotary part once per token instead of a copy per head
            return ops.prefill_varlen_shared_tail(q, k_nope, pe, v, ctx.cu_seqlens_q, ctx.cu_seqlens_k,
                                                  ctx.max_seqlen_q, self.scale, out=out, plan=ctx.prefill_plan)
        k = torch.cat([k_nope, pe.unsqueeze(1).expand(-1, H, dr)], dim=-1)
        return ops.prefill_varlen(q, k, v, ctx.cu_seqlens_q, ctx.cu_seqlens_k, ctx.max_seqlen_q,
                                  ctx.max_seqlen_k, self.scale, out=out, plan=ctx.prefill_plan)

    def _gather_context_rows(self, ctx):
        """Packed latent rows of every sequence's full context, read back through the block tables."""
        bs = self.latent_cache.shape[1]
        cu_k = ctx.cu_seqlens_k.long()
        total = int(cu_k[-1])
        seq = torch.repeat_interleave(torch.arange(cu_k.numel() - 1, device=cu_k.device), cu_k[1:] - cu_k[:-1],
                                      output_size=total)
        pos = torch.arange(total, device=cu_k.device) - cu_k[seq]
        blk = ctx.block_tables.long()[seq, pos // bs]
        return self.latent_cache.view(-1, self.latent_cache.shape[-1])[blk * bs + pos % bs]


class DecoderLayer(nn.Module):
    def __init__(self, p: _Params, i: int, cfg: ModelConfig, rope: torch.Tensor):
        super().__init__()
        prefix = f"layers.{i}"
        att_cls = MLAAttention if cfg.attention_type == "MLA" else GQAAttention
        self.att = att_cls(p, prefix + ".att", cfg, rope)
        self.ffn = MoE(p, prefix + ".ffn", cfg) if cfg.is_moe_layer(i) else MLP(p, prefix + ".ffn")
        self.att_norm, self.ffn_norm = p.f32(prefix + ".att_norm.weight"), p.f32(prefix + ".ffn_norm.weight")
        self.eps = cfg.rms_eps

    def forward(self, x, residual, ctx, positions, attn_out=None):
        if residual is None:
            h, residual = rms_norm(x, self.att_norm, self.eps), x
        else:
            h, residual = rms_norm(x, self.att_norm, self.eps, residual)
        a = self.att(h, ctx, positions, attn_out)
        h, residual = rms_norm(a, self.ffn_norm, self.eps, residual)
        return self.ffn(h), residual


class EngineTransformerLM(nn.Module):
    """``model(input_ids)`` -> hidden states [T, d]; ``compute_logits(hidden)`` -> [num_seqs, vocab]."""

    def __init__(self, cfg: ModelConfig, weights: dict, device, dtype=torch.float32):
        super().__init__()
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)
        p = _Params(weights, self.device, dtype)
        self.embed = p.f32("token_embeddings.weight")
        rope = _rope_table(cfg.rope_theta, cfg.head_dim, cfg.context_length).to(self.device)
        self.layers = nn.ModuleList([DecoderLayer(p, i, cfg, rope) for i in range(cfg.num_layers)])
        self.final_norm = p.f32("final_norm.weight")
        self.w_head, self.b_head = p.lin("lm_head")

    @property
    def attention_layers(self):
        return [layer.att for layer in self.layers]

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
        ctx = get_context()
        if positions is None:
            positions = ctx.positions if ctx.positions is not None else ctx.context_lens - 1
        x = self.embed[input_ids]
        residual = None
        attn_out = None
        if ctx.is_prefill:
            # one attention output buffer for all layers; rows of padding tokens (in no sequence) are
            # never written by the kernel and stay zero
            c = self.cfg
            dv = c.head_dim
            attn_out = torch.zeros(x.shape[0], c.num_heads, dv, dtype=self.dtype, device=x.device)
        for layer in self.layers:
            x, residual = layer(x, residual, ctx, positions, attn_out)
        h, _ = rms_norm(x, self.final_norm, self.cfg.rms_eps, residual)
        return h

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        ctx = get_context()
        if ctx.is_prefill:
            hidden = hidden[ctx.cu_seqlens_q[1:].long() - 1]
        return F.linear(hidden.to(self.dtype), self.w_head, self.b_head)

    fused_head_max_rows = 64     # rows up to which the fused head (weights as the MMA M side) beats GEMM + argmax

    def greedy_tokens(self, hidden: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """argmax of ``compute_logits(hidden)`` per sequence (first maximum), int64 [num_seqs].  In bf16, up to 64
        rows, the head projection and the argmax are one fused pass over the head matrix
        (``ops.lm_head_argmax``: the logits are never written; 20-22 us against 24-27 us on B200).  Larger batches
        take the library GEMM followed by the argmax kernel of ``ops.sample`` (the fused kernel keeps the tokens
        on the narrow side of the MMA and takes 41 us at 256 rows against 27 us)."""
        ctx = get_context()
        if ctx.is_prefill:
            hidden = hidden[ctx.cu_seqlens_q[1:].long() - 1]
        hidden = hidden.to(self.dtype)
        if hidden.shape[0] <= self.fused_head_max_rows and ops.lm_head_argmax_supported(hidden, self.w_head):
            return ops.lm_head_argmax(hidden.contiguous(), self.w_head, self.b_head, out)
        logits = F.linear(hidden, self.w_head, self.b_head)
        if logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16) and logits.shape[0] > 0:
            return ops.sample(logits, None, 0, 0, out=out)   # no temperatures: greedy rows, first maximum
        if out is None:
            return torch.argmax(logits, dim=-1)
        return torch.argmax(logits, dim=-1, out=out)
