"""fp32 CPU restatement of the attention arithmetic on the engine path (test oracle).

The reference ships no paged-attention layer; what it defines is (a) the attention arithmetic of
its dense-cache modules and (b) the paged metadata contract of engine/model_runner.py.  The
functions below apply (a) to a pool gathered through (b): gather the rows a block table names,
then run the reference's own formulas in fp32.  Inputs of any float dtype are promoted to fp32
first, so for bf16 tensors this is "the fp32 reference on the bf16-rounded inputs".
"""
from __future__ import annotations

import torch


# --------------------------------------------------------------------------- utils.py:8-12
def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    shifted = x - x.amax(dim=dim, keepdim=True)
    e = torch.exp(shifted)
    return e / e.sum(dim=dim, keepdim=True)


# --------------------------------------------------------------------------- utils.py:51-63
def sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None = None,
         scale: float | None = None) -> torch.Tensor:
    """softmax(q k^T / sqrt(d_k) + mask) v; ``mask`` is boolean, True = attend."""
    q, k, v = q.float(), k.float(), v.float()
    scores = q @ k.transpose(-2, -1)
    scores = scores / (q.size(-1) ** 0.5) if scale is None else scores * scale
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf"))
    return softmax(scores, dim=-1) @ v


# --------------------------------------------------------------------------- utils.py:18-45
def rope_table(theta: float, d_k: int, max_seq_len: int) -> torch.Tensor:
    """[max_seq_len, d_k] table whose row is cat(cos(d_k/2), sin(d_k/2)) (utils.py:25-32)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, d_k, 2).float() / d_k))
    ang = torch.einsum("i,j->ij", torch.arange(max_seq_len).float(), inv_freq)
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=-1)


def apply_rope(x: torch.Tensor, positions: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of the last dim of x [..., T, d_x] at ``positions`` [T].

    Keeps the reference's slicing ``table[pos, :d_x]`` (utils.py:38): when d_x equals the table
    width the two halves are cos and sin; when d_x is smaller (MLA's rope_dim) the slice holds
    cosines only and the "sin" half is cos of other frequencies.  The oracle reproduces that.
    """
    d_x = x.shape[-1]
    cs = table[positions, :d_x]
    cs = cs.view(*([1] * (x.ndim - 2)), *cs.shape)
    cos, sin = torch.chunk(cs, 2, dim=-1)
    x1, x2 = torch.chunk(x, 2, dim=-1)
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat((y1, y2), dim=-1)


# ------------------------------------------------------------------ model_runner.py:184-190
def gather_rows(cache: torch.Tensor, block_table, length: int) -> torch.Tensor:
    """Rows 0..length-1 of one sequence from a pool [num_blocks, block_size, ...]."""
    bs = cache.shape[1]
    nblk = (length + bs - 1) // bs
    ids = torch.as_tensor(list(block_table[:nblk]), dtype=torch.long)
    rows = cache[ids].reshape(nblk * bs, *cache.shape[2:])
    return rows[:length]


def store_kvcache(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping) -> None:
    """In place: cache row ``slot`` := token row, for every slot >= 0 (model_runner.py:226-230,261;
    -1 is the graph-replay padding of :300)."""
    kf = k_cache.view(-1, *k_cache.shape[-2:])
    vf = v_cache.view(-1, *v_cache.shape[-2:])
    for t, slot in enumerate(slot_mapping.tolist() if hasattr(slot_mapping, "tolist") else slot_mapping):
        if slot < 0:
            continue
        kf[slot] = k[t]
        vf[slot] = v[t]


def _expand_kv(x: torch.Tensor, group: int) -> torch.Tensor:
    """[Hkv, L, D] -> [Hkv*group, L, D]; query head h reads KV head h // group (GQA.py:118-125)."""
    hkv, L, d = x.shape
    return x.unsqueeze(1).expand(hkv, group, L, d).reshape(hkv * group, L, d)


def paged_decode_gqa(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables,
                     context_lens, scale: float | None = None) -> torch.Tensor:
    """q [B,Hq,D]; caches [nb,bs,Hkv,D]; returns fp32 [B,Hq,D] (GQA.py:105-130 at seq_len 1)."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    out = torch.zeros(B, Hq, D, dtype=torch.float32)
    lens = [int(x) for x in context_lens]
    for b in range(B):
        L = lens[b]
        if L <= 0:
            continue
        k = gather_rows(k_cache, block_tables[b], L).float().transpose(0, 1)  # [Hkv, L, D]
        v = gather_rows(v_cache, block_tables[b], L).float().transpose(0, 1)
        k, v = _expand_kv(k, Hq // Hkv), _expand_kv(v, Hq // Hkv)
        out[b] = sdpa(q[b].float().unsqueeze(1), k, v, None, scale).squeeze(1)
    return out


def prefill_varlen(q: torch.Tensor, k: torch.Tensor | None, v: torch.Tensor | None, cu_seqlens_q,
                   cu_seqlens_k, scale: float | None = None, k_cache=None, v_cache=None,
                   block_tables=None) -> torch.Tensor:
    """Causal attention per packed sequence; q [Tq,Hq,Dqk] -> fp32 [Tq,Hq,Dv].

    The mask is the lower-triangular mask of TransformerLM.forward (transformer.py:174-176); with a
    cached prefix (seqlen_k > seqlen_q) the new tokens see the whole prefix, i.e. the mask is
    bottom-right aligned (GQA.py:108-113 builds exactly that from the square mask).
    """
    cu_q = [int(x) for x in cu_seqlens_q]
    cu_k = [int(x) for x in cu_seqlens_k]
    Hq = q.shape[1]
    outs = []
    for s in range(len(cu_q) - 1):
        qs = q[cu_q[s]:cu_q[s + 1]].float().transpose(0, 1)  # [Hq, Lq, D]
        Lq, Lk = cu_q[s + 1] - cu_q[s], cu_k[s + 1] - cu_k[s]
        if block_tables is None:
            ks = k[cu_k[s]:cu_k[s + 1]].float().transpose(0, 1)
            vs = v[cu_k[s]:cu_k[s + 1]].float().transpose(0, 1)
        else:
            ks = gather_rows(k_cache, block_tables[s], Lk).float().transpose(0, 1)
            vs = gather_rows(v_cache, block_tables[s], Lk).float().transpose(0, 1)
        Hkv = ks.shape[0]
        ks, vs = _expand_kv(ks, Hq // Hkv), _expand_kv(vs, Hq // Hkv)
        qi = torch.arange(Lq).unsqueeze(1) + (Lk - Lq)
        mask = torch.arange(Lk).unsqueeze(0) <= qi
        outs.append(sdpa(qs, ks, vs, mask, scale).transpose(0, 1))
    Dv = outs[0].shape[-1] if outs else (v.shape[-1] if v is not None else v_cache.shape[-1])
    return torch.cat(outs, dim=0) if outs else torch.zeros(0, Hq, Dv)


def mla_decode(q_abs: torch.Tensor, q_rope: torch.Tensor, latent_cache: torch.Tensor, block_tables,
               context_lens, scale: float) -> torch.Tensor:
    """Absorbed MLA attention between the two weight einsums (MLA.py:154-177) at seq_len 1.

    q_abs [B,H,r], q_rope [B,H,dr]; latent rows are [c (r) | pe (dr)]; returns fp32 [B,H,r].
    """
    B, H, r = q_abs.shape
    out = torch.zeros(B, H, r, dtype=torch.float32)
    lens = [int(x) for x in context_lens]
    for b in range(B):
        L = lens[b]
        if L <= 0:
            continue
        rows = gather_rows(latent_cache, block_tables[b], L).float()
        c, pe = rows[:, :r], rows[:, r:]
        score = torch.einsum("hk,tk->ht", q_abs[b].float(), c)
        score = score + torch.einsum("hd,td->ht", q_rope[b].float(), pe)
        p = torch.softmax(score * scale, dim=-1)
        out[b] = torch.einsum("ht,tk->hk", p, c)
    return out


# --------------------------------------------------------------------------- model/utils.py:54-67
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None):
    """RMSNorm in fp32 returning the input dtype; with ``residual`` the sum is normalised and also
    returned as the new residual (the fused add + norm of the reference's residual stream)."""
    dt = x.dtype
    xf = x.float() if residual is None else x.float() + residual.float()
    y = (weight * xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dt)
    return y if residual is None else (y, xf.to(dt))
