"""Tensor-level wrappers over the C ABI: the calls the attention layers of the engine make.

Every function takes CUDA tensors, checks shapes/dtypes on the host, and enqueues the kernel on
the current CUDA stream.  Nothing here computes on the CPU; a CPU tensor is an error.
"""
from __future__ import annotations

import array

import torch

from . import _lib
from ._lib import lib, check

_DTYPES = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16}

# Epsilon of the reference's q / k / latent RMSNorm layers, nn.RMSNorm(eps=None) (GQA.py:39-40, MLA.py:71-72).
# With fp32 parameters and a bf16 activation (the reference's autocast mode) torch evaluates that layer in
# fp32 with the fp32 machine epsilon and rounds once at the end; in fp32 it is the same number.
VECTOR_NORM_EPS = float(torch.finfo(torch.float32).eps)

_status: dict[int, torch.Tensor] = {}
_workspaces: dict[tuple[int, str], torch.Tensor] = {}
_retired_workspaces: list[torch.Tensor] = []   # outgrown buffers that captured graphs may still address


def _dt(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; the kernels take float32 or bfloat16") from None


def _cuda(*ts: torch.Tensor | None) -> torch.device:
    dev = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("b200 ops take CUDA tensors only (there is no CPU path)")
        if dev is not None and t.device != dev:
            raise ValueError("all tensors must be on the same device")
        dev = t.device
    return dev


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 that kernels set when they skip an out-of-pool block id or slot."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[idx]


def check_status(device: torch.device | None = None) -> None:
    """Synchronises the current stream, raises if a kernel reported a device-side fault."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    st = status_word(device)
    host = array.array("i", [0])
    addr, _ = host.buffer_info()
    check(lib.b200_read_status(st.data_ptr(), addr, _stream()), "read_status")
    if host[0] != 0:
        check(host[0], "device-side check")


def selftest_bounded_wait(poll_limit: int = 1024, device: torch.device | None = None) -> list[int]:
    """Diagnostic: makes a bounded barrier wait run out inside one small CTA (``b200_selftest_bounded_wait``).
    Returns the five result words; the device status word then holds the time-out code, so the next
    ``check_status`` raises (``read_status_code`` reads and clears it without raising)."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    result = torch.full((5,), -1, dtype=torch.int32, device=device)
    check(lib.b200_selftest_bounded_wait(poll_limit, result.data_ptr(), status_word(device).data_ptr(), _stream()),
          "selftest_bounded_wait")
    return result.tolist()


def read_status_code(device: torch.device | None = None) -> int:
    """Synchronises the current stream and returns (and clears) the device status word: 0 or a B200_ERR_* code."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    host = array.array("i", [0])
    addr, _ = host.buffer_info()
    check(lib.b200_read_status(status_word(device).data_ptr(), addr, _stream()), "read_status")
    return host[0]


def workspace(device: torch.device, nbytes: int, tag: str) -> torch.Tensor:
    """Scratch buffer per (device, op); allocated outside any graph capture.

    A captured CUDA graph has the address of the buffer it was captured with baked in, so a buffer
    that has been handed out is never freed: when a later call needs more, a larger one (at least
    twice the size, so all retired buffers together stay below the live one) replaces it for new
    calls and the old one is kept alive for the graphs that still write to it.  Buffers start zero-filled
    (the decode kernels keep arrival counters at the head of theirs, which every call returns to zero);
    nothing else survives a call, so old and new buffers can be in use side by side."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, tag)
    w = _workspaces.get(key)
    if w is None or w.numel() < nbytes:
        if w is not None:
            _retired_workspaces.append(w)
            nbytes = max(nbytes, 2 * w.numel())
        w = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=device)
        _workspaces[key] = w
    return w


def store_kvcache(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  slot_mapping: torch.Tensor) -> None:
    """k_cache[slot_mapping[t]] = k[t], v likewise; slots < 0 are skipped.

    k, v: [T, Hkv, D] (rows contiguous, token stride free); caches: [..., Hkv, D] contiguous.
    """
    dev = _cuda(k, v, k_cache, v_cache, slot_mapping)
    T, Hkv, D = k.shape
    if v.shape != k.shape or k.dtype != v.dtype or k_cache.dtype != k.dtype or v_cache.dtype != k.dtype:
        raise ValueError("k/v/cache shape or dtype mismatch")
    if slot_mapping.dtype != torch.int64 or slot_mapping.numel() != T or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 tensor with one entry per token")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("caches must be contiguous")
    if k.stride(2) != 1 or k.stride(1) != D or v.stride(2) != 1 or v.stride(1) != D:
        raise ValueError("k/v rows (Hkv*D) must be contiguous")
    if k_cache.shape[-2:] != (Hkv, D) or v_cache.shape != k_cache.shape:
        raise ValueError("cache trailing dims must be (Hkv, D)")
    num_slots = k_cache.numel() // (Hkv * D)
    check(lib.b200_store_kvcache(k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0),
                                 k_cache.data_ptr(), v_cache.data_ptr(), slot_mapping.data_ptr(),
                                 T, Hkv, D, num_slots, _dt(k), status_word(dev).data_ptr(),
                                 _stream()), "store_kvcache")


def store_rows(rows: torch.Tensor, cache: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    """cache[slot_mapping[t]] = rows[t] for a single pool (the MLA latent cache).

    rows: [T, W] with contiguous rows; cache: [..., W] contiguous.
    """
    dev = _cuda(rows, cache, slot_mapping)
    T, W = rows.shape
    if cache.shape[-1] != W or cache.dtype != rows.dtype or not cache.is_contiguous() or rows.stride(1) != 1:
        raise ValueError("rows/cache shape, dtype or layout mismatch")
    if slot_mapping.dtype != torch.int64 or slot_mapping.numel() != T or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 tensor with one entry per row")
    check(lib.b200_store_kvcache(rows.data_ptr(), None, rows.stride(0), 0, cache.data_ptr(), None,
                                 slot_mapping.data_ptr(), T, 1, W, cache.numel() // W, _dt(rows),
                                 status_word(dev).data_ptr(), _stream()), "store_rows")


def paged_decode_gqa(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_tables: torch.Tensor, context_lens: torch.Tensor, scale: float,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """One query token per sequence over a paged KV pool.

    q: [B, Hq, D]; caches: [num_blocks, block_size, Hkv, D]; block_tables: [B, maxb] int32;
    context_lens: [B] int64.  Returns out [B, Hq, D].
    """
    dev = _cuda(q, k_cache, v_cache, block_tables, context_lens, out)
    B, Hq, D = q.shape
    nb, bs, Hkv, Dc = k_cache.shape
    if Dc != D or v_cache.shape != k_cache.shape or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("cache shape/dtype does not match q")
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int64:
        raise ValueError("block_tables must be int32 and context_lens int64")
    if block_tables.dim() != 2 or block_tables.shape[0] != B or block_tables.stride(1) != 1:
        raise ValueError("block_tables must be [B, maxb] with contiguous rows")
    if context_lens.numel() != B or not context_lens.is_contiguous():
        raise ValueError("context_lens must be a contiguous [B] tensor")
    if not (q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("q and caches must be contiguous")
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("out must match q")
    need = lib.b200_paged_decode_gqa_workspace_bytes(B, Hq, Hkv, D, _dt(q))
    ws = workspace(dev, need, "decode")
    check(lib.b200_paged_decode_gqa(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                    out.data_ptr(), block_tables.data_ptr(),
                                    block_tables.stride(0), context_lens.data_ptr(), B, Hq, Hkv, D,
                                    bs, nb, float(scale), ws.data_ptr(), ws.numel(), _dt(q),
                                    status_word(dev).data_ptr(), _stream()), "paged_decode_gqa")
    return out


def prefill_varlen(q: torch.Tensor, k: torch.Tensor | None, v: torch.Tensor | None,
                   cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor, max_seqlen_q: int,
                   max_seqlen_k: int, scale: float, k_cache: torch.Tensor | None = None,
                   v_cache: torch.Tensor | None = None, block_tables: torch.Tensor | None = None,
                   out: torch.Tensor | None = None, plan: "PrefillPlan | None" = None,
                   slot_mapping: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention over packed ragged sequences.

    ``slot_mapping`` (int64, one slot per row of k / v): the same call first scatters the new tokens' k / v
    rows into ``k_cache`` / ``v_cache`` (the step's store_kvcache), with or without ``block_tables``.

    q: [Tq, Hq, Dqk].  Without ``block_tables``: k [Tk, Hkv, Dqk], v [Tk, Hkv, Dv] are the packed
    keys/values.  With ``block_tables`` (a cached prefix exists) keys/values are read from the
    paged caches [num_blocks, block_size, Hkv, D*].  Returns out [Tq, Hq, Dv].  ``plan``: a tile list from
    ``prefill_plan`` for the same ``cu_seqlens_q`` (one CTA per real tile, longest first).
    """
    dev = _cuda(q, k, v, cu_seqlens_q, cu_seqlens_k, k_cache, v_cache, block_tables, out)
    Tq, Hq, Dqk = q.shape
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
        raise ValueError("cu_seqlens must be int32")
    num_seqs = cu_seqlens_q.numel() - 1
    if cu_seqlens_k.numel() != num_seqs + 1:
        raise ValueError("cu_seqlens_q and cu_seqlens_k must have the same length")
    if q.stride(2) != 1 or q.stride(1) != Dqk:
        raise ValueError("q heads must be contiguous")
    if block_tables is None:
        if k is None or v is None:
            raise ValueError("k and v are required without block_tables")
        Hkv, Dv = v.shape[1], v.shape[2]
        if k.shape[1] != Hkv or k.shape[2] != Dqk or k.dtype != q.dtype or v.dtype != q.dtype:
            raise ValueError("k/v shape or dtype mismatch")
        if k.stride(2) != 1 or k.stride(1) != Dqk or v.stride(2) != 1 or v.stride(1) != Dv:
            raise ValueError("k/v heads must be contiguous")
        kp, vp, ks, vs = k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0)
        kcp = vcp = btp = 0
        bts = bs = nb = 0
        total_k = k.shape[0]
        if slot_mapping is not None:
            if k_cache is None or v_cache is None or k_cache.shape != v_cache.shape or k_cache.dim() != 4 \
                    or k_cache.shape[2:] != (Hkv, Dqk) or k_cache.dtype != q.dtype \
                    or not (k_cache.is_contiguous() and v_cache.is_contiguous()):
                raise ValueError("the fused scatter needs contiguous caches [num_blocks, block_size, Hkv, D] of q's dtype")
            nb, bs = k_cache.shape[0], k_cache.shape[1]
            kcp, vcp = k_cache.data_ptr(), v_cache.data_ptr()
    else:
        if k_cache is None or v_cache is None:
            raise ValueError("paged prefill needs k_cache and v_cache")
        nb, bs, Hkv, Dk = k_cache.shape
        Dv = v_cache.shape[3]
        if Dk != Dqk or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
            raise ValueError("cache shape/dtype does not match q")
        if block_tables.dtype != torch.int32 or block_tables.shape[0] != num_seqs or block_tables.stride(1) != 1:
            raise ValueError("block_tables must be int32 [num_seqs, maxb]")
        if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise ValueError("caches must be contiguous")
        kp = vp = 0
        ks = vs = 0
        total_k = 0
        if slot_mapping is not None:
            if k is None or v is None or k.shape != (Tq, Hkv, Dqk) or v.shape != (Tq, Hkv, Dv) or k.stride(1) != Dqk \
                    or v.stride(1) != Dv or k.stride(2) != 1 or v.stride(2) != 1:
                raise ValueError("the fused scatter needs the new tokens' k / v [Tq, Hkv, D]")
            kp, vp, ks, vs, total_k = k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0), Tq
        kcp, vcp, btp, bts = k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr(), block_tables.stride(0)
    if slot_mapping is not None and (slot_mapping.dtype != torch.int64 or not slot_mapping.is_contiguous()
                                     or slot_mapping.numel() != min(Tq, total_k)):
        raise ValueError("slot_mapping must be a contiguous int64 tensor with one entry per new token")
    if out is None:
        out = torch.empty((Tq, Hq, Dv), dtype=q.dtype, device=q.device)
    elif out.shape != (Tq, Hq, Dv) or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous [Tq, Hq, Dv] tensor")
    check(lib.b200_prefill_varlen(q.data_ptr(), kp, vp, out.data_ptr(), q.stride(0), ks, vs, Tq, total_k,
                                  cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), num_seqs,
                                  int(max_seqlen_q), int(max_seqlen_k), Hq, Hkv, Dqk, Dv,
                                  float(scale), kcp, vcp, btp, bts, bs, nb,
                                  slot_mapping.data_ptr() if slot_mapping is not None else None,
                                  plan.buffer.data_ptr() if plan is not None else None,
                                  plan.tile_rows if plan is not None else 0,
                                  plan.capacity if plan is not None else 0, _dt(q),
                                  status_word(dev).data_ptr(), _stream()), "prefill_varlen")
    return out


def prefill_varlen_shared_tail(q: torch.Tensor, k_head: torch.Tensor, k_tail: torch.Tensor, v: torch.Tensor,
                               cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor, max_seqlen_q: int,
                               scale: float, out: torch.Tensor | None = None,
                               plan: "PrefillPlan | None" = None) -> torch.Tensor:
    """``prefill_varlen`` over packed keys given in two parts: k_head [Tk, H, Dqk - tail] per head and
    k_tail [Tk, tail], the last columns of every head's key (MLA's shared rotary part).  bf16.

    q: [Tq, H, Dqk], v: [Tk, H, Dv]; token strides are free, heads contiguous.  Returns out [Tq, H, Dv].
    """
    dev = _cuda(q, k_head, k_tail, v, cu_seqlens_q, cu_seqlens_k, out)
    Tq, H, Dqk = q.shape
    Tk, tail = k_tail.shape
    Dv = v.shape[2]
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32 \
            or cu_seqlens_q.numel() != cu_seqlens_k.numel():
        raise ValueError("cu_seqlens must be int32 tensors of the same length")
    if k_head.shape != (Tk, H, Dqk - tail) or v.shape[:2] != (Tk, H):
        raise ValueError("k_head must be [Tk, H, Dqk - tail] and v [Tk, H, Dv]")
    if any(t.dtype != torch.bfloat16 for t in (q, k_head, k_tail, v)):
        raise ValueError("prefill_varlen_shared_tail takes bf16 tensors")
    if q.stride(2) != 1 or q.stride(1) != Dqk or k_head.stride(2) != 1 or k_head.stride(1) != Dqk - tail \
            or v.stride(2) != 1 or v.stride(1) != Dv or k_tail.stride(1) != 1:
        raise ValueError("heads must be contiguous")
    if out is None:
        out = torch.empty((Tq, H, Dv), dtype=q.dtype, device=q.device)
    elif out.shape != (Tq, H, Dv) or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous [Tq, H, Dv] tensor")
    check(lib.b200_prefill_varlen_shared_tail(
        q.data_ptr(), k_head.data_ptr(), k_tail.data_ptr(), v.data_ptr(), out.data_ptr(), q.stride(0),
        k_head.stride(0), k_tail.stride(0), v.stride(0), Tq, Tk, cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(),
        cu_seqlens_q.numel() - 1, int(max_seqlen_q), H, Dqk, tail, Dv, float(scale),
        plan.buffer.data_ptr() if plan is not None else None, plan.tile_rows if plan is not None else 0,
        plan.capacity if plan is not None else 0, _dt(q), status_word(dev).data_ptr(), _stream()),
        "prefill_varlen_shared_tail")
    return out


class PrefillPlan:
    """Device-side tile list shared by all prefill attention calls of one step (``prefill_plan``)."""

    __slots__ = ("buffer", "tile_rows", "capacity")

    def __init__(self, buffer: torch.Tensor, tile_rows: int, capacity: int):
        self.buffer, self.tile_rows, self.capacity = buffer, tile_rows, capacity


def prefill_tile_rows(Hq: int, Hkv: int, Dqk: int, Dv: int, dtype: torch.dtype) -> int:
    """Query rows per tile of the prefill kernel serving this shape; 0 = no tiled kernel (no plan)."""
    if dtype not in _DTYPES:
        return 0
    return int(lib.b200_prefill_tile_rows(Hq, Hkv, Dqk, Dv, _DTYPES[dtype]))


def prefill_plan(cu_seqlens_q: torch.Tensor, total_q_tokens: int, max_seqlen_q: int, tile_rows: int,
                 buffer: torch.Tensor | None = None) -> PrefillPlan | None:
    """Builds the tile list of a prefill step on the device (one small launch).  ``total_q_tokens`` and
    ``max_seqlen_q`` are host-side upper bounds; ``buffer`` (int32) may be supplied to keep the plan
    at a fixed address (graph capture).  Returns None when no tiled kernel applies (tile_rows == 0)."""
    if tile_rows <= 0:
        return None
    dev = _cuda(cu_seqlens_q, buffer)
    if cu_seqlens_q.dtype != torch.int32:
        raise ValueError("cu_seqlens must be int32")
    num_seqs = cu_seqlens_q.numel() - 1
    nbytes = int(lib.b200_prefill_plan_bytes(total_q_tokens, num_seqs, tile_rows))
    if buffer is None:
        buffer = torch.empty(nbytes // 4, dtype=torch.int32, device=dev)
    elif buffer.dtype != torch.int32 or buffer.numel() * 4 < nbytes or not buffer.is_contiguous():
        raise ValueError(f"plan buffer must be contiguous int32 with at least {nbytes // 4} entries")
    check(lib.b200_prefill_plan(cu_seqlens_q.data_ptr(), num_seqs, int(max_seqlen_q), tile_rows, buffer.data_ptr(),
                                buffer.numel() * 4, status_word(dev).data_ptr(), _stream()), "prefill_plan")
    return PrefillPlan(buffer, tile_rows, buffer.numel() - 4)


def mla_decode(q_abs: torch.Tensor, q_rope: torch.Tensor, latent_cache: torch.Tensor,
               block_tables: torch.Tensor, context_lens: torch.Tensor, scale: float,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """Absorbed MLA decode over a paged latent pool.

    q_abs: [B, H, r]; q_rope: [B, H, dr]; latent_cache: [num_blocks, block_size, r + dr];
    returns the attention-weighted latent [B, H, r].
    """
    dev = _cuda(q_abs, q_rope, latent_cache, block_tables, context_lens, out)
    B, H, r = q_abs.shape
    dr = q_rope.shape[2]
    nb, bs, row = latent_cache.shape
    if row != r + dr or q_rope.shape[:2] != (B, H):
        raise ValueError("latent row must be kv_lora_rank + rope_dim wide")
    if latent_cache.dtype != q_abs.dtype or q_rope.dtype != q_abs.dtype:
        raise ValueError("dtype mismatch")
    if block_tables.dtype != torch.int32 or context_lens.dtype != torch.int64:
        raise ValueError("block_tables must be int32 and context_lens int64")
    if block_tables.shape[0] != B or block_tables.stride(1) != 1 or context_lens.numel() != B:
        raise ValueError("metadata batch mismatch")
    if not (q_abs.is_contiguous() and q_rope.is_contiguous() and latent_cache.is_contiguous()):
        raise ValueError("inputs must be contiguous")
    if out is None:
        out = torch.empty_like(q_abs)
    need = lib.b200_mla_decode_workspace_bytes(B, H, r, dr, _dt(q_abs))
    ws = workspace(dev, need, "mla")
    check(lib.b200_mla_decode(q_abs.data_ptr(), q_rope.data_ptr(), latent_cache.data_ptr(),
                              out.data_ptr(), block_tables.data_ptr(), block_tables.stride(0),
                              context_lens.data_ptr(), B, H, r, dr, bs, nb, float(scale),
                              ws.data_ptr(), ws.numel(), _dt(q_abs), status_word(dev).data_ptr(),
                              _stream()), "mla_decode")
    return out


def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """RMSNorm of x (+ residual) in fp32, result in x's dtype.  Returns y, or (y, new_residual) when a
    residual is given (the fused add + norm of the reference's residual stream)."""
    _cuda(x, weight, residual)
    if not x.is_contiguous() or weight.dtype != torch.float32 or weight.numel() != x.shape[-1]:
        raise ValueError("x must be contiguous and weight an fp32 vector of the row width")
    if residual is not None and (residual.shape != x.shape or not residual.is_contiguous()):
        raise ValueError("residual must match x")
    rows, dim = x.numel() // x.shape[-1], x.shape[-1]
    y = torch.empty_like(x)
    res_out = torch.empty_like(x) if residual is not None else None
    check(lib.b200_add_rmsnorm(x.data_ptr(), residual.data_ptr() if residual is not None else None,
                               weight.data_ptr(), y.data_ptr(), res_out.data_ptr() if res_out is not None else None,
                               rows, dim, float(eps), _dt(x), _dt(residual) if residual is not None else 0,
                               _stream()), "add_rmsnorm")
    return y if residual is None else (y, res_out)


def qk_norm_rope_store(qkv: torch.Tensor, q_norm_w: torch.Tensor, k_norm_w: torch.Tensor, rope_table: torch.Tensor,
                       positions: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int,
                       k_cache: torch.Tensor | None, v_cache: torch.Tensor | None,
                       slot_mapping: torch.Tensor | None):
    """q/k RMSNorm over the whole projected vectors + RoPE + scatter of K/V into the paged cache.

    qkv: [T, (Hq + 2 Hkv) * D] fused projection output; returns (q [T,Hq,D], k [T,Hkv,D], v view [T,Hkv,D]).
    """
    dev = _cuda(qkv, q_norm_w, k_norm_w, rope_table, positions, k_cache, v_cache, slot_mapping)
    T = qkv.shape[0]
    wq, wk = num_q_heads * head_dim, num_kv_heads * head_dim
    if qkv.shape[1] != wq + 2 * wk or qkv.stride(1) != 1:
        raise ValueError("qkv must be [T, (Hq + 2 Hkv) * D] with contiguous rows")
    if positions.dtype != torch.int64 or positions.numel() != T or not positions.is_contiguous():
        raise ValueError("positions must be a contiguous int64 [T] tensor")
    if rope_table.dtype != torch.float32 or rope_table.shape[1] != head_dim or not rope_table.is_contiguous():
        raise ValueError("rope_table must be fp32 [positions, head_dim]")
    use_cache = k_cache is not None and k_cache.numel() > 0
    if use_cache and (slot_mapping is None or slot_mapping.dtype != torch.int64 or slot_mapping.numel() != T):
        raise ValueError("slot_mapping must be int64 [T]")
    q = torch.empty(T, num_q_heads, head_dim, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(T, num_kv_heads, head_dim, dtype=qkv.dtype, device=qkv.device)
    eps = VECTOR_NORM_EPS
    check(lib.b200_qk_norm_rope_store(
        qkv.data_ptr(), qkv.stride(0), q_norm_w.data_ptr(), k_norm_w.data_ptr(), rope_table.data_ptr(),
        rope_table.shape[0], positions.data_ptr(), q.data_ptr(), k.data_ptr(),
        k_cache.data_ptr() if use_cache else None, v_cache.data_ptr() if use_cache else None,
        slot_mapping.data_ptr() if use_cache else None, (k_cache.numel() // wk) if use_cache else 0, T,
        num_q_heads, num_kv_heads, head_dim, float(eps), _dt(qkv), status_word(dev).data_ptr(), _stream()),
        "qk_norm_rope_store")
    v = qkv[:, wq + wk:].view(T, num_kv_heads, head_dim)
    return q, k, v


def mla_prologue_supported(head_dim: int, rope_dim: int, kv_lora_rank: int, dtype: torch.dtype) -> bool:
    """Shapes the fused MLA pre-attention kernel takes (16-byte chunks everywhere, a rotation partner a whole
    number of lanes away); other shapes run the same stage as separate tensor operations on the device."""
    rpc = rope_dim // 8
    return (dtype == torch.bfloat16 and head_dim % 8 == 0 and rope_dim % 16 == 0 and kv_lora_rank % 8 == 0
            and rpc & (rpc - 1) == 0 and rpc <= 32)


def mla_prologue(q_up: torch.Tensor, kv_down: torch.Tensor, kv_norm_w: torch.Tensor, rope_table: torch.Tensor,
                 positions: torch.Tensor, num_heads: int, head_dim: int, rope_dim: int, kv_lora_rank: int,
                 latent_cache: torch.Tensor | None = None, slot_mapping: torch.Tensor | None = None):
    """MLA stage between the projections and the attention: q = [q_nope | RoPE(q_rope)] per head and the
    latent row [kv_norm(c) | RoPE(k_rope)], also scattered into the paged latent cache.

    q_up: [T, H*head_dim + H*rope_dim]; kv_down: [T, kv_lora_rank + rope_dim]; bf16.
    Returns (q [T, H, head_dim + rope_dim], rows [T, kv_lora_rank + rope_dim]).
    """
    dev = _cuda(q_up, kv_down, kv_norm_w, rope_table, positions, latent_cache, slot_mapping)
    T = q_up.shape[0]
    if q_up.dtype != torch.bfloat16 or kv_down.dtype != torch.bfloat16:
        raise ValueError("mla_prologue takes bf16 projections")
    if q_up.shape[1] != num_heads * (head_dim + rope_dim) or q_up.stride(1) != 1:
        raise ValueError("q_up must be [T, H*(head_dim + rope_dim)] with contiguous rows")
    if kv_down.shape != (T, kv_lora_rank + rope_dim) or kv_down.stride(1) != 1:
        raise ValueError("kv_down must be [T, kv_lora_rank + rope_dim] with contiguous rows")
    if positions.dtype != torch.int64 or positions.numel() != T or not positions.is_contiguous():
        raise ValueError("positions must be a contiguous int64 [T] tensor")
    if rope_table.dtype != torch.float32 or not rope_table.is_contiguous() or rope_table.dim() != 2:
        raise ValueError("rope_table must be a contiguous fp32 [positions, width] tensor")
    if kv_norm_w.dtype != torch.float32 or kv_norm_w.numel() != kv_lora_rank:
        raise ValueError("kv_norm_w must be fp32 [kv_lora_rank]")
    use_cache = latent_cache is not None and latent_cache.numel() > 0
    if use_cache:
        if latent_cache.dtype != torch.bfloat16 or latent_cache.shape[-1] != kv_lora_rank + rope_dim \
                or not latent_cache.is_contiguous():
            raise ValueError("latent_cache must be contiguous bf16 [..., kv_lora_rank + rope_dim]")
        if slot_mapping is None or slot_mapping.dtype != torch.int64 or slot_mapping.numel() != T:
            raise ValueError("slot_mapping must be int64 [T]")
    q = torch.empty(T, num_heads, head_dim + rope_dim, dtype=q_up.dtype, device=q_up.device)
    rows = torch.empty(T, kv_lora_rank + rope_dim, dtype=q_up.dtype, device=q_up.device)
    check(lib.b200_mla_prologue(
        q_up.data_ptr(), q_up.stride(0), kv_down.data_ptr(), kv_down.stride(0), kv_norm_w.data_ptr(),
        rope_table.data_ptr(), rope_table.shape[1], rope_table.shape[0], positions.data_ptr(), q.data_ptr(),
        rows.data_ptr(), latent_cache.data_ptr() if use_cache else None,
        slot_mapping.data_ptr() if use_cache else None,
        (latent_cache.numel() // (kv_lora_rank + rope_dim)) if use_cache else 0, T, num_heads, head_dim, rope_dim,
        kv_lora_rank, VECTOR_NORM_EPS, _dt(q_up), status_word(dev).data_ptr(), _stream()),
        "mla_prologue")
    return q, rows


MOE_ROUTE_MAX_EXPERTS, MOE_ROUTE_MAX_TOPK, MOE_ROUTE_MAX_TOKENS = 64, 8, 65536
MOE_GEMM_EARLY_LAUNCH = 0x100   # B200_MOE_GEMM_EARLY_LAUNCH


def moe_route(gate_logits: torch.Tensor, expert_bias: torch.Tensor, top_k: int, identity_tail: bool = False):
    """Top-k routing + grouping by expert.  Returns (sorted_token, sorted_expert, sorted_weight,
    expert_offsets, slot_to_row); see ``b200_moe_route`` in the header for the layout.  With
    ``identity_tail`` sorted_token has T more entries 0..T-1 at its end (rows of a shared expert)."""
    _cuda(gate_logits, expert_bias)
    T, E = gate_logits.shape
    if not gate_logits.is_contiguous() or expert_bias.dtype != torch.float32 or expert_bias.numel() != E:
        raise ValueError("gate_logits must be contiguous [T, E] and expert_bias fp32 [E]")
    dev, n = gate_logits.device, T * top_k
    tok = torch.empty(n + (T if identity_tail else 0), dtype=torch.int32, device=dev)
    exp = torch.empty(n, dtype=torch.int32, device=dev)
    w = torch.empty(n, dtype=gate_logits.dtype, device=dev)
    offs = torch.empty(E, dtype=torch.int32, device=dev)
    inv = torch.empty(T, top_k, dtype=torch.int32, device=dev)
    need = int(lib.b200_moe_route_workspace_bytes(T, E))
    ws = workspace(dev, need, "moe_route") if need else None
    check(lib.b200_moe_route(gate_logits.data_ptr(), expert_bias.data_ptr(), T, E, top_k, tok.data_ptr(),
                             exp.data_ptr(), w.data_ptr(), offs.data_ptr(), inv.data_ptr(), 1 if identity_tail else 0,
                             ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                             _dt(gate_logits), _stream()), "moe_route")
    return tok, exp, w, offs, inv


MOE_GATE_ROUTE_MAX_TOKENS = 256
MOE_GATE_ROUTE_MAX_GATE_BYTES = 160 * 1024
MOE_GATE_ROUTE_GATHER_MAX_TOKENS = 32   # up to here the routing launch also copies the routed rows


def moe_gate_route(x: torch.Tensor, gate_w: torch.Tensor, expert_bias: torch.Tensor, top_k: int,
                   identity_tail: bool = False, gather: bool = False):
    """Gate projection + ``moe_route`` in one launch for at most 256 bf16 tokens.  Returns (sorted_token,
    sorted_expert, sorted_weight, expert_offsets, slot_to_row, gathered): ``gathered`` is x[sorted_token]
    when ``gather`` is set (meant for small batches: one thread block copies the rows), else None."""
    dev = _cuda(x, gate_w, expert_bias)
    T, d = x.shape
    E = gate_w.shape[0]
    if x.dtype != torch.bfloat16 or gate_w.dtype != torch.bfloat16 or not x.is_contiguous() \
            or not gate_w.is_contiguous() or gate_w.shape[1] != d:
        raise ValueError("x [T, d] and gate_w [E, d] must be contiguous bfloat16")
    if expert_bias.dtype != torch.float32 or expert_bias.numel() != E:
        raise ValueError("expert_bias must be fp32 [E]")
    n = T * top_k
    rows = n + (T if identity_tail else 0)
    tok = torch.empty(rows, dtype=torch.int32, device=dev)
    exp = torch.empty(n, dtype=torch.int32, device=dev)
    w = torch.empty(n, dtype=x.dtype, device=dev)
    offs = torch.empty(E, dtype=torch.int32, device=dev)
    inv = torch.empty(T, top_k, dtype=torch.int32, device=dev)
    xs = torch.empty(rows, d, dtype=x.dtype, device=dev) if gather else None
    ws = workspace(dev, int(lib.b200_moe_gate_route_workspace_bytes()), "moe_gate_route")
    check(lib.b200_moe_gate_route(x.data_ptr(), gate_w.data_ptr(), expert_bias.data_ptr(), T, E, top_k, d,
                                  tok.data_ptr(), exp.data_ptr(), w.data_ptr(), offs.data_ptr(), inv.data_ptr(),
                                  1 if identity_tail else 0, xs.data_ptr() if xs is not None else None,
                                  ws.data_ptr(), ws.numel(), _dt(x), _stream()), "moe_gate_route")
    return tok, exp, w, offs, inv, xs


def swiglu(h: torch.Tensor, bias: torch.Tensor | None = None, row_expert: torch.Tensor | None = None):
    """act = silu(h[:, :F] + b1) * (h[:, F:] + b3) for h [rows, 2F]; ``bias`` [experts, 2F] is indexed by
    ``row_expert`` [rows] int32 (row 0 without it); every intermediate is rounded to the dtype."""
    _cuda(h, bias, row_expert)
    rows, F2 = h.shape
    if not h.is_contiguous() or F2 % 2:
        raise ValueError("h must be contiguous [rows, 2*d_ff]")
    if bias is not None and (bias.dtype != h.dtype or not bias.is_contiguous() or bias.shape[-1] != F2):
        raise ValueError("bias must be contiguous [experts, 2*d_ff] in the dtype of h")
    if row_expert is not None and (row_expert.dtype != torch.int32 or row_expert.numel() != rows):
        raise ValueError("row_expert must be int32 [rows]")
    act = torch.empty(rows, F2 // 2, dtype=h.dtype, device=h.device)
    check(lib.b200_swiglu(h.data_ptr(), bias.data_ptr() if bias is not None else None,
                          row_expert.data_ptr() if row_expert is not None else None, act.data_ptr(), rows,
                          F2 // 2, _dt(h), _stream()), "swiglu")
    return act


def moe_grouped_gemm(x: torch.Tensor, w: torch.Tensor, expert_offsets: torch.Tensor,
                     bias: torch.Tensor | None = None, swiglu: bool = False, dense_rows: int = 0,
                     early_launch: bool = False) -> torch.Tensor:
    """Rows of x [R, k] grouped by expert (expert_offsets int32 [E], exclusive ends) times the expert's
    weight: w [E, n, k] -> [R, n]; with ``swiglu`` w is [E, 2*d_ff, k] = [w1 | w3], bias [E, 2*d_ff],
    and the result is silu(x w1^T + b1) * (x w3^T + b3) [R, d_ff].  bf16, tcgen05 tensor cores.
    ``dense_rows`` > 0: the last rows of x are not grouped and all use one more weight set, w[E] (w and
    bias then have E + 1 sets): a shared expert in the same launch."""
    _cuda(x, w, expert_offsets, bias)
    R, k = x.shape
    E, n, k2 = w.shape
    if dense_rows:
        E -= 1
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_contiguous() or not w.is_contiguous():
        raise ValueError("x and w must be contiguous bfloat16")
    if k2 != k or expert_offsets.dtype != torch.int32 or expert_offsets.numel() != E or (swiglu and n % 2):
        raise ValueError("w must be [E, n, k] with k = x.shape[1]; expert_offsets int32 [E]")
    n_out = n // 2 if swiglu else n
    if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_contiguous()
                             or tuple(bias.shape) != (w.shape[0], n)):
        raise ValueError("bias must be contiguous bfloat16 [weight sets, n]")
    if dense_rows < 0 or dense_rows > R or E < 1:
        raise ValueError("dense_rows must be within the rows of x and leave at least one routed expert")
    out = torch.empty(R, n_out, dtype=torch.bfloat16, device=x.device)
    check(lib.b200_moe_grouped_gemm(x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                                    out.data_ptr(), expert_offsets.data_ptr(), R, E, int(dense_rows), n_out, k,
                                    (1 if swiglu else 0) | (MOE_GEMM_EARLY_LAUNCH if early_launch else 0),
                                    _dt(x), status_word(x.device).data_ptr(), _stream()), "moe_grouped_gemm")
    return out


def lm_head_argmax_supported(hidden: torch.Tensor, w: torch.Tensor) -> bool:
    return (hidden.is_cuda and hidden.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and hidden.dim() == 2
            and hidden.shape[1] % 8 == 0 and hidden.shape[0] > 0)


def lm_head_argmax(hidden: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """Greedy tokens of hidden [R, d] under the head w [vocab, d] (+ bias [vocab]): argmax over the bf16 logits,
    first maximum, without materialising the logits.  bf16; returns int64 [R]."""
    dev = _cuda(hidden, w, bias, out)
    R, d = hidden.shape
    V = w.shape[0]
    if hidden.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not hidden.is_contiguous() \
            or not w.is_contiguous() or w.shape[1] != d:
        raise ValueError("hidden [R, d] and w [vocab, d] must be contiguous bfloat16")
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != V or not bias.is_contiguous()):
        raise ValueError("bias must be contiguous bfloat16 [vocab]")
    if out is None:
        out = torch.empty(R, dtype=torch.int64, device=hidden.device)
    elif out.dtype != torch.int64 or out.numel() != R or not out.is_contiguous():
        raise ValueError("out must be a contiguous int64 [R] tensor")
    need = lib.b200_lm_head_argmax_workspace_bytes(R, V)
    ws = workspace(dev, need, "lm_head")
    check(lib.b200_lm_head_argmax(hidden.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
                                  out.data_ptr(), R, V, d, ws.data_ptr(), ws.numel(), _dt(hidden),
                                  status_word(dev).data_ptr(), _stream()), "lm_head_argmax")
    return out


def moe_combine(expert_out: torch.Tensor, bias: torch.Tensor | None, row_expert: torch.Tensor,
                row_weight: torch.Tensor, slot_to_row: torch.Tensor, shared: torch.Tensor | None = None):
    """Weighted sum of every token's expert rows in ascending expert order (+ bias, + shared expert),
    rounding like the reference's accumulation in the activation dtype.  Returns [tokens, d]."""
    _cuda(expert_out, bias, row_expert, row_weight, slot_to_row, shared)
    T, K = slot_to_row.shape
    rows, d = expert_out.shape
    if rows != T * K or not expert_out.is_contiguous() or not slot_to_row.is_contiguous():
        raise ValueError("expert_out must be contiguous [tokens*top_k, d] and slot_to_row [tokens, top_k]")
    if row_weight.dtype != expert_out.dtype or row_weight.numel() != rows or row_expert.dtype != torch.int32:
        raise ValueError("row_weight must match expert_out's dtype, row_expert must be int32, both [rows]")
    if slot_to_row.dtype != torch.int32:
        raise ValueError("slot_to_row must be int32")
    for name, t, shape in (("bias", bias, None), ("shared", shared, (T, d))):
        if t is not None and (t.dtype != expert_out.dtype or not t.is_contiguous() or t.shape[-1] != d
                              or (shape is not None and tuple(t.shape) != shape)):
            raise ValueError(f"{name} must be contiguous [..., {d}] in the dtype of expert_out")
    out = torch.empty(T, d, dtype=expert_out.dtype, device=expert_out.device)
    check(lib.b200_moe_combine(expert_out.data_ptr(), bias.data_ptr() if bias is not None else None,
                               row_expert.data_ptr(), row_weight.data_ptr(), slot_to_row.data_ptr(),
                               shared.data_ptr() if shared is not None else None, out.data_ptr(), T, K, d,
                               _dt(expert_out), _stream()), "moe_combine")
    return out


def block_hash(token_ids, prefix: int = -1) -> int:
    """Chained XXH64 block hash; same value as BlockManager.compute_hash of the reference."""
    buf = array.array("i", token_ids)
    addr, n = buf.buffer_info()
    return int(lib.b200_block_hash(addr, n, 0 if prefix == -1 else prefix, 0 if prefix == -1 else 1))


def decode_advance(sampled: torch.Tensor, input_ids: torch.Tensor, context_lens: torch.Tensor,
                   slot_mapping: torch.Tensor, block_tables: torch.Tensor, block_size: int, num_blocks: int,
                   history: torch.Tensor | None = None) -> None:
    """Turns the decode inputs of the step that just sampled ``sampled`` into those of the next step, in
    place and on the device: input id = sampled token, context length + 1, slot of the new position from
    the block table (which must already list that block).  ``history`` [n] also receives the tokens."""
    dev = _cuda(sampled, input_ids, context_lens, slot_mapping, block_tables, history)
    n = sampled.numel()
    for t in (sampled, input_ids, context_lens, slot_mapping) + ((history,) if history is not None else ()):
        if t.dtype != torch.int64 or t.numel() < n or not t.is_contiguous():
            raise ValueError("sampled, input_ids, context_lens, slot_mapping, history must be contiguous int64 [n]")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.shape[0] < n \
            or block_tables.stride(1) != 1:
        raise ValueError("block_tables must be int32 [n, max_blocks]")
    check(lib.b200_decode_advance(sampled.data_ptr(), input_ids.data_ptr(), context_lens.data_ptr(),
                                  slot_mapping.data_ptr(), block_tables.data_ptr(), block_tables.stride(0),
                                  int(block_size), int(num_blocks), n,
                                  history.data_ptr() if history is not None else None,
                                  status_word(dev).data_ptr(), _stream()), "decode_advance")


def block_table_patch(patches: torch.Tensor, count: int, block_tables: torch.Tensor) -> None:
    """Writes the first ``count`` (row, column, block id) int32 triples of ``patches`` into ``block_tables``
    [rows, max_blocks] on the device (incremental update of a device-resident table)."""
    if count <= 0:
        return
    dev = _cuda(patches, block_tables)
    if patches.dtype != torch.int32 or not patches.is_contiguous() or patches.numel() < 3 * count:
        raise ValueError("patches must be a contiguous int32 tensor of at least 3 * count elements")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.stride(1) != 1:
        raise ValueError("block_tables must be int32 [rows, max_blocks]")
    check(lib.b200_block_table_patch(patches.data_ptr(), int(count), block_tables.data_ptr(), block_tables.stride(0),
                                     block_tables.shape[0], status_word(dev).data_ptr(), _stream()),
          "block_table_patch")


def block_hash_chain(token_ids, block_size: int) -> list[int]:
    """Chained XXH64 hashes of every full block of ``token_ids`` in one native call: element i is what
    ``block_hash(block i, prefix = element i-1)`` returns."""
    buf = array.array("i", token_ids)
    addr, n = buf.buffer_info()
    out = array.array("Q", bytes(8 * (n // block_size)))
    got = int(lib.b200_block_hash_chain(addr, n, block_size, out.buffer_info()[0]))
    if got != len(out):
        raise RuntimeError("b200_block_hash_chain failed")
    return out.tolist()


def sample(logits: torch.Tensor, temperatures: torch.Tensor | None, seed: int, offset: int,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of ``logits`` [B, V]: greedy where the temperature is <= 0 (or ``temperatures`` is
    None), else a draw from softmax(logits / T).  ``seed`` / ``offset`` select the random stream."""
    _cuda(logits, temperatures, out)
    B, V = logits.shape
    if logits.stride(1) != 1:
        raise ValueError("logits rows must be contiguous")
    if temperatures is not None and (temperatures.dtype != torch.float32 or temperatures.numel() != B
                                     or not temperatures.is_contiguous()):
        raise ValueError("temperatures must be contiguous float32 [B]")
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=logits.device)
    elif out.dtype != torch.int64 or out.numel() != B or not out.is_contiguous():
        raise ValueError("out must be contiguous int64 [B]")
    check(lib.b200_sample(logits.data_ptr(), logits.stride(0), temperatures.data_ptr() if temperatures is not None
                          else None, B, V, seed & 0xFFFFFFFFFFFFFFFF, offset & 0xFFFFFFFFFFFFFFFF, out.data_ptr(),
                          _dt(logits), _stream()), "sample")
    return out
