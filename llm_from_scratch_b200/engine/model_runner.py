"""Runs one scheduled batch on the GPU (reference: engine/model_runner.py).

Keeps the reference's method names — ``allocate_kv_cache``, ``prepare_prefill``,
``prepare_decode``, ``prepare_sample``, ``run_model``, ``run``, ``capture_cudagraph`` — and its
conventions: the pool is one tensor ``[2, layers, num_blocks, block_size, Hkv, D]`` whose slices are
injected into every module that has ``k_cache`` and ``v_cache`` attributes (model_runner.py:184-190);
decode can be replayed from CUDA graphs captured per batch-size bucket, with ``slot_mapping``
padded with -1 and ``context_lens`` with 0 (model_runner.py:295-310).

What differs is mechanism: the step metadata is built with numpy (engine/metadata.py), packed into
one pinned staging buffer and sent with a single host-to-device copy instead of one
``torch.tensor(..., pin_memory=True).cuda()`` per field; the single-process replica design has no
shared-memory RPC, no NCCL group and no tensor-parallel workers.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..model import EngineTransformerLM, ModelConfig, init_reference_order
from ..utils.context import get_context, reset_context, set_context
from ..utils.sampler import Sampler
from . import metadata as md
from .sequence import Sequence


def _cfg(config: dict, *names, default=None):
    for n in names:
        if n in config:
            return config[n]
    return default


class _Staging:
    """One pinned host buffer + one device buffer; arrays are packed 16-byte aligned and shipped
    with a single copy, then handed out as typed views of the device buffer."""

    def __init__(self, device):
        self.device = device
        self.host = torch.empty(1 << 16, dtype=torch.uint8).pin_memory()
        self.dev = torch.empty(1 << 16, dtype=torch.uint8, device=device)

    def upload(self, arrays: dict[str, np.ndarray]) -> dict[str, torch.Tensor]:
        offs, total = {}, 0
        for name, a in arrays.items():
            offs[name] = total
            total += (a.nbytes + 15) & ~15
        if total > self.host.numel():
            size = max(total, 2 * self.host.numel())
            self.host = torch.empty(size, dtype=torch.uint8).pin_memory()
            self.dev = torch.empty(size, dtype=torch.uint8, device=self.device)
        hview = self.host.numpy()
        for name, a in arrays.items():
            hview[offs[name]:offs[name] + a.nbytes] = np.ascontiguousarray(a).view(np.uint8).reshape(-1)
        self.dev[:total].copy_(self.host[:total], non_blocking=True)
        out = {}
        for name, a in arrays.items():
            t = self.dev[offs[name]:offs[name] + a.nbytes].view(_TORCH_DTYPES[a.dtype.str])
            out[name] = t.view(*a.shape)
        return out


_TORCH_DTYPES = {np.dtype(np.int64).str: torch.int64, np.dtype(np.int32).str: torch.int32,
                 np.dtype(np.float32).str: torch.float32}


class ModelRunner:
    def __init__(self, config: dict, model: EngineTransformerLM | None = None):
        self.config = config
        self.block_size = _cfg(config, "block_size", default=256)
        self.enforce_eager = bool(_cfg(config, "enforce_eager", default=False))
        self.max_num_seqs = _cfg(config, "max_num_sequences", "max_num_seqs", default=16)
        self.max_model_length = _cfg(config, "max_model_length", default=None)
        self.device = torch.device(_cfg(config, "device", default="cuda:0"))
        # prefill batches are padded to a multiple of this many tokens (ids 0, slot -1, in no sequence):
        # the GEMM library then meets a few dozen distinct row counts instead of a new one every step,
        # and its per-shape algorithm selection (~0.1 ms per new shape per GEMM) is paid once
        self.prefill_token_multiple = int(_cfg(config, "prefill_token_multiple", default=256))
        self.max_num_batched_tokens = int(_cfg(config, "max_num_batched_tokens", "max_num_batch_tokens", default=1024))
        torch.cuda.set_device(self.device)
        dtype = _cfg(config, "dtype", default=torch.float32)
        self.dtype = getattr(torch, dtype) if isinstance(dtype, str) else dtype
        if model is None:
            mc = config["model"]
            mc = mc if isinstance(mc, ModelConfig) else ModelConfig.from_dict(mc)
            weights = _cfg(config, "weights", "model_path", default=None)
            if isinstance(weights, (str, bytes)) or hasattr(weights, "__fspath__"):
                from ..utils.loader import load_weights     # a checkpoint in one of the reference's formats
                weights = load_weights(str(weights))
            if weights is None:
                weights = init_reference_order(mc, _cfg(config, "seed", default=0))
            model = EngineTransformerLM(mc, weights, self.device, self.dtype)
        self.model = model
        self.model_config = model.cfg
        if self.max_model_length is None:
            self.max_model_length = self.model_config.context_length
        self.sampler = Sampler()
        self.staging = _Staging(self.device)
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_vars: dict[str, torch.Tensor] = {}
        self.prefill_graphs: dict[int, tuple] = {}
        self.decode_builder = None
        # sums over the decode steps replayed from graphs: sequences stepped and context tokens attended to
        # (what the decode kernels had to read), for throughput and memory-roofline reports
        self.decode_seq_steps = 0
        self.decode_ctx_tokens = 0
        c = self.model_config
        if c.attention_type == "MLA":    # prefill runs the expanded form: 192-wide keys, 128-wide values
            self.prefill_tile_rows = ops.prefill_tile_rows(c.num_heads, c.num_heads, c.head_dim + c.rope_dim,
                                                           c.head_dim, self.dtype)
        else:
            self.prefill_tile_rows = ops.prefill_tile_rows(c.num_heads, c.num_kv_heads, c.head_dim, c.head_dim,
                                                           self.dtype)
        self.allocate_kv_cache()
        if not self.enforce_eager:
            self.capture_cudagraph()
            if self.prefill_tile_rows and _cfg(config, "prefill_graphs", default=True):
                self.capture_prefill_graphs()

    # ------------------------------------------------------------------ KV pool
    def kv_block_bytes(self) -> int:
        c = self.model_config
        itemsize = torch.empty(0, dtype=self.dtype).element_size()
        if c.attention_type == "MLA":
            return self.block_size * c.num_layers * (c.kv_lora_rank + c.rope_dim) * itemsize
        return self.block_size * 2 * c.num_layers * c.num_kv_heads * c.head_dim * itemsize

    def allocate_kv_cache(self) -> None:
        """One pool for all layers; per-layer views injected into the attention modules."""
        c = self.model_config
        num_blocks = _cfg(self.config, "max_cached_blocks", "num_kv_blocks", default=None)
        if num_blocks is None:
            free, _total = torch.cuda.mem_get_info(self.device)
            util = _cfg(self.config, "gpu_memory_utilization", default=0.5)
            num_blocks = int(free * util) // self.kv_block_bytes()
        if num_blocks < 1:
            raise RuntimeError("not enough device memory for a single KV block")
        self.num_kv_blocks = int(num_blocks)
        if c.attention_type == "MLA":
            self.kv_cache = torch.zeros(c.num_layers, num_blocks, self.block_size, c.kv_lora_rank + c.rope_dim,
                                        dtype=self.dtype, device=self.device)
            for i, att in enumerate(self.model.attention_layers):
                att.latent_cache = self.kv_cache[i]
        else:
            self.kv_cache = torch.zeros(2, c.num_layers, num_blocks, self.block_size, c.num_kv_heads, c.head_dim,
                                        dtype=self.dtype, device=self.device)
            layer = 0
            for module in self.model.modules():
                if hasattr(module, "k_cache") and hasattr(module, "v_cache"):
                    module.k_cache = self.kv_cache[0, layer]
                    module.v_cache = self.kv_cache[1, layer]
                    layer += 1

    # ------------------------------------------------------------------ metadata -> device
    def _publish(self, m: md.StepMetadata) -> torch.Tensor:
        arrays = {"input_ids": m.input_ids, "slot_mapping": m.slot_mapping, "positions": m.positions}
        for name in ("cu_seqlens_q", "cu_seqlens_k", "context_lens", "block_tables"):
            a = getattr(m, name)
            if a is not None:
                arrays[name] = a
        if len(m.slot_mapping) != len(m.input_ids):
            raise RuntimeError("slot_mapping and input_ids disagree: Sequence.reference_exact must be off "
                               "when the model runs (it reproduces a reference defect at block multiples)")
        mult = self.prefill_token_multiple
        if m.is_prefill and mult > 1 and len(m.input_ids) % mult:
            pad = mult - len(m.input_ids) % mult
            arrays["input_ids"] = np.concatenate([m.input_ids, np.zeros(pad, dtype=m.input_ids.dtype)])
            arrays["positions"] = np.concatenate([m.positions, np.zeros(pad, dtype=m.positions.dtype)])
            arrays["slot_mapping"] = np.concatenate([m.slot_mapping, np.full(pad, -1, dtype=m.slot_mapping.dtype)])
        t = self.staging.upload(arrays)
        plan = None
        if m.is_prefill and self.prefill_tile_rows:
            # one tile list per step, shared by the attention calls of all layers
            plan = ops.prefill_plan(t["cu_seqlens_q"], len(arrays["input_ids"]), m.max_seqlen_q, self.prefill_tile_rows)
        set_context(m.is_prefill, t.get("cu_seqlens_q"), t.get("cu_seqlens_k"), m.max_seqlen_q, m.max_seqlen_k,
                    t["slot_mapping"], t.get("context_lens"), t.get("block_tables"), t["positions"], plan)
        return t["input_ids"]

    def prepare_prefill(self, seqs: list[Sequence]) -> torch.Tensor:
        return self._publish(md.prepare_prefill(seqs, self.block_size))

    def prepare_decode(self, seqs: list[Sequence]) -> torch.Tensor:
        return self._publish(md.prepare_decode(seqs, self.block_size))

    def prepare_sample(self, seqs: list[Sequence]) -> torch.Tensor | None:
        temps = [s.temperature for s in seqs]
        if not any(temps):
            return None   # all greedy
        return torch.tensor(temps, dtype=torch.float32).to(self.device, non_blocking=True)

    # ------------------------------------------------------------------ execution
    @torch.inference_mode()
    def run_model(self, input_ids: torch.Tensor, is_prefill: bool) -> torch.Tensor:
        bs = input_ids.size(0)
        if is_prefill or self.enforce_eager or not self.graphs or bs > max(self.graphs):
            return self.model.compute_logits(self.model(input_ids))
        ctx = get_context()
        bucket = next(b for b in sorted(self.graphs) if b >= bs)
        v = self.graph_vars
        v["input_ids"][:bs].copy_(input_ids)
        v["slot_mapping"][:bucket].fill_(-1)
        v["slot_mapping"][:bs].copy_(ctx.slot_mapping)
        v["context_lens"][:bucket].zero_()
        v["context_lens"][:bs].copy_(ctx.context_lens)
        v["block_tables"][:bs, :ctx.block_tables.size(1)].copy_(ctx.block_tables)
        self.graphs[bucket].replay()
        return self.model.compute_logits(v["outputs"][:bs])

    def run(self, seqs: list[Sequence], is_prefill: bool) -> list[int]:
        greedy = not any(s.temperature for s in seqs)
        if not is_prefill and self.graphs and not self.enforce_eager and len(seqs) <= max(self.graphs):
            hidden = self._replay_decode(seqs)
            if greedy:
                # the fused head (projection + argmax) was part of the graph; reading it is the step's only sync
                token_ids = self.graph_vars["greedy"][:len(seqs)].tolist()
                reset_context()
                return token_ids
        elif is_prefill and self.prefill_graphs and (hidden := self._replay_prefill(seqs)) is not None:
            self.decode_builder.invalidate(seqs)
        else:
            if is_prefill and self.decode_builder is not None:
                self.decode_builder.invalidate(seqs)
            input_ids = self.prepare_prefill(seqs) if is_prefill else self.prepare_decode(seqs)
            with torch.inference_mode():
                hidden = self.model(input_ids)
        with torch.inference_mode():
            if greedy:
                token_ids = self.model.greedy_tokens(hidden).tolist()
            else:
                token_ids = self.sampler(self.model.compute_logits(hidden), self.prepare_sample(seqs)).tolist()
        reset_context()
        return token_ids

    @torch.inference_mode()
    def _replay_decode(self, seqs: list[Sequence], replay: bool = True) -> torch.Tensor:
        """Decode step from a captured graph; returns the final hidden states [n, d] (the graph has also written
        the greedy tokens).  The graph's inputs live in one device buffer mirrored by
        one pinned host buffer: the step's metadata is written straight into the host mirror (padding
        rows: slot -1, context 0) and shipped with a single copy; nothing else runs before the replay."""
        n = len(seqs)
        bucket = next(b for b in sorted(self.graphs) if b >= n)
        h, v = self.graph_host_np, self.graph_vars
        # block tables live on the device: a step ships the entries that changed (one new block per sequence
        # every block_size steps) as patches behind the small arrays, or the whole table for a new batch
        patched = self.decode_builder.build(seqs, h["input_ids"], h["slot_mapping"], h["context_lens"],
                                            h["block_tables"], patches=h["patches"])
        h["slot_mapping"][n:bucket] = -1
        h["context_lens"][n:bucket] = 0
        self.decode_seq_steps += n
        self.decode_ctx_tokens += int(h["context_lens"][:n].sum())
        if patched >= 0:
            nbytes = self.graph_patches_offset + patched * 12
        else:
            nbytes = self.graph_tables_offset + bucket * h["block_tables"].shape[1] * 4
        self.graph_dev[:nbytes].copy_(self.graph_host[:nbytes], non_blocking=True)
        if patched > 0:
            ops.block_table_patch(v["patches"], patched, v["block_tables"])
        set_context(False, slot_mapping=v["slot_mapping"][:n], context_lens=v["context_lens"][:n],
                    block_tables=v["block_tables"][:n])
        if replay:
            self.graphs[bucket].replay()
        return v["outputs"][:n]

    def can_run_window(self, seqs: list[Sequence]) -> bool:
        """Whether ``run_window`` can serve this decode batch: captured graphs, all rows greedy."""
        return bool(self.graphs) and not self.enforce_eager and len(seqs) <= max(self.graphs) \
            and not any(s.temperature for s in seqs)

    @torch.inference_mode()
    def run_window(self, seqs: list[Sequence], steps: int) -> list[list[int]]:
        """``steps`` greedy decode steps back to back from the captured graph.  Between two replays a
        small kernel turns the sampled tokens into the next step's inputs (input id, context length, slot
        from the block table, which already lists the blocks opened for the window) and records them; the
        host reads all tokens once at the end.  Returns tokens[step][sequence]."""
        n = len(seqs)
        v = self.graph_vars
        self._replay_decode(seqs, replay=False)
        bucket = next(b for b in sorted(self.graphs) if b >= n)
        graph, hist = self.graphs[bucket], v["history"]
        for j in range(steps):
            graph.replay()
            if j + 1 < steps:
                ops.decode_advance(v["greedy"][:n], v["input_ids"], v["context_lens"], v["slot_mapping"],
                                   v["block_tables"], self.block_size, self.num_kv_blocks, hist[j])
            else:
                hist[j, :n].copy_(v["greedy"][:n])
        tokens = hist[:steps, :n].tolist()
        # steps after the first (counted by _replay_decode): every context is one token longer per step
        self.decode_ctx_tokens += (steps - 1) * int(self.graph_host_np["context_lens"][:n].sum()) \
            + n * steps * (steps - 1) // 2
        self.decode_seq_steps += n * (steps - 1)
        reset_context()
        return tokens

    @torch.inference_mode()
    def run_logits(self, seqs: list[Sequence], is_prefill: bool) -> torch.Tensor:
        """Like ``run`` but returns the last-token logits [num_seqs, vocab] (used by parity tests)."""
        input_ids = self.prepare_prefill(seqs) if is_prefill else self.prepare_decode(seqs)
        logits = self.run_model(input_ids, is_prefill).float().clone()
        reset_context()
        return logits

    # ------------------------------------------------------------------ CUDA graphs for prefill
    def _prefill_layout(self, tokens: int):
        """Byte offsets of (cu_seqlens, input_ids, positions, slot_mapping) of a padded prefill batch in
        the prefill staging buffer: one contiguous run, so a step is one host-to-device copy."""
        n_cu = self.max_num_seqs + 1
        o_ids = (n_cu * 4 + 15) & ~15
        return 0, o_ids, o_ids + tokens * 8, o_ids + 2 * tokens * 8, o_ids + 3 * tokens * 8

    @torch.inference_mode()
    def capture_prefill_graphs(self) -> None:
        """One graph per padded token count (multiples of ``prefill_token_multiple`` up to
        ``max_num_batched_tokens``).  The buffers have fixed sizes — cu_seqlens for ``max_num_seqs``
        sequences (unused ones have length 0), token arrays padded with slot -1 — and the attention
        grid comes from the step's tile list, so nothing in the launch sequence depends on the batch."""
        mult = max(self.prefill_token_multiple, 1)
        buckets = list(range(mult, self.max_num_batched_tokens + 1, mult))
        if not buckets or len(buckets) > 64:
            return
        dev, tmax, n_cu = self.device, buckets[-1], self.max_num_seqs + 1
        total = self._prefill_layout(tmax)[-1]
        self.prefill_dev = torch.zeros(total, dtype=torch.uint8, device=dev)
        self.prefill_host = torch.zeros(total, dtype=torch.uint8).pin_memory()
        self.prefill_out = torch.zeros(tmax, self.model_config.d_model, dtype=self.dtype, device=dev)
        plan_entries = ops.lib.b200_prefill_plan_bytes(tmax, self.max_num_seqs, self.prefill_tile_rows) // 4
        self.prefill_plan_buffer = torch.zeros(plan_entries, dtype=torch.int32, device=dev)
        pool = self.graphs[max(self.graphs)].pool() if self.graphs else None
        for tokens in reversed(buckets):
            o_cu, o_ids, o_pos, o_slot, _end = self._prefill_layout(tokens)
            view = lambda off, n, dt: self.prefill_dev[off:off + n * dt.itemsize].view(dt)
            cu = view(o_cu, n_cu, torch.int32)
            ids, pos, slots = (view(o, tokens, torch.int64) for o in (o_ids, o_pos, o_slot))
            slots.fill_(-1)
            cu.zero_()

            def body():
                plan = ops.prefill_plan(cu, tokens, tokens, self.prefill_tile_rows, buffer=self.prefill_plan_buffer)
                set_context(True, cu, cu, tokens, tokens, slots, None, None, pos, plan)
                self.prefill_out[:tokens] = self.model(ids)

            body()                                   # warm-up: allocates workspaces, selects GEMM algorithms
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool):
                body()
            if pool is None:
                pool = g.pool()
            self.prefill_graphs[tokens] = (g, cu, ids, pos, slots)
            torch.cuda.synchronize()
            reset_context()

    @torch.inference_mode()
    def _replay_prefill(self, seqs: list[Sequence]):
        """Prefill step from a captured graph: the hidden states of the padded batch (the context is left set for
        the head), or None when the batch does not fit one (a cached
        prefix, which needs block tables, or more tokens / sequences than were captured)."""
        if len(seqs) > self.max_num_seqs:
            return None
        m = md.prepare_prefill(seqs, self.block_size)
        if m.block_tables is not None:
            return None
        T, n = len(m.input_ids), len(seqs)
        if len(m.slot_mapping) != T:
            raise RuntimeError("slot_mapping and input_ids disagree: Sequence.reference_exact must be off "
                               "when the model runs (it reproduces a reference defect at block multiples)")
        mult = self.prefill_token_multiple
        tokens = max((T + mult - 1) // mult * mult, mult)
        entry = self.prefill_graphs.get(tokens)
        if entry is None:
            return None
        g, cu, ids, pos, slots = entry
        o_cu, o_ids, o_pos, o_slot, end = self._prefill_layout(tokens)
        hb = self.prefill_host.numpy()
        h_cu = hb[o_cu:o_cu + (self.max_num_seqs + 1) * 4].view(np.int32)
        h_ids, h_pos, h_slot = (hb[o:o + tokens * 8].view(np.int64) for o in (o_ids, o_pos, o_slot))
        h_cu[:n + 1] = m.cu_seqlens_q
        h_cu[n + 1:] = T
        h_ids[:T] = m.input_ids
        h_ids[T:] = 0
        h_pos[:T] = m.positions
        h_pos[T:] = 0
        h_slot[:T] = m.slot_mapping
        h_slot[T:] = -1
        self.prefill_dev[:end].copy_(self.prefill_host[:end], non_blocking=True)
        g.replay()
        set_context(True, cu[:n + 1], cu[:n + 1], m.max_seqlen_q, m.max_seqlen_k, slots, None, None, pos)
        return self.prefill_out[:tokens]

    # ------------------------------------------------------------------ CUDA graphs for decode
    @torch.inference_mode()
    def capture_cudagraph(self) -> None:
        max_bs = min(self.max_num_seqs, 512)
        max_blocks = (self.max_model_length + self.block_size - 1) // self.block_size
        dev = self.device
        # all graph inputs in one device buffer with a pinned host mirror (block tables last, so that a
        # step copies only the prefix its batch bucket uses)
        fields = (("input_ids", np.int64, torch.int64, (max_bs,)), ("slot_mapping", np.int64, torch.int64, (max_bs,)),
                  ("context_lens", np.int64, torch.int64, (max_bs,)),
                  ("patches", np.int32, torch.int32, (8 * max_bs, 3)),
                  ("block_tables", np.int32, torch.int32, (max_bs, max_blocks)))
        offsets, total = {}, 0
        for name, npdt, _, shape in fields:
            offsets[name] = total
            total += (int(np.prod(shape)) * np.dtype(npdt).itemsize + 15) & ~15
        self.graph_dev = torch.zeros(total, dtype=torch.uint8, device=dev)
        self.graph_host = torch.zeros(total, dtype=torch.uint8).pin_memory()
        self.graph_tables_offset = offsets["block_tables"]
        self.graph_patches_offset = offsets["patches"]
        host_bytes = self.graph_host.numpy()
        v, self.graph_host_np = {}, {}
        for name, npdt, tdt, shape in fields:
            nbytes = int(np.prod(shape)) * np.dtype(npdt).itemsize
            v[name] = self.graph_dev[offsets[name]:offsets[name] + nbytes].view(tdt).view(*shape)
            self.graph_host_np[name] = host_bytes[offsets[name]:offsets[name] + nbytes].view(npdt).reshape(shape)
        v["slot_mapping"].fill_(-1)
        self.graph_host_np["slot_mapping"][:] = -1
        self.decode_builder = md.DecodeBatchBuilder(self.block_size, max_blocks, rows=4 * max_bs, device_rows=max_bs)
        v["outputs"] = torch.zeros(max_bs, self.model_config.d_model, dtype=self.dtype, device=dev)
        # the graph also holds the greedy head (lm_head projection fused with the argmax), so a greedy step
        # launches nothing else; rows with a temperature take their logits from "outputs" after the replay
        v["greedy"] = torch.zeros(max_bs, dtype=torch.int64, device=dev)
        v["history"] = torch.zeros(self.block_size, max_bs, dtype=torch.int64, device=dev)   # run_window: tokens per step
        buckets = [b for b in (1, 2, 4, 8) if b <= max_bs] + list(range(16, max_bs + 1, 16))
        if max_bs not in buckets:
            buckets.append(max_bs)
        pool = None
        for b in reversed(buckets):
            # a padded row decodes position 0 of an empty context: its output row is never read
            set_context(False, slot_mapping=v["slot_mapping"][:b], context_lens=v["context_lens"][:b],
                        block_tables=v["block_tables"][:b])
            positions = (v["context_lens"][:b] - 1).clamp_min(0)
            v["outputs"][:b] = self.model(v["input_ids"][:b], positions)       # warm-up, allocates workspaces
            self.model.greedy_tokens(v["outputs"][:b], out=v["greedy"][:b])
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool):
                positions = (v["context_lens"][:b] - 1).clamp_min(0)
                v["outputs"][:b] = self.model(v["input_ids"][:b], positions)
                self.model.greedy_tokens(v["outputs"][:b], out=v["greedy"][:b])
            if pool is None:
                pool = g.pool()
            self.graphs[b] = g
            torch.cuda.synchronize()
            reset_context()
        self.graph_vars = v

    def exit(self) -> None:
        self.graphs.clear()
        self.graph_vars.clear()
        self.prefill_graphs.clear()
        torch.cuda.synchronize()
