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
        torch.cuda.set_device(self.device)
        dtype = _cfg(config, "dtype", default=torch.float32)
        self.dtype = getattr(torch, dtype) if isinstance(dtype, str) else dtype
        if model is None:
            mc = config["model"]
            mc = mc if isinstance(mc, ModelConfig) else ModelConfig.from_dict(mc)
            weights = _cfg(config, "weights", default=None) or init_reference_order(mc, _cfg(config, "seed", default=0))
            model = EngineTransformerLM(mc, weights, self.device, self.dtype)
        self.model = model
        self.model_config = model.cfg
        if self.max_model_length is None:
            self.max_model_length = self.model_config.context_length
        self.sampler = Sampler()
        self.staging = _Staging(self.device)
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.graph_vars: dict[str, torch.Tensor] = {}
        self.allocate_kv_cache()
        if not self.enforce_eager:
            self.capture_cudagraph()

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
        set_context(m.is_prefill, t.get("cu_seqlens_q"), t.get("cu_seqlens_k"), m.max_seqlen_q, m.max_seqlen_k,
                    t["slot_mapping"], t.get("context_lens"), t.get("block_tables"), t["positions"])
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
        if not is_prefill and self.graphs and not self.enforce_eager and len(seqs) <= max(self.graphs):
            logits = self._replay_decode(seqs)
        else:
            input_ids = self.prepare_prefill(seqs) if is_prefill else self.prepare_decode(seqs)
            logits = self.run_model(input_ids, is_prefill)
        with torch.inference_mode():
            token_ids = self.sampler(logits, self.prepare_sample(seqs)).tolist()
        reset_context()
        return token_ids

    @torch.inference_mode()
    def _replay_decode(self, seqs: list[Sequence]) -> torch.Tensor:
        """Decode step from a captured graph.  The graph's inputs live in one device buffer mirrored by
        one pinned host buffer: the step's metadata is written straight into the host mirror (padding
        rows: slot -1, context 0) and shipped with a single copy; nothing else runs before the replay."""
        n = len(seqs)
        bucket = next(b for b in sorted(self.graphs) if b >= n)
        h, v = self.graph_host_np, self.graph_vars
        m = md.prepare_decode(seqs, self.block_size, tables_out=h["block_tables"])
        h["input_ids"][:n] = m.input_ids
        h["slot_mapping"][:n] = m.slot_mapping
        h["slot_mapping"][n:bucket] = -1
        h["context_lens"][:n] = m.context_lens
        h["context_lens"][n:bucket] = 0
        nbytes = self.graph_tables_offset + bucket * h["block_tables"].shape[1] * 4
        self.graph_dev[:nbytes].copy_(self.graph_host[:nbytes], non_blocking=True)
        set_context(False, slot_mapping=v["slot_mapping"][:n], context_lens=v["context_lens"][:n],
                    block_tables=v["block_tables"][:n])
        self.graphs[bucket].replay()
        return self.model.compute_logits(v["outputs"][:n])

    @torch.inference_mode()
    def run_logits(self, seqs: list[Sequence], is_prefill: bool) -> torch.Tensor:
        """Like ``run`` but returns the last-token logits [num_seqs, vocab] (used by parity tests)."""
        input_ids = self.prepare_prefill(seqs) if is_prefill else self.prepare_decode(seqs)
        logits = self.run_model(input_ids, is_prefill).float().clone()
        reset_context()
        return logits

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
                  ("block_tables", np.int32, torch.int32, (max_bs, max_blocks)))
        offsets, total = {}, 0
        for name, npdt, _, shape in fields:
            offsets[name] = total
            total += (int(np.prod(shape)) * np.dtype(npdt).itemsize + 15) & ~15
        self.graph_dev = torch.zeros(total, dtype=torch.uint8, device=dev)
        self.graph_host = torch.zeros(total, dtype=torch.uint8).pin_memory()
        self.graph_tables_offset = offsets["block_tables"]
        host_bytes = self.graph_host.numpy()
        v, self.graph_host_np = {}, {}
        for name, npdt, tdt, shape in fields:
            nbytes = int(np.prod(shape)) * np.dtype(npdt).itemsize
            v[name] = self.graph_dev[offsets[name]:offsets[name] + nbytes].view(tdt).view(*shape)
            self.graph_host_np[name] = host_bytes[offsets[name]:offsets[name] + nbytes].view(npdt).reshape(shape)
        v["slot_mapping"].fill_(-1)
        self.graph_host_np["slot_mapping"][:] = -1
        v["outputs"] = torch.zeros(max_bs, self.model_config.d_model, dtype=self.dtype, device=dev)
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
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool):
                positions = (v["context_lens"][:b] - 1).clamp_min(0)
                v["outputs"][:b] = self.model(v["input_ids"][:b], positions)
            if pool is None:
                pool = g.pool()
            self.graphs[b] = g
            torch.cuda.synchronize()
            reset_context()
        self.graph_vars = v

    def exit(self) -> None:
        self.graphs.clear()
        self.graph_vars.clear()
        torch.cuda.synchronize()
