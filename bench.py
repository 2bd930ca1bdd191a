#!/usr/bin/env python
"""Benchmark of the continuous-batching decode path on B200; the headline is the paged GQA decode attention step.

Workload (per GPU): 256 sequences, context lengths log-uniform in [128, 8192], 32 query heads,
8 KV heads, head_dim 128, KV block size 16, bf16; the physical pool is a random permutation of
block ids (seed 1) holding K, V ~ N(0,1); q ~ N(0,1); softmax scale 1/sqrt(128).  One "step" is one
decode-attention call over the whole batch (one new token per sequence).

  value     tokens/s with every input resident in HBM (kernel time only, CUDA events)
  e2e       tokens/s through the public op layer with HOST inputs: per step the new tokens' q/k/v,
            slot_mapping, block_tables and context_lens are copied from pinned host memory, the
            new K/V rows are scattered into the pool (store_kvcache), attention runs, and the
            output is copied back to the host.  The KV pool is persistent engine state and stays
            on the device, as model weights would.
  roofline  algorithmic bytes of one call / its measured duration, against the measured HBM copy
            peak of this pool's B200s.

  secondary the other kernels of the path on their benchmark shapes (store_kvcache, ragged prefill with the
            scatter, MLA decode, MLA prefill, MoE expert GEMMs), timed in this process, each with its algorithmic
            bytes or FLOPs and the fraction of the measured peak; 1 GPU only
  engine    the GQA+MoE decoder through the engine on the 2048-request continuous-batching job: output tokens/s,
            wall time per decode step, and the decode steps' fraction of the HBM roofline from the live contexts.
            Under torchrun both the fixed job (2048 requests over all replicas) and the weak job (2048 per replica)

The step region is timed ``REGIONS`` times; ms_per_step is the median region, min and max are reported beside it.

``--impl reference`` times the CPU oracle (the reference's fp32 torch arithmetic applied to the
gathered pool) on the host cores instead.  With N > 1 (torchrun) every rank runs an independent
replica of the workload on its own GPU: requests shard, nothing is exchanged.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, D, BS, BATCH = 32, 8, 128, 16, 256
CPU_SAMPLE_SEQS = 64
DECODE_KERNEL = "paged_decode_bf16_kernel<128,1> (+ combine, timed together)"
DECODE_LAUNCHES_PER_CALL = 2
REGIONS = 5   # the --steps region is timed this many times; the median is reported
# DRAM bytes read + written by one ncu-captured launch of the decode kernel over 130,732 context tokens
NCU_DRAM_BYTES_PER_CONTEXT_TOKEN = (536_459_520 + 4_956_544) / 130_732


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Reads SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.01):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "note": "NVML unavailable"}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


def cpu_oracle_sample(case, q_cpu, kc, vc, nseq):
    """(blocks gathered to the host, remapped block tables) for the first nseq sequences."""
    lens = case.context_lens[:nseq]
    nblk = (lens + BS - 1) // BS
    ids = np.concatenate([case.block_tables[i, :nblk[i]] for i in range(nseq)]).astype(np.int64)
    idt = torch.from_numpy(ids).to(kc.device)
    k_host, v_host = kc[idt].cpu(), vc[idt].cpu()
    tables, pos = [], 0
    for i in range(nseq):
        tables.append(list(range(pos, pos + int(nblk[i]))))
        pos += int(nblk[i])
    return q_cpu[:nseq], k_host, v_host, tables, lens


def time_cpu_oracle(sample, repeats=1):
    from oracle import attention as orc
    q, k, v, tables, lens = sample
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.paged_decode_gqa(q, k, v, tables, lens, D ** -0.5)
        best = min(best, time.perf_counter() - t0)
    return best


def bf16_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    except Exception:
        return 1590.0, 1400.0, "fallback"


def reference_arm(args, case, config, n_gpus):
    """The reference's CPU arithmetic for this step (gather + fp32 softmax attention) on a bounded sample of
    the same workload; inputs synthesised on the host.  Prints the JSON line."""
    torch.set_num_threads(os.cpu_count() or 1)   # torchrun pins OMP_NUM_THREADS=1; use every host core
    g = torch.Generator().manual_seed(1)
    nseq = CPU_SAMPLE_SEQS
    lens = case.context_lens[:nseq]
    nblk = int(((lens + BS - 1) // BS).sum())
    k_host = torch.randn(nblk, BS, HKV, D, generator=g).to(torch.bfloat16)
    v_host = torch.randn(nblk, BS, HKV, D, generator=g).to(torch.bfloat16)
    q_host = torch.randn(nseq, HQ, D, generator=g).to(torch.bfloat16)
    tables, pos = [], 0
    for i in range(nseq):
        n = int((lens[i] + BS - 1) // BS)
        tables.append(list(range(pos, pos + n)))
        pos += n
    sample = (q_host, k_host, v_host, tables, lens)
    # all requested steps unless that would run for more than ~2.5 minutes on these cores: every
    # step repeats the same bounded sample, so fewer steps change the noise, not the figure
    t0 = time.perf_counter()
    time_cpu_oracle(sample)
    est = time.perf_counter() - t0
    warm = max(0, min(args.warmup, 3) - 1)
    for _ in range(warm):
        time_cpu_oracle(sample)
    steps = max(1, min(args.steps, int(150.0 / max(est, 1e-3))))
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        time_cpu_oracle(sample)
        times.append(time.perf_counter() - t0)
    dt = float(np.median(times))
    val = nseq / dt
    cores = torch.get_num_threads()
    desc = f"first {nseq} of the {BATCH} sequences ({int(lens.sum())} context tokens) per step, median of {steps} steps"
    print(json.dumps({
        "impl": "reference", "metric": "decode tokens/s", "value": val, "unit": "tokens/s",
        "n_gpus": n_gpus, "steps": steps, "warmup": warm + 1, "requested_steps": args.steps,
        "ms_per_step": 1e3 * dt, "ms_per_step_min": 1e3 * min(times), "ms_per_step_max": 1e3 * max(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config,
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": desc},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_leg_in_a_fresh_process(batch: int):
    """The CPU baseline of the b200 arm: the reference arm itself (same function, same sample), run in a process of
    its own before this one touches CUDA, so that neither pinned-memory, NVML nor CUDA runtime threads share the
    host cores with it.  Returns the parsed line, or a dict with 'error'."""
    env = {k: v for k, v in os.environ.items() if k not in ("OMP_NUM_THREADS", "MKL_NUM_THREADS")}
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--gpus", "1", "--steps", "5",
           "--warmup", "3", "--batch", str(batch)]
    try:
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
        for ln in reversed(r.stdout.strip().splitlines()):
            if ln.startswith("{"):
                return json.loads(ln)
        return {"error": (r.stderr or r.stdout)[-300:]}
    except Exception as e:   # noqa: BLE001 - the baseline is reported, never needed
        return {"error": repr(e)}


def secondary_kernels(steps_scale: float = 1.0) -> dict:
    """The other kernels of the path on their benchmark shapes, each with its roofline fraction."""
    from llm_from_scratch_b200 import microbench
    hbm, hbm_kind = hbm_peak()
    burst, sustained, tf_kind = bf16_peaks()
    out = {"peaks": {"hbm_gbs": hbm, "bf16_tflops_burst": burst, "bf16_tflops_sustained": sustained,
                     "kind": f"of {hbm_kind}"}}

    def hbm_bound(res):
        res["roofline"] = {"bound": "hbm", "achieved": res["gbs"], "peak": hbm, "unit": "GB/s", "frac": res["gbs"] / hbm}
        return res

    def tensor_bound(res, tflops):
        res["roofline"] = {"bound": "tensor", "achieved": tflops, "peak": burst, "unit": "TFLOP/s",
                           "frac": tflops / burst, "frac_of_sustained": tflops / sustained}
        return res

    n = lambda k: max(3, int(k * steps_scale))

    def clocked(fn, **kw):
        """Runs one secondary benchmark with the SM clock sampled beside it."""
        smp = ClockSampler(physical_gpu_index(torch.cuda.current_device()), period=0.005)
        smp.start()
        res = fn(**kw)
        smp.stop()
        smp.join(timeout=2)
        c = smp.summary()
        res["clocks"] = {"sm_mhz": c.get("sm_mhz"), "reasons": c.get("reasons", [])}
        torch.cuda.empty_cache()
        return res

    # memory-bound kernels first: the long tensor-core runs heat the part up and the power cap then lowers the
    # SM clock, which the kernels that are bound by on-chip pipes (MLA decode) would inherit
    out["store"] = hbm_bound(clocked(microbench.store, steps=n(50), warmup=5))
    out["mla_decode"] = hbm_bound(clocked(microbench.mla_decode, steps=n(50), warmup=5))
    out["moe_experts"] = hbm_bound(clocked(microbench.moe_experts, steps=n(20), warmup=3))
    out["lm_head"] = hbm_bound(clocked(microbench.lm_head, steps=n(50), warmup=5))
    p64 = clocked(microbench.prefill64, steps=n(20), warmup=3)
    out["prefill_d64"] = tensor_bound(p64, p64["tflops"])
    mp = clocked(microbench.mla_prefill, steps=n(20), warmup=3)
    out["mla_prefill"] = tensor_bound(mp, mp["tflops"])
    pf = clocked(microbench.prefill, steps=n(5), warmup=3)
    pf["lengths"] = pf.pop("lengths")          # realised lengths of the 64 sequences, longest first
    out["prefill"] = tensor_bound(pf, pf["tflops"])
    out["prefill"]["attention_only_frac"] = pf["attention_only_tflops"] / burst
    return out


def main():
    global BATCH, CPU_SAMPLE_SEQS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-input leg (profiling runs)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary kernels (profiling runs)")
    ap.add_argument("--no-engine", action="store_true", help="skip the engine job (profiling runs)")
    ap.add_argument("--workload", default="decode", choices=["decode", "mla_decode", "prefill", "prefill64", "mla_prefill", "store", "moe_experts", "lm_head", "engine", "engine_mla", "engine_step"],
                    help="decode = the benchmark (paged GQA decode); the others time a secondary kernel on "
                         "its benchmark shape and print a short JSON line (single GPU, no reference arm)")
    ap.add_argument("--rate", type=float, default=0.0, help="engine workload: Poisson arrival rate (req/s); 0 = offline")
    ap.add_argument("--decode-window", type=int, default=1,
                    help="engine workload: decode steps per scheduling decision (1 = the reference's loop)")
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="sequences per GPU; anything but the default is a profiling case, not the benchmark")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if args.workload != "decode":
        from llm_from_scratch_b200 import microbench
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        fn = getattr(microbench, args.workload)
        kw = dict(steps=args.steps, warmup=args.warmup)
        if args.workload == "engine" and args.rate > 0:
            kw["rate"] = args.rate
        if args.workload == "engine" and args.decode_window > 1:
            kw["decode_window"] = args.decode_window
        if args.batch != BATCH:   # profiling cases: fewer sequences / tokens
            key = {"mla_decode": "batch", "engine": "batch", "prefill": "total", "store": "tokens",
                   "moe_experts": "tokens", "engine_mla": "batch", "mla_prefill": "seqs", "engine_step": "batch",
                   "prefill64": "seqs", "lm_head": "rows"}[args.workload]
            kw[key] = args.batch
        res = fn(**kw)
        if not res:       # a non-zero rank of a multi-replica engine run
            return
        peak, kind = hbm_peak()
        if "gbs" in res:
            res["hbm_frac"] = res["gbs"] / peak
            res["hbm_peak"] = f"{peak} GB/s of {kind}"
        print(json.dumps(res))
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n_gpus = max(args.gpus, world)

    from llm_from_scratch_b200.workloads import c2_decode_case, decode_algorithmic_bytes
    BATCH = args.batch
    CPU_SAMPLE_SEQS = min(CPU_SAMPLE_SEQS, BATCH)
    case = c2_decode_case(BATCH, 128, 8192, BS, seed=1)
    config = {"workload": f"paged GQA decode attention microbenchmark: {BATCH} seqs/GPU, ctx log-uniform "
                          "[128,8192], 32 q heads / 8 kv heads, head_dim 128, block 16, bf16",
              "batch_per_gpu": BATCH, "context_tokens_per_gpu": case.total_tokens,
              "l2": "inputs (>2 GB of K/V per GPU) exceed the 126 MB L2; no flush needed",
              "parallelism": f"replicas x{n_gpus} (requests shard, no collective)"}

    if args.impl == "reference":
        if rank == 0:
            reference_arm(args, case, config, n_gpus)
        return

    # the CPU baseline runs first, in a process of its own, while this process has not touched CUDA yet
    cpu_line = None
    if n_gpus == 1 and not args.no_cpu_baseline:
        cpu_line = cpu_leg_in_a_fresh_process(BATCH)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the b200 arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from llm_from_scratch_b200 import ops

    gen = torch.Generator(device=dev).manual_seed(1)
    kc = torch.randn(case.num_blocks, BS, HKV, D, generator=gen, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(case.num_blocks, BS, HKV, D, generator=gen, device=dev, dtype=torch.bfloat16)
    q = torch.randn(BATCH, HQ, D, generator=gen, device=dev, dtype=torch.bfloat16)
    bt = torch.from_numpy(case.block_tables).to(dev)
    cl = torch.from_numpy(case.context_lens).to(dev)
    out = torch.empty_like(q)
    scale = D ** -0.5

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(ms: float) -> float:
        if dist is None:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_regions(step_fn, wall: bool):
        """REGIONS x args.steps calls of step_fn; per region the device time between two events on the launching
        stream (and, for the host-input leg, the wall time if longer), max over ranks.  ms per step per region."""
        res = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(REGIONS):
            barrier()
            t0 = time.perf_counter()
            e0.record()
            for _ in range(args.steps):
                step_fn()
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1)
            if wall:
                ms = max(ms, (time.perf_counter() - t0) * 1e3)   # host-side stalls between steps count
            res.append(reduce_max(ms) / args.steps)
        return res

    # ---------------------------------------------------------------- kernel-resident timing
    for _ in range(args.warmup):
        ops.paged_decode_gqa(q, kc, vc, bt, cl, scale, out=out)
    ops.check_status(dev)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    barrier()
    sampler.start()
    kernel_ms = timed_regions(lambda: ops.paged_decode_gqa(q, kc, vc, bt, cl, scale, out=out), wall=False)
    ms_step = float(np.median(kernel_ms))

    # ---------------------------------------------------------------- end-to-end with host inputs
    # The engine's own input path (engine/model_runner.py of this package): the block table is resident on the
    # device; a step ships, in ONE copy from one pinned buffer, the new tokens' q / k / v, slot_mapping,
    # context_lens and the (row, column, block id) triples of the table entries that changed — one new block
    # per sequence every 16 steps — which b200_block_table_patch applies; then store_kvcache, attention, and the
    # output is copied back.  The KV pool is engine state and stays resident, as weights do.
    max_patches = BATCH
    fields = [("q", torch.bfloat16, (BATCH, HQ, D)), ("k", torch.bfloat16, (BATCH, HKV, D)),
              ("v", torch.bfloat16, (BATCH, HKV, D)), ("slots", torch.int64, (BATCH,)),
              ("cl", torch.int64, (BATCH,)), ("patches", torch.int32, (max_patches, 3))]
    offs, total = {}, 0
    for name, dt, shape in fields:
        offs[name] = total
        total += (int(np.prod(shape)) * torch.empty(0, dtype=dt).element_size() + 255) & ~255
    hbuf = torch.empty(total, dtype=torch.uint8).pin_memory()
    dbuf = torch.empty(total, dtype=torch.uint8, device=dev)

    def views(buf):
        out_ = {}
        for name, dt, shape in fields:
            n = int(np.prod(shape)) * torch.empty(0, dtype=dt).element_size()
            out_[name] = buf[offs[name]:offs[name] + n].view(dt).view(*shape)
        return out_

    hv_, dv_ = views(hbuf), views(dbuf)
    hv_["q"].copy_(torch.randn(BATCH, HQ, D).to(torch.bfloat16))
    hv_["k"].copy_(torch.randn(BATCH, HKV, D).to(torch.bfloat16))
    hv_["v"].copy_(torch.randn(BATCH, HKV, D).to(torch.bfloat16))
    hv_["slots"].copy_(torch.from_numpy(case.slot_mapping))
    hv_["cl"].copy_(torch.from_numpy(case.context_lens))
    hout = torch.empty(BATCH, HQ, D, dtype=torch.bfloat16).pin_memory()
    # table entries a step of a steady batch changes: the sequences that enter a new block on that step, i.e.
    # (length + step) % 16 == 1; the workload itself stays fixed, so a patch rewrites the entry's own value
    last_col = (case.context_lens - 1) // BS
    patch_sets = []
    for t in range(BS):
        rows = np.nonzero((case.context_lens + t) % BS == 1)[0]
        patch_sets.append(np.stack([rows, last_col[rows], case.block_tables[rows, last_col[rows]]], axis=1).astype(np.int32))
    patch_np = hv_["patches"].numpy()
    bt_dev = bt.clone()
    e2e_state = {"t": 0, "h2d": 0}
    fixed_bytes = sum(hv_[n].numel() * hv_[n].element_size() for n in ("q", "k", "v", "slots", "cl"))
    # (host view, device view) of the buffer prefix a step with m patches ships
    prefix = {len(p_): (hbuf[:offs["patches"] + len(p_) * 12], dbuf[:offs["patches"] + len(p_) * 12]) for p_ in patch_sets}

    def e2e_step():
        pt = patch_sets[e2e_state["t"] % BS]
        e2e_state["t"] += 1
        m = len(pt)
        patch_np[:m] = pt
        e2e_state["h2d"] += fixed_bytes + m * 12
        src, dst = prefix[m]
        dst.copy_(src, non_blocking=True)
        if m:
            ops.block_table_patch(dv_["patches"], m, bt_dev)
        ops.store_kvcache(dv_["k"], dv_["v"], kc, vc, dv_["slots"])
        ops.paged_decode_gqa(dv_["q"], kc, vc, bt_dev, dv_["cl"], scale, out=out)
        hout.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result every step

    e2e_ms, h2d, d2h = None, 0, hout.numel() * hout.element_size()
    if not args.no_e2e:
        for _ in range(args.warmup):
            e2e_step()
        e2e_state["h2d"], calls0 = 0, e2e_state["t"]
        e2e_ms = timed_regions(e2e_step, wall=True)
        h2d = e2e_state["h2d"] / max(e2e_state["t"] - calls0, 1)
        assert torch.equal(bt_dev, bt), "patches must leave the benchmark's block table as it was"
    sampler.stop()
    sampler.join(timeout=2)
    ops.check_status(dev)
    clocks = sampler.summary()
    del kc, vc, q, bt, cl, out, dbuf, bt_dev
    torch.cuda.empty_cache()

    # ---------------------------------------------------------------- the rest of the path
    secondary = None
    if n_gpus == 1 and not args.no_secondary:
        secondary = secondary_kernels()
    engine = None
    if not args.no_engine:
        from llm_from_scratch_b200 import microbench
        engine = microbench.engine_jobs(hbm_peak_gbs=hbm_peak()[0])
        if n_gpus == 1:
            # the MLA+MoE decoder's mixed step (16 prefills + 240 decodes per step pair) through the engine
            torch.cuda.empty_cache()
            engine["mla_mixed_step"] = microbench.engine_mla(steps=5, warmup=2)

    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    tokens_per_step = BATCH * n_gpus
    value = tokens_per_step / (ms_step * 1e-3)
    alg_bytes = decode_algorithmic_bytes(case, HQ, HKV, D, 2)
    peak, peak_kind = hbm_peak()
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s", "value": value, "unit": "tokens/s", "n_gpus": n_gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "timing": {"regions": REGIONS, "steps_per_region": args.steps, "ms_per_step_median": ms_step,
                   "ms_per_step_min": min(kernel_ms), "ms_per_step_max": max(kernel_ms),
                   "how": "CUDA events on the launching stream around each region, max over ranks"},
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": config,
        "per_gpu_tokens_per_s": value / n_gpus,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                     "frac_of_nominal_8TBs": achieved / 8000.0,
                     "algorithmic_bytes_per_launch": alg_bytes,
                     # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the 64-sequence
                     # case (541.4 MB for 130,732 context tokens), scaled by context tokens to this launch
                     "traffic": NCU_DRAM_BYTES_PER_CONTEXT_TOKEN * case.total_tokens,
                     "kernel": DECODE_KERNEL},
        "e2e": None if e2e_ms is None else {
            "value": tokens_per_step / (float(np.median(e2e_ms)) * 1e-3), "unit": "tokens/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": float(np.median(e2e_ms)),
            "ms_per_step_min": min(e2e_ms), "ms_per_step_max": max(e2e_ms),
            "input_path": "device-resident block table + per-step patches, one pinned H2D copy, one D2H copy"},
        "gpu_launches": DECODE_LAUNCHES_PER_CALL * args.steps,
        "gpu_launches_note": f"per timed region of {args.steps} steps; {REGIONS} regions",
        "clocks": clocks,
    }
    if cpu_line is not None:
        if "error" in cpu_line:
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": "failed: " + cpu_line["error"]}
        else:
            line["cpu_baseline"] = dict(cpu_line["cpu_baseline"],
                                        how="the reference arm of this file run in a fresh process before CUDA start-up")
    if secondary is not None:
        line["secondary"] = secondary
    if engine:
        line["engine"] = engine
    print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
