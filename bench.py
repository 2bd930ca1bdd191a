#!/usr/bin/env python
"""Benchmark of the paged GQA decode attention step on B200.

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

``--impl reference`` times the CPU oracle (the reference's fp32 torch arithmetic applied to the
gathered pool) on the host cores instead.  With N > 1 (torchrun) every rank runs an independent
replica of the workload on its own GPU: requests shard, nothing is exchanged.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, D, BS, BATCH = 32, 8, 128, 16, 256
CPU_SAMPLE_SEQS = 64
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


def main():
    global BATCH, CPU_SAMPLE_SEQS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-input leg (profiling runs)")
    ap.add_argument("--workload", default="decode", choices=["decode", "mla_decode", "prefill", "mla_prefill", "store", "moe_experts", "engine", "engine_mla", "engine_step"],
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
                   "moe_experts": "tokens", "engine_mla": "batch", "mla_prefill": "seqs", "engine_step": "batch"}[args.workload]
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
        if rank != 0:
            return
        torch.set_num_threads(os.cpu_count() or 1)   # torchrun pins OMP_NUM_THREADS=1; use every host core
        # The reference's CPU arithmetic for this step (gather + fp32 softmax attention) on a
        # bounded sample of the same workload; inputs synthesised on the host.
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
        t0 = time.perf_counter()
        for _ in range(steps):
            time_cpu_oracle(sample)
        dt = time.perf_counter() - t0
        val = nseq * steps / dt
        cores = torch.get_num_threads()
        desc = f"first {nseq} of the {BATCH} sequences ({int(lens.sum())} context tokens) per step"
        print(json.dumps({
            "impl": "reference", "metric": "decode tokens/s", "value": val, "unit": "tokens/s",
            "n_gpus": n_gpus, "steps": steps, "warmup": warm + 1, "requested_steps": args.steps,
            "ms_per_step": 1e3 * dt / steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config,
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": cores, "kind": "port",
                             "sample": desc},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }))
        return

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

    # ---------------------------------------------------------------- kernel-resident timing
    for _ in range(args.warmup):
        ops.paged_decode_gqa(q, kc, vc, bt, cl, scale, out=out)
    ops.check_status(dev)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        ops.paged_decode_gqa(q, kc, vc, bt, cl, scale, out=out)
    e1.record()
    barrier()
    ms_total = reduce_max(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps

    # ---------------------------------------------------------------- end-to-end with host inputs
    # The step's inputs live in one pinned host buffer and are shipped with a single copy (as the engine's
    # model runner does with its step metadata); typed views of the device copy go to the kernels.
    fields = [("q", torch.bfloat16, (BATCH, HQ, D)), ("k", torch.bfloat16, (BATCH, HKV, D)),
              ("v", torch.bfloat16, (BATCH, HKV, D)), ("slots", torch.int64, (BATCH,)),
              ("cl", torch.int64, (BATCH,)), ("bt", torch.int32, tuple(case.block_tables.shape))]
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
    hv_["bt"].copy_(torch.from_numpy(case.block_tables))
    hout = torch.empty(BATCH, HQ, D, dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in hv_.values())
    d2h = hout.numel() * hout.element_size()

    def e2e_step():
        dbuf.copy_(hbuf, non_blocking=True)
        ops.store_kvcache(dv_["k"], dv_["v"], kc, vc, dv_["slots"])
        ops.paged_decode_gqa(dv_["q"], kc, vc, dv_["bt"], dv_["cl"], scale, out=out)
        hout.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller reads the result every step

    e2e_ms = float("nan")
    if not args.no_e2e:
        for _ in range(args.warmup):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = reduce_max(max(e0.elapsed_time(e1), 0.0))
        e2e_wall_ms = reduce_max((time.perf_counter() - t0) * 1e3)
        e2e_ms = max(e2e_ms, e2e_wall_ms)  # host-side stalls between steps count
    sampler.stop()
    sampler.join(timeout=2)
    ops.check_status(dev)

    if rank != 0:
        if dist is not None:
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
                     "kernel": "paged_decode_bf16_kernel<128,1> (+ combine, timed together)"},
        "e2e": None if args.no_e2e else {
            "value": tokens_per_step / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": 2 * args.steps,
        "clocks": sampler.summary(),
    }
    if n_gpus == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        nseq = CPU_SAMPLE_SEQS
        sample = cpu_oracle_sample(case, q.cpu(), kc, vc, nseq)
        time_cpu_oracle(sample)  # warm-up
        dt = time_cpu_oracle(sample, repeats=3)
        line["cpu_baseline"] = {
            "value": nseq / dt, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"first {nseq} of the {BATCH} sequences ({int(sample[4].sum())} context tokens), best of 3"}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
