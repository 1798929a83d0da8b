#!/usr/bin/env python
"""Benchmark of the TurboQuant paged KV decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

One step = one pass of the hot path over one batch: append one token per sequence into the quantized paged cache (the
oldest token of every full residual window is quantized, packed and written into its page), then single-token GQA
decode attention over [packed pages | window] for every sequence.

The headline workload is the fifth benchmark configuration: 4-bit TurboQuant KV, 32 query / 8 KV heads, head_dim 128,
page size 16, residual window 128, 512 sequences of 32768 tokens, N(0,1) bf16 keys and values.  With N GPUs (one
process per GPU under torchrun) the 512 sequences are split evenly over the ranks (strong scaling, no data-path
collective); the reported value is all sequences decoded per second over the slowest rank's device time.

Prints ONE JSON line.  ``value`` is device-timed with inputs resident in HBM; ``e2e`` goes through the public cache
API with pinned host buffers (H2D of q, k, v and D2H of the output inside the timed region); ``roofline`` is the
algorithmic bytes of the decode call over its CUDA-event duration against the measured copy bandwidth;
``cpu_baseline`` is the CPU oracle (a port of the reference's CPU path for the same rows) timed on this host;
``extra`` holds the other benchmark configurations measured the same way (un-quantized paged decode, 2-bit ragged
decode, the 3-bit mixed continuous-batching step with page churn, the CPU-runnable configuration, prefill attention).

``--impl reference`` times the CPU port alone (rank 0 only) and prints the same line shape.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "kv_decode_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read + dram__bytes_write over the algorithmic bytes, from ncu captures of the small profile cases
# (same kernels, contexts of 8 K - 32 K tokens); traffic grows with the bytes streamed.
NCU_TRAFFIC_RATIO = {"packed": 1.023, "paged": 1.019}
NCU_TRAFFIC_SOURCE = {
    "packed": "ncu capture of --profile-case tq4long, packed kernel (329.3 MB moved for 321.9 MB algorithmic), scaled by bytes",
    "paged": "ncu capture of --profile-case paged (253.9 MB moved for 249.2 MB algorithmic), scaled by bytes",
}


# ---------------------------------------------------------------------------------------------------------------
# workload definitions


def cfg5_spec(world: int = 1) -> dict:
    return {"workload": "cfg5: TurboQuant 4-bit paged GQA decode, 512 sequences x 32768 tokens", "sequences": 512,
            "q_heads": 32, "kv_heads": 8, "head_dim": 128, "bits": 4, "page_size": 16, "residual_len": 128,
            "context": 32768, "dtype": "bf16", "append_per_step": 1,
            "parallelism": f"sequences sharded over {world} GPU(s), {512 // world} per rank, no collective"}


def cfg2_spec() -> dict:
    return {"workload": "cfg2: unquantized paged bf16 GQA decode", "batch": 32, "q_heads": 32, "kv_heads": 8,
            "head_dim": 128, "page_size": 16, "context": "uniform[1024,8192]", "dtype": "bf16",
            "block_tables": "seeded random permutation of a shared page pool", "append_per_step": 1}


def cfg2_lengths(seed: int, batch: int = 32) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(1024, 8193, (batch,), generator=gen).tolist()


def uniform_lengths(seed: int, batch: int, low: int, high: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(low, high + 1, (batch,), generator=gen).tolist()


def measured_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001 - fall through to the stated fallback
            pass
    return FALLBACK_HBM_GBS, "fallback"


def packed_token_bytes(dim: int, bits: int, elem: int = 2) -> tuple[int, int]:
    """(key bytes, value bytes) stored per packed token and kv head: codes plus per-token metadata."""
    key = dim * bits // 8 + 8
    value = dim // (4 if bits == 2 else 2) + 2 * (dim // 32) * elem
    return key, value


def tq_decode_bytes(lengths: list[int], *, q_heads: int, kv_heads: int, dim: int, bits: int, residual: int, page: int,
                    elem: int = 2) -> int:
    """Algorithmic bytes of one packed decode call: every packed token and every window token once per KV head (the
    GQA group shares it), q in, out, and the block-table entries."""
    key, value = packed_token_bytes(dim, bits, elem)
    total = 0
    for n in lengths:
        quantized = max(0, n - residual)
        total += kv_heads * (quantized * (key + value) + min(n, residual) * 2 * dim * elem)
        total += (quantized + page - 1) // page * 4
    return total + len(lengths) * q_heads * dim * elem * 2


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, enabled: bool = True) -> None:
        self.gpu_index = gpu_index
        self.enabled = enabled
        self.proc: subprocess.Popen | None = None
        self.lines: list[str] = []
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        if not self.enabled:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump() -> None:
            assert self.proc is not None and self.proc.stdout is not None
            for line in self.proc.stdout:
                self.lines.append(line.strip())

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if not self.enabled:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["sampled on rank 0 only"]}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxes, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                maxes.append(float(parts[2]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxes) if maxes else None, "samples": len(clocks), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------------------
# distributed plumbing (torchrun env; NCCL only for the barrier and the max over ranks)


class Dist:
    def __init__(self, want_gpus: int, use_cuda: bool) -> None:
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.enabled = self.world > 1
        if self.enabled:
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl" if use_cuda else "gloo")
            self.dist = dist
        if want_gpus != self.world and self.rank == 0:
            print(f"[bench] --gpus {want_gpus} but WORLD_SIZE={self.world}; using {self.world}", file=sys.stderr)

    def pin_cores(self) -> None:
        """Give every rank its own slice of the host cores, so that eight Python step loops on one host do not migrate
        over each other (the step loop is host-bound for the small configurations)."""
        if not self.enabled or not hasattr(os, "sched_setaffinity"):
            return
        try:
            cores = sorted(os.sched_getaffinity(0))
            per_rank = max(1, len(cores) // self.world)
            mine = cores[self.local_rank * per_rank:(self.local_rank + 1) * per_rank]
            if mine:
                os.sched_setaffinity(0, mine)
        except OSError:
            pass

    def barrier(self) -> None:
        if self.enabled:
            self.dist.barrier()

    def max(self, value: float, device) -> float:
        if not self.enabled:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self) -> None:
        if self.enabled:
            self.dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
# cache builders


def build_tq_cache_uniform(device, *, rows: int, context: int, q_heads: int, kv_heads: int, dim: int, bits: int,
                           residual: int, page: int, headroom: int, seed: int, kv_slice: slice | None = None,
                           row_group: int = 128):
    """A batched TurboQuant cache whose `rows` sequences all hold `context` tokens of seeded N(0,1) bf16 K/V.  The
    page pool is sized once up front (growing it would copy it)."""
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache

    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    cache = Qwen3DynamicCache(config, batch_size=rows, kv_cache_quantization="turboquant", kv_cache_quant_bits=bits,
                              kv_cache_residual_len=residual)
    cache.reserve_sequence_capacity(context + headroom)
    local_kv = kv_heads if kv_slice is None else len(range(*kv_slice.indices(kv_heads)))
    pool = cache.allocator.turboquant_layers[0]
    pool.configure(kv_heads=local_kv, head_dim=dim, bits=bits, residual_len=residual, dtype=torch.bfloat16,
                   device=device)
    pool.ensure_capacity(rows * ((context + headroom + page - 1) // page) + 16)
    pool.ensure_slot_capacity(rows)
    gen = torch.Generator(device=device).manual_seed(seed)
    chunk = max(256, min(2048, (1 << 28) // max(1, rows * kv_heads * dim)))  # bounds the staging tensors to 0.5 GB each
    done = 0
    while done < context:
        step = min(chunk, context - done)
        k = torch.randn(rows, kv_heads, step, dim, device=device, dtype=torch.bfloat16, generator=gen)
        v = torch.randn(rows, kv_heads, step, dim, device=device, dtype=torch.bfloat16, generator=gen)
        if kv_slice is not None:
            k, v = k[:, kv_slice], v[:, kv_slice]
        cache.update(k, v, 0, require_dense_cache=False)
        done += step
        del k, v
    return cache


def build_tq_cache_ragged(device, *, lengths: list[int], kv_heads: int, dim: int, bits: int, residual: int, page: int,
                          headroom: int, seed: int, channel_sigma: float = 0.0, extra_pages: int = 0):
    """Per-sequence caches on one allocator, filled with their own context lengths and stacked into one batch (the
    way the scheduler builds a decode batch).  channel_sigma > 0 multiplies K and V by per-channel log-normal scales."""
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache, Qwen3PageAllocator

    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    allocator = Qwen3PageAllocator(config)
    pool = allocator.turboquant_layers[0]
    pool.configure(kv_heads=kv_heads, head_dim=dim, bits=bits, residual_len=residual, dtype=torch.bfloat16,
                   device=device)
    pool.ensure_capacity(sum((n + headroom + page - 1) // page for n in lengths) + 16 + extra_pages)
    pool.ensure_slot_capacity(len(lengths) + 16)
    gen = torch.Generator(device=device).manual_seed(seed)
    scale = None
    if channel_sigma > 0:
        scale = torch.exp(channel_sigma * torch.randn(kv_heads, 1, dim, device=device, generator=gen))
    rows = []
    for n in lengths:
        row = Qwen3DynamicCache(config, allocator=allocator, batch_size=1, kv_cache_quantization="turboquant",
                                kv_cache_quant_bits=bits, kv_cache_residual_len=residual)
        row.reserve_sequence_capacity(n + headroom)
        k = torch.randn(1, kv_heads, n, dim, device=device, generator=gen)
        v = torch.randn(1, kv_heads, n, dim, device=device, generator=gen)
        if scale is not None:
            k, v = k * scale, v * scale
        row.update(k.to(torch.bfloat16), v.to(torch.bfloat16), 0, require_dense_cache=False)
        rows.append(row)
        del k, v
    cache = Qwen3DynamicCache.stack(rows, config, clone_turboquant_rows=False)
    cache.reserve_sequence_capacity(0)  # every row already holds the pages for its own headroom
    return cache, scale


# ---------------------------------------------------------------------------------------------------------------
# GPU arm, headline: cfg5


def time_steps(step, decode_events: list | None, steps: int, device, dist: Dist) -> float:
    """K back-to-back steps between two CUDA events, bracketed by barrier + synchronize; max over ranks, in ms."""
    torch.cuda.synchronize(device)
    dist.barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        step(decode_events)
    end.record()
    torch.cuda.synchronize(device)
    dist.barrier()
    return dist.max(begin.elapsed_time(end), device)


def run_tq_decode_loops(args, dist: Dist, device, cache, lengths: list[int], *, q_heads: int, kv_heads: int,
                        dim: int, bits: int, residual: int, page: int, seed: int, with_e2e: bool,
                        scale=None) -> dict:
    """Device-resident and end-to-end step loops over one TurboQuant cache; returns the measured pieces."""
    batch = len(lengths)
    scaling = dim ** -0.5
    groups = q_heads // kv_heads
    gen = torch.Generator(device=device).manual_seed(seed)
    q_dev = torch.randn(batch, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    k_dev = torch.randn(batch, kv_heads, 1, dim, device=device, generator=gen)
    v_dev = torch.randn(batch, kv_heads, 1, dim, device=device, generator=gen)
    if scale is not None:
        k_dev, v_dev = k_dev * scale, v_dev * scale
    k_dev, v_dev = k_dev.to(torch.bfloat16), v_dev.to(torch.bfloat16)

    def step(events: list | None):
        cache.update(k_dev, v_dev, 0, require_dense_cache=False)
        if events is not None:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        out = cache.turboquant_single_token_decode_attention(0, q_dev, scaling=scaling, num_key_value_groups=groups)
        if events is not None:
            stop.record()
            events.append((start, stop))
        return out

    sampler = ClockSampler(device.index or 0, enabled=dist.rank == 0)
    sampler.start()
    for _ in range(args.warmup):
        step(None)
    # keep the GPU under this load until nvidia-smi has delivered a few samples, then time
    spin_deadline = time.perf_counter() + 3.0
    spun = 0
    while (sampler.enabled and not args.no_clock_spin and len(sampler.lines) < 6
           and time.perf_counter() < spin_deadline and spun < args.spin_steps):
        step(None)
        torch.cuda.synchronize(device)
        spun += 1
    decode_events: list = []
    total_ms = time_steps(step, decode_events, args.steps, device, dist)
    clocks = sampler.stop()
    step_ms = total_ms / args.steps
    decode_ms = statistics.mean(a.elapsed_time(b) for a, b in decode_events)
    done_steps = args.warmup + spun + args.steps
    lengths_mid = [n + args.warmup + spun + args.steps // 2 + 1 for n in lengths]
    algo_bytes = tq_decode_bytes(lengths_mid, q_heads=q_heads, kv_heads=kv_heads, dim=dim, bits=bits,
                                 residual=residual, page=page)
    result = {"step_ms": step_ms, "decode_ms": decode_ms, "algo_bytes": algo_bytes, "clocks": clocks,
              "steps_done": done_steps}
    if not with_e2e:
        return result

    # ---- end to end through the public API with host buffers -------------------------------------------------------
    # the step's inputs (q, new k, new v) sit in one pinned host buffer and cross PCIe as one copy
    q_count, kv_count = q_dev.numel(), k_dev.numel()
    in_host = torch.cat([q_dev.reshape(-1), k_dev.reshape(-1), v_dev.reshape(-1)]).cpu().pin_memory()
    out_hosts = [torch.empty(batch, q_heads, 1, dim, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    landed_events = [torch.cuda.Event(), torch.cuda.Event()]
    landed: list = [None, None]

    def step_e2e(index: int, pipelined: bool):
        """One step from pinned host inputs to a pinned host result.  Serial: the host waits for the result of every
        step before it prepares the next one.  Pipelined (depth 2): the result goes back asynchronously into one of
        two pinned buffers and the host waits for a buffer only when it is about to be reused, so the host work of
        step i+1 overlaps the kernels of step i, as a serving loop with asynchronous scheduling does."""
        slot = index & 1
        if pipelined and landed[slot] is not None:
            landed[slot].synchronize()  # the result of step index - 2 is in host memory
        staged = in_host.to(device, non_blocking=True)
        q = staged[:q_count].view(batch, q_heads, 1, dim)
        k = staged[q_count:q_count + kv_count].view(batch, kv_heads, 1, dim)
        v = staged[q_count + kv_count:].view(batch, kv_heads, 1, dim)
        cache.update(k, v, 0, require_dense_cache=False)
        out = cache.turboquant_single_token_decode_attention(0, q, scaling=scaling, num_key_value_groups=groups)
        if not pipelined:
            out_hosts[slot].copy_(out, non_blocking=False)
            return
        out_hosts[slot].copy_(out, non_blocking=True)
        landed[slot] = landed_events[slot]
        landed[slot].record()

    def timed_e2e(pipelined: bool) -> float:
        for i in range(args.warmup):
            step_e2e(i, pipelined)
        torch.cuda.synchronize(device)
        dist.barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            step_e2e(i, pipelined)
        torch.cuda.synchronize(device)  # every result has landed in host memory
        local = time.perf_counter() - t0
        dist.barrier()
        return dist.max(local, device)

    result["e2e_serial_s"] = timed_e2e(False)
    result["e2e_s"] = timed_e2e(True)
    result["h2d"] = in_host.numel() * 2
    result["d2h"] = out_hosts[0].numel() * 2
    return result


def run_cfg5_gpu(args, dist: Dist, device) -> dict:
    spec = cfg5_spec(dist.world)
    total, context = spec["sequences"], spec["context"]
    q_heads, kv_heads, dim = spec["q_heads"], spec["kv_heads"], spec["head_dim"]
    bits, residual, page = spec["bits"], spec["residual_len"], spec["page_size"]
    from anna_b200.sharding import shard_sequences

    shard = shard_sequences(total, dist.world, dist.rank)
    rows = shard.count
    headroom = 3 * (args.steps + args.warmup) + args.spin_steps + 64
    cache = build_tq_cache_uniform(device, rows=rows, context=context, q_heads=q_heads, kv_heads=kv_heads, dim=dim,
                                   bits=bits, residual=residual, page=page, headroom=headroom, seed=1234 + dist.rank)
    lengths = [context] * rows
    m = run_tq_decode_loops(args, dist, device, cache, lengths, q_heads=q_heads, kv_heads=kv_heads, dim=dim,
                            bits=bits, residual=residual, page=page, seed=99 + dist.rank, with_e2e=True)
    peak, peak_kind = measured_peak_gbs()
    achieved = m["algo_bytes"] / (m["decode_ms"] / 1e3) / 1e9
    value = total / (m["step_ms"] / 1e3)
    e2e_value = total * args.steps / m["e2e_s"]
    result = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": dist.world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": m["step_ms"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded N(0,1) bf16 keys, values and queries; no public dataset is involved)",
        "config": {**spec, "sequences_per_rank": rows,
                   "l2_policy": f"{m['algo_bytes'] / 1e9:.2f} GB of packed KV per rank and step exceed the 126 MB L2",
                   "key_codes": "this build's own definition of the TurboQuant key quantizer (unpinned against the "
                                "un-vendored turboquant 0.2.x package)"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": m["h2d"], "d2h_bytes_per_step": m["d2h"],
                "ms_per_step": m["e2e_s"] / args.steps * 1e3, "pipeline_depth": 2,
                "serial_value": total * args.steps / m["e2e_serial_s"],
                "note": "value: results return asynchronously into two pinned buffers, the host waits for a buffer "
                        "only before reusing it; serial_value: the host waits for every step's result before the next"},
        # per step: tq_append_kernel, tq_prepare_queries_kernel, tq_window_split_mma_kernel, tq_decode_split_mma_kernel
        # (the merge of the split-K partials is fused into the tail of the last one)
        "gpu_launches": 4 * args.steps,
        "clocks": m["clocks"],
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": int(m["algo_bytes"] * NCU_TRAFFIC_RATIO["packed"]),
                     "traffic_source": NCU_TRAFFIC_SOURCE["packed"], "peak_kind": peak_kind,
                     "kernel": "tq_decode_split_mma_kernel (timed with the query-preparation and window launches of "
                               "the same decode call; the split-K merge runs in its tail)",
                     "algorithmic_bytes_per_launch": m["algo_bytes"], "launch_ms": m["decode_ms"],
                     "frac_of_8TBps_nominal": achieved / 8000.0},
    }
    cache.release()
    cache.allocator.clear()
    return result


# ---------------------------------------------------------------------------------------------------------------
# KV-head-sharded variant of cfg5 (--variant kvhead): every rank holds all sequences but only its KV heads


def run_kvhead_variant(args, dist: Dist, device) -> dict:
    """TurboQuant 4-bit decode, all sequences on every rank, Hkv / N KV heads per rank; the outputs reach every rank by
    peer stores from the decode kernel's merge epilogue plus one flag exchange (--gather peer, the default) or by one
    NCCL all-gather (--gather nccl).  Total work is fixed, so the scaling is "strong"."""
    from anna_b200.sharding import HeadGather, PeerHeadGather, shard_kv_heads

    q_heads, kv_heads, dim, page, bits, residual = 32, 8, 128, 16, 4, 128
    batch, context = args.kvhead_batch, args.kvhead_context
    shard = shard_kv_heads(q_heads, kv_heads, dist.world, dist.rank)
    local_kv, local_q = shard.kv_stop - shard.kv_start, shard.q_stop - shard.q_start
    gather = HeadGather() if dist.enabled else (lambda out: out)
    groups = q_heads // kv_heads

    def build(rows: int, tokens: int, kv_slice: slice, seed: int, headroom: int):
        # the same stream of random numbers on every rank, each rank keeps its own KV heads
        return build_tq_cache_uniform(device, rows=rows, context=tokens, q_heads=q_heads, kv_heads=kv_heads, dim=dim,
                                      bits=bits, residual=residual, page=page, headroom=headroom, seed=seed,
                                      kv_slice=kv_slice)

    # self-check on a small problem: gathered sharded outputs == the unsharded computation of the same data
    check_rows, check_tokens = 2, 700
    full = build(check_rows, check_tokens, slice(0, kv_heads), 5, 16)
    part = build(check_rows, check_tokens, slice(shard.kv_start, shard.kv_stop), 5, 16)
    q_check = torch.randn(check_rows, q_heads, 1, dim, device=device, dtype=torch.bfloat16,
                          generator=torch.Generator(device=device).manual_seed(6))
    want = full.turboquant_single_token_decode_attention(0, q_check, scaling=dim ** -0.5, num_key_value_groups=groups)
    got = gather(part.turboquant_single_token_decode_attention(0, shard.slice_q(q_check), scaling=dim ** -0.5,
                                                               num_key_value_groups=groups))
    check_err = float((got.float() - want.float()).abs().max())
    if not check_err <= 2e-2:
        raise RuntimeError(f"KV-head-sharded decode disagrees with the unsharded one: max abs {check_err}")
    full.release()
    part.release()

    cache = build(batch, context, slice(shard.kv_start, shard.kv_stop), 11, args.steps + args.warmup + 64)
    peer = None
    if dist.enabled and args.gather == "peer":
        peer = PeerHeadGather(shard, batch=batch, q_heads=q_heads, head_dim=dim, dtype=torch.bfloat16, device=device)
    gen = torch.Generator(device=device).manual_seed(12)
    q = torch.randn(batch, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    k1 = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    v1 = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    q_local, k_local, v_local = shard.slice_q(q), shard.slice_kv(k1), shard.slice_kv(v1)

    def step(_events=None):
        cache.update(k_local, v_local, 0, require_dense_cache=False)
        if peer is not None:
            local_out, peer_ptrs = peer.begin()
            cache.turboquant_single_token_decode_attention(0, q_local, scaling=dim ** -0.5, num_key_value_groups=groups,
                                                           output=local_out, peer_outputs=peer_ptrs)
            return peer.finish()
        local = cache.turboquant_single_token_decode_attention(0, q_local, scaling=dim ** -0.5,
                                                               num_key_value_groups=groups)
        return gather(local)

    if peer is not None:
        # the peer-store path against the collective on the same cache state: every rank must see the same tensor
        local = cache.turboquant_single_token_decode_attention(0, q_local, scaling=dim ** -0.5,
                                                               num_key_value_groups=groups)
        want_full = gather(local).clone()
        local_out, peer_ptrs = peer.begin()
        cache.turboquant_single_token_decode_attention(0, q_local, scaling=dim ** -0.5, num_key_value_groups=groups,
                                                       output=local_out, peer_outputs=peer_ptrs)
        got_full = peer.finish()
        torch.cuda.synchronize(device)
        peer.check()
        if not torch.equal(got_full, want_full):
            raise RuntimeError("peer-store gather disagrees with the all-gather of the same outputs")

    sampler = ClockSampler(device.index or 0, enabled=dist.rank == 0)
    sampler.start()
    out = None
    for _ in range(args.warmup):
        out = step()
    step_ms = time_steps(step, None, args.steps, device, dist) / args.steps
    clocks = sampler.stop()
    if peer is not None:
        peer.check()
    key_bytes, value_bytes = packed_token_bytes(dim, bits)
    per_rank_bytes = batch * local_kv * ((context - residual) * (key_bytes + value_bytes) + residual * 2 * dim * 2)
    peak, peak_kind = measured_peak_gbs()
    achieved = per_rank_bytes / (step_ms / 1e3) / 1e9
    cache.release()
    return {
        "metric": METRIC, "value": batch / (step_ms / 1e3), "unit": UNIT, "n_gpus": dist.world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded N(0,1) bf16)",
        "config": {"workload": "cfg5 variant: TurboQuant 4-bit, KV heads sharded, outputs all-gathered", "batch": batch,
                   "q_heads": q_heads, "kv_heads": kv_heads, "head_dim": dim, "bits": bits, "context": context,
                   "page_size": page, "residual_len": residual, "append_per_step": 1,
                   "kv_heads_per_rank": local_kv, "q_heads_per_rank": local_q,
                   "parallelism": f"kv-head-sharded x{dist.world}, " + (
                       "outputs stored into every rank's [B, Hq, D] tensor by the decode kernel's merge epilogue "
                       "(peer stores over NVLink) and one flag exchange per step" if peer is not None else
                       "one all-gather of [B, Hq/N, D] per step"),
                   "l2_policy": f"{per_rank_bytes / 1e6:.0f} MB of packed KV per rank and step exceed the 126 MB L2"},
        # per step: tq_append, tq_prepare_queries, tq_window_split_mma, tq_decode_split_mma, and either the flag
        # exchange kernel or NCCL's all-gather with one strided copy (library kernels, not counted)
        "gpu_launches": (5 if peer is not None else 4) * args.steps, "clocks": clocks,
        "self_check": {"max_abs_vs_unsharded": check_err, "rows": check_rows, "context": check_tokens},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_kind": peak_kind,
                     "kernel": "tq_decode_split_mma_kernel (whole step incl. append and all-gather)",
                     "algorithmic_bytes_per_launch": per_rank_bytes, "launch_ms": step_ms},
        "out_shape": None if out is None else list(out.shape),
    }


# ---------------------------------------------------------------------------------------------------------------
# extras (single GPU)


def _time_device(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for start, stop in events:
        start.record()
        fn()
        stop.record()
    torch.cuda.synchronize()
    return statistics.median(a.elapsed_time(b) for a, b in events)


def run_cfg2_extra(args, device) -> dict:
    """Un-quantized paged bf16 decode (cfg2), device-resident step loop."""
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache, Qwen3PageAllocator, fused_ops

    spec = cfg2_spec()
    batch, q_heads, kv_heads, dim, page = spec["batch"], spec["q_heads"], spec["kv_heads"], spec["head_dim"], \
        spec["page_size"]
    steps, warmup = min(args.steps, 30), 3
    headroom = steps + warmup + 8
    lengths = cfg2_lengths(1234, batch)
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    allocator = Qwen3PageAllocator(config)
    total_pages = sum((n + headroom + page - 1) // page for n in lengths) + 32
    template = torch.empty(1, kv_heads, 1, dim, device=device, dtype=torch.bfloat16)
    layer = allocator.layers[0]
    layer.ensure_capacity(total_pages, key_template=template, value_template=template)
    layer.free_pages[:] = torch.randperm(layer.capacity(), generator=torch.Generator().manual_seed(1235)).tolist()
    gen = torch.Generator(device=device).manual_seed(1236)
    caches = []
    for n in lengths:
        row = Qwen3DynamicCache(config, allocator=allocator)
        row.reserve_sequence_capacity(n + headroom)
        k = torch.randn(1, kv_heads, n, dim, device=device, dtype=torch.bfloat16, generator=gen)
        v = torch.randn(1, kv_heads, n, dim, device=device, dtype=torch.bfloat16, generator=gen)
        row.update(k, v, 0, require_dense_cache=False)
        caches.append(row)
    cache = Qwen3DynamicCache.stack(caches, config)
    cache.reserve_sequence_capacity(0)
    q = torch.randn(batch, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    k1 = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    v1 = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    events: list = []

    def step(record: bool):
        cache.update(k1, v1, 0, require_dense_cache=False)
        key_pages, value_pages, table, visible = cache.paged_attention_state(0)
        if record:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        fused_ops.run_paged_gqa_decode_fused(query=q, key_pages=key_pages, value_pages=value_pages, page_table=table,
                                             visible_lengths=visible, scaling=dim ** -0.5)
        if record:
            stop.record()
            events.append((start, stop))

    for _ in range(warmup):
        step(False)
    torch.cuda.synchronize(device)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        step(True)
    end.record()
    torch.cuda.synchronize(device)
    step_ms = begin.elapsed_time(end) / steps
    decode_ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    mid = [n + warmup + steps // 2 + 1 for n in lengths]
    algo = (sum(mid) * kv_heads * 2 * dim * 2 + batch * q_heads * dim * 2 * 2
            + sum((n + page - 1) // page for n in mid) * 4)
    peak, _ = measured_peak_gbs()
    cache.release()
    allocator.clear()
    return {**spec, "steps": steps, "ms_per_step": step_ms, "tokens_per_s": batch / (step_ms / 1e3),
            "decode_ms": decode_ms, "decode_algorithmic_bytes": algo, "decode_GBps": algo / (decode_ms / 1e3) / 1e9,
            "decode_frac_of_measured_peak": algo / (decode_ms / 1e3) / 1e9 / peak,
            "kernel": "dense_decode_balanced_mma_kernel"}


def run_cfg3_extra(args, device) -> dict:
    """cfg3 as written: 2-bit TurboQuant, 64 sequences, contexts uniform in [4096, 32768], 16 q / 2 kv heads,
    head_dim 256, window 128, K and V = N(0,1) times per-channel log-normal scales (sigma 0.5); step = append one
    token per sequence + decode."""
    batch, q_heads, kv_heads, dim, bits, residual, page = 64, 16, 2, 256, 2, 128, 16
    sub = argparse.Namespace(**{**vars(args), "steps": min(args.steps, 30), "warmup": 3, "spin_steps": 0})
    lengths = uniform_lengths(3003, batch, 4096, 32768)
    cache, scale = build_tq_cache_ragged(device, lengths=lengths, kv_heads=kv_heads, dim=dim, bits=bits,
                                         residual=residual, page=page, headroom=sub.steps + sub.warmup + 8, seed=3004,
                                         channel_sigma=0.5)
    m = run_tq_decode_loops(sub, _SOLO, device, cache, lengths, q_heads=q_heads, kv_heads=kv_heads, dim=dim,
                            bits=bits, residual=residual, page=page, seed=3005, with_e2e=False, scale=scale)
    peak, _ = measured_peak_gbs()
    gbps = m["algo_bytes"] / (m["decode_ms"] / 1e3) / 1e9
    cache.release()
    cache.allocator.clear()
    return {"workload": "cfg3: TurboQuant 2-bit, 64 sequences, contexts uniform[4096,32768], 16q/2kv, D=256, window 128, "
                        "per-channel log-normal scales (sigma 0.5)",
            "context_min_mean_max": [min(lengths), sum(lengths) / batch, max(lengths)], "steps": sub.steps,
            "ms_per_step": m["step_ms"], "tokens_per_s": batch / (m["step_ms"] / 1e3), "decode_ms": m["decode_ms"],
            "decode_algorithmic_bytes": m["algo_bytes"], "decode_GBps": gbps,
            "decode_frac_of_measured_peak": gbps / peak, "kernel": "tq_decode_split_mma_kernel<bf16,256,2>"}


def run_cfg4_extra(args, device) -> dict:
    """cfg4 as written, one mixed continuous-batching step: 3-bit TurboQuant, 16 q / 4 kv heads, head_dim 128; per
    step 8 new sequences get a 2048-token prefill chunk quantize-appended and 128 decode sequences (contexts uniform
    in [512, 16384]) append one token and decode; the packed pool is 80 % occupied; every step 10 % of the decode
    sequences finish (pages back to the allocator) and as many are admitted in their place (seeded).

    An admitted sequence takes a fresh context length, its pages from the allocator's free list (most recently freed
    first) and a window slot; what those recycled pages hold stands in for its K/V (the data is synthetic), so
    admission costs what the scheduler's admission costs here: allocator calls, a new batch object and a block-table
    upload, not a replay of the prompt."""
    from anna_b200 import Qwen3DynamicCache
    from anna_b200.turboquant import TurboQuantKVRow

    q_heads, kv_heads, dim, bits, residual, page = 16, 4, 128, 3, 128, 16
    decode_rows, new_rows, chunk, prompt_chunks = 128, 8, 2048, 4
    steps, warmup = min(args.steps, 20), 3
    rng = np.random.default_rng(4004)
    lengths = uniform_lengths(4005, decode_rows, 512, 16384)
    spare = (decode_rows // 10 + 1) * (16384 // page + 2) + new_rows * (prompt_chunks * chunk // page + 2)
    cache, _ = build_tq_cache_ragged(device, lengths=lengths, kv_heads=kv_heads, dim=dim, bits=bits, residual=residual,
                                     page=page, headroom=steps + warmup + 8, seed=4006, extra_pages=spare)
    allocator, config = cache.allocator, cache.config
    pool = allocator.turboquant_layers[0]
    used_target = pool.used_pages() + new_rows * (prompt_chunks * chunk // page) // 2
    pool.ensure_capacity(int(used_target / 0.8) + 1)  # 80 % occupancy in the steady state of the loop below
    pool.ensure_slot_capacity(decode_rows + 2 * new_rows + 16)
    gen = torch.Generator(device=device).manual_seed(4007)
    q = torch.randn(decode_rows, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    k1 = torch.randn(decode_rows, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    v1 = torch.randn(decode_rows, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    kc = torch.randn(new_rows, kv_heads, chunk, dim, device=device, dtype=torch.bfloat16, generator=gen)
    vc = torch.randn(new_rows, kv_heads, chunk, dim, device=device, dtype=torch.bfloat16, generator=gen)
    key_bytes, value_bytes = packed_token_bytes(dim, bits)

    def new_prefill_batch():
        batch_cache = Qwen3DynamicCache(config, allocator=allocator, batch_size=new_rows,
                                        kv_cache_quantization="turboquant", kv_cache_quant_bits=bits,
                                        kv_cache_residual_len=residual)
        batch_cache.reserve_sequence_capacity(prompt_chunks * chunk)
        return batch_cache

    def admit(length: int):
        """A single-row cache whose row holds `length` tokens in pages taken from the allocator."""
        single = Qwen3DynamicCache(config, allocator=allocator, batch_size=1, kv_cache_quantization="turboquant",
                                   kv_cache_quant_bits=bits, kv_cache_residual_len=residual)
        row = TurboQuantKVRow(bits=bits, residual_len=residual)
        row._bind(pool, kv_heads=kv_heads, head_dim=dim, dtype=torch.bfloat16, device=device)
        row._reserve_blocks(length + steps + warmup + 8)
        row._length = length
        single.turboquant_rows[0][0] = row
        single.layer_lengths[0][0] = length
        single.seen_tokens = length
        return single

    state = {"decode": cache, "prefill": new_prefill_batch(), "chunks_done": 0, "lengths": list(lengths)}
    decode_ev, append_ev = [], []

    def mixed_step(record: bool):
        # 1. churn: 10 % of the decode sequences finish and are replaced
        finished = set(rng.choice(decode_rows, size=decode_rows // 10, replace=False).tolist())
        keep = [i for i in range(decode_rows) if i not in finished]
        kept = state["decode"].compact_batch_rows(keep)
        kept_lengths = [state["lengths"][i] for i in keep]
        fresh_lengths = rng.integers(512, 16385, size=len(finished)).tolist()
        fresh = [admit(int(n)) for n in fresh_lengths]
        # the scheduler's order of calls: compact the finished rows away, split the group into per-request caches
        # without cloning, stack them again together with the admitted requests (scheduler.py:814-823, :640-648, :516-522)
        singles = kept.split_batch(clone_turboquant_rows=False)
        state["decode"] = Qwen3DynamicCache.stack(singles + fresh, config, clone_turboquant_rows=False)
        state["decode"].reserve_sequence_capacity(0)
        state["lengths"] = kept_lengths + [int(n) for n in fresh_lengths]
        # 2. prefill side: a 2048-token chunk for each of the 8 new sequences (fresh ones every prompt_chunks steps)
        if state["chunks_done"] == prompt_chunks:
            state["prefill"].release()
            state["prefill"] = new_prefill_batch()
            state["chunks_done"] = 0
        if record:
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
        state["prefill"].update(kc, vc, 0, require_dense_cache=False)
        if record:
            a1.record()
            append_ev.append((a0, a1))
        state["chunks_done"] += 1
        # 3. decode side: one token per sequence, then attention
        state["decode"].update(k1, v1, 0, require_dense_cache=False)
        state["lengths"] = [n + 1 for n in state["lengths"]]
        if record:
            d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            d0.record()
        state["decode"].turboquant_single_token_decode_attention(0, q, scaling=dim ** -0.5,
                                                                 num_key_value_groups=q_heads // kv_heads)
        if record:
            d1.record()
            decode_ev.append((d0, d1, tq_decode_bytes(state["lengths"], q_heads=q_heads, kv_heads=kv_heads, dim=dim,
                                                      bits=bits, residual=residual, page=page)))

    for _ in range(warmup):
        mixed_step(False)
    torch.cuda.synchronize(device)
    occupancy = pool.used_pages() / pool.capacity()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    begin.record()
    for _ in range(steps):
        mixed_step(True)
    end.record()
    torch.cuda.synchronize(device)
    wall_ms = (time.perf_counter() - t0) * 1e3 / steps
    step_ms = begin.elapsed_time(end) / steps
    peak, _ = measured_peak_gbs()
    decode_gbps = statistics.mean(nbytes / (a.elapsed_time(b) / 1e3) / 1e9 for a, b, nbytes in decode_ev)
    decode_ms = statistics.mean(a.elapsed_time(b) for a, b, _ in decode_ev)
    append_ms = statistics.mean(a.elapsed_time(b) for a, b in append_ev)
    append_bytes = append_algorithmic_bytes(new_rows * kv_heads, chunk, 128, dim, 2, key_bytes + value_bytes)
    state["decode"].release()
    state["prefill"].release()
    allocator.clear()
    return {"workload": "cfg4: mixed continuous-batching step, TurboQuant 3-bit, 16q/4kv, D=128: 8 x 2048-token "
                        "quantize-appends + 128 decodes (contexts uniform[512,16384]), pool 80 % occupied, 10 % of the "
                        "decode sequences finished and re-admitted per step",
            "steps": steps, "ms_per_step": step_ms, "ms_per_step_host_wall": wall_ms,
            "decode_tokens_per_s": decode_rows / (step_ms / 1e3),
            "prefill_tokens_per_s": new_rows * chunk / (step_ms / 1e3), "pool_occupancy": occupancy,
            "decode_ms": decode_ms, "decode_GBps": decode_gbps, "decode_frac_of_measured_peak": decode_gbps / peak,
            "quant_append_ms": append_ms, "quant_append_algorithmic_bytes": append_bytes,
            "quant_append_GBps": append_bytes / (append_ms / 1e3) / 1e9,
            "quant_append_frac_of_measured_peak": append_bytes / (append_ms / 1e3) / 1e9 / peak,
            "note": "quant_append_ms brackets the update() call of the chunk (host bookkeeping + tq_append_kernel); the "
                    "kernel is bound by instruction issue, not by HBM"}


def append_algorithmic_bytes(row_heads: int, new_tokens: int, residual: int, dim: int, elem_bytes: int,
                              packed_token_bytes_kv: int) -> int:
    """Bytes one fused quantize-append must move for ``row_heads`` (row, kv head) pairs whose window is already full:
    the new K and V are read once, every new token pushes one token into packed form (codes, norms, scales written),
    and the window ring has min(T, R) old tokens read out of it and min(T, R) new tokens written into it."""
    vec = 2 * dim * elem_bytes
    ring = 2 * min(new_tokens, residual) * vec
    return row_heads * (new_tokens * (vec + packed_token_bytes_kv) + ring)


def run_bulk_append_extra(device) -> dict:
    """Fused quantize-append alone, kernel-timed: 64 sequences x 8 kv heads x 2048-token chunks, 4-bit, D=128."""
    from anna_b200.turboquant import launch_tq_append

    batch, kv_heads, dim, bits, residual, page, chunk = 64, 8, 128, 4, 128, 16, 2048
    cache = build_tq_cache_uniform(device, rows=batch, context=2176, q_heads=32, kv_heads=kv_heads, dim=dim, bits=bits,
                                   residual=residual, page=page, headroom=8 * chunk, seed=77)
    pool = cache.allocator.turboquant_layers[0]
    gen = torch.Generator(device=device).manual_seed(78)
    k = torch.randn(batch, kv_heads, chunk, dim, device=device, dtype=torch.bfloat16, generator=gen)
    v = torch.randn(batch, kv_heads, chunk, dim, device=device, dtype=torch.bfloat16, generator=gen)
    kernel_ms, api_ms = [], []
    for it in range(5):
        rows = cache.turboquant_rows[0]
        past = [row.length for row in rows]
        if it % 2 == 0:  # the launch alone between two events, bookkeeping done before
            for row in rows:
                row._reserve_blocks(row.length + chunk)
            table = cache._sync_page_table_layer_buffer(0, batch_size=batch, device=device)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            launch_tq_append(pool, k, v, table, [row.slot for row in rows], past)
            stop.record()
            torch.cuda.synchronize()
            kernel_ms.append(start.elapsed_time(stop))
            for idx, row in enumerate(rows):
                row._length += chunk
                cache.layer_lengths[0][idx] = row.length
            dev_state = cache._dev_lengths[0]
            if dev_state is not None:
                dev_state.host = None
        else:  # the public call, host-timed
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            cache.update(k, v, 0, require_dense_cache=False)
            torch.cuda.synchronize()
            api_ms.append((time.perf_counter() - t0) * 1e3)
    key_bytes, value_bytes = packed_token_bytes(dim, bits)
    nbytes = append_algorithmic_bytes(batch * kv_heads, chunk, residual, dim, 2, key_bytes + value_bytes)
    peak, _ = measured_peak_gbs()
    ms = statistics.median(kernel_ms)
    cache.release()
    cache.allocator.clear()
    # The kernel is bound by fp32 instruction issue (about 64 fused multiply-adds' worth of butterflies, compares and
    # exact divisions per coordinate), so the second fraction is against the fp32 pipe, not against HBM.
    return {"workload": "fused quantize-append alone: 64 sequences x 8 kv heads x 2048 tokens, 4-bit, D=128",
            "kernel_ms": ms, "api_ms_host_timed": statistics.median(api_ms), "quant_append_algorithmic_bytes": nbytes,
            "quant_append_GBps": nbytes / (ms / 1e3) / 1e9,
            "quant_append_frac_of_measured_peak": nbytes / (ms / 1e3) / 1e9 / peak,
            "token_heads_per_s": batch * kv_heads * chunk / (ms / 1e3), "bound": "fp32 instruction issue"}


def run_cfg1_extra(device) -> dict:
    """cfg1, the CPU-runnable configuration, in full on both sides: fp32, batch 2, 8 q / 2 kv heads, head_dim 128,
    page 16, 4-bit keys and values, window 128, N(0,1) with 4 outlier channels per head scaled by 8; prefill 512
    tokens, then 64 steps of (append one token, decode).  GPU path against the oracle, both timed."""
    import oracle
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache

    batch, q_heads, kv_heads, dim, bits, residual, page = 2, 8, 2, 128, 4, 128, 16
    gen = torch.Generator().manual_seed(1001)

    def draw(tokens: int) -> torch.Tensor:
        x = torch.randn(batch, kv_heads, tokens, dim, generator=gen)
        for h in range(kv_heads):
            x[:, h, :, outliers[h]] *= 8.0
        return x

    outliers = [torch.randperm(dim, generator=gen)[:4] for _ in range(kv_heads)]
    prefill_k, prefill_v = draw(512), draw(512)
    step_k = [draw(1) for _ in range(64)]
    step_v = [draw(1) for _ in range(64)]
    queries = [torch.randn(batch, q_heads, 1, dim, generator=gen) for _ in range(64)]

    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    cache = Qwen3DynamicCache(config, batch_size=batch, kv_cache_quantization="turboquant", kv_cache_quant_bits=bits,
                              kv_cache_residual_len=residual)
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    cache.update(prefill_k.to(device), prefill_v.to(device), 0, require_dense_cache=False)
    gpu_out = []
    for i in range(64):
        cache.update(step_k[i].to(device), step_v[i].to(device), 0, require_dense_cache=False)
        gpu_out.append(cache.turboquant_single_token_decode_attention(0, queries[i].to(device), scaling=dim ** -0.5,
                                                                      num_key_value_groups=q_heads // kv_heads))
    gpu_out = torch.stack(gpu_out).cpu().numpy()
    gpu_s = time.perf_counter() - t0
    cache.release()

    t0 = time.perf_counter()
    rows = [oracle.OracleTurboQuantRow(bits=bits, residual_len=residual, dtype=oracle.DTYPE_F32, block_size=page,
                                       keep_decode_cache=True) for _ in range(batch)]
    for b, row in enumerate(rows):
        row.append(prefill_k[b].numpy(), prefill_v[b].numpy())
    cpu_out = np.zeros_like(gpu_out)
    for i in range(64):
        for b, row in enumerate(rows):
            row.append(step_k[i][b].numpy(), step_v[i][b].numpy())
            cpu_out[i, b, :, 0] = row.decode_attention(queries[i][b, :, 0].numpy(), scaling=dim ** -0.5, blas=True)
    cpu_s = time.perf_counter() - t0
    err = np.abs(gpu_out - cpu_out)
    return {"workload": "cfg1: fp32, batch 2, 8q/2kv, D=128, 4-bit, window 128, prefill 512 + 64 decode steps",
            "gpu_seconds_whole_run_host_timed": gpu_s, "cpu_oracle_seconds_whole_run": cpu_s,
            "decode_steps": 64, "max_abs_vs_oracle": float(err.max()),
            "rel_l2_vs_oracle": float(np.linalg.norm(err.ravel()) / np.linalg.norm(cpu_out.ravel())),
            "tolerance": 2e-3, "kernel": "tq_decode_split_kernel (CUDA-core path of fp32 caches)"}


def run_prefill_extra(device, *, batch: int = 8, q_heads: int = 16, kv_heads: int = 4, dim: int = 128,
                      chunk: int = 2048, past: int = 8192, iters: int = 10) -> dict:
    """cfg4's prefill side: causal attention of a 2048-token chunk over (past + chunk) dense bf16 keys, the operands
    `update(require_dense_cache=True)` hands to grouped_query_attention.  Tensor-bound: flops against the measured
    bf16 GEMM peak."""
    from anna_b200 import grouped_query_attention

    gen = torch.Generator(device=device).manual_seed(11)
    total = past + chunk
    q = torch.randn(batch, q_heads, chunk, dim, device=device, dtype=torch.bfloat16, generator=gen)
    k = torch.randn(batch, kv_heads, total, dim, device=device, dtype=torch.bfloat16, generator=gen)
    v = torch.randn(batch, kv_heads, total, dim, device=device, dtype=torch.bfloat16, generator=gen)
    lengths = torch.full((batch,), total, dtype=torch.long, device=device)
    fn = lambda: grouped_query_attention(q, k, v, scaling=dim ** -0.5, key_lengths=lengths, causal=True)  # noqa: E731
    ms = _time_device(fn, iters=iters, warmup=3)
    visible_pairs = batch * q_heads * (chunk * past + chunk * (chunk + 1) // 2)
    flops = 4.0 * visible_pairs * dim
    peak_tflops = None
    try:
        peak_tflops = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"])
    except Exception:  # noqa: BLE001
        pass
    tflops = flops / (ms / 1e3) / 1e12
    out = {"workload": f"cfg4 prefill attention: {batch} seq x {chunk}-token chunk over {past} cached tokens, "
                       f"{q_heads}q/{kv_heads}kv heads, D={dim}, bf16 dense K/V",
           "prefill_ms": ms, "prefill_tokens_per_s": batch * chunk / (ms / 1e3), "algorithmic_flops": flops,
           "TFLOPs": tflops, "frac_of_measured_bf16_peak": None if peak_tflops is None else tflops / peak_tflops,
           "bound": "tensor"}
    del k, v
    # The same chunk shape with cfg3's heads (16 q / 2 kv, head_dim 256): the other tensor-memory kernel
    dim2, kv2 = 256, 2
    q2 = torch.randn(batch, q_heads, chunk, dim2, device=device, dtype=torch.bfloat16, generator=gen)
    k2 = torch.randn(batch, kv2, total, dim2, device=device, dtype=torch.bfloat16, generator=gen)
    v2 = torch.randn(batch, kv2, total, dim2, device=device, dtype=torch.bfloat16, generator=gen)
    ms2 = _time_device(lambda: grouped_query_attention(q2, k2, v2, scaling=dim2 ** -0.5, key_lengths=lengths, causal=True),
                       iters=iters, warmup=3)
    tflops2 = 4.0 * visible_pairs * dim2 / (ms2 / 1e3) / 1e12
    out["head_dim_256"] = {"workload": f"the same chunk with {q_heads}q/{kv2}kv heads, D={dim2}", "prefill_ms": ms2,
                           "TFLOPs": tflops2,
                           "frac_of_measured_bf16_peak": None if peak_tflops is None else tflops2 / peak_tflops}
    del q2, k2, v2
    # The same chunk on a quantized cache (cfg4: 3-bit): the dense view update(require_dense_cache=True) builds first
    # (de-quantized prefix + window, one launch), through the cache's own call.
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache

    cache = Qwen3DynamicCache(KVCacheConfig(num_hidden_layers=1, cache_block_size=16), batch_size=batch,
                              kv_cache_quantization="turboquant", kv_cache_quant_bits=3, kv_cache_residual_len=128)
    kq = torch.randn(batch, kv_heads, total, dim, device=device, dtype=torch.bfloat16, generator=gen)
    cache.update(kq, torch.randn(kq.shape, device=device, dtype=torch.bfloat16, generator=gen), 0,
                 require_dense_cache=False)
    del kq
    view_ms = _time_device(lambda: cache.visible_key_cache(0), iters=iters, warmup=3)
    written = 2.0 * batch * kv_heads * total * dim * 2
    out["dense_view"] = {"workload": f"de-quantized dense K and V of the same {batch} x {total} tokens from a 3-bit cache",
                         "ms": view_ms, "written_GBps": written / (view_ms / 1e3) / 1e9, "bound": "instruction issue"}
    cache.release()
    return out


# ---------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU path for TurboQuant rows


def cpu_cfg5_row_step_seconds(rows: int, steps: int, seed: int) -> tuple[float, int, float]:
    """Times `steps` decode steps of the CPU port on `rows` sequences of the cfg5 shape; returns (seconds per row and
    step, host threads used, seconds spent on the untimed prefill).

    Port of Qwen3DynamicCache.update + turboquant_single_token_decode_attention on CPU
    (src/anna/model/ops.py:618-660, :1024-1070 -> TurboQuantKVRow.append / decode_attention,
    src/anna/model/turboquant.py:1027-1140, :1275-1293): per row, quantize the token that leaves the window, extend the
    dense de-quantized decode cache in place (the reference's _KEEP_DECODE_CACHE), then fp32 attention over the dense
    cache with multi-threaded BLAS."""
    import oracle

    spec = cfg5_spec()
    q_heads, kv_heads, dim = spec["q_heads"], spec["kv_heads"], spec["head_dim"]
    bits, residual, page, context = spec["bits"], spec["residual_len"], spec["page_size"], spec["context"]
    from threadpoolctl import threadpool_limits

    try:
        threads = len(os.sched_getaffinity(0))
    except AttributeError:
        threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    # a launcher that exports OMP_NUM_THREADS=1 for its ranks must not turn this into a single-threaded baseline
    blas_threads = threadpool_limits(limits=threads)
    rng = np.random.default_rng(seed)
    t0 = time.perf_counter()
    cpu_rows = []
    for _ in range(rows):
        row = oracle.OracleTurboQuantRow(bits=bits, residual_len=residual, dtype=oracle.DTYPE_BF16, block_size=page,
                                         allocator=oracle.OracleLayerAllocator(), keep_decode_cache=True)
        k = oracle.round_bf16(rng.standard_normal((kv_heads, context, dim), dtype=np.float32))
        v = oracle.round_bf16(rng.standard_normal((kv_heads, context, dim), dtype=np.float32))
        row.append(k, v)
        cpu_rows.append(row)
        del k, v
    prefill_s = time.perf_counter() - t0
    q = oracle.round_bf16(rng.standard_normal((rows, q_heads, dim), dtype=np.float32))
    new_k = oracle.round_bf16(rng.standard_normal((rows, kv_heads, 1, dim), dtype=np.float32))
    new_v = oracle.round_bf16(rng.standard_normal((rows, kv_heads, 1, dim), dtype=np.float32))

    def one_step():
        for r, row in enumerate(cpu_rows):
            row.append(new_k[r], new_v[r])
            row.decode_attention(q[r], scaling=dim ** -0.5, blas=True)

    one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    elapsed = time.perf_counter() - t0
    blas_threads.restore_original_limits()
    return elapsed / (steps * rows), threads, prefill_s


def cpu_line(rows: int, steps: int) -> dict:
    per_row_step, threads, prefill_s = cpu_cfg5_row_step_seconds(rows, steps, 1234)
    total = cfg5_spec()["sequences"]
    return {"value": 1.0 / per_row_step, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{rows} of {total} sequences (each with its full 32768-token context), {steps} timed steps, the "
                      f"step time scaled linearly by rows (the reference loops over rows in Python); numpy fp32 BLAS "
                      f"port of the reference's CPU TurboQuant path with its incremental dense decode cache; prefill "
                      f"of the sample ({prefill_s:.0f} s) not timed",
            "ms_per_step_all_sequences": per_row_step * total * 1e3}


def run_reference_arm(args, dist: Dist) -> dict | None:
    if dist.rank != 0:
        return None
    rows = 2
    base = cpu_line(rows, max(3, min(args.steps + args.warmup, 60)))
    spec = cfg5_spec(dist.world)
    return {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": dist.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step_all_sequences"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic (seeded N(0,1) rounded to bf16)",
        "config": {**spec, "note": "CPU port of the reference's CPU path (oracle/), host cores only; the same 512 "
                                   "sequences whatever the GPU count"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ---------------------------------------------------------------------------------------------------------------
# small cases for profiler captures (inputs larger than L2, at most a few GB on the device, a handful of launches)


def run_profile_case(case: str, device) -> dict:
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache, Qwen3PageAllocator, fused_ops

    gen = torch.Generator(device=device).manual_seed(3)
    if case == "paged":
        # half of the cfg2 batch: 16 ragged rows drawn like cfg2's, block tables a permutation of the pool
        batch, q_heads, kv_heads, dim, page = 16, 32, 8, 128, 16
        lengths = cfg2_lengths(7, batch)
        config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
        allocator = Qwen3PageAllocator(config)
        template = torch.empty(1, kv_heads, 1, dim, device=device, dtype=torch.bfloat16)
        layer = allocator.layers[0]
        layer.ensure_capacity(sum((n + page - 1) // page for n in lengths) + 8, key_template=template,
                              value_template=template)
        layer.free_pages[:] = torch.randperm(layer.capacity(), generator=torch.Generator().manual_seed(8)).tolist()
        rows = []
        for n in lengths:
            row = Qwen3DynamicCache(config, allocator=allocator)
            k = torch.randn(1, kv_heads, n, dim, device=device, dtype=torch.bfloat16, generator=gen)
            v = torch.randn(1, kv_heads, n, dim, device=device, dtype=torch.bfloat16, generator=gen)
            row.update(k, v, 0, require_dense_cache=False)
            rows.append(row)
        cache = Qwen3DynamicCache.stack(rows, config)
        q = torch.randn(batch, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
        key_pages, value_pages, table, visible = cache.paged_attention_state(0)
        fn = lambda: fused_ops.run_paged_gqa_decode_fused(  # noqa: E731
            query=q, key_pages=key_pages, value_pages=value_pages, page_table=table, visible_lengths=visible,
            scaling=dim ** -0.5)
        algo = sum(lengths) * kv_heads * 2 * dim * 2
    elif case == "prefill":
        result = run_prefill_extra(device, batch=2, iters=3)
        return {"profile_case": case, **result}
    elif case == "tqappend":
        # bulk append: 2048 new tokens on top of 2176 cached ones, all 2048 oldest window/incoming tokens get packed
        batch, kv_heads, dim, page, tokens = 16, 8, 128, 16, 2048
        config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
        cache = Qwen3DynamicCache(config, batch_size=batch, kv_cache_quantization="turboquant",
                                  kv_cache_quant_bits=4, kv_cache_residual_len=128)
        cache.reserve_sequence_capacity(2176 + 8 * tokens)
        k = torch.randn(batch, kv_heads, 2176, dim, device=device, dtype=torch.bfloat16, generator=gen)
        cache.update(k, torch.randn_like(k), 0, require_dense_cache=False)
        k = torch.randn(batch, kv_heads, tokens, dim, device=device, dtype=torch.bfloat16, generator=gen)
        v = torch.randn(batch, kv_heads, tokens, dim, device=device, dtype=torch.bfloat16, generator=gen)
        fn = lambda: cache.update(k, v, 0, require_dense_cache=False)  # noqa: E731
        packed = sum(packed_token_bytes(dim, 4))
        algo = batch * kv_heads * tokens * (2 * 2 * dim * 2 + packed)  # ring/incoming read + ring write + packed write
    else:
        # tq4 / tq3 / tq2: contexts of 8 K tokens; tq4long / tq2long: few rows with the full 32 K context, so that a
        # CTA walks a 4096-token chunk as it does in the headline workload
        bits = {"tq4": 4, "tq3": 3, "tq2": 2, "tq4long": 4, "tq2long": 2, "tq4shard": 4}[case]
        long_case = case.endswith("long") or case.endswith("shard")
        if bits == 2:
            batch, q_heads, kv_heads, dim = (16, 16, 2, 256) if long_case else (32, 16, 2, 256)
        else:
            batch, q_heads, kv_heads, dim = (8, 32, 8, 128) if long_case else (16, 32, 8, 128)
        if case == "tq4shard":  # the per-GPU share of the headline workload at 8 GPUs (2.6 GB of packed pages)
            batch = 64
        page, context = 16, (32768 if long_case else 8320)
        cache = build_tq_cache_uniform(device, rows=batch, context=context, q_heads=q_heads, kv_heads=kv_heads,
                                       dim=dim, bits=bits, residual=128, page=page, headroom=64, seed=3)
        q = torch.randn(batch, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
        fn = lambda: cache.turboquant_single_token_decode_attention(  # noqa: E731
            0, q, scaling=dim ** -0.5, num_key_value_groups=q_heads // kv_heads)
        algo = tq_decode_bytes([context] * batch, q_heads=q_heads, kv_heads=kv_heads, dim=dim, bits=bits,
                               residual=128, page=page)
    ms = _time_device(fn, iters=3, warmup=2)
    return {"profile_case": case, "decode_ms": ms, "algorithmic_bytes": algo, "GBps": algo / (ms / 1e3) / 1e9}


class _Solo:
    """Stand-in for Dist inside the single-GPU extras."""
    world, rank, local_rank, enabled = 1, 0, 0, False

    @staticmethod
    def barrier() -> None:
        return None

    @staticmethod
    def max(value: float, device) -> float:
        return value


_SOLO = _Solo()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=30)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-extras", action="store_true", help="skip the other benchmark configurations")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--gather", choices=("peer", "nccl"), default="peer",
                        help="KV-head variant: how the per-rank outputs reach every rank")
    parser.add_argument("--variant", choices=("sequence", "kvhead"), default="sequence",
                        help="sequence: sequences sharded over ranks (default, the headline); kvhead: the same decode "
                             "with KV heads sharded over ranks and an all-gather of the outputs")
    parser.add_argument("--kvhead-batch", type=int, default=128)
    parser.add_argument("--kvhead-context", type=int, default=32768)
    parser.add_argument("--no-clock-spin", action="store_true",
                        help="do not add untimed steps while waiting for clock samples (for profiler runs)")
    parser.add_argument("--spin-steps", type=int, default=40,
                        help="at most this many untimed steps while waiting for nvidia-smi samples under load")
    parser.add_argument("--profile-case", default=None,
                        choices=("paged", "tq4", "tq3", "tq2", "tq4long", "tq2long", "tq4shard", "tqappend", "prefill"),
                        help="run one small case a few times and exit (meant to be wrapped by ncu)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        dist = Dist(args.gpus, use_cuda=False)
        line = run_reference_arm(args, dist)
        dist.barrier()
        if line is not None:
            print(json.dumps(line))
        dist.close()
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the "
                         "CPU port of the reference).")
    if args.profile_case:
        device = torch.device("cuda", 0)
        torch.cuda.set_device(device)
        print(json.dumps(run_profile_case(args.profile_case, device)))
        return
    dist = Dist(args.gpus, use_cuda=True)
    dist.pin_cores()
    device = torch.device("cuda", dist.local_rank)
    torch.cuda.set_device(device)
    if args.variant == "kvhead":
        result = run_kvhead_variant(args, dist, device)
        dist.barrier()
        if dist.rank == 0:
            print(json.dumps(result))
        dist.close()
        return
    result = run_cfg5_gpu(args, dist, device)

    if dist.rank == 0 and dist.world == 1:
        if not args.no_cpu_baseline:
            base = cpu_line(1, 3)
            result["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        if not args.no_extras:
            extras = []
            for fn in (lambda: run_cfg2_extra(args, device), lambda: run_cfg3_extra(args, device),
                       lambda: run_cfg4_extra(args, device), lambda: run_bulk_append_extra(device),
                       lambda: run_cfg1_extra(device), lambda: run_prefill_extra(device)):
                try:
                    extras.append(fn())
                except Exception as exc:  # noqa: BLE001 - extras never take the headline down
                    extras.append({"error": repr(exc)})
                torch.cuda.empty_cache()
            result["extra"] = extras
    dist.barrier()
    if dist.rank == 0:
        print(json.dumps(result))
    dist.close()


if __name__ == "__main__":
    main()
