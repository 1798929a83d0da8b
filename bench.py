#!/usr/bin/env python
"""Benchmark of the paged KV decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

One step = one pass of the hot path over one batch: append one token per sequence into the paged cache, then
single-token GQA decode attention for every sequence.  The headline workload is the second benchmark configuration
(un-quantized paged bf16 GQA decode: 32 sequences, 32 query / 8 KV heads, head_dim 128, page size 16, contexts
uniform in [1024, 8192], block tables a seeded random permutation of a shared page pool, N(0,1) data).  With N > 1
(one process per GPU under torchrun) every rank runs its own batch of the same shape (weak scaling, no data-path
collective); the reported value is all ranks' sequences per second over the slowest rank's device time.

Prints ONE JSON line.  ``value`` is device-timed with inputs resident in HBM; ``e2e`` goes through the public cache /
operator API with pinned host buffers (H2D of q, k, v and D2H of the output inside the timed region); ``roofline``
is algorithmic bytes of the decode call over its CUDA-event duration against the measured copy bandwidth;
``cpu_baseline`` is the CPU oracle (a port of the reference's CPU path) timed on this host; ``extra`` holds the
TurboQuant configurations (packed decode, fused append) measured the same way.

``--impl reference`` times that CPU port alone (rank 0 only) and prints the same line shape.
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
# dram__bytes_read + dram__bytes_write of the decode kernel over its algorithmic bytes, from the ncu capture of
# `--profile-case paged` (same kernel and shape at half the batch); traffic grows with the bytes streamed.
NCU_TRAFFIC_RATIO = 1.019
NCU_TRAFFIC_SOURCE = "ncu capture of --profile-case paged (253.9 MB moved for 249.2 MB algorithmic), scaled by bytes"


# ---------------------------------------------------------------------------------------------------------------
# workload definitions


def cfg2_spec() -> dict:
    return {"workload": "cfg2: unquantized paged bf16 GQA decode", "batch": 32, "q_heads": 32, "kv_heads": 8,
            "head_dim": 128, "page_size": 16, "context": "uniform[1024,8192]", "dtype": "bf16",
            "block_tables": "seeded random permutation of a shared page pool", "append_per_step": 1}


def cfg2_lengths(seed: int, batch: int = 32) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(1024, 8193, (batch,), generator=gen).tolist()


def measured_peak_gbs() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001 - fall through to the stated fallback
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc: subprocess.Popen | None = None
        self.lines: list[str] = []
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
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

    def barrier(self) -> None:
        if self.enabled:
            self.dist.barrier()

    def max(self, value: float, device) -> float:
        if not self.enabled:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum(self, value: float, device) -> float:
        if not self.enabled:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=device)
        self.dist.all_reduce(t)
        return float(t.item())

    def close(self) -> None:
        if self.enabled:
            self.dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
# GPU arm: cfg2


def build_cfg2_state(device, seed: int, headroom_tokens: int):
    """Paged bf16 cache holding the cfg2 batch; returns (cache, lengths, host copies for the CPU baseline)."""
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache, Qwen3PageAllocator

    spec = cfg2_spec()
    batch, kv_heads, dim, page = spec["batch"], spec["kv_heads"], spec["head_dim"], spec["page_size"]
    lengths = cfg2_lengths(seed, batch)
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    allocator = Qwen3PageAllocator(config)
    total_pages = sum((n + headroom_tokens + page - 1) // page for n in lengths) + 32
    template = torch.empty(1, kv_heads, 1, dim, device=device, dtype=torch.bfloat16)
    layer = allocator.layers[0]
    layer.ensure_capacity(total_pages, key_template=template, value_template=template)
    perm = torch.randperm(layer.capacity(), generator=torch.Generator().manual_seed(seed + 1)).tolist()
    layer.free_pages[:] = perm  # block tables become a seeded random permutation of the shared pool
    caches = []
    gen = torch.Generator(device=device).manual_seed(seed + 2)
    for n in lengths:
        cache = Qwen3DynamicCache(config, allocator=allocator)
        cache.reserve_sequence_capacity(n + headroom_tokens)
        k = torch.randn(1, kv_heads, n, dim, device=device, dtype=torch.bfloat16, generator=gen)
        v = torch.randn(1, kv_heads, n, dim, device=device, dtype=torch.bfloat16, generator=gen)
        cache.update(k, v, 0, require_dense_cache=False)
        caches.append(cache)
    stacked = Qwen3DynamicCache.stack(caches, config)
    stacked.reserve_sequence_capacity(0)  # every row already holds the pages for its own headroom
    return stacked, lengths


def cfg2_bytes(lengths: list[int], spec: dict) -> int:
    """Algorithmic bytes of one decode call: every visible K and V element once per KV head (the GQA group shares
    it), q in, out, and the block-table entries."""
    dim, kv_heads, q_heads, page = spec["head_dim"], spec["kv_heads"], spec["q_heads"], spec["page_size"]
    kv = sum(lengths) * kv_heads * 2 * dim * 2
    qo = len(lengths) * q_heads * dim * 2 * 2
    table = sum((n + page - 1) // page for n in lengths) * 4
    return kv + qo + table


def run_cfg2_gpu(args, dist: Dist, device) -> dict:
    from anna_b200 import fused_ops

    spec = cfg2_spec()
    batch, q_heads, kv_heads, dim = spec["batch"], spec["q_heads"], spec["kv_heads"], spec["head_dim"]
    total_steps = 3 * (args.steps + args.warmup) + 8  # device-resident, serial and pipelined host loops
    cache, lengths = build_cfg2_state(device, seed=1234 + dist.rank, headroom_tokens=total_steps)
    scaling = dim ** -0.5
    gen = torch.Generator(device=device).manual_seed(99 + dist.rank)
    q_dev = torch.randn(batch, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    k_dev = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    v_dev = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)

    def step_resident():
        cache.update(k_dev, v_dev, 0, require_dense_cache=False)
        key_pages, value_pages, table, visible = cache.paged_attention_state(0)
        return key_pages, value_pages, table, visible

    decode_ms: list[float] = []

    def decode(state, record: bool):
        key_pages, value_pages, table, visible = state
        if record:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        out = fused_ops.run_paged_gqa_decode_fused(query=q_dev, key_pages=key_pages, value_pages=value_pages,
                                                   page_table=table, visible_lengths=visible, scaling=scaling)
        if record:
            stop.record()
            decode_events.append((start, stop))
        return out

    # ---- device-resident timing ------------------------------------------------------------------------------------
    # The clock sampler starts before warm-up; after the W warm-up steps the same decode launch is repeated (no
    # append, so no extra pages) until nvidia-smi has delivered samples under this load, then the K timed steps run
    # back to back with the sampler still on.
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    state = None
    for _ in range(args.warmup):
        state = step_resident()
        decode(state, False)
    spin_deadline = time.perf_counter() + 3.0
    while not args.no_clock_spin and len(sampler.lines) < 8 and time.perf_counter() < spin_deadline:
        for _ in range(50):
            decode(state, False)
        torch.cuda.synchronize(device)
    decode_events: list = []
    torch.cuda.synchronize(device)
    dist.barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(args.steps):
        decode(step_resident(), True)
    end.record()
    torch.cuda.synchronize(device)
    dist.barrier()
    clocks = sampler.stop()
    local_ms = begin.elapsed_time(end)
    decode_ms = [a.elapsed_time(b) for a, b in decode_events]
    step_ms = dist.max(local_ms, device) / args.steps
    value = dist.world * batch / (step_ms / 1e3)

    lengths_mid = [n + args.warmup + args.steps // 2 + 1 for n in lengths]
    algo_bytes = cfg2_bytes(lengths_mid, spec)
    kernel_ms = statistics.mean(decode_ms)
    peak, peak_kind = measured_peak_gbs()
    achieved = algo_bytes / (kernel_ms / 1e3) / 1e9

    # ---- end to end through the public API with host buffers --------------------------------------------------------
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
        key_pages, value_pages, table, visible = cache.paged_attention_state(0)
        out = fused_ops.run_paged_gqa_decode_fused(query=q, key_pages=key_pages, value_pages=value_pages,
                                                   page_table=table, visible_lengths=visible, scaling=scaling)
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

    e2e_serial_s = timed_e2e(False)
    e2e_s = timed_e2e(True)
    e2e_value = dist.world * batch * args.steps / e2e_s
    out_host = out_hosts[0]
    h2d = in_host.numel() * 2
    d2h = out_host.numel() * 2

    result = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": dist.world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded N(0,1) bf16, random-permutation block tables)",
        "config": {**spec, "l2_policy": "working set (705 MB of K/V per step) exceeds the 126 MB L2",
                   "per_rank_batch": batch, "parallelism": f"sequence-sharded x{dist.world}, no collective"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_s / args.steps * 1e3, "pipeline_depth": 2,
                "serial_value": dist.world * batch * args.steps / e2e_serial_s,
                "note": "value: results return asynchronously into two pinned buffers, the host waits for a buffer "
                        "only before reusing it; serial_value: the host waits for every step's result before the next"},
        "gpu_launches": 2 * args.steps,  # per step: paged_kv_write_kernel + the decode kernel (merge fused in its tail)
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": int(algo_bytes * NCU_TRAFFIC_RATIO), "traffic_source": NCU_TRAFFIC_SOURCE,
                     "peak_kind": peak_kind, "kernel": "dense_decode_balanced_mma_kernel (split pass with the merge fused into its tail)",
                     "algorithmic_bytes_per_launch": algo_bytes, "launch_ms": kernel_ms,
                     "frac_of_8TBps_nominal": achieved / 8000.0},
    }
    cache.release()
    return result


# ---------------------------------------------------------------------------------------------------------------
# KV-head-sharded variant of cfg5 (--variant kvhead): every rank holds all sequences but only its KV heads


def run_kvhead_variant(args, dist: Dist, device) -> dict:
    """TurboQuant 4-bit decode, all sequences on every rank, Hkv / N KV heads per rank, one all-gather of the outputs
    per step.  Total work is fixed, so the scaling is "strong"."""
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache
    from anna_b200.sharding import HeadGather, shard_kv_heads

    q_heads, kv_heads, dim, page, bits, residual = 32, 8, 128, 16, 4, 128
    batch, context = args.kvhead_batch, args.kvhead_context
    shard = shard_kv_heads(q_heads, kv_heads, dist.world, dist.rank)
    local_kv, local_q = shard.kv_stop - shard.kv_start, shard.q_stop - shard.q_start
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    gather = HeadGather() if dist.enabled else (lambda out: out)

    def build(rows: int, tokens: int, kv_slice: slice, seed: int):
        cache = Qwen3DynamicCache(config, batch_size=rows, kv_cache_quantization="turboquant",
                                  kv_cache_quant_bits=bits, kv_cache_residual_len=residual)
        cache.reserve_sequence_capacity(tokens + 8 * (args.steps + args.warmup) + 64)
        gen = torch.Generator(device=device).manual_seed(seed)  # the same stream of numbers on every rank
        done = 0
        while done < tokens:
            step = min(2048, tokens - done)
            k = torch.randn(rows, kv_heads, step, dim, device=device, dtype=torch.bfloat16, generator=gen)
            v = torch.randn(rows, kv_heads, step, dim, device=device, dtype=torch.bfloat16, generator=gen)
            cache.update(k[:, kv_slice], v[:, kv_slice], 0, require_dense_cache=False)
            done += step
            del k, v
        return cache

    # self-check on a small problem: gathered sharded outputs == the unsharded computation of the same data
    check_rows, check_tokens = 2, 700
    full = build(check_rows, check_tokens, slice(0, kv_heads), seed=5)
    part = build(check_rows, check_tokens, slice(shard.kv_start, shard.kv_stop), seed=5)
    q_check = torch.randn(check_rows, q_heads, 1, dim, device=device, dtype=torch.bfloat16,
                          generator=torch.Generator(device=device).manual_seed(6))
    want = full.turboquant_single_token_decode_attention(0, q_check, scaling=dim ** -0.5,
                                                         num_key_value_groups=q_heads // kv_heads)
    got = gather(part.turboquant_single_token_decode_attention(0, shard.slice_q(q_check), scaling=dim ** -0.5,
                                                               num_key_value_groups=q_heads // kv_heads))
    check_err = float((got.float() - want.float()).abs().max())
    if not check_err <= 2e-2:
        raise RuntimeError(f"KV-head-sharded decode disagrees with the unsharded one: max abs {check_err}")
    full.release()
    part.release()

    cache = build(batch, context, slice(shard.kv_start, shard.kv_stop), seed=11)
    gen = torch.Generator(device=device).manual_seed(12)
    q = torch.randn(batch, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    k1 = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    v1 = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    q_local, k_local, v_local = shard.slice_q(q), shard.slice_kv(k1), shard.slice_kv(v1)

    def step():
        cache.update(k_local, v_local, 0, require_dense_cache=False)
        local = cache.turboquant_single_token_decode_attention(0, q_local, scaling=dim ** -0.5,
                                                               num_key_value_groups=q_heads // kv_heads)
        return gather(local)

    sampler = ClockSampler(device.index or 0)
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(device)
    dist.barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(args.steps):
        out = step()
    end.record()
    torch.cuda.synchronize(device)
    dist.barrier()
    clocks = sampler.stop()
    step_ms = dist.max(begin.elapsed_time(end), device) / args.steps
    key_bytes = dim * bits // 8 + 8
    value_bytes = dim // 2 + 2 * (dim // 32) * 2
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
                   "parallelism": f"kv-head-sharded x{dist.world}, one all-gather of [B, Hq/N, D] per step",
                   "l2_policy": f"{per_rank_bytes / 1e6:.0f} MB of packed KV per rank and step exceed the 126 MB L2"},
        # per step: tq_append, tq_prepare_queries, tq_window_split_mma, tq_decode_split_mma (+ NCCL's all-gather and
        # one strided copy, which are library kernels and not counted)
        "gpu_launches": 4 * args.steps, "clocks": clocks,
        "self_check": {"max_abs_vs_unsharded": check_err, "rows": check_rows, "context": check_tokens},
        "roofline": {"bound": "hbm (issue-bound today)", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_kind": peak_kind,
                     "kernel": "tq_decode_split_mma_kernel (whole step incl. append and all-gather)",
                     "algorithmic_bytes_per_launch": per_rank_bytes, "launch_ms": step_ms},
        "out_shape": list(out.shape),
    }


# ---------------------------------------------------------------------------------------------------------------
# TurboQuant extras (single GPU): packed decode and fused append, device-timed


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


def run_turboquant_extra(device, *, name: str, batch: int, q_heads: int, kv_heads: int, dim: int, bits: int,
                         context: int, residual: int = 128, page: int = 16, chunk: int = 2048) -> dict:
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache

    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    cache = Qwen3DynamicCache(config, batch_size=batch, kv_cache_quantization="turboquant", kv_cache_quant_bits=bits,
                              kv_cache_residual_len=residual)
    gen = torch.Generator(device=device).manual_seed(7)
    key_bytes = dim * bits // 8 + 8
    value_bytes = dim // (4 if bits == 2 else 2) + 2 * (dim // 32) * 2
    from anna_b200.turboquant import launch_tq_append

    cache.reserve_sequence_capacity(context + 64)
    done, bulk_ms, bulk_api_ms, bulk_tokens = 0, None, None, 0
    while done < context:
        tokens = min(chunk, context - done)
        k = torch.randn(batch, kv_heads, tokens, dim, device=device, dtype=torch.bfloat16, generator=gen)
        v = torch.randn(batch, kv_heads, tokens, dim, device=device, dtype=torch.bfloat16, generator=gen)
        if done == 0:
            cache.update(k, v, 0, require_dense_cache=False)  # binds rows, sizes the pool
            pool = cache.allocator.turboquant_layers[0]
            pool.ensure_capacity(batch * ((context + 64 + page - 1) // page) + 16)
        elif tokens == chunk and bulk_ms is None:
            # host bookkeeping first, then the launch alone between two events
            rows = cache.turboquant_rows[0]
            past = [row.length for row in rows]
            for row in rows:
                row._reserve_blocks(row.length + tokens)
            table = cache._sync_page_table_layer_buffer(0, batch_size=batch, device=device)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            launch_tq_append(pool, k, v, table, [row.slot for row in rows], past)
            stop.record()
            torch.cuda.synchronize()
            bulk_ms, bulk_tokens = start.elapsed_time(stop), tokens
            for idx, row in enumerate(rows):
                row._length += tokens
                cache.layer_lengths[0][idx] = row.length
        else:
            t0 = time.perf_counter()
            cache.update(k, v, 0, require_dense_cache=False)
            torch.cuda.synchronize()
            if tokens == chunk:
                bulk_api_ms = (time.perf_counter() - t0) * 1e3
        done += tokens
        del k, v
    q = torch.randn(batch, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    k1 = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    v1 = torch.randn(batch, kv_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
    decode_ms = _time_device(lambda: cache.turboquant_single_token_decode_attention(
        0, q, scaling=dim ** -0.5, num_key_value_groups=q_heads // kv_heads), iters=10, warmup=3)
    append_ms = _time_device(lambda: cache.update(k1, v1, 0, require_dense_cache=False), iters=10, warmup=3)
    quantized = context - residual
    decode_bytes = (batch * kv_heads * (quantized * (key_bytes + value_bytes) + residual * 2 * dim * 2)
                    + batch * q_heads * dim * 2 * 2 + batch * ((quantized + page - 1) // page) * 4)
    peak, _ = measured_peak_gbs()
    out = {"workload": name, "batch": batch, "q_heads": q_heads, "kv_heads": kv_heads, "head_dim": dim, "bits": bits,
           "context": context, "decode_ms": decode_ms, "decode_tokens_per_s": batch / (decode_ms / 1e3),
           "decode_algorithmic_bytes": decode_bytes, "decode_GBps": decode_bytes / (decode_ms / 1e3) / 1e9,
           "decode_frac_of_measured_peak": decode_bytes / (decode_ms / 1e3) / 1e9 / peak,
           "step_append_ms": append_ms,
           "step_tokens_per_s": batch / ((decode_ms + append_ms) / 1e3)}
    if bulk_ms:
        bulk_bytes = batch * kv_heads * bulk_tokens * (2 * dim * 2 + key_bytes + value_bytes)
        out.update({"bulk_append_tokens": bulk_tokens, "bulk_append_kernel_ms": bulk_ms,
                    "bulk_append_api_ms_host_timed": bulk_api_ms, "quant_append_algorithmic_bytes": bulk_bytes,
                    "quant_append_GBps": bulk_bytes / (bulk_ms / 1e3) / 1e9,
                    "quant_append_frac_of_measured_peak": bulk_bytes / (bulk_ms / 1e3) / 1e9 / peak})
    cache.release()
    cache.allocator.trim()
    return out


# ---------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU path for cfg2 (gather pages -> dense K/V -> fp32 attention)


def cpu_cfg2_step_seconds(rows: int, seed: int, steps: int) -> tuple[float, int]:
    """Times `steps` decode steps of the CPU port on `rows` sequences of the cfg2 batch; returns (seconds per step
    for those rows, host threads used).  Port of Qwen3DynamicCache.update + _gather_layer_cache +
    materialized_kv_single_token_decode_attention, CPU branch (src/anna/model/ops.py:662-777, :931-1006, :1604-1615)."""
    import oracle

    spec = cfg2_spec()
    kv_heads, q_heads, dim, page = spec["kv_heads"], spec["q_heads"], spec["head_dim"], spec["page_size"]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    lengths = cfg2_lengths(seed)[:rows]
    rng = np.random.default_rng(seed)
    blocks = [(n + steps + page - 1) // page for n in lengths]
    total = sum(blocks)
    perm = rng.permutation(total)
    key_pages = oracle.round_bf16(rng.standard_normal((total, kv_heads, page, dim), dtype=np.float32))
    value_pages = oracle.round_bf16(rng.standard_normal((total, kv_heads, page, dim), dtype=np.float32))
    tables, offset = [], 0
    for count in blocks:
        tables.append(perm[offset:offset + count])
        offset += count
    q = oracle.round_bf16(rng.standard_normal((rows, q_heads, dim), dtype=np.float32))
    new_k = oracle.round_bf16(rng.standard_normal((rows, kv_heads, dim), dtype=np.float32))
    new_v = oracle.round_bf16(rng.standard_normal((rows, kv_heads, dim), dtype=np.float32))
    cur = list(lengths)

    def one_step():
        for r in range(rows):
            pos = cur[r]
            pid = tables[r][pos // page]
            key_pages[pid, :, pos % page] = new_k[r]
            value_pages[pid, :, pos % page] = new_v[r]
            cur[r] = pos + 1
            n = cur[r]
            used = tables[r][: (n + page - 1) // page]
            k = key_pages[used].transpose(1, 0, 2, 3).reshape(kv_heads, -1, dim)[:, :n]
            v = value_pages[used].transpose(1, 0, 2, 3).reshape(kv_heads, -1, dim)[:, :n]
            oracle.gqa_decode_blas(q[r], k, v, dim ** -0.5)

    one_step()
    t0 = time.perf_counter()
    for _ in range(steps - 1):
        one_step()
    return (time.perf_counter() - t0) / max(1, steps - 1), threads


def run_reference_arm(args, dist: Dist) -> dict | None:
    if dist.rank != 0:
        return None
    spec = cfg2_spec()
    batch = spec["batch"]
    rows = batch
    probe, threads = cpu_cfg2_step_seconds(4, 1234, 2)
    if probe * (batch / 4) * (args.steps + args.warmup) > 150.0:
        rows = 8
    seconds, threads = cpu_cfg2_step_seconds(rows, 1234, args.steps + args.warmup + 1)
    step_s = seconds * (batch / rows)
    value = batch * dist.world / step_s
    sample = (f"{rows} of {batch} sequences per step" + (", scaled linearly by rows" if rows != batch else "")
              + f", {args.steps + args.warmup} steps, numpy fp32 BLAS")
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": dist.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded N(0,1) rounded to bf16)",
        "config": {**spec, "note": "CPU port of the reference's CPU path (oracle/), host cores only"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ---------------------------------------------------------------------------------------------------------------
# small cases for profiler captures (inputs larger than L2, well under a GB on the device, a handful of launches)


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
    return {"workload": f"cfg4-like prefill attention: {batch} seq x {chunk}-token chunk over {past} cached tokens, "
                        f"{q_heads}q/{kv_heads}kv heads, D={dim}, bf16 dense K/V",
            "prefill_ms": ms, "prefill_tokens_per_s": batch * chunk / (ms / 1e3), "algorithmic_flops": flops,
            "TFLOPs": tflops, "frac_of_measured_bf16_peak": None if peak_tflops is None else tflops / peak_tflops,
            "bound": "tensor"}


def run_profile_case(case: str, device) -> dict:
    from anna_b200 import KVCacheConfig, Qwen3DynamicCache, Qwen3PageAllocator, fused_ops

    gen = torch.Generator(device=device).manual_seed(3)
    if case == "paged":
        # half of the headline batch: 16 ragged rows drawn like cfg2's, block tables a permutation of the pool
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
        packed = dim * 4 // 8 + 8 + dim // 2 + 2 * (dim // 32) * 2
        algo = batch * kv_heads * tokens * (2 * 2 * dim * 2 + packed)  # ring/incoming read + ring write + packed write
    else:
        bits = {"tq4": 4, "tq3": 3, "tq2": 2}[case]
        batch, q_heads, kv_heads, dim, page, context = (32, 16, 2, 256, 16, 8320) if bits == 2 else \
            (16, 32, 8, 128, 16, 8320)
        config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
        cache = Qwen3DynamicCache(config, batch_size=batch, kv_cache_quantization="turboquant",
                                  kv_cache_quant_bits=bits, kv_cache_residual_len=128)
        for _ in range(context // 2080):
            k = torch.randn(batch, kv_heads, 2080, dim, device=device, dtype=torch.bfloat16, generator=gen)
            v = torch.randn(batch, kv_heads, 2080, dim, device=device, dtype=torch.bfloat16, generator=gen)
            cache.update(k, v, 0, require_dense_cache=False)
        q = torch.randn(batch, q_heads, 1, dim, device=device, dtype=torch.bfloat16, generator=gen)
        fn = lambda: cache.turboquant_single_token_decode_attention(  # noqa: E731
            0, q, scaling=dim ** -0.5, num_key_value_groups=q_heads // kv_heads)
        per_token = dim * bits // 8 + 8 + dim // (4 if bits == 2 else 2) + 2 * (dim // 32) * 2
        algo = batch * kv_heads * ((context - 128) * per_token + 128 * 2 * dim * 2)
    ms = _time_device(fn, iters=3, warmup=2)
    return {"profile_case": case, "decode_ms": ms, "algorithmic_bytes": algo, "GBps": algo / (ms / 1e3) / 1e9}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-extras", action="store_true", help="skip the TurboQuant configurations")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--variant", choices=("sequence", "kvhead"), default="sequence",
                        help="sequence: rows sharded over ranks (default, the headline); kvhead: the TurboQuant 4-bit "
                             "decode with KV heads sharded over ranks and an all-gather of the outputs")
    parser.add_argument("--kvhead-batch", type=int, default=128)
    parser.add_argument("--kvhead-context", type=int, default=32768)
    parser.add_argument("--no-clock-spin", action="store_true",
                        help="do not repeat the decode launch while waiting for clock samples (for profiler runs)")
    parser.add_argument("--profile-case", choices=("paged", "tq4", "tq3", "tq2", "tqappend", "prefill"), default=None,
                        help="run one small decode case a few times and exit (meant to be wrapped by ncu)")
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
    device = torch.device("cuda", dist.local_rank)
    torch.cuda.set_device(device)
    if args.variant == "kvhead":
        result = run_kvhead_variant(args, dist, device)
        dist.barrier()
        if dist.rank == 0:
            print(json.dumps(result))
        dist.close()
        return
    result = run_cfg2_gpu(args, dist, device)

    if dist.rank == 0 and dist.world == 1:
        if not args.no_cpu_baseline:
            rows = 8
            seconds, threads = cpu_cfg2_step_seconds(rows, 1234, 4)
            batch = cfg2_spec()["batch"]
            result["cpu_baseline"] = {
                "value": batch / (seconds * batch / rows), "unit": UNIT, "cores": threads, "kind": "port",
                "sample": f"{rows} of {batch} sequences, 3 timed steps, scaled linearly by rows (numpy fp32 BLAS port "
                          "of the reference's gather + attention CPU path)"}
        if not args.no_extras:
            extras = []
            for kwargs in (
                dict(name="cfg3-like: TurboQuant 2-bit, 64 seq x 18432 ctx (mean of uniform[4096,32768])", batch=64,
                     q_heads=16, kv_heads=2, dim=256, bits=2, context=18432),
                dict(name="cfg5 per-GPU shard at 8 GPUs: TurboQuant 4-bit, 64 seq x 32768 ctx", batch=64, q_heads=32,
                     kv_heads=8, dim=128, bits=4, context=32768),
                dict(name="cfg4-like: TurboQuant 3-bit, 128 seq x 8448 ctx + 2048-token chunk appends", batch=128,
                     q_heads=16, kv_heads=4, dim=128, bits=3, context=8448),
            ):
                try:
                    extras.append(run_turboquant_extra(device, **kwargs))
                except Exception as exc:  # noqa: BLE001 - extras never take the headline down
                    extras.append({"workload": kwargs["name"], "error": repr(exc)})
            try:
                extras.append(run_prefill_extra(device))
            except Exception as exc:  # noqa: BLE001
                extras.append({"workload": "cfg4-like prefill attention", "error": repr(exc)})
            result["extra"] = extras
    dist.barrier()
    if dist.rank == 0:
        print(json.dumps(result))
    dist.close()


if __name__ == "__main__":
    main()
