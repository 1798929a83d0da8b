"""GPU: replay of what Anna's real scheduler does to the KV cache.

tests/golden/scheduler_trace.* was recorded by running the reference's AnnaScheduler and AnnaQwen3_5TextEngine on CPU
around a stand-in model (tests/golden/make_scheduler_trace.py): every update / stack / compact_batch_rows / release /
reserve_sequence_capacity call that reached the reference's Qwen3DynamicCache, with the cache state after it (row
lengths, block tables, pages in use) and, at every decode step, the query and the reference's own attention output.
The same calls are made here on the CUDA cache: block tables, lengths and page counts must be identical after every
call (the engine's kv_cache_used_pages metric is computed from them, src/anna/runtime/qwen3_5_text_engine.py:1335-1346)
and the decode outputs must agree with the reference's."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from anna_b200 import KVCacheConfig, Qwen3DynamicCache, Qwen3PageAllocator, fused_ops
from tests.helpers import to_np

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _used_and_total_pages(allocator) -> tuple[int, int]:
    """AnnaQwen3_5TextEngine._kv_cache_page_counts over this allocator's un-quantized layers."""
    used = total = 0
    for layer in allocator.layers:
        if layer.key_pages is None:
            continue
        capacity = int(layer.key_pages.shape[0])
        used += max(0, min(capacity, capacity - len(layer.free_pages)))
        total += capacity
    return used, total


@pytest.mark.parametrize("run_index", [0, 1, 2])
def test_replay_of_the_reference_scheduler_trace(cuda_device, run_index):
    trace = json.loads((GOLDEN / "scheduler_trace.json").read_text())
    tensors = np.load(GOLDEN / "scheduler_trace.npz")
    run = trace["runs"][run_index]
    heads, kv_heads, dim, block = trace["heads"], trace["kv_heads"], trace["head_dim"], trace["block_size"]
    quantized = run["quantization"] == "turboquant"
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=block)
    allocator = Qwen3PageAllocator(config)
    caches: dict[int, Qwen3DynamicCache] = {}

    def tensor(name: str) -> torch.Tensor:
        return torch.from_numpy(tensors[f"run{run_index}_{name}"]).to(cuda_device)

    probes = 0
    for event in run["events"]:
        op = event["op"]
        if op == "new":
            caches[event["id"]] = Qwen3DynamicCache(
                config, allocator=allocator, batch_size=event["batch_size"],
                kv_cache_quantization=event["quantization"], kv_cache_quant_bits=event["bits"],
                kv_cache_residual_len=event["residual_len"])
        elif op == "update":
            caches[event["id"]].update(tensor(event["key"]), tensor(event["value"]), 0,
                                       require_dense_cache=event["require_dense_cache"])
        elif op == "stack":
            caches[event["out"]] = Qwen3DynamicCache.stack([caches[i] for i in event["inputs"]], config,
                                                           clone_turboquant_rows=event["clone_turboquant_rows"])
        elif op == "split_batch":
            parts = caches[event["id"]].split_batch(clone_turboquant_rows=event["clone_turboquant_rows"])
            for handle, part in zip(event["out"], parts):
                caches[handle] = part
        elif op == "compact_batch_rows":
            caches[event["out"]] = caches[event["id"]].compact_batch_rows(
                event["rows"], release_unselected=event["release_unselected"])
        elif op == "release":
            caches[event["id"]].release()
        elif op == "reserve_sequence_capacity":
            caches[event["id"]].reserve_sequence_capacity(event["seq_length"])
        elif op == "decode_probe":
            cache = caches[event["id"]]
            assert cache.layer_lengths[0] == event["lengths"]
            query = tensor(event["query"])
            if quantized:
                out = cache.turboquant_single_token_decode_attention(0, query, scaling=dim ** -0.5,
                                                                     num_key_value_groups=heads // kv_heads)
                tol = 2e-3   # fp32 TurboQuant tolerance of the parity tests
            else:
                key_pages, value_pages, table, visible = cache.paged_attention_state(0)
                out = fused_ops.run_paged_gqa_decode_fused(query=query, key_pages=key_pages, value_pages=value_pages,
                                                           page_table=table, visible_lengths=visible,
                                                           scaling=dim ** -0.5)
                tol = 2e-4   # fp32 tolerance of the paged decode parity tests
            np.testing.assert_allclose(to_np(out), tensors[f"run{run_index}_{event['output']}"], atol=tol, rtol=tol)
            probes += 1
        else:
            raise AssertionError(f"unknown trace event {op}")
        for handle, want in (event.get("after") or {}).items():
            cache = caches[int(handle)]
            got_lengths = cache.layer_lengths[0] if cache.layer_lengths else []
            assert list(got_lengths) == want["lengths"], (op, handle)
            if quantized:
                rows = cache.turboquant_rows[0] if cache.turboquant_rows else []
                if "quantized" in want:
                    assert [0 if r is None else r.quantized_length for r in rows] == want["quantized"], (op, handle)
                    assert [0 if r is None else r.residual_length for r in rows] == want["residual"], (op, handle)
            else:
                got_tables = cache.page_tables[0] if cache.page_tables else []
                assert [list(t) for t in got_tables] == want["tables"], (op, handle)
        if not quantized and "used_pages" in event:
            # what the engine publishes as kv_cache_used_pages / kv_cache_total_pages
            assert _used_and_total_pages(allocator) == (event["used_pages"], event["capacity"]), op
    assert probes > 0
    if not quantized:
        assert _used_and_total_pages(allocator)[0] == run["final_used_pages"]
