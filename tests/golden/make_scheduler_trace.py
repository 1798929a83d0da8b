"""Record what Anna's real scheduler does to the KV cache, as a replayable trace.

    python tests/golden/make_scheduler_trace.py --reference /path/to/Anna

The reference's ``AnnaScheduler`` and ``AnnaQwen3_5TextEngine`` run unchanged on CPU (imported from ``<reference>/src``;
``soundfile`` is stubbed because the runtime package imports it, ``turboquant.core`` comes from
oracle/turboquant_core_shim.py) around a stand-in model with one attention layer that does what ``Qwen3Attention`` does
to the cache: ``update`` with the new keys / values of every forward, and a single-token attention read in decode
steps.  Every top-level call that reaches ``Qwen3DynamicCache`` -- construction, ``update``, ``stack``, ``split_batch``,
``compact_batch_rows``, ``reserve_sequence_capacity``, ``release`` -- is written down with its arguments, followed by
what the reference's cache looked like afterwards (row lengths, block tables, pages in use).  Decode steps also store
the query and the reference's own attention output.

Three runs are recorded: un-quantized and TurboQuant (4 bit, window 8) with requests of different prompt and
completion lengths submitted together, so that the scheduler stacks single-row caches into a decode group, compacts
the group when rows finish and releases caches; and an un-quantized run whose requests arrive in waves while earlier
ones decode.  Output: ``scheduler_trace.json`` (events) and ``scheduler_trace.npz`` (tensors).
"""
from __future__ import annotations

import argparse
import json
import sys
import threading
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

HEADS, KV_HEADS, HEAD_DIM, BLOCK = 8, 2, 64, 16


class Recorder:
    """Wraps the cache class of the reference; only calls made from outside the class are recorded."""

    def __init__(self, cache_cls, allocator_of) -> None:
        self.cache_cls = cache_cls
        self.allocator_of = allocator_of
        self.events: list[dict] = []
        self.tensors: dict[str, np.ndarray] = {}
        self.ids: dict[int, int] = {}
        self.keep: list[object] = []   # keeps recorded caches alive so that id() values are never reused
        self.depth = threading.local()
        self.lock = threading.RLock()

    def handle(self, cache) -> int:
        key = id(cache)
        if key not in self.ids:
            self.ids[key] = len(self.ids)
            self.keep.append(cache)
        return self.ids[key]

    def tensor(self, value: torch.Tensor) -> str:
        name = f"t{len(self.tensors)}"
        self.tensors[name] = value.detach().to(torch.float32).cpu().numpy()
        return name

    def state(self, caches) -> dict:
        out = {}
        for cache in caches:
            rows = cache.turboquant_rows[0] if cache.turboquant_rows and cache.turboquant_rows[0] else []
            entry = {"lengths": [int(n) for n in cache.layer_lengths[0]] if cache.layer_lengths else [],
                     "tables": [list(map(int, t)) for t in cache.page_tables[0]] if cache.page_tables else []}
            if any(row is not None for row in rows):
                entry["quantized"] = [0 if row is None else int(row.quantized_length) for row in rows]
                entry["residual"] = [0 if row is None else int(row.residual_length) for row in rows]
            out[str(self.handle(cache))] = entry
        return out

    def wrap(self, name: str, describe):
        original = getattr(self.cache_cls, name)
        is_classmethod = isinstance(self.cache_cls.__dict__[name], classmethod)
        func = original.__func__ if is_classmethod else original
        recorder = self

        def wrapped(first, *args, **kwargs):
            depth = getattr(recorder.depth, "value", 0)
            recorder.depth.value = depth + 1
            try:
                result = func(first, *args, **kwargs)
            finally:
                recorder.depth.value = depth
            if depth == 0:
                with recorder.lock:
                    event, touched = describe(first, args, kwargs, result)
                    event["op"] = name
                    allocator = recorder.allocator_of(touched[0]) if touched else None
                    event["after"] = recorder.state(touched)
                    if allocator is not None:
                        layer = allocator.layers[0]
                        event["used_pages"] = int(layer.used_pages())
                        event["capacity"] = int(layer.capacity())
                    recorder.events.append(event)
            return result

        setattr(self.cache_cls, name, classmethod(wrapped) if is_classmethod else wrapped)


def install_recorder(ref_ops) -> Recorder:
    cls = ref_ops.Qwen3DynamicCache
    rec = Recorder(cls, lambda cache: cache.allocator)

    original_init = cls.__init__

    def init(self, config, **kwargs):
        original_init(self, config, **kwargs)
        if getattr(rec.depth, "value", 0) == 0:
            with rec.lock:
                rec.events.append({"op": "new", "id": rec.handle(self), "batch_size": int(kwargs.get("batch_size", 0)),
                                   "quantization": kwargs.get("kv_cache_quantization", "none"),
                                   "bits": int(kwargs.get("kv_cache_quant_bits", 4)),
                                   "residual_len": int(kwargs.get("kv_cache_residual_len", 128))})

    cls.__init__ = init
    rec.wrap("update", lambda self, a, kw, res: (
        {"id": rec.handle(self), "key": rec.tensor(a[0]), "value": rec.tensor(a[1]),
         "require_dense_cache": bool(kw.get("require_dense_cache", True))}, [self]))
    rec.wrap("stack", lambda cls_, a, kw, res: (
        {"inputs": [rec.handle(c) for c in a[0]], "out": rec.handle(res),
         "clone_turboquant_rows": bool(kw.get("clone_turboquant_rows", True))}, [res]))
    rec.wrap("split_batch", lambda self, a, kw, res: (
        {"id": rec.handle(self), "out": [rec.handle(c) for c in res],
         "clone_turboquant_rows": bool(kw.get("clone_turboquant_rows", True))}, list(res)))
    rec.wrap("compact_batch_rows", lambda self, a, kw, res: (
        {"id": rec.handle(self), "rows": [int(i) for i in a[0]], "out": rec.handle(res),
         "release_unselected": bool(kw.get("release_unselected", True))}, [res]))
    rec.wrap("release", lambda self, a, kw, res: ({"id": rec.handle(self)}, [self]))
    rec.wrap("reserve_sequence_capacity", lambda self, a, kw, res: (
        {"id": rec.handle(self), "seq_length": int(a[0] if a else kw["seq_length"])}, [self]))
    return rec


class StandInModel:
    """One attention layer's worth of cache traffic behind the model interface the engine and the scheduler use."""

    def __init__(self, config, ref_ops, recorder: Recorder, quantization: str, seed: int) -> None:
        self.config = config
        self.ref_ops = ref_ops
        self.recorder = recorder
        self.quantization = quantization
        self.cache_allocator = ref_ops.Qwen3PageAllocator(config.text_config)
        self.gen = torch.Generator().manual_seed(seed)
        self.model = self._prefill_hidden
        self.lm_head = self._logits_from_hidden

    def _new_kv(self, batch: int, tokens: int):
        shape = (batch, KV_HEADS, tokens, HEAD_DIM)
        return torch.randn(shape, generator=self.gen), torch.randn(shape, generator=self.gen)

    def _fresh_cache(self, batch: int):
        return self.ref_ops.Qwen3DynamicCache(
            self.config.text_config, allocator=self.cache_allocator, batch_size=batch,
            kv_cache_quantization=self.quantization, kv_cache_quant_bits=4, kv_cache_residual_len=8)

    def _logits(self, batch: int) -> torch.Tensor:
        logits = torch.full((batch, 1, self.config.text_config.vocab_size), -1000.0)
        logits[:, 0, 1] = 1000.0  # always the same ordinary token: requests end by their completion budget
        return logits

    def _forward(self, input_ids: torch.Tensor, cache):
        batch, tokens = int(input_ids.shape[0]), int(input_ids.shape[1])
        if cache is None:
            cache = self._fresh_cache(batch)
        key, value = self._new_kv(batch, tokens)
        decode = tokens == 1 and cache.get_seq_length() > 0
        cache.update(key, value, 0, require_dense_cache=False)
        if decode:
            self._attention_probe(cache, batch)
        return cache

    def _attention_probe(self, cache, batch: int) -> None:
        """The decode-step attention read of Qwen3Attention (ops.py:1877-2028), recorded with its result."""
        query = torch.randn((batch, HEADS, 1, HEAD_DIM), generator=self.gen)
        scaling = HEAD_DIM ** -0.5
        if cache.uses_turboquant_for_layer(0):
            out = cache.turboquant_single_token_decode_attention(0, query, scaling=scaling,
                                                                 num_key_value_groups=HEADS // KV_HEADS)
        else:
            keys, values, visible = cache._gather_layer_cache(0)
            positions = torch.arange(keys.shape[2])[None, :]
            out = self.ref_ops.grouped_query_attention(query, keys, values, scaling=scaling,
                                                       visible_mask=positions < visible[:, None])
        rec = self.recorder
        with rec.lock:
            rec.events.append({"op": "decode_probe", "id": rec.handle(cache), "query": rec.tensor(query),
                               "output": rec.tensor(out), "lengths": [int(n) for n in cache.layer_lengths[0]]})

    # -- the interface the engine calls (prefill through .model / .lm_head, text-only fast paths, generic call) ------
    def _prefill_hidden(self, *, input_ids, attention_mask=None, mm_token_type_ids=None, use_cache=None):
        cache = self._forward(input_ids, None)
        hidden = torch.zeros((input_ids.shape[0], input_ids.shape[1], self.config.text_config.hidden_size))
        return types.SimpleNamespace(last_hidden_state=hidden, past_key_values=cache)

    def _logits_from_hidden(self, hidden_states):
        return self._logits(int(hidden_states.shape[0]))[:, 0]

    def forward_text_only(self, *, input_ids, attention_mask=None, past_key_values=None, use_cache=None,
                          logits_to_keep=None):
        cache = self._forward(input_ids, past_key_values)
        return types.SimpleNamespace(logits=self._logits(int(input_ids.shape[0])), past_key_values=cache)

    def forward_text_only_topk(self, *, input_ids, attention_mask=None, past_key_values=None, use_cache=None,
                               logits_to_keep=None, top_k=1):
        cache = self._forward(input_ids, past_key_values)
        batch = int(input_ids.shape[0])
        candidate_logits = torch.full((batch, 1, top_k), -1000.0)
        candidate_logits[:, 0, 0] = 1000.0
        candidate_ids = torch.zeros((batch, 1, top_k), dtype=torch.long)
        candidate_ids[:, 0, 0] = 1
        return types.SimpleNamespace(candidate_logits=candidate_logits, candidate_token_ids=candidate_ids,
                                     past_key_values=cache)

    def __call__(self, *, input_ids, past_key_values=None, use_cache=None, logits_to_keep=None, **_):
        cache = self._forward(input_ids, past_key_values)
        return types.SimpleNamespace(logits=self._logits(int(input_ids.shape[0])), past_key_values=cache)


class PlainTokenizer:
    eos_token_ids = {9}

    def decode(self, token_ids, *, skip_special_tokens=False):
        return "".join("x" for _ in token_ids)


class CpuDeviceContext:
    def __init__(self, policy) -> None:
        self.device = torch.device("cpu")
        self.dtype = torch.float32
        self.safety_policy = policy

    def get_memory_info(self):
        return None

    def element_size(self, dtype):
        return torch.empty((), dtype=dtype).element_size()

    def move_prepared_inputs(self, prepared):
        return prepared

    def move_token_ids(self, token_ids):
        return token_ids


def record_run(quantization: str, requests: list[tuple], seed: int, ref) -> dict:
    """requests: (prompt tokens, completion tokens[, seconds to wait before submitting]) per request."""
    import time

    ref_ops, cfg_mod, engine_mod, sched_mod, prepared_mod, device_mod = ref
    text = cfg_mod.Qwen3_5TextConfig(
        hidden_size=8, intermediate_size=16, num_hidden_layers=1, num_attention_heads=HEADS,
        num_key_value_heads=KV_HEADS, head_dim=HEAD_DIM, linear_key_head_dim=4, linear_value_head_dim=4,
        linear_num_key_heads=1, linear_num_value_heads=1, vocab_size=16, eos_token_id=9, pad_token_id=0,
        cache_block_size=BLOCK, layer_types=["full_attention"])
    config = cfg_mod.Qwen3_5TextModelConfig(text_config=text)
    recorder = install_recorder(ref_ops)
    model = StandInModel(config, ref_ops, recorder, quantization, seed)
    engine = engine_mod.AnnaQwen3_5TextEngine(model=model, tokenizer=PlainTokenizer(), processor=object(),
                                               model_id="stand-in",
                                               device_context=CpuDeviceContext(device_mod.RuntimeSafetyPolicy()))
    scheduler = sched_mod.AnnaScheduler(engine, max_batch_size=8, batch_wait_ms=50.0)
    engine.set_scheduler(scheduler)
    try:
        submitted = []
        for prompt_len, completion, *delay in requests:
            if delay:
                time.sleep(delay[0])
            ids = torch.randint(2, 8, (1, prompt_len), generator=model.gen)
            prepared = prepared_mod.PreparedInputs(prompt="", input_ids=ids, attention_mask=torch.ones_like(ids),
                                                   mm_token_type_ids=torch.zeros_like(ids, dtype=torch.int32))
            submitted.append(scheduler._submit(
                prepared, stream=False,
                config=engine_mod.GenerationConfig(max_new_tokens=completion, temperature=0.0, top_p=1.0, top_k=0,
                                                   repetition_penalty=1.0)))
        for request in submitted:
            assert request.done.wait(timeout=60.0) and request.error is None, request.error
    finally:
        scheduler.shutdown()
    used = int(model.cache_allocator.layers[0].used_pages())
    return {"quantization": quantization, "requests": requests, "events": recorder.events,
            "tensors": recorder.tensors, "final_used_pages": used}


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of funkpopo/Anna to import from")
    args = parser.parse_args()
    sys.path.insert(0, str(Path(args.reference) / "src"))
    sys.modules.setdefault("soundfile", types.ModuleType("soundfile"))
    from oracle import turboquant_core_shim

    turboquant_core_shim.install()
    import importlib

    from anna.mm import prepared_inputs as prepared_mod
    from anna.model import ops as ref_ops
    from anna.model import qwen3_5_text_config as cfg_mod
    from anna.runtime import device as device_mod
    from anna.runtime import qwen3_5_text_engine as engine_mod
    from anna.runtime import scheduler as sched_mod

    runs, tensors = [], {}
    for index, (quantization, requests) in enumerate((
            ("none", [(23, 3), (23, 6), (23, 9), (40, 4), (7, 7)]),
            ("turboquant", [(30, 4), (30, 8), (30, 5), (19, 6)]),
            # a second wave arrives while the first one decodes: the running group is split and stacked again
            ("none", [(12, 40), (12, 40), (12, 30, 0.3), (33, 25, 0.0), (12, 20, 0.3)]))):
        importlib.reload(ref_ops)  # a fresh, un-wrapped cache class for every run
        ref = (ref_ops, cfg_mod, engine_mod, sched_mod, prepared_mod, device_mod)
        run = record_run(quantization, requests, 100 + index, ref)
        for name, value in run.pop("tensors").items():
            tensors[f"run{index}_{name}"] = value
        runs.append(run)
    (HERE / "scheduler_trace.json").write_text(json.dumps({"heads": HEADS, "kv_heads": KV_HEADS, "head_dim": HEAD_DIM,
                                                           "block_size": BLOCK, "runs": runs}))
    np.savez_compressed(HERE / "scheduler_trace.npz", **tensors)
    for run in runs:
        ops = [e["op"] for e in run["events"]]
        print(run["quantization"], {op: ops.count(op) for op in sorted(set(ops))})


if __name__ == "__main__":
    main()
