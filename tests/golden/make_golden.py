"""Generate the golden fixtures under tests/golden/ from the reference itself.

Run in a container that has the reference checkout:

    python tests/golden/make_golden.py --reference /path/to/Anna

It imports ``anna.model.turboquant`` and ``anna.model.ops`` from ``<reference>/src`` unchanged.  The one piece the
reference cannot supply, the un-vendored ``turboquant.core`` module, is provided by oracle/turboquant_core_shim.py,
so fixtures that involve key codes pin the oracle's *definition* through the reference's own row / cache code,
while everything else (value quantizer, window/flush order, allocator policy, CPU decode math) is the reference's
own arithmetic.  Inputs are regenerated from seeds by the tests; a checksum of every input is stored so that a
change in the random generator is detected instead of silently comparing different data.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))


def digest(array: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def config1_inputs(seed: int = 1):
    """Benchmark configuration 1: B=2, Hkv=2, D=128, K,V ~ N(0,1) with 4 outlier channels per head scaled x8."""
    from tests.helpers import outlier_kv

    gen = torch.Generator().manual_seed(seed)
    prefill_k = outlier_kv(gen, (2, 2, 512, 128), torch.float32)
    prefill_v = outlier_kv(gen, (2, 2, 512, 128), torch.float32)
    steps = []
    for _ in range(64):
        steps.append((outlier_kv(gen, (2, 2, 1, 128), torch.float32), outlier_kv(gen, (2, 2, 1, 128), torch.float32),
                      torch.randn(2, 8, 1, 128, generator=gen)))
    return prefill_k, prefill_v, steps


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="checkout of funkpopo/Anna to import from")
    parser.add_argument("--only", choices=("prefill",), default=None, help="write just this fixture")
    args = parser.parse_args()
    sys.path.insert(0, str(Path(args.reference) / "src"))

    from oracle import turboquant_core_shim

    turboquant_core_shim.install()
    from anna.model import ops as ref_ops
    from anna.model import turboquant as ref_tq

    # ---- 5. multi-token attention with the model's masks (ops.py:1552-1574, masks as in :1840-1852, :2008-2016) ------
    prefill = {}
    gen = torch.Generator().manual_seed(31)
    cases = {"chunk": (2, 4, 2, 70, 160, 128, (160, 101), True), "full": (2, 4, 4, 33, 33, 64, (33, 20), True),
             "padding_only": (3, 6, 2, 5, 90, 256, (90, 64, 7), False)}
    for name, (batch, heads, kv_heads, q_len, key_len, dim, lengths, causal) in cases.items():
        # inputs are fp16-representable so that the fixture stores them exactly in half the space
        q = torch.randn(batch, heads, q_len, dim, generator=gen).half().float()
        k = torch.randn(batch, kv_heads, key_len, dim, generator=gen).half().float()
        v = torch.randn(batch, kv_heads, key_len, dim, generator=gen).half().float()
        visible = torch.tensor(lengths, dtype=torch.long)
        past = visible - q_len
        positions = torch.arange(key_len)[None, :]
        visible_mask = positions < visible[:, None]
        causal_mask = None
        if causal:
            q_positions = past[:, None] + torch.arange(q_len)[None, :]
            causal_mask = positions[:, None, :] > q_positions[:, :, None]
        ref = ref_ops.grouped_query_attention(q, k, v, scaling=dim ** -0.5, causal_mask=causal_mask,
                                              visible_mask=visible_mask)
        prefill[f"{name}_q"], prefill[f"{name}_k"], prefill[f"{name}_v"] = (t.numpy().astype(np.float16) for t in (q, k, v))
        prefill[f"{name}_lengths"] = visible.numpy()
        prefill[f"{name}_causal"] = np.array(int(causal))
        prefill[f"{name}_ref"] = ref.numpy()
    np.savez_compressed(HERE / "prefill_attention.npz", **prefill)
    if args.only == "prefill":
        print("prefill fixture written to", HERE)
        return

    # ---- 1. value quantizer (turboquant.py:199-252) --------------------------------------------------------------
    values = {}
    gen = torch.Generator().manual_seed(7)
    for dtype_name, dtype in (("bf16", torch.bfloat16), ("f16", torch.float16), ("f32", torch.float32)):
        for bits in (2, 3, 4):
            for dim, group in ((64, 16), (128, 32), (256, 32)):
                x = (torch.randn(2, 9, dim, generator=gen) * 2.5).to(dtype)
                x[0, 0] = 0.5  # constant group: scale clamps to 1e-8
                state = ref_tq.quantize_turboquant_values(x, bits=bits, group_size=group)
                deq = ref_tq.dequantize_turboquant_values(state)
                key = f"{dtype_name}_b{bits}_d{dim}_g{group}"
                values[key + "_x"] = x.float().numpy()
                values[key + "_data"] = state.data.numpy()
                values[key + "_scales"] = state.scales.float().numpy()
                values[key + "_zeros"] = state.zeros.float().numpy()
                values[key + "_deq"] = deq.numpy()
    np.savez_compressed(HERE / "value_quantizer.npz", **values)

    # ---- 2. allocator policy trace (ops.py:92-245) ------------------------------------------------------------------
    alloc = ref_ops.Qwen3PagedLayerAllocator(16)
    template = torch.zeros(1, 2, 1, 8)
    trace = []

    def snap(op, arg, result):
        trace.append({"op": op, "arg": arg, "result": result, "capacity": alloc.capacity(),
                      "free": list(alloc.free_pages), "used": alloc.used_pages()})

    a = alloc.allocate(3, key_template=template, value_template=template); snap("allocate", 3, a)
    b = alloc.allocate(3, key_template=template, value_template=template); snap("allocate", 3, b)
    alloc.release_pages(a); snap("release", a, None)
    c = alloc.allocate(4, key_template=template, value_template=template); snap("allocate", 4, c)
    snap("ensure_capacity", 40, alloc.ensure_capacity(40, key_template=template, value_template=template))
    d = alloc.allocate(20, key_template=template, value_template=template); snap("allocate", 20, d)
    alloc.retain_page(d[0]); snap("retain", d[0], None)
    alloc.release_pages(d); snap("release", d, None)
    alloc.release_pages([d[0]]); snap("release", [d[0]], None)
    e = alloc.allocate(30, key_template=template, value_template=template); snap("allocate", 30, e)
    alloc.release_pages(b); alloc.release_pages(c); alloc.release_pages(e); snap("release_all", None, None)
    snap("trim", None, alloc.trim())
    (HERE / "allocator_trace.json").write_text(json.dumps(trace, indent=1) + "\n")

    # block tables of the un-quantized cache (ops.py:696-729): B=2, 40 tokens, S=16, then release row 0 and re-admit
    class Cfg:
        num_hidden_layers = 1
        layer_types = ("full_attention",)
        cache_block_size = 16

    page_alloc = ref_ops.Qwen3PageAllocator(Cfg())
    cache = ref_ops.Qwen3DynamicCache(Cfg(), allocator=page_alloc, batch_size=2)
    kv = torch.zeros(2, 2, 40, 8)
    cache.update(kv, kv, 0, require_dense_cache=False)
    tables = {"after_prefill": [list(t) for t in cache.page_tables[0]], "free_after_prefill": list(page_alloc.layers[0].free_pages)}
    for _ in range(9):
        cache.update(kv[:, :, :1], kv[:, :, :1], 0, require_dense_cache=False)
    tables["after_9_steps"] = [list(t) for t in cache.page_tables[0]]
    compacted = cache.compact_batch_rows([1])
    tables["free_after_compact"] = list(page_alloc.layers[0].free_pages)
    fresh = ref_ops.Qwen3DynamicCache(Cfg(), allocator=page_alloc, batch_size=1)
    fresh.update(kv[:1, :, :33], kv[:1, :, :33], 0, require_dense_cache=False)
    tables["readmitted"] = [list(t) for t in fresh.page_tables[0]]
    tables["survivor"] = [list(t) for t in compacted.page_tables[0]]
    (HERE / "paged_block_tables.json").write_text(json.dumps(tables, indent=1) + "\n")

    # ---- 3. config 1 end to end through the reference's TurboQuantKVRow / Qwen3DynamicCache (fp32) ----------------
    prefill_k, prefill_v, steps = config1_inputs()
    cache = ref_ops.Qwen3DynamicCache(Cfg(), batch_size=2, kv_cache_quantization="turboquant", kv_cache_quant_bits=4,
                                      kv_cache_residual_len=128)
    cache.update(prefill_k, prefill_v, 0, require_dense_cache=False)
    outputs = {}
    checks = {"prefill_k": digest(prefill_k.numpy()), "prefill_v": digest(prefill_v.numpy())}
    for step, (k, v, q) in enumerate(steps):
        cache.update(k, v, 0, require_dense_cache=False)
        out = cache.turboquant_single_token_decode_attention(0, q, scaling=128 ** -0.5, num_key_value_groups=4)
        if step in (0, 21, 42, 63):
            outputs[f"out_step{step}"] = out.numpy()
            checks[f"q_step{step}"] = digest(q.numpy())
    cfg1 = dict(outputs)
    for b in range(2):
        row = cache.turboquant_rows[0][b]
        ks, vs = row._active_quantized_keys(), row._active_quantized_values()
        cfg1[f"row{b}_idx"] = ks.mse_indices.numpy().astype(np.uint8)
        cfg1[f"row{b}_sign_bits"] = np.packbits(ks.qjl_signs.numpy().astype(np.uint8), axis=-1, bitorder="little")
        cfg1[f"row{b}_norms"] = ks.norms.numpy()[..., 0]
        cfg1[f"row{b}_rnorms"] = ks.residual_norms.numpy()[..., 0]
        cfg1[f"row{b}_vdata"] = vs.data.numpy()
        cfg1[f"row{b}_vscales"] = vs.scales.numpy()
        cfg1[f"row{b}_vzeros"] = vs.zeros.numpy()
        cfg1[f"row{b}_lengths"] = np.array([row.length, row.quantized_length, row.residual_length])
    np.savez_compressed(HERE / "config1_turboquant.npz", **cfg1)
    (HERE / "config1_input_digests.json").write_text(json.dumps(checks, indent=1) + "\n")

    # ---- 4. the reference's TurboQuant split-KV kernel test on CPU semantics (tests/test_fused_op_xpu.py:647-703) ---
    xpu = {}
    for bits in (2, 3, 4):
        torch.manual_seed(24 + bits)
        query = torch.randn(1, 8, 1, 128, dtype=torch.bfloat16)[..., ::2]
        qkey = torch.randn(1, 2, 77, 64, dtype=torch.bfloat16)
        dense_v = torch.randn(2, 77, 64, dtype=torch.bfloat16)
        state = ref_tq.quantize_turboquant_values(dense_v, bits=bits, group_size=16)
        rkey = torch.randn(1, 2, 5, 64, dtype=torch.bfloat16)
        rvalue = torch.randn(1, 2, 5, 64, dtype=torch.bfloat16)
        gate = torch.randn(1, 1, 8 * 64, dtype=torch.bfloat16).view(1, 1, 8, 64).transpose(1, 2)
        deq = ref_tq.dequantize_turboquant_values(state, dtype=torch.bfloat16).unsqueeze(0)
        ref = ref_ops.grouped_query_attention(query, torch.cat((qkey, rkey), dim=2), torch.cat((deq, rvalue), dim=2),
                                              scaling=64 ** -0.5) * torch.sigmoid(gate)
        for name, tensor in (("query", query), ("qkey", qkey), ("dense_v", dense_v), ("rkey", rkey), ("rvalue", rvalue),
                             ("gate", gate), ("ref", ref)):
            xpu[f"b{bits}_{name}"] = tensor.float().numpy()
        xpu[f"b{bits}_vdata"] = state.data.numpy()
        xpu[f"b{bits}_vscales"] = state.scales.float().numpy()
        xpu[f"b{bits}_vzeros"] = state.zeros.float().numpy()
    np.savez_compressed(HERE / "splitkv_turboquant_case.npz", **xpu)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
