"""KV-head-sharded decode on two GPUs of one box: the peer-store epilogue and flag exchange (`PeerHeadGather`) against
the all-gather of the same per-rank outputs (`HeadGather`) and against the unsharded computation.  Skipped on boxes with
one GPU; the single-GPU pieces are covered by tests/test_gpu_peer_outputs.py."""
from __future__ import annotations

import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rank_main(rank: int, world: int, port: int, result_path: str) -> None:
    import torch.distributed as dist

    from anna_b200 import KVCacheConfig, Qwen3DynamicCache
    from anna_b200.sharding import HeadGather, PeerHeadGather, shard_kv_heads

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        q_heads, kv_heads, dim, batch, tokens = 16, 4, 128, 3, 600
        shard = shard_kv_heads(q_heads, kv_heads, world, rank)
        gen = torch.Generator().manual_seed(21)  # the same numbers on both ranks
        k = torch.randn(batch, kv_heads, tokens, dim, generator=gen).to(torch.bfloat16).to(device)
        v = torch.randn(batch, kv_heads, tokens, dim, generator=gen).to(torch.bfloat16).to(device)
        q = torch.randn(batch, q_heads, 1, dim, generator=gen).to(torch.bfloat16).to(device)

        def build(kv_slice):
            config = KVCacheConfig(num_hidden_layers=1, cache_block_size=16)
            cache = Qwen3DynamicCache(config, batch_size=batch, kv_cache_quantization="turboquant",
                                      kv_cache_quant_bits=4, kv_cache_residual_len=64)
            cache.update(k[:, kv_slice].contiguous(), v[:, kv_slice].contiguous(), 0, require_dense_cache=False)
            return cache

        full = build(slice(0, kv_heads))
        want = full.turboquant_single_token_decode_attention(0, q, scaling=dim ** -0.5, num_key_value_groups=4)
        part = build(slice(shard.kv_start, shard.kv_stop))
        q_local = shard.slice_q(q)
        gathered = HeadGather()(part.turboquant_single_token_decode_attention(
            0, q_local, scaling=dim ** -0.5, num_key_value_groups=4)).clone()
        peer = PeerHeadGather(shard, batch=batch, q_heads=q_heads, head_dim=dim, dtype=torch.bfloat16, device=device,
                              timeout_ms=5000)
        outs = []
        for _ in range(3):  # three steps: both output tensors of the gather are used, the flags keep growing
            local_out, peers = peer.begin()
            part.turboquant_single_token_decode_attention(0, q_local, scaling=dim ** -0.5, num_key_value_groups=4,
                                                          output=local_out, peer_outputs=peers)
            outs.append(peer.finish().clone())
        torch.cuda.synchronize(device)
        peer.check()
        ok = all(torch.equal(o, gathered) for o in outs) and torch.equal(gathered, want)
        dist.barrier()
        if rank == 0:
            with open(result_path, "w") as handle:
                handle.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_peer_store_gather_equals_all_gather_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    result = tmp_path / "result.txt"
    mp.spawn(_rank_main, args=(2, 29611, str(result)), nprocs=2, join=True)
    assert result.read_text() == "ok"
