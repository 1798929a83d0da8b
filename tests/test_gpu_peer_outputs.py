"""Peer-store epilogue of the KV-head-sharded decode and its arrival flags, on one GPU: the "peer" tensors and flag
arrays are ordinary allocations of the same device, so no kernel ever waits for another kernel."""
import ctypes

import numpy as np
import pytest
import torch

from anna_b200 import _lib
from anna_b200.fused_ops import ptr, stream_ptr
from tests.helpers import TqPair, to_np

pytestmark = pytest.mark.gpu

DEV_PEER_TIMEOUT = 2


def test_decode_stores_its_rows_into_local_and_peer_tensors(cuda_device):
    """Heads 4..11 of a 16-head output tensor are this rank's: the merge writes them into the local tensor and, at the
    same offset, into two more tensors; nothing else in the three tensors changes and the rows equal a plain decode."""
    pair = TqPair(device=cuda_device, batch=3, kv_heads=2, head_dim=128, bits=4, residual_len=16, block_size=16,
                  dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(5)
    pair.append(torch.randn(3, 2, 300, 128, generator=gen).to(torch.bfloat16),
                torch.randn(3, 2, 300, 128, generator=gen).to(torch.bfloat16))
    query = torch.randn(3, 8, 1, 128, generator=gen).to(torch.bfloat16).to(cuda_device)
    want = pair.cache.turboquant_single_token_decode_attention(0, query, scaling=128 ** -0.5, num_key_value_groups=4)
    tensors = [torch.full((3, 16, 1, 128), 7.0, dtype=torch.bfloat16, device=cuda_device) for _ in range(3)]
    local = tensors[0][:, 4:12]
    peers = tuple(t[:, 4:12].data_ptr() for t in tensors[1:])
    got = pair.cache.turboquant_single_token_decode_attention(0, query, scaling=128 ** -0.5, num_key_value_groups=4,
                                                              output=local, peer_outputs=peers)
    assert got.data_ptr() == local.data_ptr()
    torch.cuda.synchronize()
    for t in tensors:
        assert torch.equal(t[:, 4:12], want)
        assert bool((t[:, :4] == 7.0).all()) and bool((t[:, 12:] == 7.0).all())


def _flag_table(arrays):
    return (ctypes.c_void_p * len(arrays))(*[a.data_ptr() for a in arrays])


def test_signal_wait_publishes_the_step_and_sees_arrived_peers(cuda_device):
    """Rank 1 of 3: the other ranks' flags are already at the step, so the wait ends at once; this rank's flag shows up
    in slot 1 of both other arrays."""
    arrays = [torch.zeros(3, dtype=torch.int64, device=cuda_device) for _ in range(3)]
    arrays[1][0] = 5
    arrays[1][2] = 6
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    _lib.check(_lib.lib().anna_peer_signal_wait(_flag_table(arrays), 1, 3, 5, 500, ptr(status), stream_ptr(cuda_device)),
               "anna_peer_signal_wait")
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert arrays[0].tolist() == [0, 5, 0] and arrays[2].tolist() == [0, 5, 0] and arrays[1].tolist() == [5, 0, 6]


def test_signal_wait_gives_up_after_its_time_limit(cuda_device):
    """Nobody ever sets the awaited flag: the kernel returns after the limit with the time-out bit set and the context
    still works."""
    arrays = [torch.zeros(2, dtype=torch.int64, device=cuda_device) for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    _lib.check(_lib.lib().anna_peer_signal_wait(_flag_table(arrays), 0, 2, 1, 100, ptr(status), stream_ptr(cuda_device)),
               "anna_peer_signal_wait")
    torch.cuda.synchronize()
    assert int(status.item()) & DEV_PEER_TIMEOUT
    assert arrays[1].tolist() == [1, 0]
    assert float(torch.ones(4, device=cuda_device).sum().item()) == 4.0


def test_signal_wait_rejects_bad_arguments(cuda_device):
    arrays = [torch.zeros(2, dtype=torch.int64, device=cuda_device) for _ in range(2)]
    lib = _lib.lib()
    assert lib.anna_peer_signal_wait(_flag_table(arrays), 2, 2, 1, 100, None, stream_ptr(cuda_device)) != 0
    assert lib.anna_peer_signal_wait(_flag_table(arrays), 0, 2, 1, 0, None, stream_ptr(cuda_device)) != 0
    assert lib.anna_peer_signal_wait(None, 0, 2, 1, 100, None, stream_ptr(cuda_device)) != 0
