"""Multi-token grouped-query attention (prefill and chunked prefill) over dense K/V on the GPU.

``grouped_query_attention`` keeps the signature of the reference function (``src/anna/model/ops.py:1552-1574``).  The
reference materialises three boolean masks and a ``[B, Hkv, G, T, L]`` score tensor; the kernel behind this function
(``csrc/gqa_prefill.cu``) needs only the number of visible keys per row and a causal flag, which is exactly the
information in the masks the model builds (``ops.py:1840-1852``, ``:2008-2016``): ``visible_mask`` and
``key_padding_mask`` hide a suffix of the keys, ``causal_mask`` hides the keys after each query's own position, the
chunk's queries being the last ``T`` visible positions of their row.  Masks of any other shape are rejected by
``check_masks=True`` (which reads them back, so callers on the hot path pass ``key_lengths`` and leave it off).
"""
from __future__ import annotations

import torch

from . import _lib
from .fused_ops import dtype_code, on_device, ptr, run_gqa_decode_fused, stream_ptr

_FAST_DIMS = (64, 128, 256)


def _lengths_from_masks(batch: int, key_len: int, device, visible_mask, key_padding_mask) -> torch.Tensor | None:
    allowed = None
    for mask in (visible_mask, key_padding_mask):
        if mask is None:
            continue
        if mask.dim() != 2 or tuple(mask.shape) != (batch, key_len):
            raise ValueError("visible_mask / key_padding_mask must be [batch, key_len]")
        mask = mask.to(dtype=torch.bool)
        allowed = mask if allowed is None else (allowed & mask)
    if allowed is None:
        return None
    return allowed.sum(dim=-1, dtype=torch.long)


def _verify_masks(lengths, query_len, key_len, causal_mask, visible_mask, key_padding_mask) -> None:
    positions = torch.arange(key_len, device=lengths.device)[None, :]
    prefix = positions < lengths[:, None]
    for mask in (visible_mask, key_padding_mask):
        if mask is not None and not bool(torch.equal(mask.to(torch.bool) | prefix, prefix)):
            raise ValueError("grouped_query_attention: key masks must hide a suffix of the keys only")
    if causal_mask is not None:
        q_positions = (lengths - query_len)[:, None] + torch.arange(query_len, device=lengths.device)[None, :]
        expected = positions[:, None, :] > q_positions[:, :, None]
        # only the keys a row can see matter: the rest is hidden by the key masks anyway
        differs = (causal_mask.to(torch.bool) ^ expected) & prefix[:, None, :]
        if bool(differs.any()):
            raise ValueError("grouped_query_attention: causal_mask must be the model's causal mask for a chunk that "
                             "ends at each row's last visible key")


def grouped_query_attention(query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor, *,
                            scaling: float, causal_mask: torch.Tensor | None = None,
                            visible_mask: torch.Tensor | None = None, key_padding_mask: torch.Tensor | None = None,
                            key_lengths: torch.Tensor | None = None, causal: bool | None = None,
                            check_masks: bool = False) -> torch.Tensor:
    """``softmax_fp32(Q K^T * scaling + masks) V`` grouped by KV head: q ``[B, Hq, T, D]``, k / v ``[B, Hkv, L, D]``.

    ``key_lengths`` (int64 ``[B]`` on the device) and ``causal`` may be given instead of the masks; a query that sees
    no key gives zeros (the reference gives NaN there)."""
    if query_states.dim() != 4 or key_states.dim() != 4 or value_states.dim() != 4:
        raise ValueError("grouped_query_attention expects [batch, heads, tokens, head_dim] tensors")
    if not query_states.is_cuda:
        raise RuntimeError("grouped_query_attention: tensors must live on a CUDA device (there is no CPU path)")
    batch, heads, query_len, dim = (int(v) for v in query_states.shape)
    kv_heads, key_len = int(key_states.shape[1]), int(key_states.shape[2])
    if key_states.shape != value_states.shape or key_states.shape[0] != batch or key_states.shape[3] != dim:
        raise ValueError("grouped_query_attention: query / key / value shape mismatch")
    if kv_heads < 1 or heads % kv_heads != 0:
        raise ValueError("grouped_query_attention: query heads must be a multiple of kv heads")
    if not (query_states.dtype == key_states.dtype == value_states.dtype):
        raise ValueError("grouped_query_attention: query, key and value must share the dtype")
    device = query_states.device
    if causal is None:
        causal = causal_mask is not None
    if key_lengths is None:
        key_lengths = _lengths_from_masks(batch, key_len, device, visible_mask, key_padding_mask)
    elif key_lengths.dtype != torch.long or tuple(key_lengths.shape) != (batch,):
        raise ValueError("key_lengths must be int64 [batch]")
    if check_masks:
        lengths = key_lengths if key_lengths is not None else torch.full((batch,), key_len, dtype=torch.long,
                                                                         device=device)
        _verify_masks(lengths, query_len, key_len, causal_mask, visible_mask, key_padding_mask)
    if query_len == 0 or batch == 0:
        return torch.empty_like(query_states)
    if key_len == 0:
        return torch.zeros_like(query_states)
    if query_states.dtype in (torch.float16, torch.bfloat16) and dim in _FAST_DIMS:
        return _prefill_tensor_core(query_states, key_states, value_states, key_lengths, float(scaling), bool(causal))
    return _prefill_by_rows(query_states, key_states, value_states, key_lengths, float(scaling), bool(causal))


def _aligned(tensor: torch.Tensor) -> torch.Tensor:
    """Last dim contiguous, every other stride a multiple of 8 elements, base 16-byte aligned (what 16-byte copies need)."""
    ok = tensor.stride(3) == 1 and all(tensor.stride(i) % 8 == 0 for i in range(3)) and tensor.data_ptr() % 16 == 0
    return tensor if ok else tensor.contiguous()


def _prefill_tensor_core(query, key, value, key_lengths, scaling: float, causal: bool) -> torch.Tensor:
    batch, heads, query_len, dim = (int(v) for v in query.shape)
    query, key, value = _aligned(query), _aligned(key), _aligned(value)
    if value.stride() != key.stride():
        key, value = key.contiguous(), value.contiguous()
    if key_lengths is not None:
        key_lengths = key_lengths.contiguous()
    out = torch.empty((batch, heads, query_len, dim), dtype=query.dtype, device=query.device)
    with on_device(query.device):
        _lib.check(_lib.lib().anna_gqa_prefill(
            ptr(query), query.stride(0), query.stride(1), query.stride(2), ptr(key), ptr(value), key.stride(0),
            key.stride(1), key.stride(2), ptr(key_lengths), ptr(out), out.stride(0), out.stride(1), out.stride(2),
            batch, heads, int(key.shape[1]), query_len, int(key.shape[2]), dim, scaling, int(causal),
            dtype_code(query.dtype), stream_ptr(query.device)), "anna_gqa_prefill")
    return out


def _prefill_by_rows(query, key, value, key_lengths, scaling: float, causal: bool) -> torch.Tensor:
    """fp32 caches: every query token becomes one row of the single-token decode kernel, all rows
    of a sequence reading the same K/V (batch stride 0), with its own visible length."""
    batch, heads, query_len, dim = (int(v) for v in query.shape)
    key_len = int(key.shape[2])
    device = query.device
    if key_lengths is None:
        key_lengths = torch.full((batch,), key_len, dtype=torch.long, device=device)
    steps = torch.arange(query_len, device=device, dtype=torch.long)
    out = torch.empty((batch, heads, query_len, dim), dtype=query.dtype, device=device)
    for row in range(batch):
        n = key_lengths[row]
        visible = (n - query_len + steps + 1).clamp(min=0) if causal else n.expand(query_len)
        visible = torch.minimum(visible, n).contiguous()
        q_rows = query[row].transpose(0, 1).unsqueeze(2)  # [T, Hq, 1, D]
        k_rows = key[row].unsqueeze(0).expand(query_len, -1, -1, -1)
        v_rows = value[row].unsqueeze(0).expand(query_len, -1, -1, -1)
        result = run_gqa_decode_fused(query=q_rows, key=k_rows, value=v_rows, visible_lengths=visible, scaling=scaling)
        out[row].copy_(result.squeeze(2).transpose(0, 1))
    return out
