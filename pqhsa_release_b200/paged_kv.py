"""Readers of vLLM FLASH_ATTN KV pages, both layouts
(benchmarks/vllm_backend/paged_kv_fa.py:44-156 in the reference):

* 5-D ``[2, num_blocks, block_size, kv_heads, dim]`` (vLLM <= 0.8.5),
* 4-D ``[num_blocks, kv_heads, block_size, 2 * dim]`` with K and V concatenated in the
  last dim and arbitrary outer strides (vLLM >= 0.10).

The decode kernels read pages in place through the block table; these helpers are
only used when an index has to be (re)built from a range of tokens, and for tests.
"""

from __future__ import annotations

import torch


def is_new_kv_layout(kv_cache: torch.Tensor) -> bool:
    return kv_cache.dim() == 4


def split_kv_cache(kv_cache: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Views ``(key_cache, value_cache)`` shaped [num_blocks, block_size, kv_heads, dim] for either layout."""
    if kv_cache.dim() == 5:
        return kv_cache[0], kv_cache[1]
    if kv_cache.dim() == 4:
        head = int(kv_cache.shape[-1]) // 2
        k, v = kv_cache.transpose(1, 2).split(head, dim=-1)
        return k, v
    raise ValueError(f"unsupported FLASH_ATTN kv_cache shape {tuple(kv_cache.shape)}")


def kv_cache_dims(kv_cache: torch.Tensor) -> tuple[int, int, int]:
    """(block_size, kv_heads, head_dim) for either layout."""
    k, _ = split_kv_cache(kv_cache)
    return int(k.shape[1]), int(k.shape[2]), int(k.shape[3])


def gather_paged_range(kv_cache: torch.Tensor, block_table: torch.Tensor, seq_idx: int, start: int, end: int):
    """Token range [start, end) of request ``seq_idx`` -> contiguous keys / values [kv_heads, n, dim]."""
    k_cache, v_cache = split_kv_cache(kv_cache)
    bs, heads, dim = int(k_cache.shape[1]), int(k_cache.shape[2]), int(k_cache.shape[3])
    n = int(end) - int(start)
    if n <= 0:
        empty = kv_cache.new_empty(heads, 0, dim)
        return empty, empty
    first, last = start // bs, (end - 1) // bs
    blocks = block_table[seq_idx, first : last + 1].long()
    keys = k_cache[blocks].reshape(-1, heads, dim)
    values = v_cache[blocks].reshape(-1, heads, dim)
    r0 = start - first * bs
    return (keys[r0 : r0 + n].permute(1, 0, 2).contiguous(), values[r0 : r0 + n].permute(1, 0, 2).contiguous())


def gather_paged_kv(kv_cache: torch.Tensor, block_table: torch.Tensor, seq_idx: int, seq_len: int):
    """Whole request -> keys / values [1, kv_heads, seq, dim] (the reference's ``gather_flashattn_kv``)."""
    k, v = gather_paged_range(kv_cache, block_table, seq_idx, 0, seq_len)
    return k.unsqueeze(0), v.unsqueeze(0)


def write_paged_token(kv_cache: torch.Tensor, block_table: torch.Tensor, seq_idx: int, pos: int, key: torch.Tensor,
                      value: torch.Tensor) -> None:
    """Store one token's K/V [kv_heads, dim] at position ``pos`` (what vLLM's
    ``reshape_and_cache_flash`` does for the real engine; used by tests and the benchmark)."""
    k_cache, v_cache = split_kv_cache(kv_cache)
    bs = int(k_cache.shape[1])
    blk = int(block_table[seq_idx, pos // bs])
    k_cache[blk, pos % bs] = key
    v_cache[blk, pos % bs] = value
