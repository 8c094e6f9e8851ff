"""GQA sidecar: the object the vLLM decode runtime drives per (layer, request), with
the duck-typed surface of the reference's ``GQASidecar`` / ``GQASidecarFast``
(benchmarks/vllm_backend/gqa_sidecar.py:11-76, gqa_sidecar_fast.py:48-187):
one IVF-PQ stream per KV head, the G query heads h*G .. h*G+G-1 share stream h.

    build_cache(keys[1, Hkv, S, D], values)          append(keys[1, Hkv, D], values)
    lean_append(key[T, Hkv, D], value, q) -> bool    forward(queries[1, Hq, D]) -> [1, Hq, D]
    set_paged_kv_context(kv_cache, attn_metadata, seq_idx)
    apply_pending_index_update() / .adapter.apply_pending_index_update()

With a paged context set before ``build_cache`` the sidecar keeps no K/V copy: the
kernels read vLLM's pages in place through the block table.
"""

from __future__ import annotations

import torch

from .config import IVFPQConfig, SparseAttentionConfig
from .engine import PoolAttention
from .paged_kv import kv_cache_dims


class GQASidecar:
    def __init__(self, index_config: IVFPQConfig, attention_config: SparseAttentionConfig, *,
                 num_query_heads: int, num_kv_heads: int) -> None:
        if num_query_heads % num_kv_heads != 0:
            raise ValueError("GQA requires num_query_heads % num_kv_heads == 0")
        self.index_config = index_config
        self.attention_config = attention_config
        self.num_query_heads = int(num_query_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.num_groups = self.num_query_heads // self.num_kv_heads
        self.engine = PoolAttention(index_config, attention_config, group=self.num_groups)
        self.adapter = self  # the runtime calls sidecar.adapter.apply_pending_index_update()
        self.length = 0
        self._paged = None  # (kv_cache, block_table [1, max_blocks] int32, token capacity)

    # the reference's fast sidecar reports these; here they are always true
    batched_heads_active = True
    cuda_graph_active = False

    @property
    def streams(self) -> tuple[int, ...]:
        return tuple(range(self.num_kv_heads))

    def set_paged_kv_context(self, kv_cache: torch.Tensor, attn_metadata, seq_idx: int = 0) -> None:
        """Read K/V in place from vLLM's pages (benchmarks/e2e_pq_param_sweep.py set_paged_kv_context;
        the runtime calls it before every build / step: pq_hsa_decode_runtime.py:500-522)."""
        bs, heads, dim = kv_cache_dims(kv_cache)
        if heads != self.num_kv_heads:
            raise ValueError(f"kv_cache has {heads} KV heads, sidecar was made for {self.num_kv_heads}")
        table = attn_metadata.block_table[seq_idx : seq_idx + 1]
        if table.dtype != torch.int32 or not table.is_contiguous():
            table = table.to(torch.int32).contiguous()
        self._paged = (kv_cache, table, int(table.shape[1]) * bs)
        if self.engine.pool is not None and self.engine.paged:
            self.engine._paged = (kv_cache, table)
            self.engine.pool.bind_kv_paged(kv_cache, table)

    def build_cache(self, keys: torch.Tensor, values: torch.Tensor) -> "GQASidecar":
        if keys.ndim != 4 or values.ndim != 4:
            raise ValueError("keys/values must be [1, kv_heads, seq, dim]")
        if keys.shape[0] != 1 or keys.shape[1] != self.num_kv_heads:
            raise ValueError(f"expected keys [1, {self.num_kv_heads}, S, D], got {tuple(keys.shape)}")
        if self._paged is not None:
            kv_cache, table, cap = self._paged
            self.engine.build_paged(kv_cache, table, [int(keys.shape[2])], self.num_kv_heads, cap)
        else:
            self.engine.build(keys, values)
        self.length = int(keys.shape[2])
        return self

    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        if keys.ndim != 3 or values.ndim != 3:
            raise ValueError("append keys/values must be [1, kv_heads, dim]")
        self.engine.append(keys, values)
        self.length += 1

    def lean_append(self, key: torch.Tensor, value: torch.Tensor, q: torch.Tensor | None = None) -> bool:
        """One-launch append of the step's token, ``key``/``value`` [T=1, Hkv, D]
        (benchmarks/e2e_pq_param_sweep.py:4575-4645).  Returns False if the shape is not a single token."""
        if key.ndim != 3 or key.shape[0] != 1:
            return False
        self.append(key, value)
        return True

    def append_many(self, keys: torch.Tensor, values: torch.Tensor, *, flush_every: int = 0) -> int:
        if keys.ndim == 4:
            keys, values = keys[0], values[0]
        for i in range(int(keys.shape[1])):
            self.append(keys[:, i].unsqueeze(0), values[:, i].unsqueeze(0))
        return 0

    def apply_pending_index_update(self) -> int:
        return self.num_kv_heads if self.engine.apply_pending_index_update() else 0

    def forward(self, queries: torch.Tensor) -> torch.Tensor:
        """queries ``[1, q_heads, dim]`` -> context ``[1, q_heads, dim]``."""
        if queries.ndim != 3 or queries.shape[0] != 1:
            raise ValueError(f"queries must be [1, q_heads, dim], got {tuple(queries.shape)}")
        return self.engine.forward(queries)

    # prefix checkpoints (benchmarks/e2e_pq_param_sweep.py:3358-3432) are not kept by this build
    prefix_checkpoint_length = 0

    def checkpoint_prefix(self) -> None:
        return None

    def restore_prefix(self, keys, values, *, kv_cache=None, attn_metadata=None, seq_idx: int = 0) -> bool:
        return False
