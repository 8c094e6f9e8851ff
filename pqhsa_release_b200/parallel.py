"""KV-head sharding across the GPUs of one node, in vLLM's tensor-parallel layout:
rank r owns KV heads [r * Hkv / W, (r + 1) * Hkv / W) and their G query heads; the
index, codes and pages of a head live only on its owner.  Streams are independent, so
the data path has exactly one collective: the all-gather of the output slices.

The reference has no distributed layer of its own (its only rank lookup is
benchmarks/vllm_backend/worker_hook.py:91-94); under vLLM each TP worker simply sees
its shard of heads, which is what these helpers reproduce for stand-alone use.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def kv_head_shard(num_kv_heads: int, rank: int, world: int) -> range:
    """KV heads owned by ``rank``."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if num_kv_heads % world != 0:
        raise ValueError(f"{num_kv_heads} KV heads do not shard evenly over {world} ranks")
    per = num_kv_heads // world
    return range(rank * per, (rank + 1) * per)


def query_head_shard(num_kv_heads: int, group: int, rank: int, world: int) -> range:
    """Query heads owned by ``rank`` (the G heads of each owned KV head)."""
    kv = kv_head_shard(num_kv_heads, rank, world)
    return range(kv.start * group, kv.stop * group)


def gather_context(local: torch.Tensor, out: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """All-gather of the per-rank contexts [B, Hq / W, D] into [B, Hq, D] (head order = rank
    order).  ``out`` may be a preallocated [W, B, Hq / W, D] staging tensor (needed when the call
    is captured in a CUDA graph).  With one rank this is the identity."""
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if world == 1:
        return local
    local = local.contiguous()
    if out is None:
        out = torch.empty((world, *local.shape), dtype=local.dtype, device=local.device)
    b, hl, d = local.shape
    # the output is the ranks' tensors concatenated along dim 0
    dist.all_gather_into_tensor(out.view(world * b, hl, d), local, group=group)
    return out.permute(1, 0, 2, 3).reshape(b, world * hl, d)
