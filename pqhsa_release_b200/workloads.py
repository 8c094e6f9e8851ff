"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (they stand in for model KV; no weights or datasets are
needed).  The same generators feed the parity tests and ``bench.py``.

* ``config0_stream``  : one fp32 head, keys ~ N(0,1) with 4 outlier channels x8 and
  per-key norms ~ lognormal(0, 0.3) (times sqrt(D)), values ~ N(0,1), query =
  0.5 * (one random key) + N(0,1).
* ``mixture_kv``      : per KV head a 64-component Gaussian mixture (random means,
  unit covariance) plus outlier channels; values ~ N(0,1); ``planted_queries`` puts
  each query head near 16 random keys of its KV head.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Workload:
    """Shape of one benchmark configuration."""

    name: str
    batch: int
    kv_heads: int
    group: int
    context: int
    dtype: torch.dtype
    head_dim: int = 128
    num_lists: int = 512
    top_fraction: float = 0.02
    sink_tokens: int = 4
    local_window: int = 128
    paged: bool = False
    block_size: int = 16

    @property
    def q_heads(self) -> int:
        return self.kv_heads * self.group

    def retrieval_len(self, context: int | None = None) -> int:
        c = self.context if context is None else context
        return max(c - min(self.sink_tokens, c) - self.local_window, 0)

    def topk(self, context: int | None = None) -> int:
        n = self.retrieval_len(context)
        return min(max(math.ceil(n * self.top_fraction), 0), n)

    def algorithmic_bytes(self, contexts=None, kv_heads: int | None = None) -> int:
        """Bytes one layer-step must move: 8 B per indexed key (code 4 + list id 2 +
        norm 2), the selected K and V rows per query head, the sink+local rows, the
        value means, centroids + code words, and q in / out."""
        e = 4 if self.dtype == torch.float32 else 2
        hkv = self.kv_heads if kv_heads is None else kv_heads
        hq = hkv * self.group
        d, l = self.head_dim, self.num_lists
        total = 0
        for c in (contexts if contexts is not None else [self.context] * self.batch):
            n = self.retrieval_len(c)
            k = self.topk(c)
            f = c - n
            total += hkv * n * 8 + hq * k * 2 * d * e + hkv * f * 2 * d * e + hkv * l * d * e
            total += hkv * (l * d + 8 * 16 * (d // 8)) * e + 2 * hq * d * e
        return total


WORKLOADS = {
    "c0": Workload("c0: 1 head fp32 8K", 1, 1, 1, 8192, torch.float32),
    "c1": Workload("c1: Llama-3-8B shape, 32K, batch 1", 1, 8, 4, 32768, torch.bfloat16),
    "c2": Workload("c2: Llama-3-8B shape, 128K, batch 4", 4, 8, 4, 131072, torch.bfloat16),
    "c3": Workload("c3: paged, batch 16, contexts U[8192, 65536]", 16, 8, 4, 65536, torch.bfloat16, paged=True),
    "c4": Workload("c4: Llama-3-70B shape, 256K, batch 8", 8, 8, 8, 262144, torch.bfloat16, paged=True),
}


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def config0_stream(seed: int = 0, context: int = 8192, dim: int = 128, device="cpu"):
    """(keys [S, D], values [S, D], query [D]) in fp32."""
    g = _gen(seed, device)
    k = torch.randn(context, dim, generator=g, device=device)
    ch = torch.randperm(dim, generator=g, device=device)[:4]
    k[:, ch] *= 8.0
    target = torch.exp(0.3 * torch.randn(context, generator=g, device=device)) * math.sqrt(dim)
    k = k * (target / k.norm(dim=1)).unsqueeze(1)
    v = torch.randn(context, dim, generator=g, device=device)
    j = int(torch.randint(0, context, (1,), generator=g, device=device))
    q = 0.5 * k[j] + torch.randn(dim, generator=g, device=device)
    return k, v, q


def mixture_kv(seed: int, heads: int, context: int, dim: int = 128, components: int = 64,
               dtype=torch.bfloat16, device="cpu"):
    """(keys, values) of shape [heads, context, dim]: Gaussian mixture keys with 4
    outlier channels x8 per head, N(0,1) values."""
    g = _gen(seed, device)
    keys = torch.empty(heads, context, dim, dtype=dtype, device=device)
    values = torch.empty(heads, context, dim, dtype=dtype, device=device)
    for h in range(heads):
        means = torch.randn(components, dim, generator=g, device=device)
        comp = torch.randint(0, components, (context,), generator=g, device=device)
        k = means[comp] + torch.randn(context, dim, generator=g, device=device)
        ch = torch.randperm(dim, generator=g, device=device)[:4]
        k[:, ch] *= 8.0
        keys[h] = k.to(dtype)
        values[h] = torch.randn(context, dim, generator=g, device=device).to(dtype)
    return keys, values


def planted_queries(seed: int, keys: torch.Tensor, group: int, near: int = 16):
    """keys [heads, context, dim] -> queries [heads * group, dim]: each query is
    (0.25 / sqrt(near)) * sum of ``near`` random keys of its KV head + N(0,1)."""
    heads, context, dim = keys.shape
    g = _gen(seed, keys.device)
    qs = []
    for h in range(heads):
        for _ in range(group):
            idx = torch.randint(0, context, (near,), generator=g, device=keys.device)
            q = (0.25 / math.sqrt(near)) * keys[h, idx].float().sum(0) + torch.randn(dim, generator=g, device=keys.device)
            qs.append(q)
    return torch.stack(qs).to(keys.dtype)
