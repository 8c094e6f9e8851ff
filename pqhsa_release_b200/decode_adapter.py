"""Model-facing decode adapter with the call signatures of the reference's
``IVFPQDecodeAttentionAdapter`` (pq_hsa/attention/decode_adapter.py:18-132) on
top of the CUDA library.

    keys / values : [batch, heads, seq, 128]
    queries       : [batch, heads, 128] or [batch, heads, query_len, 128]

One independent stream per (batch, head), as in the reference
(pq_hsa/attention/multihead.py:30-42).  Errors are the reference's: ``ValueError``
for shapes, ``RuntimeError`` for use before ``build_cache``.  Tensors must live on
a CUDA device; there is no CPU path.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass

import torch

from .config import IVFPQConfig, SparseAttentionConfig
from .engine import PoolAttention


@dataclass(slots=True)
class DecodeAttentionOutput:
    """``context`` has the shape of the queries.  ``per_query`` is empty: the B200
    path runs with ``collect_attention_details=False`` (the production setting)."""

    context: torch.Tensor
    per_query: tuple = ()


class IVFPQDecodeAttentionAdapter:
    def __init__(self, index_config: IVFPQConfig, attention_config: SparseAttentionConfig):
        self.index_config = index_config
        self.attention_config = attention_config
        self.attention = PoolAttention(index_config, attention_config, group=1)

    @property
    def streams(self) -> tuple[int, ...]:
        """Stream ids, one per (batch, head), in row-major order."""
        return tuple(range(self.attention.B * self.attention.H))

    @property
    def leading_shape(self) -> tuple[int, ...]:
        if self.attention.pool is None:
            raise RuntimeError("build_cache must be called before reading leading_shape")
        return (self.attention.B, self.attention.H)

    def build_cache(self, keys: torch.Tensor, values: torch.Tensor) -> "IVFPQDecodeAttentionAdapter":
        if keys.ndim != 4 or values.ndim != 4:
            raise ValueError("keys and values must be [batch, heads, seq, dim]")
        self.attention.build(keys, values)
        return self

    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        self.attention.append(_squeeze_decode_token(keys, "keys"), _squeeze_decode_token(values, "values"))

    def apply_pending_index_update(self) -> int:
        """Number of streams whose deferred update was applied (all or none)."""
        n = self.attention.B * self.attention.H
        return n if self.attention.apply_pending_index_update() else 0

    def forward(self, queries: torch.Tensor) -> DecodeAttentionOutput:
        if queries.ndim == 3:
            return DecodeAttentionOutput(context=self.attention.forward(queries))
        if queries.ndim == 4:
            outs = [self.attention.forward(queries[:, :, i].contiguous()) for i in range(queries.shape[2])]
            return DecodeAttentionOutput(context=torch.stack(outs, dim=2))
        raise ValueError("queries must be [batch, heads, dim] or [batch, heads, query_len, dim]")

    def decode_step(self, queries: torch.Tensor, keys: torch.Tensor | None = None,
                    values: torch.Tensor | None = None, *, append_kv: bool = True) -> DecodeAttentionOutput:
        if append_kv:
            if keys is None or values is None:
                raise ValueError("keys and values are required when append_kv=True")
            self.append(keys, values)
        return self.forward(queries)

    # ---- checkpoint / resume (pq_hsa/attention/decode_adapter.py:55-78) ------------
    def state_dict(self) -> dict[str, object]:
        a = self.attention
        if a.pool is None:
            raise RuntimeError("build_cache must be called before state_dict")
        n = a.length
        return {
            "attention": {
                "index_config": asdict(self.index_config),
                "attention_config": asdict(self.attention_config),
                "leading_shape": (a.B, a.H),
                "keys": a.keys[:, :, :n].clone(),
                "values": a.values[:, :, :n].clone(),
                "indexed_length": a.indexed_length,
                "pending": a.pending,
                "deferred_pending": a.deferred_pending,
                "streams": tuple(a.pool.export_stream_state(s) for s in range(a.B * a.H)),
            }
        }

    @classmethod
    def from_state_dict(cls, state: dict[str, object], *, index_config: IVFPQConfig | None = None,
                        attention_config: SparseAttentionConfig | None = None) -> "IVFPQDecodeAttentionAdapter":
        att = _attention_state(state)
        ic = index_config or IVFPQConfig(**att["index_config"])
        ac = attention_config or SparseAttentionConfig(**att["attention_config"])
        return cls(ic, ac).load_state_dict(state)

    def load_state_dict(self, state: dict[str, object]) -> "IVFPQDecodeAttentionAdapter":
        att = _attention_state(state)
        if asdict(self.index_config) != dict(att["index_config"]):
            raise ValueError("state index_config does not match this adapter")
        if asdict(self.attention_config) != dict(att["attention_config"]):
            raise ValueError("state attention_config does not match this adapter")
        self.attention.restore(att)
        return self


def _squeeze_decode_token(tensor: torch.Tensor, name: str) -> torch.Tensor:
    if tensor.ndim == 3:
        return tensor
    if tensor.ndim == 4 and tensor.shape[-2] == 1:
        return tensor.squeeze(-2)
    raise ValueError(f"{name} must be [batch, heads, dim] or [batch, heads, 1, dim]")


def _attention_state(state: dict[str, object]) -> dict[str, object]:
    attention = state.get("attention")
    if not isinstance(attention, dict):
        raise ValueError("adapter state must contain an attention dict")
    return attention
