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
            if queries.ndim == 3:
                # the token append, the index update and the attention as one library call
                k, v = _squeeze_decode_token(keys, "keys"), _squeeze_decode_token(values, "values")
                return DecodeAttentionOutput(context=self.attention.step(queries, k, v))
            self.append(keys, values)
        return self.forward(queries)

    # ---- checkpoint / resume (pq_hsa/attention/decode_adapter.py:55-78) ------------
    def state_dict(self) -> dict[str, object]:
        """The reference's own checkpoint layout, so that either side loads the other's snapshots:
        ``{"attention": {index_config, attention_config, leading_shape, key_dim, value_dim, streams}}``
        (pq_hsa/attention/multihead.py:88-103) with one ``SparseKVCache`` state per (batch, head) stream
        (pq_hsa/attention/kv_cache.py:337-366) holding an ``IVFPQIndex`` state (pq_hsa/index/ivfpq.py:448-472).
        Index entries are in token order, as the reference keeps them."""
        a = self.attention
        if a.pool is None:
            raise RuntimeError("build_cache must be called before state_dict")
        n = a.length
        streams = []
        for s in range(a.B * a.H):
            b, h = divmod(s, a.H)
            e = a.pool.export_stream_state(s)
            index = None
            if e is not None:
                lists = int(e.coarse_centroids.shape[0])
                index = {
                    "config": asdict(self.index_config),
                    "coarse_centroids": e.coarse_centroids,
                    "list_ids": e.list_ids.to(torch.uint16 if lists - 1 <= 0xFFFF else torch.int64),
                    "codes": None,
                    "packed_codes": e.packed_codes,
                    "pq_codebooks": e.codebooks,
                    "rotation_matrix": None,
                    "key_norms": e.key_norms,
                    "dim": int(e.coarse_centroids.shape[1]),
                    "num_vectors": int(e.list_ids.numel()),
                }
            ac = self.attention_config
            streams.append({
                "index_config": asdict(self.index_config),
                "metadata": {
                    "sink_tokens": ac.sink_tokens, "local_window": ac.local_window,
                    "index_update_interval": ac.index_update_interval, "index_update_strategy": ac.index_update_strategy,
                    "codebook_refresh_interval": ac.codebook_refresh_interval, "kv_storage": ac.kv_storage,
                    "pin_offloaded_kv": ac.pin_offloaded_kv, "indexed_length": a.indexed_length,
                    "pending_update_tokens": a.pending, "deferred_index_update_pending": a.deferred_pending,
                    "tokens_since_codebook_refresh": 0, "index_rebuilds": a.index_rebuilds, "index_adds": a.index_adds,
                    "online_codebook_updates": a.online_updates, "codebook_refreshes": 0,
                    "deferred_index_updates": a.online_updates if ac.index_update_strategy == "deferred" else 0,
                },
                "keys": a.keys[b, h, :n].clone(),
                "values": a.values[b, h, :n].clone(),
                "index": index,
                "retrieval_value_centroids": None if e is None else e.value_means,
                "retrieval_value_sums": None if e is None else e.value_sums,
                "retrieval_value_counts": None if e is None else e.value_counts.to(e.value_sums.dtype),
            })
        return {
            "attention": {
                "index_config": asdict(self.index_config),
                "attention_config": asdict(self.attention_config),
                "leading_shape": (a.B, a.H),
                "key_dim": int(a.keys.shape[-1]),
                "value_dim": int(a.values.shape[-1]),
                "streams": tuple(streams),
            }
        }

    @classmethod
    def from_state_dict(cls, state: dict[str, object], *, index_config: IVFPQConfig | None = None,
                        attention_config: SparseAttentionConfig | None = None) -> "IVFPQDecodeAttentionAdapter":
        att = _attention_state(state)
        ic = index_config or IVFPQConfig(**att["index_config"])
        ac = attention_config or SparseAttentionConfig(**att["attention_config"])
        return cls(ic, ac).load_state_dict(state)

    def load_state_dict(self, state: dict[str, object], device: torch.device | str = "cuda") -> "IVFPQDecodeAttentionAdapter":
        """Load a snapshot in the reference's layout (one made here or by the reference's adapter) without
        rebuilding any index.  All streams must have the same length (the pool steps them together)."""
        att = _attention_state(state)
        if asdict(self.index_config) != dict(att["index_config"]):
            raise ValueError("state index_config does not match this adapter")
        if asdict(self.attention_config) != dict(att["attention_config"]):
            raise ValueError("state attention_config does not match this adapter")
        self.attention.restore(reference_attention_state(att, device))
        return self


def reference_attention_state(att: dict, device="cuda") -> dict:
    """The multi-head state of the reference's layout (pq_hsa/attention/multihead.py:88-154) as what
    ``PoolAttention.restore`` takes: stacked keys / values, the shared counters, one StreamIndexTensors per stream."""
    from .device_index import StreamIndexTensors

    streams = att.get("streams")
    if not isinstance(streams, (tuple, list)):
        raise ValueError("state must contain a tuple/list of stream states")
    lead = tuple(int(x) for x in att["leading_shape"])
    if len(lead) != 2:
        raise ValueError("leading_shape must be (batch, heads)")
    B, H = lead
    if len(streams) != B * H:
        raise ValueError("stream state count does not match leading_shape")
    if int(att.get("key_dim", 128)) != 128 or int(att.get("value_dim", 128)) != 128:
        raise ValueError("the B200 kernels are built for key_dim = value_dim = 128")
    lens = {int(st["keys"].shape[0]) for st in streams}
    metas = [st["metadata"] for st in streams]
    if len(lens) != 1 or len({(int(m["indexed_length"]), int(m["pending_update_tokens"])) for m in metas}) != 1:
        raise ValueError("all streams of a snapshot must have the same length and update counters")
    keys = torch.stack([st["keys"] for st in streams]).reshape(B, H, -1, 128).to(device)
    values = torch.stack([st["values"] for st in streams]).reshape(B, H, -1, 128).to(device)
    idx = []
    for st in streams:
        ix = st.get("index")
        if ix is None:
            idx.append(None)
            continue
        if ix.get("packed_codes") is None:
            raise ValueError("the snapshot must hold packed 4-bit codes")
        if ix.get("rotation_matrix") is not None:
            raise ValueError("rotated indexes are not supported")
        cnt = st.get("retrieval_value_counts")
        idx.append(StreamIndexTensors(
            packed_codes=ix["packed_codes"], list_ids=ix["list_ids"].to(torch.int64), key_norms=ix["key_norms"],
            coarse_centroids=ix["coarse_centroids"], codebooks=ix["pq_codebooks"],
            value_means=st["retrieval_value_centroids"], value_sums=st.get("retrieval_value_sums"),
            value_counts=None if cnt is None else cnt.to(torch.int32)))
    m = metas[0]
    return {"keys": keys, "values": values, "indexed_length": int(m["indexed_length"]),
            "pending": int(m["pending_update_tokens"]),
            "deferred_pending": bool(m.get("deferred_index_update_pending", False)), "streams": tuple(idx)}


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
