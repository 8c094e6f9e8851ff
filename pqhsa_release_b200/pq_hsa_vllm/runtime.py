"""Decode runtime behind the plugin: the admission test and the per-layer, per-request
state machine of the reference's ``benchmarks/vllm_backend/pq_hsa_decode_runtime.py``
(should_pq_decode :302-341, run_pq_decode :492-716, pq_or_dense_forward :790-822),
driving the B200 sidecar.

The wrapped ``FlashAttentionImpl.forward`` keeps vLLM's signature and writes its result
in place into ``output``.  A step is taken by the PQ path only if it is a single-token
decode of requests that are long enough; everything else goes to the original forward.
Errors re-raise unless ``PQ_HSA_FALLBACK=1`` (then the original forward runs instead).
"""

from __future__ import annotations

import os
from typing import Any

STATS: dict[str, int] = {"pq_steps": 0, "dense_steps": 0, "builds": 0, "flushes": 0, "fallbacks": 0}
_REJECTS: dict[str, int] = {}
_STATE: dict[tuple[int, int], Any] = {}  # (layer id, request slot) -> sidecar


def reject(reason: str) -> bool:
    _REJECTS[reason] = _REJECTS.get(reason, 0) + 1
    return False


def rejects() -> dict[str, int]:
    return dict(_REJECTS)


def min_pq_seq() -> int:
    """sink + local + 16, the shortest context worth indexing (pq_hsa_decode_runtime.py:269-272)."""
    return int(os.environ.get("PQ_HSA_SINK", "4")) + int(os.environ.get("PQ_HSA_LOCAL", "128")) + 16


def batch_enabled() -> bool:
    return os.environ.get("PQ_HSA_BATCH", "0") == "1"


def should_pq_decode(attn_metadata) -> bool:
    if os.environ.get("PQ_HSA_ENABLE", "1") != "1":
        return reject("disabled")
    if attn_metadata is None:
        return reject("no_metadata")
    if getattr(attn_metadata, "use_cascade", False):
        return reject("cascade")
    if int(getattr(attn_metadata, "max_query_len", 0)) != 1:
        return reject("max_query_len!=1")
    seq_lens = getattr(attn_metadata, "seq_lens", None)
    if seq_lens is None:
        return reject("no_seq_lens")
    num_reqs = int(seq_lens.shape[0])
    if int(getattr(attn_metadata, "num_actual_tokens", 0)) != num_reqs:
        return reject("num_actual_tokens!=num_reqs")
    if num_reqs != 1 and not batch_enabled():
        return reject("num_reqs!=1")
    # max_seq_len comes from the runner's host-side lengths: no device sync
    # (benchmarks/vllm_backend/paged_kv_fa.py:15-27)
    if num_reqs == 1 and int(getattr(attn_metadata, "max_seq_len", 0)) < min_pq_seq():
        return reject("seq_too_short")
    return True


def index_config():
    from ..config import paper_index_config

    return paper_index_config(
        num_lists=int(os.environ.get("PQ_HSA_NUM_LISTS", "512")), nprobe=int(os.environ.get("PQ_HSA_NPROBE", "64")),
        num_subspaces=int(os.environ.get("PQ_HSA_SUBSPACES", "8")), num_bits=int(os.environ.get("PQ_HSA_BITS", "4")),
        coarse_max_iter=int(os.environ.get("PQ_HSA_COARSE_ITER", "1")),
        pq_max_iter=int(os.environ.get("PQ_HSA_PQ_ITER", "2")),
    )


def attention_config(scale: float):
    from ..config import paper_attention_config

    return paper_attention_config(
        scale=float(scale), sink_tokens=int(os.environ.get("PQ_HSA_SINK", "4")),
        local_window=int(os.environ.get("PQ_HSA_LOCAL", "128")),
        retrieval_top_fraction=float(os.environ.get("PQ_HSA_TOP_FRAC", "0.01")),
        index_update_interval=int(os.environ.get("PQ_HSA_UPD_INTERVAL", "256")),
    )


def _seq_len(attn_metadata, i: int, num_reqs: int) -> int:
    if num_reqs == 1:
        return int(attn_metadata.max_seq_len)
    host = getattr(attn_metadata, "seq_lens_cpu", None)
    return int(host[i]) if host is not None else int(attn_metadata.seq_lens[i].item())


def run_pq_decode(impl, layer, query, key, value, kv_cache, attn_metadata, output):
    """One decode token of every request of the step through its sidecar
    (pq_hsa_decode_runtime.py:492-716; batch loop: pq_hsa_batch_decode.py:383-432)."""
    from ..gqa_sidecar import GQASidecar
    from ..paged_kv import gather_paged_kv

    num_reqs = int(attn_metadata.seq_lens.shape[0])
    flush_every = int(os.environ.get("PQ_HSA_FLUSH_INTERVAL", "256"))
    for i in range(num_reqs):
        seq_len = _seq_len(attn_metadata, i, num_reqs)
        key_id = (id(layer), i)
        side = _STATE.get(key_id)
        q = query[i : i + 1]
        if seq_len < min_pq_seq():
            raise RuntimeError("request too short for the PQ path")
        if side is None or side.length + 1 != seq_len:
            # first call for this request, or a non-sequential step: (re)build from the pages
            side = GQASidecar(index_config(), attention_config(impl.scale), num_query_heads=impl.num_heads,
                              num_kv_heads=impl.num_kv_heads)
            side.set_paged_kv_context(kv_cache, attn_metadata, i)
            keys, values = gather_paged_kv(kv_cache, attn_metadata.block_table.to("cuda").int(), i, seq_len)
            side.build_cache(keys, values)
            side.appended_since_flush = 0
            _STATE[key_id] = side
            STATS["builds"] += 1
        else:
            side.set_paged_kv_context(kv_cache, attn_metadata, i)
            side.lean_append(key[i : i + 1], value[i : i + 1], q)
            side.appended_since_flush += 1
            if flush_every > 0 and side.appended_since_flush >= flush_every:
                side.apply_pending_index_update()
                side.appended_since_flush = 0
                STATS["flushes"] += 1
        ctx = side.forward(q.reshape(1, impl.num_heads, -1))
        output[i : i + 1].copy_(ctx.reshape(output[i : i + 1].shape))
    STATS["pq_steps"] += 1
    return output


def pq_or_dense_forward(original, impl, layer, query, key, value, kv_cache, attn_metadata, output=None, **extra):
    if not should_pq_decode(attn_metadata) or output is None:
        STATS["dense_steps"] += 1
        return original(impl, layer, query, key, value, kv_cache, attn_metadata, output=output, **extra)
    try:
        return run_pq_decode(impl, layer, query, key, value, kv_cache, attn_metadata, output)
    except Exception:
        if os.environ.get("PQ_HSA_FALLBACK", "0") != "1":
            raise
        STATS["fallbacks"] += 1
        return original(impl, layer, query, key, value, kv_cache, attn_metadata, output=output, **extra)


def install_flashattn_backend(impl_cls=None) -> dict[str, Any]:
    """Replace ``FlashAttentionImpl.forward`` with the PQ-or-dense wrapper, once
    (benchmarks/vllm_backend/pq_hsa_flashattn_wrap.py:41-97)."""
    if impl_cls is None:
        from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl as impl_cls  # type: ignore
    if getattr(impl_cls.forward, "_pq_hsa_wrapped", False):
        return {"installed": True, "already": True}
    original = impl_cls.forward

    def wrapped(self, layer, query, key, value, kv_cache, attn_metadata, output=None, **extra):
        return pq_or_dense_forward(original, self, layer, query, key, value, kv_cache, attn_metadata, output, **extra)

    wrapped._pq_hsa_wrapped = True
    wrapped._pq_hsa_original = original
    impl_cls.forward = wrapped
    return {"installed": True, "already": False}
