"""Decode runtime behind the plugin: the admission test and the per-layer state machine of the
reference's ``benchmarks/vllm_backend/pq_hsa_decode_runtime.py`` (should_pq_decode :302-341,
run_pq_decode :492-716, run_pq_decode_into_output :719-787, pq_or_dense_forward :790-822) and of its
batch driver ``pq_hsa_batch_decode.py`` (:383-432), on the B200 library.

The wrapped ``FlashAttentionImpl.forward`` keeps vLLM's signature and writes its result in place
into ``output``.  A step is taken by the PQ path only if it is a pure single-token decode step of
requests that are long enough; everything else goes to the original forward.  Errors re-raise
unless ``PQ_HSA_FALLBACK=1`` (then the original forward runs instead).

Where the reference keeps one sidecar per (layer, request) and loops the requests in Python, a
layer here owns one :class:`~pqhsa_release_b200.batch_engine.PagedBatchEngine`: all requests of
the step - any number, any mix of lengths - are one fused library call that reads vLLM's pages in
place and writes the contexts straight into ``output``.  Requests are told apart by vLLM's request
ids (reachable through the model runner attached to the metadata, as in the reference,
pq_hsa_batch_decode.py:99-118); a finished request's slot is cleared and reused; nothing on the
path synchronises with the device (lengths come from the runner's host-side arrays,
benchmarks/vllm_backend/paged_kv_fa.py:15-27).
"""

from __future__ import annotations

import os
from typing import Any

STATS: dict[str, int] = {"pq_steps": 0, "dense_steps": 0, "builds": 0, "flushes": 0, "fallbacks": 0,
                         "restores": 0, "evictions": 0, "kv_writes": 0}
_REJECTS: dict[str, int] = {}
_LAYERS: dict[int, Any] = {}  # id(layer) -> PagedBatchEngine


def reject(reason: str) -> bool:
    _REJECTS[reason] = _REJECTS.get(reason, 0) + 1
    return False


def rejects() -> dict[str, int]:
    return dict(_REJECTS)


def reset() -> None:
    """Forget every layer's engine (tests; a worker that reloads its model)."""
    _LAYERS.clear()
    _REJECTS.clear()
    for k in STATS:
        STATS[k] = 0


def min_pq_seq() -> int:
    """sink + local + 16, the shortest context worth indexing (pq_hsa_decode_runtime.py:269-272)."""
    return int(os.environ.get("PQ_HSA_SINK", "4")) + int(os.environ.get("PQ_HSA_LOCAL", "128")) + 16


def batch_enabled() -> bool:
    return os.environ.get("PQ_HSA_BATCH", "0") == "1"


def batch_seq_lens(attn_metadata) -> list[int]:
    """Per-request lengths from host memory, no device sync: the metadata's own CPU copy, else the runner's
    ``seq_lens_np`` (pq_hsa_batch_decode.py:72-96).  Cached on the metadata object: every layer of the step
    asks for it."""
    cached = getattr(attn_metadata, "_pq_batch_seq_lens", None)
    if cached is not None:
        return cached
    n = int(attn_metadata.seq_lens.shape[0])
    lens = None
    host = getattr(attn_metadata, "seq_lens_cpu", None)
    if host is not None:
        lens = [int(x) for x in host[:n]]
    if lens is None:
        runner = getattr(attn_metadata, "_pq_runner", None)
        np_lens = getattr(runner, "seq_lens_np", None) if runner is not None else None
        if np_lens is not None and len(np_lens) >= n:
            lens = [int(x) for x in np_lens[:n]]
    if lens is None and n == 1:
        lens = [int(attn_metadata.max_seq_len)]
    if lens is None:
        # last resort, one device sync per STEP (the result is cached for the step's other layers)
        lens = [int(x) for x in attn_metadata.seq_lens[:n].tolist()]
    try:
        attn_metadata._pq_batch_seq_lens = lens
    except Exception:  # a frozen metadata object: recomputed per layer
        pass
    return lens


def batch_req_keys(attn_metadata, num_reqs: int) -> list:
    """vLLM request ids when the runner is reachable, else the batch slot (pq_hsa_batch_decode.py:99-118)."""
    keys: list = [("slot", i) for i in range(num_reqs)]
    runner = getattr(attn_metadata, "_pq_runner", None)
    req_ids = getattr(getattr(runner, "input_batch", None), "req_ids", None) if runner is not None else None
    if req_ids is not None and len(req_ids) >= num_reqs:
        for i in range(num_reqs):
            if req_ids[i] is not None:
                keys[i] = req_ids[i]
    return keys


def req_ids_available(attn_metadata, num_reqs: int) -> bool:
    runner = getattr(attn_metadata, "_pq_runner", None)
    req_ids = getattr(getattr(runner, "input_batch", None), "req_ids", None) if runner is not None else None
    return req_ids is not None and len(req_ids) >= num_reqs and all(req_ids[i] is not None for i in range(num_reqs))


def prefix_keys(attn_metadata, lens: list[int]) -> list:
    """(context length, digest of the prompt ids) per request, or None where the prompt is not reachable
    (pq_hsa_decode_runtime.py:403-422, per request: pq_hsa_batch_decode.py:132-153)."""
    from ..batch_engine import prompt_key

    runner = getattr(attn_metadata, "_pq_runner", None)
    out: list = [None] * len(lens)
    if runner is None or os.environ.get("PQ_HSA_PREFIX_CACHE", "1") != "1":
        return out
    req_ids = getattr(getattr(runner, "input_batch", None), "req_ids", None)
    requests = getattr(runner, "requests", None)
    if req_ids is None or requests is None:
        return out
    for i, n in enumerate(lens):
        if i < len(req_ids) and req_ids[i] is not None:
            request = requests.get(req_ids[i])
            ids = None if request is None else getattr(request, "prompt_token_ids", None)
            if ids is not None:
                out[i] = prompt_key(n - int(attn_metadata.max_query_len), ids)
    return out


def should_pq_decode(attn_metadata) -> bool:
    if os.environ.get("PQ_HSA_ENABLE", "1") != "1":
        return reject("disabled")
    if attn_metadata is None:
        return reject("no_metadata")
    if getattr(attn_metadata, "use_cascade", False):
        return reject("cascade")
    if int(getattr(attn_metadata, "max_query_len", 0)) != 1:
        if not multi_query_enabled():
            return reject("max_query_len!=1")
        return should_pq_decode_mq(attn_metadata)
    seq_lens = getattr(attn_metadata, "seq_lens", None)
    if seq_lens is None:
        return reject("no_seq_lens")
    num_reqs = int(seq_lens.shape[0])
    if num_reqs < 1:
        return reject("num_reqs<1")
    if int(getattr(attn_metadata, "num_actual_tokens", 0)) != num_reqs:
        return reject("num_actual_tokens!=num_reqs")
    if num_reqs != 1:
        if not batch_enabled():
            return reject("num_reqs!=1")
        if not req_ids_available(attn_metadata, num_reqs):
            return reject("no_req_ids")  # batch slots are reshuffled when a request ends: ids are needed
        floor = min_pq_seq()
        if any(n < floor for n in batch_seq_lens(attn_metadata)):
            return reject("seq_too_short")
        return True
    # max_seq_len comes from the runner's host-side lengths: no device sync
    # (benchmarks/vllm_backend/paged_kv_fa.py:15-27)
    if int(getattr(attn_metadata, "max_seq_len", 0)) < min_pq_seq():
        return reject("seq_too_short")
    return True


def multi_query_enabled() -> bool:
    """PQ_HSA_MULTI_QUERY=1 (default 0): speculative-decoding steps of one request take the PQ path
    (benchmarks/vllm_backend/pq_hsa_multi_query.py:1-12)."""
    return os.environ.get("PQ_HSA_MULTI_QUERY", "0") == "1"


def should_pq_decode_mq(attn_metadata) -> bool:
    """Admission of a step with ``T = max_query_len > 1`` query tokens (pq_hsa_multi_query.py:112-160): one
    request, T within PQ_HSA_MQ_MAX, every token of the step a query token, the committed context long enough,
    and not a prefill chunk (a chunk starts inside the prompt; a speculative step starts after it)."""
    seq_lens = getattr(attn_metadata, "seq_lens", None)
    if seq_lens is None or int(seq_lens.shape[0]) != 1:
        return reject("mq_num_reqs!=1")
    T = int(getattr(attn_metadata, "max_query_len", 0))
    if T < 1 or T > int(os.environ.get("PQ_HSA_MQ_MAX", "8")):
        return reject("mq_query_len_out_of_range")
    if int(getattr(attn_metadata, "num_actual_tokens", 0)) != T:
        return reject("mq_num_actual_tokens!=T")
    context = batch_seq_lens(attn_metadata)[0] - T
    if context < min_pq_seq():
        return reject("seq_too_short")
    runner = getattr(attn_metadata, "_pq_runner", None)
    req_ids = getattr(getattr(runner, "input_batch", None), "req_ids", None) if runner is not None else None
    request = runner.requests.get(req_ids[0]) if req_ids and req_ids[0] is not None and hasattr(runner, "requests") else None
    if request is None:
        return reject("mq_no_request")  # without the request a prefill chunk cannot be told from a speculative step
    prompt = getattr(request, "num_prompt_tokens", None)
    if prompt is None:
        ids = getattr(request, "prompt_token_ids", None)
        prompt = None if ids is None else len(ids)
    if prompt is None or context < int(prompt):
        return reject("mq_prefill_chunk")
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
        index_update_strategy=os.environ.get("PQ_HSA_UPD_STRATEGY", "deferred"),
    )


def write_step_kv(key, value, kv_cache, attn_metadata) -> None:
    """vLLM <= 0.8.5 pages ``[2, blocks, block_size, Hkv, D]``: the attention forward itself stores the step's
    K/V at ``slot_mapping`` (what reshape_and_cache_flash does, pq_hsa_decode_runtime.py:734-744); with the
    ``[blocks, Hkv, block_size, 2D]`` pages of vLLM >= 0.10 the write has happened before the forward."""
    if kv_cache.dim() != 5:
        return
    slots = attn_metadata.slot_mapping[: key.shape[0]].long()
    nb, bs, heads, dim = kv_cache.shape[1:]
    kv_cache[0].view(nb * bs, heads, dim).index_copy_(0, slots, key.to(kv_cache.dtype))
    kv_cache[1].view(nb * bs, heads, dim).index_copy_(0, slots, value.to(kv_cache.dtype))
    STATS["kv_writes"] += 1


def layer_engine(impl, layer, kv_cache, attn_metadata):
    """The layer's engine, made on its first PQ step: request slots for PQ_HSA_MAX_REQUESTS requests
    (default: 1 without PQ_HSA_BATCH, else 16), index slots for PQ_HSA_MAX_CONTEXT tokens each (default: what
    the block table can address, at most 262144 + 4096)."""
    from ..batch_engine import PagedBatchEngine
    from ..paged_kv import kv_cache_dims

    eng = _LAYERS.get(id(layer))
    if eng is None:
        bs, _, _ = kv_cache_dims(kv_cache)
        addressable = int(attn_metadata.block_table.shape[1]) * bs
        cap = min(addressable, int(os.environ.get("PQ_HSA_MAX_CONTEXT", str(262144 + 4096))))
        max_reqs = int(os.environ.get("PQ_HSA_MAX_REQUESTS", "16" if batch_enabled() else "1"))
        eng = PagedBatchEngine(
            index_config(), attention_config(impl.scale), num_query_heads=impl.num_heads,
            num_kv_heads=impl.num_kv_heads, max_requests=max_reqs, token_capacity=cap, dtype=kv_cache.dtype,
            device=kv_cache.device, flush_every=int(os.environ.get("PQ_HSA_FLUSH_INTERVAL", "256")),
        )
        _LAYERS[id(layer)] = eng
    return eng


def run_pq_decode(impl, layer, query, key, value, kv_cache, attn_metadata, output):
    """One decode token of every request of the step: K/V store (old page layout only), then ONE fused
    library call for the whole batch, the contexts landing in ``output``
    (pq_hsa_decode_runtime.py:719-787 + :492-716; batch: pq_hsa_batch_decode.py:383-432)."""
    import torch

    if int(getattr(attn_metadata, "max_query_len", 1)) > 1:
        return run_pq_decode_mq(impl, layer, query, key, value, kv_cache, attn_metadata, output)
    lens = batch_seq_lens(attn_metadata)
    num_reqs = len(lens)
    if any(n < min_pq_seq() for n in lens):
        raise RuntimeError("request too short for the PQ path")
    write_step_kv(key, value, kv_cache, attn_metadata)
    eng = layer_engine(impl, layer, kv_cache, attn_metadata)
    table = attn_metadata.block_table
    if table.dtype != torch.int32 or not table.is_contiguous():
        table = table.to(torch.int32).contiguous()
    q = query[:num_reqs].reshape(num_reqs, impl.num_heads, -1)
    direct = (output.is_contiguous() and output.dtype == q.dtype and q.is_contiguous()
              and output[:num_reqs].numel() == q.numel())
    out = output[:num_reqs].view(q.shape) if direct else torch.empty_like(q.contiguous())
    before = dict(eng.stats)
    eng.step(q.contiguous(), kv_cache, table, batch_req_keys(attn_metadata, num_reqs), lens, out,
             prefix_keys(attn_metadata, lens))
    if not direct:
        output[:num_reqs].copy_(out.reshape(output[:num_reqs].shape))
    for k in ("builds", "flushes", "restores", "evictions"):
        STATS[k] += eng.stats[k] - before[k]
    STATS["pq_steps"] += 1
    return output


def run_pq_decode_mq(impl, layer, query, key, value, kv_cache, attn_metadata, output):
    """A speculative-decoding step of one request: T query tokens at the consecutive positions C .. C + T - 1
    (pq_hsa_multi_query.py:14-60).  Causality by sequential replay, as there: for j < T the request advances by
    token C + j (already in the pages) and query j attends with the steady path's sink / local / retrieval
    semantics - T fused library calls.  Where the reference checkpoints the sidecar before the step and restores
    it when drafts are rejected, nothing needs saving here: the pages are read in place and an appended token
    changes only the counters, so the engine takes the request's length back when the next step starts at a
    lower position (``PagedBatchEngine._rollback``).  No deferred flush runs on an unverified token: the first
    token of a step is the one the previous step committed, the flush check happens there."""
    import torch

    T = int(attn_metadata.max_query_len)
    total = batch_seq_lens(attn_metadata)[0]
    context = total - T
    if context < min_pq_seq():
        raise RuntimeError("request too short for the PQ path")
    write_step_kv(key, value, kv_cache, attn_metadata)
    eng = layer_engine(impl, layer, kv_cache, attn_metadata)
    table = attn_metadata.block_table
    if table.dtype != torch.int32 or not table.is_contiguous():
        table = table.to(torch.int32).contiguous()
    q = query[:T].reshape(T, impl.num_heads, -1).contiguous()
    direct = output.is_contiguous() and output.dtype == q.dtype and output[:T].numel() == q.numel()
    out = output[:T].view(q.shape) if direct else torch.empty_like(q)
    keys = batch_req_keys(attn_metadata, 1)
    pkeys = prefix_keys(attn_metadata, [total])
    before = dict(eng.stats)
    for j in range(T):
        eng.step(q[j : j + 1], kv_cache, table, keys, [context + j + 1], out[j : j + 1], pkeys if j == 0 else None,
                 hold_flush=j > 0)
    if not direct:
        output[:T].copy_(out.reshape(output[:T].shape))
    for k in ("builds", "flushes", "restores", "evictions"):
        STATS[k] += eng.stats[k] - before[k]
    STATS["pq_steps"] += 1
    STATS["mq_steps"] = STATS.get("mq_steps", 0) + 1
    STATS["mq_tokens"] = STATS.get("mq_tokens", 0) + T
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


def attach_runner(builder_cls=None) -> dict[str, Any]:
    """Wrap ``FlashAttentionMetadataBuilder.build`` so that the metadata it returns carries the model runner
    (``_pq_runner``): request ids, host-side lengths and prompt ids are read from it
    (pq_hsa_decode_runtime.py:874-902)."""
    if builder_cls is None:
        from vllm.v1.attention.backends.flash_attn import FlashAttentionMetadataBuilder as builder_cls  # type: ignore
    if getattr(builder_cls.build, "_pq_hsa_wrapped", False):
        return {"attached": True, "already": True}
    original = builder_cls.build

    def build(self, *args, **kwargs):
        md = original(self, *args, **kwargs)
        runner = getattr(self, "runner", None) or getattr(self, "model_runner", None)
        if md is not None and runner is not None:
            try:
                md._pq_runner = runner
            except Exception:
                pass
        return md

    build._pq_hsa_wrapped = True
    builder_cls.build = build
    return {"attached": True, "already": False}


def install_flashattn_backend(impl_cls=None, builder_cls=None) -> dict[str, Any]:
    """Replace ``FlashAttentionImpl.forward`` with the PQ-or-dense wrapper, once, and attach the runner to the
    metadata (benchmarks/vllm_backend/pq_hsa_flashattn_wrap.py:41-97)."""
    attached = False
    if impl_cls is None:
        from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl as impl_cls  # type: ignore

        attached = attach_runner(builder_cls)["attached"]
    elif builder_cls is not None:
        attached = attach_runner(builder_cls)["attached"]
    if getattr(impl_cls.forward, "_pq_hsa_wrapped", False):
        return {"installed": True, "already": True, "runner_attached": attached}
    original = impl_cls.forward

    def wrapped(self, layer, query, key, value, kv_cache, attn_metadata, output=None, **extra):
        return pq_or_dense_forward(original, self, layer, query, key, value, kv_cache, attn_metadata, output, **extra)

    wrapped._pq_hsa_wrapped = True
    wrapped._pq_hsa_original = original
    impl_cls.forward = wrapped
    return {"installed": True, "already": False, "runner_attached": attached}
