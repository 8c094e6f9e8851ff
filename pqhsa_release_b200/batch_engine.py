"""All running requests of one attention layer behind ONE index pool, reading vLLM's pages in place.

The reference's vLLM runtime keeps one sidecar per (layer, request) and loops the requests of a
decode step in Python (benchmarks/vllm_backend/pq_hsa_batch_decode.py:383-432: per request an
append launch, a graph replay and a context copy).  Here a layer owns one ``DeviceIndexPool``
whose streams are (request slot, KV head) pairs; a decode step of any number of requests with
any mix of context lengths is ONE fused library call - five launches, the result written
straight into vLLM's output tensor:

* a request keeps its slot for life, whatever row of the batch it sits in at a given step: the
  ``io_map`` of the call says which block of the query / output tensor a stream uses and the
  stream's request index says which block-table row addresses its pages;
* requests that are new in a step (or whose length jumped) get their index built from the pages
  (or restored from a prefix checkpoint) before the call; the others advance by the one token
  vLLM has just stored;
* the index follows the production policy per request: appended tokens stay in the exact local
  region until ``flush_every`` of them have gathered, then the keys that left the local window
  move the codebooks (EMA) and are encoded (``deferred``); or every step encodes the key that
  leaves the window (``incremental`` with interval 1, the c3 benchmark configuration);
* slots of requests that have left the batch are cleared and reused.
"""

from __future__ import annotations

import hashlib
from array import array

import numpy as np
import torch

from . import _lib
from .config import IVFPQConfig, SparseAttentionConfig, softmax_scale, validate_attention_config, validate_index_config
from .device_index import DeviceIndexPool
from .index_build import build_index_batch
from .paged_kv import gather_paged_range, kv_cache_dims


def prompt_key(context_len: int, prompt_token_ids) -> tuple[int, bytes]:
    """Key of a prefix checkpoint: (context length, blake2b of the prompt ids), as
    benchmarks/vllm_backend/pq_hsa_decode_runtime.py:403-422 builds it."""
    digest = hashlib.blake2b(array("I", prompt_token_ids).tobytes(), digest_size=16).digest()
    return int(context_len), digest


class PagedBatchEngine:
    def __init__(self, index_config: IVFPQConfig, attention_config: SparseAttentionConfig, *, num_query_heads: int,
                 num_kv_heads: int, max_requests: int, token_capacity: int, dtype: torch.dtype, device,
                 flush_every: int = 256, max_checkpoints: int = 4):
        validate_index_config(index_config)
        validate_attention_config(attention_config)
        if num_query_heads % num_kv_heads:
            raise ValueError("GQA requires num_query_heads % num_kv_heads == 0")
        self.icfg, self.acfg = index_config, attention_config
        self.Hq, self.H = int(num_query_heads), int(num_kv_heads)
        self.G = self.Hq // self.H
        self.max_requests = int(max_requests)
        self.flush_every = int(flush_every)
        a = attention_config
        window = max(a.index_update_interval, self.flush_every if a.index_update_strategy == "deferred" else 1, 1)
        self.pool = DeviceIndexPool(
            num_streams=self.max_requests * self.H, group=self.G, dtype=dtype, device=device,
            slot_capacity=int(token_capacity), num_lists=index_config.num_lists, sink_tokens=a.sink_tokens,
            local_window=a.local_window, scale=softmax_scale(a, _lib.HEAD_DIM), top_fraction=a.retrieval_top_fraction,
            topk_fixed=a.retrieval_topk, tail_capacity=min(int(token_capacity), max(4096, 4 * window)),
            max_full=a.sink_tokens + a.local_window + 2 * window + 64,
        )
        S = self.pool.S
        dev = self.pool.device
        self.io_map = torch.full((S,), -1, dtype=torch.int32, device=dev)
        self.enc = torch.zeros(S, dtype=torch.int32, device=dev)
        self._h_io = np.full(S, -1, dtype=np.int32)
        self._h_enc = np.zeros(S, dtype=np.int32)
        self._h_req = np.zeros(S, dtype=np.int32)
        self._last_io = self._last_enc = None
        self.pool.p.io_map = self.io_map.data_ptr()
        self.slots: dict[object, int] = {}
        self.free = list(range(self.max_requests - 1, -1, -1))
        z = np.zeros(self.max_requests, dtype=np.int64)
        self.length, self.indexed_length, self.pending = z.copy(), z.copy(), z.copy()
        self.since_flush = z.copy()
        self.row_of = np.full(self.max_requests, -1, dtype=np.int64)
        self.checkpoints: dict[tuple[int, bytes], dict] = {}
        self.max_checkpoints = int(max_checkpoints)
        self.stats = {"steps": 0, "builds": 0, "restores": 0, "flushes": 0, "evictions": 0, "launch_calls": 0}
        self._bound = None

    # ---- regions of one request (pq_hsa/attention/kv_cache.py:1160-1170) ----------------------------
    def _bounds(self, length: int, indexed: int) -> tuple[int, int]:
        a = self.acfg
        indexed = min(indexed, length)
        sink_end = min(a.sink_tokens, length)
        retr_end = max(sink_end, indexed - a.local_window) if a.local_window > 0 else max(sink_end, indexed)
        return sink_end, retr_end

    def _streams(self, slot: int) -> range:
        return range(slot * self.H, (slot + 1) * self.H)

    # ---- pages ----------------------------------------------------------------------------------------
    def bind(self, kv_cache: torch.Tensor, block_table: torch.Tensor) -> None:
        """vLLM's pages and this step's block table (int32 [requests, max_blocks], contiguous)."""
        tag = (kv_cache.data_ptr(), block_table.data_ptr(), tuple(block_table.shape), tuple(kv_cache.shape))
        if tag != self._bound:
            bs, heads, dim = kv_cache_dims(kv_cache)
            if heads != self.H or dim != _lib.HEAD_DIM:
                raise ValueError(f"kv_cache has {heads} KV heads of dim {dim}, engine was made for {self.H} x 128")
            self.pool.bind_kv_paged(kv_cache, block_table)
            self._bound = tag
        self._kv = (kv_cache, block_table)

    # ---- slots ----------------------------------------------------------------------------------------
    def _release(self, key) -> None:
        slot = self.slots.pop(key)
        st = list(self._streams(slot))
        self.pool.state[st[0] : st[-1] + 1].zero_()
        self.pool.h_sorted[st], self.pool.h_tail[st], self.pool.h_seq[st] = 0, 0, 0
        self.length[slot] = self.indexed_length[slot] = self.pending[slot] = self.since_flush[slot] = 0
        self.row_of[slot] = -1
        self.free.append(slot)
        self.stats["evictions"] += 1

    def _rollback(self, slot: int, length: int) -> None:
        """The request keeps its first ``length`` tokens (benchmarks/vllm_backend/pq_hsa_multi_query.py:30-45: the
        rejected tail of a speculative step disappears).  Only called when the index does not cover a dropped token:
        the pages are read in place and appended tokens touch nothing but the counters, so the counters go back and
        that is all.  ``stats["rollbacks"]`` counts the tokens dropped."""
        drop = int(self.length[slot]) - length
        if drop <= 0:
            return
        st = list(self._streams(slot))
        self.length[slot] = length
        self.pending[slot] = max(int(self.pending[slot]) - drop, 0)
        self.since_flush[slot] = max(int(self.since_flush[slot]) - drop, 0)
        self.pool.state[st[0] : st[-1] + 1, _lib.ST_SEQ_LEN] = length
        self.pool.h_seq[st] = length
        self.stats["rollbacks"] = self.stats.get("rollbacks", 0) + drop

    def _install(self, slot: int, row: int, length: int, pkey) -> None:
        """Index of a request that is new to the layer (or jumped): restored from the prefix checkpoint of the
        same prompt, else built from its pages.  ``length`` counts this step's token, which is in the pages."""
        kv_cache, table = self._kv
        snap = self.checkpoints.get(pkey) if pkey is not None else None
        st = list(self._streams(slot))
        if snap is not None and snap["length"] == length:
            self._restore(slot, snap, row)
            self.stats["restores"] += 1
        else:
            s, r = self._bounds(length, length)
            idx = None
            if r > s:
                if r - s > self.pool.cap:
                    raise RuntimeError(f"request of {length} tokens exceeds the pool's capacity of {self.pool.cap} keys")
                k, v = gather_paged_range(kv_cache, table, row, s, r)
                idx = build_index_batch(k, v, self.icfg)
            for h, sidx in enumerate(st):
                # the fused call advances every live stream by this step's token: load one short of it
                self.pool.load_stream(sidx, None if idx is None else idx[h], seq_len=length - 1, req=row, kv_head=h)
            self.stats["builds"] += 1
            if pkey is not None:
                self._checkpoint(slot, pkey, length)
        self.length[slot], self.indexed_length[slot], self.pending[slot] = length - 1, length, 0
        self.since_flush[slot] = 0
        self.row_of[slot] = row

    # ---- prefix checkpoints (benchmarks/e2e_pq_param_sweep.py:3358-3432, :3735-3899) -------------------
    _SNAP_SLOT = ("codes", "norms", "list_ids", "slot_pos", "slot_unit")
    _SNAP_FULL = ("unit_off", "unit_list", "coarse", "codebooks", "vmeans", "vsum", "vcnt", "state", "norm_max",
                  "sample")

    def _checkpoint(self, slot: int, pkey, length: int) -> None:
        p = self.pool
        st = list(self._streams(slot))
        lo, hi = st[0], st[-1] + 1
        n = int((p.h_sorted[st] + p.h_tail[st]).max())
        snap = {name: getattr(p, name)[lo:hi, :n].clone() for name in self._SNAP_SLOT}
        snap.update({name: getattr(p, name)[lo:hi].clone() for name in self._SNAP_FULL})
        snap.update(n=n, h_sorted=p.h_sorted[st].copy(), h_tail=p.h_tail[st].copy(), length=length)
        while len(self.checkpoints) >= self.max_checkpoints:
            self.checkpoints.pop(next(iter(self.checkpoints)))
        self.checkpoints[pkey] = snap

    def _restore(self, slot: int, snap: dict, row: int) -> None:
        p = self.pool
        st = list(self._streams(slot))
        lo, hi = st[0], st[-1] + 1
        n = snap["n"]
        for name in self._SNAP_SLOT:
            getattr(p, name)[lo:hi, :n].copy_(snap[name])
        for name in self._SNAP_FULL:
            getattr(p, name)[lo:hi].copy_(snap[name])
        p.state[lo:hi, _lib.ST_REQ] = row
        p.state[lo:hi, _lib.ST_SEQ_LEN] = snap["length"] - 1
        p.h_sorted[st], p.h_tail[st] = snap["h_sorted"], snap["h_tail"]
        p.h_seq[st] = snap["length"] - 1

    # ---- deferred flush of one request (benchmarks/e2e_pq_param_sweep.py:3021-3344) ---------------------
    @torch.no_grad()
    def _flush(self, slot: int) -> None:
        """The keys of this request that left the local window since its last update move the coarse centroids
        and the code words by one EMA step and are then encoded against them; old entries stay."""
        length = int(self.length[slot])
        s, old_r = self._bounds(length, int(self.indexed_length[slot]))
        self.indexed_length[slot], self.pending[slot], self.since_flush[slot] = length, 0, 0
        s, r = self._bounds(length, length)
        new = r - old_r
        if new <= 0:
            return
        p = self.pool
        st = list(self._streams(slot))
        lo, hi = st[0], st[-1] + 1
        kv_cache, table = self._kv
        row = int(self.row_of[slot])
        if old_r <= s:  # no index yet: build one
            k, v = gather_paged_range(kv_cache, table, row, s, r)
            idx = build_index_batch(k, v, self.icfg)
            for h, sidx in enumerate(st):
                p.load_stream(sidx, idx[h], seq_len=length, req=row, kv_head=h)
            self.stats["builds"] += 1
            return
        if int(p.h_tail[st].max()) + new > p.tail_capacity:
            p.compact()
        if new > p.tail_capacity or int((p.h_sorted[st] + p.h_tail[st]).max()) + new > p.cap:
            raise RuntimeError("index capacity exhausted: flush more often or raise the token capacity")
        lr, eps = self.icfg.online_codebook_lr, self.icfg.eps
        k, _ = gather_paged_range(kv_cache, table, row, old_r, r)  # [H, U, D]
        D = _lib.HEAD_DIM
        kf = k.float()
        nrm = torch.linalg.vector_norm(kf, dim=-1).to(k.dtype).float().clamp_min(eps)
        uu = kf / nrm.unsqueeze(-1)
        lists = int(p.state[lo, _lib.ST_N_LISTS])

        def ema(cent, x):
            ids = torch.cdist(x, cent, p=2).argmin(dim=-1)
            sums = torch.zeros_like(cent)
            sums.scatter_add_(1, ids.unsqueeze(-1).expand(-1, -1, x.shape[-1]), x)
            cnt = torch.zeros(cent.shape[:2], dtype=torch.float32, device=x.device)
            cnt.scatter_add_(1, ids, torch.ones_like(ids, dtype=torch.float32))
            means = sums / cnt.unsqueeze(-1).clamp_min(eps)
            return torch.where((cnt > 0).unsqueeze(-1), (1.0 - lr) * cent + lr * means, cent)

        coarse = ema(p.coarse[lo:hi, :lists].float(), uu).to(p.dtype)
        p.coarse[lo:hi, :lists] = coarse
        cf = coarse.float()
        ids = torch.cdist(uu, cf, p=2).argmin(dim=-1)
        ures = uu - torch.gather(cf, 1, ids.unsqueeze(-1).expand(-1, -1, D))
        M, sub = _lib.SUBSPACES, D // _lib.SUBSPACES
        chunks = ures.reshape(self.H, new, M, sub).permute(0, 2, 1, 3).reshape(self.H * M, new, sub)
        books = ema(p.codebooks[lo:hi].float().reshape(self.H * M, _lib.CODES, sub), chunks)
        p.codebooks[lo:hi] = books.reshape(self.H, M, _lib.CODES, sub).to(p.dtype)
        counts = np.zeros(p.S, dtype=np.int64)
        counts[st] = new
        p.append_encode(counts)
        self.stats["flushes"] += 1

    # ---- one decode step of the layer ---------------------------------------------------------------
    def step(self, query: torch.Tensor, kv_cache: torch.Tensor, block_table: torch.Tensor, req_keys: list,
             seq_lens: list[int], output: torch.Tensor, prompt_keys: list | None = None,
             hold_flush: bool = False) -> torch.Tensor:
        """query / output: ``[T, Hq, 128]`` contiguous, one token per request, row i = request ``req_keys[i]`` of
        ``seq_lens[i]`` tokens (this step's token included and already stored in the pages).  Writes the context
        into ``output`` and returns it.  A request whose length went BACK since its last step (speculative tokens
        were rejected) keeps its index as long as the index does not cover a dropped token.  ``hold_flush``: no
        deferred flush after this step (the step's token is not verified yet)."""
        T = len(req_keys)
        if T > self.max_requests:
            raise RuntimeError(f"{T} requests in the step, the layer's pool holds {self.max_requests}")
        if query.shape[0] < T or tuple(query.shape[1:]) != (self.Hq, _lib.HEAD_DIM) or not query.is_contiguous():
            raise ValueError(f"query must be a contiguous [T, {self.Hq}, 128] tensor")
        if not output.is_contiguous() or output.dtype != query.dtype or output.shape != query.shape:
            raise ValueError("output must match query in shape and dtype and be contiguous")
        self.bind(kv_cache, block_table)
        p = self.pool
        live = set(req_keys)
        for key in [k for k in self.slots if k not in live]:
            self._release(key)
        self._h_enc[:] = 0
        self._h_io[:] = -1
        incremental = self.acfg.index_update_strategy == "incremental"
        interval = max(self.acfg.index_update_interval, 1)
        req_changed = False
        for i, (key, length) in enumerate(zip(req_keys, seq_lens)):
            length = int(length)
            slot = self.slots.get(key)
            if slot is None:
                if not self.free:
                    raise RuntimeError("no free request slot in the layer's pool")
                slot = self.slots[key] = self.free.pop()
                self.length[slot] = -1
            st = self._streams(slot)
            self._h_io[st.start : st.stop] = np.arange(i * self.H, (i + 1) * self.H)
            self._h_req[st.start : st.stop] = i
            prev, prev_indexed = int(self.length[slot]), int(self.indexed_length[slot])
            if prev >= length and prev_indexed <= length - 1 and prev > 0:
                self._rollback(slot, length - 1)
                prev = length - 1
            s0, old_r = self._bounds(max(prev, 0), prev_indexed)
            _, r = self._bounds(length, length)
            sequential = prev + 1 == length
            if not sequential or (old_r <= s0 and r > s0 and incremental):
                # new to the layer, a jump in length, or the retrieval region only now begins: (re)install
                self._install(slot, i, length, None if prompt_keys is None else prompt_keys[i])
                self.length[slot] = length
                continue
            if int(self.row_of[slot]) != i:
                self.row_of[slot] = i
                req_changed = True
            # index policy of the token this step adds (pq_hsa/attention/kv_cache.py:195-226)
            self.pending[slot] += 1
            self.since_flush[slot] += 1
            if incremental and self.pending[slot] >= interval:
                new = r - old_r
                if new > 0:
                    if int(p.h_tail[list(st)].max()) + new > p.tail_capacity:
                        p.compact()
                    self._h_enc[st.start : st.stop] = new
                self.indexed_length[slot], self.pending[slot] = length, 0
            self.length[slot] = length
        if req_changed:
            p.state[:, _lib.ST_REQ].copy_(torch.from_numpy(self._h_req.copy()).pin_memory().to(p.device, non_blocking=True))
        io_now = self._h_io.tobytes()
        if io_now != self._last_io:
            self.io_map.copy_(torch.from_numpy(self._h_io.copy()).pin_memory(), non_blocking=True)
            self._last_io = io_now
        enc_now = self._h_enc.tobytes()
        if enc_now != self._last_enc:
            self.enc.copy_(torch.from_numpy(self._h_enc.copy()).pin_memory(), non_blocking=True)
            self._last_enc = enc_now
        if self._h_enc.any():
            # host mirror of what the fused call will encode
            p.h_tail += self._h_enc.astype(np.int64)
        p.enqueue_step_append(query, None, None, self.enc, 0, output, external=True, mapped=True)
        p.h_seq[p.h_seq > 0] += 1
        self.stats["steps"] += 1
        self.stats["launch_calls"] += 1
        # deferred policy: a request flushes once flush_every tokens have gathered since its last update
        if self.acfg.index_update_strategy == "deferred" and self.flush_every > 0 and not hold_flush:
            for key in req_keys:
                slot = self.slots[key]
                if self.since_flush[slot] >= self.flush_every:
                    self._flush(slot)
        elif not incremental and self.acfg.index_update_strategy != "deferred":
            raise RuntimeError("the batched vLLM path supports the 'deferred' and 'incremental' update strategies")
        return output
