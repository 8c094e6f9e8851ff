"""Host-side engine shared by the adapters: one KV store + one device index pool
for B requests x Hkv KV heads x G query heads per KV head.

It keeps the bookkeeping of the reference's ``SparseKVCache`` (regions, pending
tokens, update strategies: pq_hsa/attention/kv_cache.py:195-314, :1160-1201) on
the host as plain integers and leaves every per-step computation to the CUDA
library.  Index construction and the codebook-moving refresh are set-up work and
run as torch tensor operations on the device (``index_build``).
"""

from __future__ import annotations

import torch

from . import _lib
from .config import (IVFPQConfig, SparseAttentionConfig, softmax_scale, validate_attention_config,
                     validate_index_config)
from .device_index import DeviceIndexPool, StreamIndexTensors
from .index_build import build_index_batch, online_refresh_batch


class PoolAttention:
    """B x Hkv streams with G query rows each, contiguous K/V owned here or pages owned by the caller."""

    def __init__(self, index_config: IVFPQConfig, attention_config: SparseAttentionConfig, *, group: int = 1,
                 growth_margin: int = 4096):
        validate_index_config(index_config)
        validate_attention_config(attention_config)
        self.icfg, self.acfg = index_config, attention_config
        self.G = int(group)
        self.growth_margin = int(growth_margin)
        self.pool: DeviceIndexPool | None = None
        self.keys = self.values = None       # [B, Hkv, capacity, D] when the engine owns the cache
        self.B = self.H = 0
        self.length = 0                      # tokens per request (all requests advance together)
        self.indexed_length = 0
        self.pending = 0
        self.deferred_pending = False
        self.paged = False
        self.index_adds = self.index_rebuilds = self.online_updates = 0
        self.generation = 0                  # bumped whenever a device address the library sees changes

    # ---- regions (pq_hsa/attention/kv_cache.py:1160-1170) -------------------
    def bounds(self, length=None, indexed=None):
        length = self.length if length is None else length
        indexed = min(self.indexed_length if indexed is None else indexed, length)
        sink_end = min(self.acfg.sink_tokens, length)
        if self.acfg.local_window > 0:
            retr_end = max(sink_end, indexed - self.acfg.local_window)
        else:
            retr_end = max(sink_end, indexed)
        return sink_end, retr_end

    # ---- build ---------------------------------------------------------------
    def build(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """keys/values [B, Hkv, S, 128] on a CUDA device."""
        if keys.dim() != 4 or values.dim() != 4:
            raise ValueError("keys and values must be [batch, heads, seq, dim]")
        if keys.shape != values.shape:
            raise ValueError("keys and values must have the same shape")
        if keys.shape[-1] != _lib.HEAD_DIM:
            raise ValueError(f"head_dim must be {_lib.HEAD_DIM}")
        if not keys.is_cuda:
            raise RuntimeError("the B200 path needs CUDA tensors: there is no CPU fallback")
        B, H, S, D = keys.shape
        self.B, self.H = B, H
        cap = S + self.growth_margin
        self.keys = torch.zeros(B, H, cap, D, dtype=keys.dtype, device=keys.device)
        self.values = torch.zeros_like(self.keys)
        self.keys[:, :, :S] = keys
        self.values[:, :, :S] = values
        self.length = self.indexed_length = S
        self.pending = 0
        self.deferred_pending = False
        self.paged = False
        self._make_pool(keys.dtype, keys.device, cap)
        self.pool.bind_kv_contiguous(self.keys, self.values)
        self.generation += 1
        self._rebuild_index()

    def _make_pool(self, dtype, device, token_capacity: int) -> None:
        a = self.acfg
        interval = max(a.index_update_interval, 1)
        self.pool = DeviceIndexPool(
            num_streams=self.B * self.H, group=self.G, dtype=dtype, device=device,
            slot_capacity=token_capacity, num_lists=self.icfg.num_lists, sink_tokens=a.sink_tokens,
            local_window=a.local_window, scale=softmax_scale(a, _lib.HEAD_DIM),
            top_fraction=a.retrieval_top_fraction, topk_fixed=a.retrieval_topk,
            tail_capacity=min(token_capacity, 4096),
            max_full=a.sink_tokens + a.local_window + 2 * max(interval, 256) + 64,
        )

    def _kv_rows(self, lo: int, hi: int):
        """K/V rows [B, Hkv, hi - lo, D] of token range [lo, hi)."""
        if self.paged:
            from .paged_kv import gather_paged_range

            kv_cache, block_table = self._paged
            pairs = [gather_paged_range(kv_cache, block_table, b, lo, hi) for b in range(self.B)]
            return torch.stack([p[0] for p in pairs]), torch.stack([p[1] for p in pairs])
        return self.keys[:, :, lo:hi], self.values[:, :, lo:hi]

    def _rebuild_index(self) -> None:
        s, r = self.bounds()
        for b in range(self.B):
            idx = None
            if r > s:
                k, v = self._kv_rows(s, r)
                idx = build_index_batch(k[b], v[b], self.icfg)
            for h in range(self.H):
                self.pool.load_stream(b * self.H + h, None if idx is None else idx[h], seq_len=self.length, req=b,
                                      kv_head=h)
        self.index_rebuilds += 1

    # ---- append (pq_hsa/attention/kv_cache.py:195-314) --------------------------
    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """keys/values [B, Hkv, 128]: one new token per stream."""
        if self.pool is None:
            raise RuntimeError("build_cache must be called first")
        exp = (self.B, self.H, _lib.HEAD_DIM)
        if tuple(keys.shape) != exp or tuple(values.shape) != exp:
            raise ValueError(f"keys/values must have shape {exp}, got {tuple(keys.shape)}")
        if not self.paged:
            if self.length + 1 > self.keys.shape[2]:
                self._grow()
            self.pool.append_kv(keys.reshape(-1, _lib.HEAD_DIM).contiguous(),
                                values.reshape(-1, _lib.HEAD_DIM).contiguous())
        else:
            self.pool.note_external_append(1)
        self._after_append()

    def apply_pending_index_update(self) -> bool:
        if not self.deferred_pending:
            return False
        self._refresh_now()
        self.deferred_pending = False
        return True

    @torch.no_grad()
    def apply_pending_incremental_flush(self) -> bool:
        """The production form of the deferred update (benchmarks/e2e_pq_param_sweep.py:3021-3344 with
        PQ_HSA_INCREMENTAL_FLUSH=1, its default): the keys that left the local window since the last update move
        the coarse centroids and the code words by one EMA step, then ONLY those keys are assigned and encoded
        against the moved codebooks - by the library's append-encode kernel, into the unsorted tail; old list ids
        and codes stay - and the value means follow as running sums (the count-weighted merge of :3259-3281).
        The EMA itself is a handful of tensor operations over the update batch (S x U x L distances)."""
        if not self.deferred_pending:
            return False
        self.deferred_pending = False
        s, old_r = self.bounds()
        if old_r <= s:            # no index yet: build one
            self._refresh_now()
            return True
        self.indexed_length = self.length
        self.pending = 0
        s, r = self.bounds()
        new = r - old_r
        if new <= 0:
            return True
        p = self.pool
        if r - s > p.cap:
            raise RuntimeError("index slot capacity exhausted: rebuild the cache with a larger margin")
        if int(p.h_tail.max()) + new > p.tail_capacity:
            p.compact()
        if new > p.tail_capacity:
            raise RuntimeError("the update batch exceeds the tail capacity: flush more often")
        lr, eps = self.icfg.online_codebook_lr, self.icfg.eps
        k, _ = self._kv_rows(old_r, r)                       # [B, H, U, D]
        S, D = self.B * self.H, _lib.HEAD_DIM
        kf = k.reshape(S, new, D).float()
        nrm = torch.linalg.vector_norm(kf, dim=-1).to(k.dtype).float().clamp_min(eps)
        uu = kf / nrm.unsqueeze(-1)
        lists = int(p.state[0, _lib.ST_N_LISTS])
        coarse = p.coarse[:, :lists].float()

        def ema(cent, x):
            ids = torch.cdist(x, cent, p=2).argmin(dim=-1)
            sums = torch.zeros_like(cent)
            sums.scatter_add_(1, ids.unsqueeze(-1).expand(-1, -1, x.shape[-1]), x)
            cnt = torch.zeros(cent.shape[:2], dtype=torch.float32, device=x.device)
            cnt.scatter_add_(1, ids, torch.ones_like(ids, dtype=torch.float32))
            means = sums / cnt.unsqueeze(-1).clamp_min(eps)
            return torch.where((cnt > 0).unsqueeze(-1), (1.0 - lr) * cent + lr * means, cent)

        coarse = ema(coarse, uu).to(p.dtype)
        p.coarse[:, :lists] = coarse
        cf = coarse.float()
        ids = torch.cdist(uu, cf, p=2).argmin(dim=-1)
        ures = uu - torch.gather(cf, 1, ids.unsqueeze(-1).expand(-1, -1, D))
        M, sub = _lib.SUBSPACES, D // _lib.SUBSPACES
        books = p.codebooks.float()                          # [S, M, 16, sub]
        chunks = ures.reshape(S, new, M, sub).permute(0, 2, 1, 3).reshape(S * M, new, sub)
        books = ema(books.reshape(S * M, _lib.CODES, sub), chunks).reshape(S, M, _lib.CODES, sub)
        p.codebooks.copy_(books.to(p.dtype))
        p.append_encode(int(new))                            # assign + encode the batch, value sums and means
        self.online_updates += 1
        return True

    def _grow(self) -> None:
        B, H, cap, D = self.keys.shape
        ncap = cap + max(self.growth_margin, cap // 2)
        nk = torch.zeros(B, H, ncap, D, dtype=self.keys.dtype, device=self.keys.device)
        nv = torch.zeros_like(nk)
        nk[:, :, :cap], nv[:, :, :cap] = self.keys, self.values
        self.keys, self.values = nk, nv
        self.pool.bind_kv_contiguous(self.keys, self.values)
        self.generation += 1

    def _refresh_now(self) -> None:
        strategy = self.acfg.index_update_strategy
        s, old_r = self.bounds()
        had_index = old_r > s
        self.indexed_length = self.length
        self.pending = 0
        s, r = self.bounds()
        if strategy == "rebuild" or not had_index:
            if r > s:
                if r - s > self.pool.cap:
                    raise RuntimeError("index slot capacity exhausted: rebuild the cache with a larger margin")
                self._rebuild_index()
            return
        new = r - old_r
        if new <= 0:
            return
        if strategy == "incremental":
            if int(self.pool.h_tail.max()) + new > self.pool.tail_capacity:
                self.pool.compact()
            self.pool.append_encode(int(new))
            self.index_adds += 1
            return
        # "online" / "deferred": move the codebooks towards the new keys and re-encode everything
        # (pq_hsa/index/ivfpq.py:647-707)
        if r - s > self.pool.cap:
            raise RuntimeError("index slot capacity exhausted: rebuild the cache with a larger margin")
        for b in range(self.B):
            k, v = self._kv_rows(s, r)
            cur = [self.pool.export_index(b * self.H + h) for h in range(self.H)]
            idx = online_refresh_batch(k[b], v[b], cur, new, self.icfg)
            for h in range(self.H):
                self.pool.load_stream(b * self.H + h, idx[h], seq_len=self.length, req=b, kv_head=h)
        self.online_updates += 1

    # ---- checkpoint / resume ----------------------------------------------------------
    def restore(self, att: dict) -> None:
        """Reinstall the state produced by the adapter's ``state_dict`` without rebuilding
        any index (pq_hsa/attention/multihead.py:120-154 does the same per stream)."""
        keys, values = att["keys"], att["values"]
        if not keys.is_cuda:
            raise RuntimeError("the B200 path needs CUDA tensors: there is no CPU fallback")
        B, H, S, D = keys.shape
        self.B, self.H = B, H
        cap = S + self.growth_margin
        self.keys = torch.zeros(B, H, cap, D, dtype=keys.dtype, device=keys.device)
        self.values = torch.zeros_like(self.keys)
        self.keys[:, :, :S], self.values[:, :, :S] = keys, values
        self.length = S
        self.indexed_length = int(att["indexed_length"])
        self.pending = int(att["pending"])
        self.deferred_pending = bool(att["deferred_pending"])
        self.paged = False
        self._make_pool(keys.dtype, keys.device, cap)
        self.pool.bind_kv_contiguous(self.keys, self.values)
        self.generation += 1
        streams = att["streams"]
        if len(streams) != B * H:
            raise ValueError("stream state count does not match leading_shape")
        for s, st in enumerate(streams):
            self.pool.load_stream(s, st, seq_len=S, req=s // H, kv_head=s % H)

    # ---- pages owned by the caller (vLLM) -----------------------------------------------
    def build_paged(self, kv_cache: torch.Tensor, block_table: torch.Tensor, seq_lens: list[int], num_kv_heads: int,
                    token_capacity: int) -> None:
        """Index the requests of a paged cache in place: nothing is copied, the attend kernel
        reads K/V rows through ``block_table``.  All requests must currently have the same
        length (ragged batches build one engine per request, as the reference does:
        benchmarks/vllm_backend/pq_hsa_batch_decode.py:383-432)."""
        from .paged_kv import gather_paged_range

        if len(set(seq_lens)) != 1:
            raise ValueError("build_paged needs equal sequence lengths; build one engine per request otherwise")
        self.B, self.H = len(seq_lens), int(num_kv_heads)
        self.length = self.indexed_length = int(seq_lens[0])
        self.pending = 0
        self.deferred_pending = False
        self.paged = True
        self.keys = self.values = None
        self._paged = (kv_cache, block_table)
        self._make_pool(kv_cache.dtype, kv_cache.device, token_capacity)
        self.pool.bind_kv_paged(kv_cache, block_table)
        self.generation += 1
        s, r = self.bounds()
        for b in range(self.B):
            idx = None
            if r > s:
                k, v = gather_paged_range(kv_cache, block_table, b, s, r)
                idx = build_index_batch(k, v, self.icfg)
            for h in range(self.H):
                self.pool.load_stream(b * self.H + h, None if idx is None else idx[h], seq_len=self.length, req=b,
                                      kv_head=h)
        self.index_rebuilds += 1

    # ---- one decode step: append + index update + attention as ONE library call ---------------
    def step_plan(self) -> tuple[int, bool]:
        """Bookkeeping of :meth:`append` for a token that the next :meth:`step` call will carry: advances the
        host counters and returns ``(encode, fused)`` - how many keys per stream the fused library call has
        to encode, and whether the update can ride in that call at all (rebuild / online refreshes and a full
        tail cannot: the caller then appends and refreshes with the separate calls first)."""
        a = self.acfg
        pending = self.pending + 1
        if pending < a.index_update_interval or a.index_update_strategy == "deferred":
            return 0, True
        if a.index_update_strategy != "incremental":
            return 0, False
        s, old_r = self.bounds()
        if old_r <= s:
            return 0, False                      # no index yet: the refresh builds one
        _, r = self.bounds(self.length + 1, self.length + 1)
        new = r - old_r
        if new <= 0:
            return 0, True
        if int(self.pool.h_tail.max()) + new > self.pool.tail_capacity:
            return 0, False                      # the tail has to be folded into the sorted region first
        return int(new), True

    def step(self, queries: torch.Tensor, keys: torch.Tensor | None = None, values: torch.Tensor | None = None,
             out: torch.Tensor | None = None, *, external_write: bool = False) -> torch.Tensor:
        """``append(keys, values)`` followed by ``forward(queries)`` as one fused library call (token row
        write, incremental encode of the keys that leave the local window, tables, scan, selection,
        attention: five launches), with the bookkeeping of :meth:`append`.  ``external_write``: the
        caller's own cache write already stored the row (vLLM's pages), only the length advances."""
        if self.pool is None:
            raise RuntimeError("build_cache must be called first")
        if keys is None and not external_write:
            return self.forward(queries, out)
        exp = (self.B, self.H * self.G, _lib.HEAD_DIM)
        if tuple(queries.shape) != exp:
            raise ValueError(f"queries must have shape {exp}, got {tuple(queries.shape)}")
        encode, fused = self.step_plan()
        if not fused or (keys is not None and not self.paged and self.length + 1 > self.keys.shape[2]):
            if keys is None:
                self.pool.note_external_append(1)
                self._after_append()
            else:
                self.append(keys, values)
            return self.forward(queries, out)
        p = self.pool
        if keys is not None:
            exp_kv = (self.B, self.H, _lib.HEAD_DIM)
            if tuple(keys.shape) != exp_kv or tuple(values.shape) != exp_kv:
                raise ValueError(f"keys/values must have shape {exp_kv}, got {tuple(keys.shape)}")
            nk = keys.reshape(-1, _lib.HEAD_DIM).contiguous()
            nv = values.reshape(-1, _lib.HEAD_DIM).contiguous()
            res = p.decode_step_append(queries.contiguous(), nk, nv, encode=encode, out=out)
        else:
            res = p.decode_step_append(queries.contiguous(), None, None, encode=encode, out=out, external=True)
        self.note_fused_step(encode)
        return res

    def note_fused_step(self, encode: int) -> None:
        """The host counters of append() / _refresh_now() after a fused step that encoded ``encode`` keys."""
        self.length += 1
        self.pending += 1
        if self.pending >= self.acfg.index_update_interval:
            if self.acfg.index_update_strategy == "deferred":
                self.deferred_pending = True
            else:
                self.indexed_length = self.length
                self.pending = 0
                if encode:
                    self.index_adds += 1

    # ---- prefix checkpoint (benchmarks/e2e_pq_param_sweep.py:3358-3432, :3735-3899) ---------------------
    _SNAP_SLOT = ("codes", "norms", "list_ids", "slot_pos", "slot_unit")
    _SNAP_FULL = ("unit_off", "unit_list", "coarse", "codebooks", "vmeans", "vsum", "vcnt", "state", "norm_max",
                  "sample")

    def snapshot(self) -> dict:
        """Device-side copy of everything the index holds (slot arrays up to the longest stream, tables,
        counters) plus the host counters: what :meth:`restore_snapshot` needs to put the engine back without
        rebuilding anything."""
        if self.pool is None:
            raise RuntimeError("build_cache must be called first")
        p = self.pool
        n = int((p.h_sorted + p.h_tail).max()) if p.S else 0
        snap = {name: getattr(p, name)[:, :n].clone() for name in self._SNAP_SLOT}
        snap.update({name: getattr(p, name).clone() for name in self._SNAP_FULL})
        snap.update(n=n, h_sorted=p.h_sorted.copy(), h_tail=p.h_tail.copy(), h_seq=p.h_seq.copy(), length=self.length,
                    indexed_length=self.indexed_length, pending=self.pending, deferred_pending=self.deferred_pending,
                    shape=(self.B, self.H, p.cap, p.L))
        return snap

    def restore_snapshot(self, snap: dict) -> None:
        """Inverse of :meth:`snapshot` on the same pool (same request count, heads and capacity).  The K/V
        rows are not touched: tokens past the checkpoint simply stop counting."""
        p = self.pool
        if p is None or snap["shape"] != (self.B, self.H, p.cap, p.L):
            raise ValueError("the checkpoint was taken from a different pool")
        n = snap["n"]
        for name in self._SNAP_SLOT:
            getattr(p, name)[:, :n].copy_(snap[name])
        for name in self._SNAP_FULL:
            getattr(p, name).copy_(snap[name])
        p.h_sorted[:], p.h_tail[:], p.h_seq[:] = snap["h_sorted"], snap["h_tail"], snap["h_seq"]
        self.length, self.indexed_length = snap["length"], snap["indexed_length"]
        self.pending, self.deferred_pending = snap["pending"], snap["deferred_pending"]

    def _after_append(self) -> None:
        self.length += 1
        self.pending += 1
        if self.pending >= self.acfg.index_update_interval:
            if self.acfg.index_update_strategy == "deferred":
                self.deferred_pending = True
            else:
                self._refresh_now()

    # ---- forward -------------------------------------------------------------------
    def forward(self, queries: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """queries [B, Hkv * G, 128] -> context of the same shape."""
        if self.pool is None:
            raise RuntimeError("build_cache must be called first")
        exp = (self.B, self.H * self.G, _lib.HEAD_DIM)
        if tuple(queries.shape) != exp:
            raise ValueError(f"queries must have shape {exp}, got {tuple(queries.shape)}")
        q = queries.contiguous()
        res = self.pool.decode_step(q, out)
        return res
