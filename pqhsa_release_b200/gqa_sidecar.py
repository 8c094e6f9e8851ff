"""GQA sidecar: the object the vLLM decode runtime drives per (layer, request), with
the duck-typed surface of the reference's ``GQASidecar`` / ``GQASidecarFast``
(benchmarks/vllm_backend/gqa_sidecar.py:11-76, gqa_sidecar_fast.py:48-187):
one IVF-PQ stream per KV head, the G query heads h*G .. h*G+G-1 share stream h.

    build_cache(keys[B, Hkv, S, D], values)          append(keys[B, Hkv, D], values)
    lean_append(key[B, Hkv, D], value, q) -> bool    forward(queries[B, Hq, D]) -> [B, Hq, D]
    set_paged_kv_context(kv_cache, attn_metadata, seq_idx)
    checkpoint_prefix() / restore_prefix(...) / prefix_checkpoint_length
    apply_pending_index_update() / .adapter.apply_pending_index_update()

B is 1 in the reference (one sidecar per request); here a sidecar may also carry several
requests that advance together.  With a paged context set before ``build_cache`` the sidecar
keeps no K/V copy: the kernels read vLLM's pages in place through the block table (so the
reference's K/V ring, benchmarks/e2e_pq_param_sweep.py:2912-2986, has nothing to hold here).

Fast path.  ``lean_append`` only parks the step's K/V row; the ``forward`` that follows issues
ONE fused library call (row write + incremental encode + tables + scan + selection + attention,
five launches), and replays it as a CUDA graph over static input / output buffers once the
graph has validated itself: the output buffer is poisoned with NaN, the graph is replayed and
its result compared with the eager call on the same state - the self-check of
benchmarks/e2e_pq_param_sweep.py:6170-6201, at most three capture attempts (:7099-7107).
``forward`` may therefore return a view of a static buffer: callers copy it at once, as the
reference's runtime does (pq_hsa_decode_runtime.py:384-400).
"""

from __future__ import annotations

import os

import torch

from . import _lib
from .config import IVFPQConfig, SparseAttentionConfig
from .engine import PoolAttention
from .paged_kv import kv_cache_dims


class _StepGraph:
    """The fused step of one engine as a validated CUDA graph over static buffers."""

    def __init__(self, engine: PoolAttention, external: bool):
        pool = engine.pool
        S, G, D = pool.S, pool.G, _lib.HEAD_DIM
        dev, dt = pool.device, pool.dtype
        self.engine, self.external = engine, external
        self.generation = engine.generation
        # one buffer for the step's inputs: query rows, then the new K rows, then the new V rows
        self.inbuf = torch.zeros(S * G * D + 2 * S * D, dtype=dt, device=dev)
        self.q = self.inbuf[: S * G * D].view(engine.B, engine.H * G, D)
        self.nk = self.inbuf[S * G * D : S * G * D + S * D].view(S, D)
        self.nv = self.inbuf[S * G * D + S * D :].view(S, D)
        self.out = torch.zeros(engine.B, engine.H * G, D, dtype=dt, device=dev)
        self.enc = torch.zeros(S, dtype=torch.int32, device=dev)  # keys to encode per stream in the next replay
        self.enc_value = 0
        self.graph = None
        self.attempts = 0
        self.max_attempts = 3

    def _enqueue(self) -> None:
        self.engine.pool.enqueue_step_append(self.q, None if self.external else self.nk, None if self.external else self.nv,
                                             self.enc, 0, self.out, self.external)

    def _load(self, queries, keys, values, encode: int) -> None:
        # a caller that filled the static buffers itself (GQASidecar.static_inputs) passes their views: nothing to copy
        if queries.data_ptr() != self.q.data_ptr():
            self.q.copy_(queries)
        if not self.external:
            if keys.data_ptr() != self.nk.data_ptr():
                self.nk.copy_(keys.reshape(self.nk.shape))
            if values.data_ptr() != self.nv.data_ptr():
                self.nv.copy_(values.reshape(self.nv.shape))
        if encode != self.enc_value:
            self.enc.fill_(encode)
            self.enc_value = encode

    def run(self, queries, keys, values, encode: int) -> torch.Tensor:
        """One step.  The first call captures and validates; later calls replay."""
        pool = self.engine.pool
        self._load(queries, keys, values, encode)
        if self.graph is not None:
            self.graph.replay()
            return self.out
        if self.attempts >= self.max_attempts:
            self._enqueue()  # the graph never validated: eager launches over the same buffers
            return self.out
        # ---- capture + self-validation on this very step ----
        snap = [t.clone() for t in (pool.state, pool.norm_max, pool.vsum, pool.vcnt, pool.vmeans)]
        pool.graph_headroom = pool.cap  # grids sized for any growth the graph will see
        self._enqueue()                 # eager: also warms the lazy set-up outside the capture
        want = self.out.clone()
        while self.attempts < self.max_attempts:
            self.attempts += 1
            for t, s0 in zip((pool.state, pool.norm_max, pool.vsum, pool.vcnt, pool.vmeans), snap):
                t.copy_(s0)             # undo the step: the replay below is the one that counts
            torch.cuda.synchronize(pool.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._enqueue()
            self.out.fill_(float("nan"))
            g.replay()
            torch.cuda.synchronize(pool.device)
            if bool(torch.isfinite(self.out.float()).all()) and torch.allclose(self.out.float(), want.float(), rtol=2e-2, atol=2e-2):
                self.graph = g
                return self.out
        # no attempt validated: the state holds the last replay's step, its output is not trusted
        for t, s0 in zip((pool.state, pool.norm_max, pool.vsum, pool.vcnt, pool.vmeans), snap):
            t.copy_(s0)
        self._enqueue()
        return self.out


class GQASidecar:
    def __init__(self, index_config: IVFPQConfig, attention_config: SparseAttentionConfig, *,
                 num_query_heads: int, num_kv_heads: int, cuda_graph: bool | None = None) -> None:
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
        self._paged = None    # (kv_cache, block_table [B, max_blocks] int32, token capacity)
        self._pending = None  # (key, value) parked by lean_append for the next forward; (None, None) = stored by the caller
        self._use_graph = (os.environ.get("PQ_HSA_CUDA_GRAPH", "1") == "1") if cuda_graph is None else bool(cuda_graph)
        self._step_graph: _StepGraph | None = None
        self._checkpoint = None
        self.external_kv_write = False  # True: the caller stores each step's K/V in the pages itself (vLLM >= 0.10 layout)

    batched_heads_active = True  # all KV heads of all requests go through one launch sequence

    @property
    def cuda_graph_active(self) -> bool:
        return self._step_graph is not None and self._step_graph.graph is not None

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
        old = self._paged
        self._paged = (kv_cache, table, int(table.shape[1]) * bs)
        if self.engine.pool is not None and self.engine.paged:
            if old is None or old[0].data_ptr() != kv_cache.data_ptr() or old[1].data_ptr() != table.data_ptr():
                self.engine._paged = (kv_cache, table)
                self.engine.pool.bind_kv_paged(kv_cache, table)
                self.engine.generation += 1  # a captured graph holds the old addresses

    def build_cache(self, keys: torch.Tensor, values: torch.Tensor) -> "GQASidecar":
        if keys.ndim != 4 or values.ndim != 4:
            raise ValueError("keys/values must be [batch, kv_heads, seq, dim]")
        if keys.shape[1] != self.num_kv_heads:
            raise ValueError(f"expected keys [B, {self.num_kv_heads}, S, D], got {tuple(keys.shape)}")
        if self._paged is not None:
            kv_cache, table, cap = self._paged
            if keys.shape[0] != table.shape[0]:
                raise ValueError("one block-table row per request is needed")
            self.engine.build_paged(kv_cache, table, [int(keys.shape[2])] * int(keys.shape[0]), self.num_kv_heads, cap)
        else:
            self.engine.build(keys, values)
        self.length = int(keys.shape[2])
        self._pending = None
        self._step_graph = None
        return self

    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        if keys.ndim != 3 or values.ndim != 3:
            raise ValueError("append keys/values must be [batch, kv_heads, dim]")
        self._flush_pending()
        self.engine.append(keys, values)
        self.length += 1

    def _flush_pending(self) -> None:
        if self._pending is not None:
            k, v = self._pending
            self._pending = None
            if k is None:
                self.engine.pool.note_external_append(1)
                self.engine._after_append()
            else:
                self.engine.append(k, v)

    def lean_append(self, key: torch.Tensor, value: torch.Tensor, q: torch.Tensor | None = None) -> bool:
        """The step's token, ``key``/``value`` [B, Hkv, D] (one token per request), parked for the
        ``forward`` that follows, which appends it inside its own launch sequence - the one-launch
        append of benchmarks/e2e_pq_param_sweep.py:4575-4645 costs no launch at all here.  Returns
        False if the shape is not one token per request (the caller then uses ``append``)."""
        if key.ndim != 3 or self.engine.pool is None or key.shape[0] != self.engine.B:
            return False
        self._flush_pending()
        self._pending = (None, None) if (self.engine.paged and self.external_kv_write) else (key, value)
        self.length += 1
        return True

    def append_many(self, keys: torch.Tensor, values: torch.Tensor, *, flush_every: int = 0) -> int:
        if keys.ndim == 4:
            keys, values = keys[0], values[0]
        for i in range(int(keys.shape[1])):
            self.append(keys[:, i].unsqueeze(0), values[:, i].unsqueeze(0))
        return 0

    def apply_pending_index_update(self) -> int:
        """The deferred flush.  As in the production adapter, PQ_HSA_INCREMENTAL_FLUSH=1 (the default) moves the
        codebooks and encodes only the keys that became indexable since the last flush
        (benchmarks/e2e_pq_param_sweep.py:3213); 0 re-encodes every key as the library's online refresh does."""
        self._flush_pending()
        if os.environ.get("PQ_HSA_INCREMENTAL_FLUSH", "1") == "1":
            done = self.engine.apply_pending_incremental_flush()
        else:
            done = self.engine.apply_pending_index_update()
        return self.num_kv_heads * self.engine.B if done else 0

    def _graph_for(self, external: bool) -> _StepGraph:
        eng, sg = self.engine, self._step_graph
        if sg is None or sg.generation != eng.generation or sg.external != external:
            sg = self._step_graph = _StepGraph(eng, external)
        return sg

    def static_inputs(self):
        """Views of the fused step's static input buffer: ``(queries [B, Hq, D], key [B, Hkv, D], value [B, Hkv, D],
        flat)`` where ``flat`` is the one contiguous buffer behind the three (queries, then keys, then values).  A caller
        that writes a step's inputs there (one host-to-device copy into ``flat``) and passes these very views to
        ``lean_append`` and ``forward`` spares the copies into the buffer.  Valid until the cache is rebuilt or restored.
        No counterpart in the reference (its runtime copies: pq_hsa_decode_runtime.py:384-400)."""
        if self.engine.pool is None:
            raise RuntimeError("build_cache first")
        sg = self._graph_for(bool(self.engine.paged and self.external_kv_write))
        B, H, D = self.engine.B, self.engine.H, _lib.HEAD_DIM
        return sg.q, sg.nk.view(B, H, D), sg.nv.view(B, H, D), sg.inbuf

    def forward(self, queries: torch.Tensor) -> torch.Tensor:
        """queries ``[B, q_heads, dim]`` -> context ``[B, q_heads, dim]`` (possibly a view of a static buffer)."""
        if queries.ndim != 3 or queries.shape[0] != max(self.engine.B, 1):
            raise ValueError(f"queries must be [{max(self.engine.B, 1)}, q_heads, dim], got {tuple(queries.shape)}")
        if self._pending is None:
            return self.engine.forward(queries)
        k, v = self._pending
        self._pending = None
        eng = self.engine
        external = k is None
        if not self._use_graph:
            return eng.step(queries, k, v, external_write=external)
        encode, fused = eng.step_plan()
        grow = k is not None and not eng.paged and eng.length + 1 > eng.keys.shape[2]
        if not fused or grow:
            return eng.step(queries, k, v, external_write=external)  # refresh / growth steps run eagerly
        sg = self._graph_for(external)
        eng.pool.check_step(not external, external, encode)
        out = sg.run(queries, k, v, encode)
        eng.pool.note_step(not external, external, encode)
        eng.note_fused_step(encode)
        return out

    # ---- prefix checkpoints (benchmarks/e2e_pq_param_sweep.py:3358-3432, :3735-3899) -----------------
    @property
    def prefix_checkpoint_length(self) -> int | None:
        return None if self._checkpoint is None else int(self._checkpoint["length"])

    def checkpoint_prefix(self) -> None:
        """Keep the index as it stands (after the prefill build, before any decode token) so that the same
        prompt arriving again skips the k-means build: a device-side copy of the streams' index tensors and
        counters, about 12 bytes per key."""
        self._flush_pending()
        self._checkpoint = self.engine.snapshot()

    def restore_prefix(self, keys=None, values=None, *, kv_cache=None, attn_metadata=None, seq_idx: int = 0) -> bool:
        """Put the checkpointed index back (the request starts again from the prompt).  With pages the K/V
        rows are vLLM's and stay where they are; a sidecar that owns its cache truncates it to the prefix.
        Returns False if there is no checkpoint."""
        if self._checkpoint is None:
            return False
        self._pending = None
        if kv_cache is not None and attn_metadata is not None:
            self.set_paged_kv_context(kv_cache, attn_metadata, seq_idx)
        self.engine.restore_snapshot(self._checkpoint)
        self.length = int(self._checkpoint["length"])
        return True
