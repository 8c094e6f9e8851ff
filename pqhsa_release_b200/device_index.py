"""Device-resident IVF-PQ index pool and the thin wrappers over the C ABI.

A pool holds the index of S independent streams (stream = one request x one KV
head) in the list-sorted snapshot layout described in ``include/pqhsa.h``:
per-stream slots sorted by IVF list (so the list of a scan unit is uniform and
the per-list log-sum-exp needs no atomics) followed by an unsorted tail that
incremental encoding appends to.  This is the layout of the reference's
production snapshot (benchmarks/e2e_pq_param_sweep.py:4182-4305) with the tail
added so that a new key costs O(1).

torch is used for device memory and streams only; every computation of the
decode path happens in ``libpqhsa_b200.so``.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import Params, WsLayout

_DTYPE_CODE = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


@dataclass
class StreamIndexTensors:
    """One stream's index in insertion order, as the reference's ``IVFPQIndex`` +
    ``SparseKVCache`` hold it (pq_hsa/index/ivfpq.py:160-173,
    pq_hsa/attention/kv_cache.py:190)."""

    packed_codes: torch.Tensor   # uint8 [N, 4]
    list_ids: torch.Tensor       # integer [N]
    key_norms: torch.Tensor      # float [N]
    coarse_centroids: torch.Tensor   # float [L, 128]
    codebooks: torch.Tensor      # float [8, 16, 16]
    value_means: torch.Tensor    # float [L, 128]
    value_sums: torch.Tensor | None = None    # float [L, 128] (fp32 running sums)
    value_counts: torch.Tensor | None = None  # integer [L]


def codes_to_words(packed: torch.Tensor) -> torch.Tensor:
    """uint8 [N, 4] -> int32 [N] holding the little-endian word (subspace s in bits 4s..4s+3)."""
    p = packed.to(torch.int64)
    w = p[:, 0] | (p[:, 1] << 8) | (p[:, 2] << 16) | (p[:, 3] << 24)
    return w.to(torch.int32)


def words_to_codes(words: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`codes_to_words`: integer [..., N] -> uint8 [..., N, 4]."""
    w = words.to(torch.int64) & 0xFFFFFFFF
    return torch.stack([(w >> (8 * i)) & 0xFF for i in range(4)], dim=-1).to(torch.uint8)


def list_sorted_layout(list_ids: torch.Tensor, num_lists: int):
    """Stable sort by list (the CSR order of pq_hsa/index/ivfpq.py:864-882) and
    the scan units: ranges of at most 128 slots inside one list.
    Returns (perm, unit_off [U+1], unit_list [U])."""
    ids = list_ids.to(torch.int64)
    n = ids.numel()
    if ids.is_cuda and n and 0 < num_lists <= _lib.MAX_LISTS:
        # the counting sort of the index build's kernels: the same stable order, and the lists' sizes with it
        raw = ids.to(torch.int16).contiguous()  # u16 bit patterns
        order = torch.empty(n, dtype=torch.int32, device=ids.device)
        start = torch.empty(num_lists + 1, dtype=torch.int32, device=ids.device)
        with torch.cuda.device(ids.device):
            _lib.call("pqhsa_cluster_order", raw.data_ptr(), 1, n, num_lists, order.data_ptr(), start.data_ptr(),
                      torch.cuda.current_stream(ids.device).cuda_stream)
        perm = order.long()
        counts = (start[1:] - start[:-1]).long()
    else:
        perm = torch.argsort(ids, stable=True)
        counts = torch.bincount(ids, minlength=num_lists)
    off = torch.zeros(num_lists + 1, dtype=torch.int64, device=ids.device)
    off[1:] = torch.cumsum(counts, 0)
    per = (counts + _lib.UNIT_KEYS - 1) // _lib.UNIT_KEYS
    unit_list = torch.repeat_interleave(torch.arange(num_lists, device=ids.device), per)
    first = torch.cumsum(per, 0) - per
    within = torch.arange(unit_list.numel(), device=ids.device) - first[unit_list]
    start = off[unit_list] + within * _lib.UNIT_KEYS
    unit_off = torch.cat([start, torch.tensor([n], device=ids.device, dtype=torch.int64)])
    return perm, unit_off, unit_list


def _slot_units(unit_off: torch.Tensor, n: int) -> torch.Tensor:
    """Unit index of every slot of the sorted region, from the unit offsets."""
    if n == 0:
        return torch.zeros(0, dtype=torch.int64, device=unit_off.device)
    lens = unit_off[1:] - unit_off[:-1]
    return torch.repeat_interleave(torch.arange(lens.numel(), device=unit_off.device), lens)


class DeviceIndexPool:
    """Index pool + workspace + KV binding of a batch of streams on one GPU."""

    def __init__(
        self,
        *,
        num_streams: int,
        group: int,
        dtype: torch.dtype,
        device: torch.device | str,
        slot_capacity: int,
        num_lists: int,
        sink_tokens: int,
        local_window: int,
        scale: float,
        top_fraction: float | None,
        topk_fixed: int = 100,
        tail_capacity: int = 1024,
        max_full: int | None = None,
        hist_lo: float = 0.0,
        hist_width: float | None = None,
        select_margin: float = 0.0,
    ):
        if dtype not in _DTYPE_CODE:
            raise ValueError(f"unsupported dtype {dtype}: need float32, bfloat16 or float16")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("DeviceIndexPool needs a CUDA device: there is no CPU path")
        self.S, self.G, self.dtype = int(num_streams), int(group), dtype
        self.L = int(num_lists)
        self.cap = (int(slot_capacity) + 7) // 8 * 8
        self.tail_capacity = min(int(tail_capacity), self.cap)
        self.ucap = self.L + self.cap // _lib.UNIT_KEYS + 1
        self.sink, self.local = int(sink_tokens), int(local_window)
        self.max_full = int(max_full) if max_full is not None else self.sink + self.local + 512
        D = _lib.HEAD_DIM
        dev = self.device
        S, cap, L, ucap = self.S, self.cap, self.L, self.ucap
        self.codes = torch.zeros(S, cap, dtype=torch.int32, device=dev)
        self.norms = torch.zeros(S, cap, dtype=dtype, device=dev)
        self.list_ids = torch.zeros(S, cap, dtype=torch.int16, device=dev)
        self.slot_pos = torch.zeros(S, cap, dtype=torch.int32, device=dev)
        self.slot_unit = torch.zeros(S, cap, dtype=torch.int16, device=dev)
        self.norm_max = torch.zeros(S, dtype=torch.float32, device=dev)
        self.unit_off = torch.zeros(S, ucap + 1, dtype=torch.int32, device=dev)
        self.unit_list = torch.zeros(S, ucap, dtype=torch.int16, device=dev)
        self.coarse = torch.zeros(S, L, D, dtype=dtype, device=dev)
        self.codebooks = torch.zeros(S, _lib.SUBSPACES, _lib.CODES, D // _lib.SUBSPACES, dtype=dtype, device=dev)
        self.vmeans = torch.zeros(S, L, D, dtype=dtype, device=dev)
        self.vsum = torch.zeros(S, L, D, dtype=torch.float32, device=dev)
        self.vcnt = torch.zeros(S, L, dtype=torch.int32, device=dev)
        self.state = torch.zeros(S, _lib.STATE_INTS, dtype=torch.int32, device=dev)
        # contiguous copy of the slots the threshold estimate samples: (code, norm bits, list, slot)
        self.sample = torch.zeros(S, _lib.SAMPLE_KEYS, 4, dtype=torch.int32, device=dev)
        # host mirrors of the device counters (every update is deterministic)
        self.h_sorted = np.zeros(S, dtype=np.int64)
        self.h_tail = np.zeros(S, dtype=np.int64)
        self.h_seq = np.zeros(S, dtype=np.int64)

        p = Params()
        p.abi_version = _lib.ABI_VERSION
        p.dtype = _DTYPE_CODE[dtype]
        p.num_streams, p.group, p.head_dim = S, self.G, D
        p.num_lists, p.slot_capacity, p.unit_capacity = L, cap, ucap
        p.sink_tokens, p.local_window = self.sink, self.local
        p.max_slots, p.max_full = 0, self.max_full
        p.topk_fixed = int(topk_fixed)
        p.tail_capacity = self.tail_capacity
        p.top_fraction = -1.0 if top_fraction is None else float(top_fraction)
        p.scale = float(scale)
        p.hist_lo = float(hist_lo)
        p.hist_inv_width = 0.0 if hist_width is None else float(1.0 / hist_width)
        p.select_margin = float(select_margin)
        for name in ("codes", "norms", "list_ids", "slot_pos", "slot_unit", "unit_off", "unit_list", "coarse",
                     "codebooks", "vmeans", "vsum", "vcnt", "state", "norm_max", "sample"):
            setattr(p, name, getattr(self, name).data_ptr())
        self.p = p
        self.layout = WsLayout()
        _lib.call("pqhsa_workspace_layout", C.byref(p), C.byref(self.layout))
        self.workspace = torch.zeros(int(self.layout.total_bytes), dtype=torch.uint8, device=dev)
        p.workspace = self.workspace.data_ptr()
        p.workspace_bytes = int(self.layout.total_bytes)
        self._kv_keepalive = None
        self.graph_headroom = 0
        self._compact_error = None

    # ---- loading ---------------------------------------------------------
    def load_stream(self, s: int, idx: StreamIndexTensors | None, *, seq_len: int, req: int, kv_head: int) -> None:
        """Install one stream's index (insertion order in, list-sorted on the
        device).  ``idx`` None means no retrieval region yet (short context)."""
        dev = self.device
        sink_end = min(self.sink, seq_len)
        st = torch.zeros(_lib.STATE_INTS, dtype=torch.int32)
        st[_lib.ST_SEQ_LEN], st[_lib.ST_REQ], st[_lib.ST_KV_HEAD] = seq_len, req, kv_head
        n = 0
        if idx is not None:
            n = int(idx.list_ids.numel())
            lists = int(idx.coarse_centroids.shape[0])
            if n > self.cap:
                raise ValueError(f"stream has {n} indexed keys, pool capacity is {self.cap}")
            if lists > self.L:
                raise ValueError(f"stream has {lists} lists, pool is built for {self.L}")
            ids = idx.list_ids.to(dev).to(torch.int64)
            perm, unit_off, unit_list = list_sorted_layout(ids, lists)
            u = int(unit_list.numel())
            if u > self.ucap:
                raise ValueError("unit table overflow")
            self.codes[s, :n] = codes_to_words(idx.packed_codes.to(dev))[perm]
            self.norms[s, :n] = idx.key_norms.to(dev)[perm].to(self.dtype)
            self.list_ids[s, :n] = ids[perm].to(torch.int16)
            self.slot_pos[s, :n] = (perm + sink_end).to(torch.int32)
            self.unit_off[s, : u + 1] = unit_off.to(torch.int32)
            self.unit_list[s, :u] = unit_list.to(torch.int16)
            self.slot_unit[s, :n] = _slot_units(unit_off, n).to(torch.int16)
            self.norm_max[s] = self.norms[s, :n].float().max() if n else 0.0
            self.coarse[s].zero_()
            self.coarse[s, :lists] = idx.coarse_centroids.to(dev).to(self.dtype)
            self.codebooks[s] = idx.codebooks.to(dev).to(self.dtype)
            self.vmeans[s].zero_()
            self.vmeans[s, :lists] = idx.value_means.to(dev).to(self.dtype)
            self.vsum[s].zero_()
            self.vcnt[s].zero_()
            if idx.value_sums is not None and idx.value_counts is not None:
                self.vsum[s, :lists] = idx.value_sums.to(dev).float()
                self.vcnt[s, :lists] = idx.value_counts.to(dev).to(torch.int32)
            else:
                # running sums for later appends, rebuilt from the means and the list sizes
                cnt = torch.bincount(ids, minlength=lists)[:lists]
                self.vcnt[s, :lists] = cnt.to(torch.int32)
                self.vsum[s, :lists] = idx.value_means.to(dev).float() * cnt.unsqueeze(-1).float()
            st[_lib.ST_N_SORTED], st[_lib.ST_N_UNITS], st[_lib.ST_N_LISTS] = n, u, lists
        self.state[s] = st.to(dev)
        self.h_sorted[s], self.h_tail[s], self.h_seq[s] = n, 0, seq_len
        self._refresh_sample(s, n)

    def _refresh_sample(self, s: int, n_sorted: int) -> None:
        """Copy the slots floor(i * n_sorted / 4096), i < 4096, of the sorted region of stream ``s``
        into the sample array (streams with at most 4096 sorted slots are never sampled)."""
        ns = _lib.SAMPLE_KEYS
        if n_sorted <= ns:
            return
        j = (torch.arange(ns, device=self.device, dtype=torch.int64) * n_sorted) // ns
        rec = self.sample[s]
        rec[:, 0] = self.codes[s][j]
        rec[:, 1] = self.norms[s][j].float().view(torch.int32)
        rec[:, 2] = self.list_ids[s][j].to(torch.int32) & 0xFFFF
        rec[:, 3] = j.to(torch.int32)

    def export_stream(self, s: int) -> dict[str, torch.Tensor]:
        """Slots of stream ``s`` back in token order (for tests and state dicts)."""
        n = int(self.h_sorted[s] + self.h_tail[s])
        pos = self.slot_pos[s, :n].to(torch.int64)
        order = torch.argsort(pos)
        return {
            "packed_codes": words_to_codes(self.codes[s, :n][order]),
            "list_ids": self.list_ids[s, :n][order].to(torch.int64),
            "key_norms": self.norms[s, :n][order],
            "positions": pos[order],
        }

    def export_stream_state(self, s: int) -> StreamIndexTensors | None:
        """Everything needed to reinstall stream ``s`` with :meth:`load_stream` (token order)."""
        n = int(self.h_sorted[s] + self.h_tail[s])
        if n == 0:
            return None
        lists = int(self.state[s, _lib.ST_N_LISTS])
        e = self.export_stream(s)
        return StreamIndexTensors(
            packed_codes=e["packed_codes"].clone(), list_ids=e["list_ids"].clone(), key_norms=e["key_norms"].clone(),
            coarse_centroids=self.coarse[s, :lists].clone(), codebooks=self.codebooks[s].clone(),
            value_means=self.vmeans[s, :lists].clone(), value_sums=self.vsum[s, :lists].clone(),
            value_counts=self.vcnt[s, :lists].clone(),
        )

    def export_index(self, s: int) -> dict[str, torch.Tensor]:
        """Codebooks of stream ``s`` (the rows in use) for a refresh or a state dict."""
        lists = int(self.state[s, _lib.ST_N_LISTS])
        return {"coarse": self.coarse[s, :lists], "codebooks": self.codebooks[s], "value_means": self.vmeans[s, :lists]}

    # ---- KV cache binding ------------------------------------------------
    def bind_kv_contiguous(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """keys/values: [B, Hkv, capacity, 128] of the pool dtype (any strides
        that keep rows contiguous)."""
        if keys.dtype != self.dtype or values.dtype != self.dtype:
            raise ValueError("KV cache dtype does not match the pool dtype")
        if keys.shape != values.shape or keys.stride() != values.stride() or keys.stride(-1) != 1:
            raise ValueError("keys and values must have the same shape and strides with contiguous rows")
        p = self.p
        p.k_base, p.v_base = keys.data_ptr(), values.data_ptr()
        p.block_table = None
        p.max_blocks, p.block_size = 0, 0
        p.stride_block, p.stride_head, p.stride_row = keys.stride(0), keys.stride(1), keys.stride(2)
        self._kv_keepalive = (keys, values)

    def bind_kv_paged(self, kv_cache: torch.Tensor, block_table: torch.Tensor) -> None:
        """vLLM FLASH_ATTN pages, either layout (benchmarks/vllm_backend/paged_kv_fa.py:44-58):
        5-D ``[2, blocks, block_size, Hkv, 128]`` or 4-D ``[blocks, Hkv, block_size, 256]``
        (K then V in the last dim, arbitrary outer strides).  ``block_table``: int32
        [requests, max_blocks]."""
        if kv_cache.dtype != self.dtype:
            raise ValueError("KV cache dtype does not match the pool dtype")
        if block_table.dtype != torch.int32 or block_table.dim() != 2 or not block_table.is_contiguous():
            raise ValueError("block_table must be a contiguous int32 [requests, max_blocks] tensor")
        p = self.p
        esz = kv_cache.element_size()
        if kv_cache.dim() == 5:
            if kv_cache.stride(-1) != 1:
                raise ValueError("rows of the KV pages must be contiguous")
            p.k_base = kv_cache[0].data_ptr()
            p.v_base = kv_cache[1].data_ptr()
            p.block_size = kv_cache.shape[2]
            p.stride_block, p.stride_row, p.stride_head = kv_cache.stride(1), kv_cache.stride(2), kv_cache.stride(3)
        elif kv_cache.dim() == 4:
            if kv_cache.stride(-1) != 1 or kv_cache.shape[-1] != 2 * _lib.HEAD_DIM:
                raise ValueError("4-D KV pages must be [blocks, Hkv, block_size, 2*128] with contiguous rows")
            p.k_base = kv_cache.data_ptr()
            p.v_base = kv_cache.data_ptr() + _lib.HEAD_DIM * esz
            p.block_size = kv_cache.shape[2]
            p.stride_block, p.stride_head, p.stride_row = kv_cache.stride(0), kv_cache.stride(1), kv_cache.stride(2)
        else:
            raise ValueError(f"unsupported FLASH_ATTN kv_cache shape {tuple(kv_cache.shape)}")
        p.block_table = block_table.data_ptr()
        p.max_blocks = block_table.shape[1]
        self._kv_keepalive = (kv_cache, block_table)

    # ---- calls -----------------------------------------------------------
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _prep(self, q: torch.Tensor | None = None, out: torch.Tensor | None = None, mapped: bool = False) -> None:
        # grids are sized for the largest stream plus the growth a captured graph may see
        self.p.max_slots = min(int((self.h_sorted + self.h_tail).max()) + int(self.graph_headroom), self.cap)
        full = int((np.minimum(self.sink, self.h_seq) + np.maximum(
            self.h_seq - (np.minimum(self.sink, self.h_seq) + self.h_sorted + self.h_tail), 0)).max())
        if full > self.max_full:
            raise RuntimeError(
                f"{full} sink+local rows exceed max_full={self.max_full}: apply the pending index update "
                "or build the pool with a larger max_full")
        # with an io_map the streams pick their blocks of q / out themselves: the tensors may hold fewer blocks
        if q is not None:
            if q.dtype != self.dtype or not q.is_contiguous() or (not mapped and q.numel() != self.S * self.G * _lib.HEAD_DIM):
                raise ValueError(f"q must be a contiguous {self.dtype} tensor of {self.S}x{self.G}x128 elements")
            self.p.q = q.data_ptr()
        if out is not None:
            if out.dtype != self.dtype or not out.is_contiguous() or (not mapped and out.numel() != self.S * self.G * _lib.HEAD_DIM):
                raise ValueError("out must match q in dtype and size")
            self.p.out = out.data_ptr()

    def lut_build(self, q: torch.Tensor) -> None:
        self._prep(q)
        _lib.call("pqhsa_lut_build", C.byref(self.p), self._stream())

    def scan_select(self) -> None:
        self._prep()
        _lib.call("pqhsa_scan_select", C.byref(self.p), self._stream())

    def attend_merge(self, q: torch.Tensor, out: torch.Tensor) -> None:
        self._prep(q, out)
        _lib.call("pqhsa_attend_merge", C.byref(self.p), self._stream())

    def decode_step(self, q: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """q: [..., 128] with S*G rows in (stream, group) order -> context of the same shape."""
        if out is None:
            out = torch.empty_like(q)
        self._prep(q, out)
        _lib.call("pqhsa_decode_step", C.byref(self.p), self._stream())
        return out

    def run_stage(self, stage: int, q: torch.Tensor | None = None, out: torch.Tensor | None = None) -> None:
        """One kernel group of the step (``_lib.STAGE_*``), for per-kernel timing."""
        self._prep(q, out)
        _lib.call("pqhsa_run_stage", C.byref(self.p), int(stage), self._stream())

    def scan_scores(self, q: torch.Tensor) -> torch.Tensor:
        """Approximate logits of every slot, float32 [S*G, cap] (slot order)."""
        self.lut_build(q)
        scores = torch.zeros(self.S * self.G, self.cap, dtype=torch.float32, device=self.device)
        _lib.call("pqhsa_scan_scores", C.byref(self.p), scores.data_ptr(), self._stream())
        return scores

    def decode_step_append(self, q: torch.Tensor, new_k: torch.Tensor | None, new_v: torch.Tensor | None,
                           encode: int = 0, out: torch.Tensor | None = None, external: bool = False) -> torch.Tensor:
        """append_kv(new_k, new_v) + append_encode(encode) + decode_step(q) as one call of five
        launches (the first kernel does the append, the encode and the tables side by side).
        ``external`` (with new_k None): the caller already stored this step's rows in the cache;
        every live stream's length advances by one."""
        if (new_k is None) != (new_v is None):
            raise ValueError("new_k and new_v go together")
        if external and new_k is not None:
            raise ValueError("external=True goes with new_k=None")
        encode = int(encode)
        self.check_step(new_k is not None, external, encode)
        if out is None:
            out = torch.empty_like(q)
        self.enqueue_step_append(q, new_k, new_v, None, encode, out, external)
        self.note_step(new_k is not None, external, encode)
        return out

    def check_step(self, appended: bool, external: bool, encode: int) -> None:
        """Host-side admission of a fused step that encodes ``encode`` keys per stream."""
        if not encode:
            return
        if int((self.h_tail + encode).max()) > self.tail_capacity:
            raise RuntimeError("tail capacity exhausted: compact() the pool first")
        # the fused call encodes tokens that were in the cache before it (all of them with local_window == 0,
        # where the library appends first): the host mirror must not run ahead of the device
        room = self.h_seq - (np.minimum(self.sink, self.h_seq) + self.h_sorted + self.h_tail)
        if (appended and self.local == 0) or external:
            room = room + 1  # the new row is in the cache before the encode looks for it
        if int((room - encode).min()) < 0:
            raise ValueError("decode_step_append asked to index tokens that are not in the cache yet")

    def enqueue_step_append(self, q: torch.Tensor, new_k, new_v, enc_count: torch.Tensor | None, uniform: int,
                            out: torch.Tensor, external: bool, mapped: bool = False) -> None:
        """The library call of :meth:`decode_step_append` and nothing else (no host bookkeeping): what a
        CUDA-graph capture records.  ``enc_count``: device int32 [S] or None for ``uniform`` on every stream."""
        for t in (new_k, new_v):
            if t is not None and (t.dtype != self.dtype or not t.is_contiguous() or t.numel() != self.S * _lib.HEAD_DIM):
                raise ValueError(f"new_k/new_v must be contiguous {self.dtype} tensors of {self.S}x128 elements")
        if enc_count is not None and (enc_count.dtype != torch.int32 or enc_count.numel() != self.S or not enc_count.is_cuda):
            raise ValueError("enc_count must be a device int32 tensor with one entry per stream")
        self.p.external_append = 1 if external else 0
        self._prep(q, out, mapped)
        _lib.call("pqhsa_decode_step_append", C.byref(self.p), new_k.data_ptr() if new_k is not None else None,
                  new_v.data_ptr() if new_v is not None else None,
                  enc_count.data_ptr() if enc_count is not None else None, int(uniform), self._stream())

    def note_step(self, appended: bool, external: bool, encode: int) -> None:
        """Advance the host mirrors by one fused step (the device counters advance by themselves)."""
        if encode:
            self.h_tail += int(encode)
        if appended:
            self.h_seq += 1
        elif external:
            self.h_seq[self.h_seq > 0] += 1

    def append_kv(self, new_k: torch.Tensor, new_v: torch.Tensor) -> None:
        """Write one K/V row per stream at its current length and advance it."""
        for t in (new_k, new_v):
            if t.dtype != self.dtype or not t.is_contiguous() or t.numel() != self.S * _lib.HEAD_DIM:
                raise ValueError(f"new_k/new_v must be contiguous {self.dtype} tensors of {self.S}x128 elements")
        _lib.call("pqhsa_append_kv", C.byref(self.p), new_k.data_ptr(), new_v.data_ptr(), self._stream())
        self.h_seq += 1

    def note_replayed(self, appends: int = 0, encodes: int = 0) -> None:
        """Advance the host mirrors after replaying a captured CUDA graph that held
        ``appends`` append_kv and ``encodes`` single-key append_encode calls per stream
        (the device counters advance by themselves).  Negative values undo the
        bookkeeping of the capture pass, which runs no kernels."""
        self.h_seq += appends
        self.h_tail += encodes

    def note_external_append(self, count: int = 1) -> None:
        """The caller (e.g. vLLM) already wrote ``count`` new rows per request into the pages."""
        self.state[:, _lib.ST_SEQ_LEN] += count
        self.h_seq += count

    def append_encode(self, counts) -> None:
        """Encode the next ``counts[s]`` (or a uniform int) tokens after each stream's indexed region."""
        if isinstance(counts, int):
            cnt = np.full(self.S, counts, dtype=np.int64)
        else:
            cnt = np.asarray(counts, dtype=np.int64)
        sink_end = np.minimum(self.sink, self.h_seq)
        room = self.h_seq - (sink_end + self.h_sorted + self.h_tail)
        if (cnt > room).any():
            raise ValueError("append_encode asked to index tokens that are not in the cache")
        if ((self.h_tail + cnt) > self.tail_capacity).any() or ((self.h_sorted + self.h_tail + cnt) > self.cap).any():
            raise RuntimeError("index tail or slot capacity exhausted: call compact() or rebuild with more capacity")
        if isinstance(counts, int):
            _lib.call("pqhsa_append_encode", C.byref(self.p), None, int(counts), self._stream())
        else:
            dcnt = torch.as_tensor(cnt, dtype=torch.int32).to(self.device)
            _lib.call("pqhsa_append_encode", C.byref(self.p), dcnt.data_ptr(), 0, self._stream())
        self.h_tail += cnt

    def compact(self) -> None:
        """Merge every stream's tail into its list-sorted region and rebuild the scan units: one
        kernel over all streams, in place, no host round trip (``pqhsa_compact``).  The analogue of the
        reference's snapshot refresh after a flush (benchmarks/e2e_pq_param_sweep.py:4163-4363)."""
        if int(self.h_tail.max()) == 0:
            return
        if int(self.h_tail.max()) > _lib.COMPACT_MAX_TAIL:
            self._compact_by_sort()
            return
        if self._compact_error is None:
            self._compact_error = torch.zeros(1, dtype=torch.int32, device=self.device)
        _lib.call("pqhsa_compact", C.byref(self.p), self._compact_error.data_ptr(), self._stream())
        self.h_sorted += self.h_tail
        self.h_tail[:] = 0

    def compact_failed(self) -> bool:
        """True if a ``compact`` left a stream as it was (never with a pool built by this class)."""
        return self._compact_error is not None and bool(int(self._compact_error.item()) != 0)

    def _compact_by_sort(self) -> None:
        """``compact`` for tails too long for the kernel: a stable sort by (list, token position) per stream."""
        for s in range(self.S):
            if self.h_tail[s] == 0:
                continue
            n = int(self.h_sorted[s] + self.h_tail[s])
            lists = int(self.state[s, _lib.ST_N_LISTS])
            ids = self.list_ids[s, :n].to(torch.int64)
            # stable order: by list, then by token position
            pos = self.slot_pos[s, :n].to(torch.int64)
            by_pos = torch.argsort(pos)
            perm, unit_off, unit_list = list_sorted_layout(ids[by_pos], lists)
            order = by_pos[perm]
            u = int(unit_list.numel())
            self.codes[s, :n] = self.codes[s, :n][order]
            self.norms[s, :n] = self.norms[s, :n][order]
            self.list_ids[s, :n] = self.list_ids[s, :n][order]
            self.slot_pos[s, :n] = self.slot_pos[s, :n][order]
            self.unit_off[s, : u + 1] = unit_off.to(torch.int32)
            self.unit_list[s, :u] = unit_list.to(torch.int16)
            self.slot_unit[s, :n] = _slot_units(unit_off, n).to(torch.int16)
            self.state[s, _lib.ST_N_SORTED] = n
            self.state[s, _lib.ST_N_TAIL] = 0
            self.state[s, _lib.ST_N_UNITS] = u
            self.h_sorted[s], self.h_tail[s] = n, 0
            self._refresh_sample(s, n)

    # ---- workspace views (after a synchronise) ----------------------------
    def ws_view(self, name: str) -> torch.Tensor:
        lay, R = self.layout, self.S * self.G
        spec = {
            "lut": (torch.float32, (self.S, self.G, _lib.SUBSPACES, _lib.CODES)),
            "list_scores": (torch.float32, (self.S, self.G, _lib.MAX_LISTS)),
            "row_bin": (torch.float32, (R, 2)),
            "row_tau": (torch.float32, (R,)),
            "unit_max": (torch.float32, (R, self.ucap)),
            "unit_sum": (torch.float32, (R, self.ucap)),
            "tail_logit": (torch.float32, (R, lay.tail_cap)),
            "row_info": (torch.int32, (R, _lib.ROW_INFO_INTS)),
            "hitmap": (torch.int32, (R, self.ucap, _lib.UNIT_KEYS // 32)),
            "sel_slot": (torch.int32, (R, lay.kcap)),
            "sel_off": (torch.int64, (R, lay.kcap)),
            "partial": (torch.float32, (R, lay.chunks + 5, _lib.HEAD_DIM + 2)),
        }[name]
        dt, shape = spec
        nbytes = int(np.prod(shape)) * torch.empty(0, dtype=dt).element_size()
        off = int(getattr(lay, name))
        return self.workspace[off : off + nbytes].view(dt).view(*shape)

    def selected_positions(self, row: int) -> torch.Tensor:
        """Token positions of the keys selected for query row ``row`` in the last step (sorted)."""
        info = self.ws_view("row_info")[row]
        k = int(info[_lib.RI_K])
        slots = self.ws_view("sel_slot")[row, :k].to(torch.int64)
        return torch.sort(self.slot_pos[row // self.G][slots].to(torch.int64)).values
