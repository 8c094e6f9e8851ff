"""CPU oracle for the PQ-HSA per-step decode operator.  TEST INFRASTRUCTURE ONLY.

This file restates, in torch-on-CPU, the arithmetic of the reference's decode
path so that the CUDA kernels can be checked against it on a machine that does
not have the reference checked out.  Only ``tests/``, the smoke check and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import it; the
product package never does.

Parity status: PINNED.  ``tests/golden/make_golden.py`` imports the reference
package itself and stores its index tensors, scores, top-k sets and outputs;
``tests/test_oracle_golden.py`` requires this restatement to reproduce them
bit for bit (integers, indices) or to 1e-6 (floats).

Every function names the reference lines it follows (paths are relative to the
reference project root).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from math import ceil, sqrt

import torch

# --------------------------------------------------------------------------
# 4-bit code packing                          pq_hsa/index/packing.py:6-60
# --------------------------------------------------------------------------


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[N, M] codes in 0..15 -> [N, ceil(M/2)] uint8; subspace 2j sits in the
    low nibble of byte j and subspace 2j+1 in the high nibble
    (pq_hsa/index/packing.py:6-34)."""
    if codes.ndim != 2:
        raise ValueError("codes must be [N, M]")
    if codes.numel() and (int(codes.min()) < 0 or int(codes.max()) > 15):
        raise ValueError("4-bit packing requires codes in [0, 15]")
    n, m = codes.shape
    c = codes.to(torch.uint8)
    if m % 2:
        c = torch.cat([c, torch.zeros(n, 1, dtype=torch.uint8)], dim=1)
    return (c[:, 0::2] & 0x0F) | (c[:, 1::2] << 4)


def unpack_nibbles(packed: torch.Tensor, num_subspaces: int) -> torch.Tensor:
    """Inverse of :func:`pack_nibbles` -> int64 [N, M]
    (pq_hsa/index/packing.py:37-60)."""
    if packed.ndim != 2 or packed.shape[1] != (num_subspaces + 1) // 2:
        raise ValueError("packed width does not match num_subspaces")
    out = torch.empty(packed.shape[0], num_subspaces, dtype=torch.long)
    out[:, 0::2] = (packed[:, : (num_subspaces + 1) // 2] & 0x0F).long()
    if num_subspaces > 1:
        out[:, 1::2] = (packed[:, : num_subspaces // 2] >> 4).long()
    return out


def codes_as_u32(packed: torch.Tensor) -> torch.Tensor:
    """[N, 4] uint8 -> [N] int64 holding the little-endian 32-bit word, i.e.
    subspace s occupies bits 4s..4s+3
    (pq_hsa/kernels/triton_lut_scan_h20.py:728-738)."""
    p = packed.long()
    return p[:, 0] | (p[:, 1] << 8) | (p[:, 2] << 16) | (p[:, 3] << 24)


# --------------------------------------------------------------------------
# k-means                                      pq_hsa/index/kmeans.py:108-227
# --------------------------------------------------------------------------


def nearest_centroid(vectors: torch.Tensor, centroids: torch.Tensor, chunk: int = 16384) -> torch.Tensor:
    """argmin_k (|c_k|^2 - 2 v.c_k), evaluated in fp32 in chunks of rows
    (pq_hsa/index/kmeans.py:108-131)."""
    cf = centroids.float()
    csq = (cf * cf).sum(dim=1)
    out = torch.empty(vectors.shape[0], dtype=torch.long)
    for lo in range(0, vectors.shape[0], chunk):
        hi = min(vectors.shape[0], lo + chunk)
        sc = csq.unsqueeze(0) - 2.0 * vectors[lo:hi].float().matmul(cf.t())
        out[lo:hi] = sc.argmin(dim=1)
    return out


def kmeans_l2(vectors: torch.Tensor, k: int, *, max_iter: int, seed: int, eps: float = 1e-12):
    """Seeded Lloyd iterations: random-permutation init, early stop when the
    assignment repeats, empty clusters re-seeded from random rows, final
    assignment against the final centroids (pq_hsa/index/kmeans.py:134-227)."""
    n, d = vectors.shape
    if n == 0:
        raise ValueError("cannot train k-means with zero vectors")
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    if n >= k:
        perm = torch.randperm(n, generator=gen)
        cent = vectors[perm[:k]].clone()
    else:
        extra = torch.randint(0, n, (k - n,), generator=gen)
        cent = torch.cat([vectors, vectors[extra]], dim=0).clone()
    assign = torch.zeros(n, dtype=torch.long)
    for _ in range(max_iter):
        nxt = nearest_centroid(vectors, cent)
        same = torch.equal(assign, nxt)
        assign = nxt
        if same:
            break
        acc = torch.zeros(k, d, dtype=torch.float32)
        cnt = torch.bincount(assign, minlength=k).to(torch.float32)
        acc.index_add_(0, assign, vectors.float())
        live = cnt > 0
        acc[live] /= cnt[live].unsqueeze(1).clamp_min(eps)
        if (~live).any():
            repl = torch.randint(0, n, (int((~live).sum()),), generator=gen)
            acc[~live] = vectors[repl].float()
        cent = acc.to(vectors.dtype)
    return cent, nearest_centroid(vectors, cent)


# --------------------------------------------------------------------------
# product quantiser                               pq_hsa/index/pq.py:47-217
# --------------------------------------------------------------------------


def pq_train(vectors: torch.Tensor, m: int, bits: int, *, max_iter: int, seed: int, eps: float = 1e-12):
    """One k-means per subspace with seed ``seed + subspace``
    (pq_hsa/index/pq.py:81-94)."""
    n, d = vectors.shape
    sub = d // m
    chunks = vectors.reshape(n, m, sub)
    books = [
        kmeans_l2(chunks[:, j, :].contiguous(), 1 << bits, max_iter=max_iter, seed=seed + j, eps=eps)[0]
        for j in range(m)
    ]
    return torch.stack(books, dim=0)


def pq_encode(vectors: torch.Tensor, codebooks: torch.Tensor) -> torch.Tensor:
    """Per subspace: argmin over code words of the fp32 Euclidean distance as
    torch.cdist computes it (pq_hsa/index/pq.py:97-115)."""
    m, _, sub = codebooks.shape
    chunks = vectors.reshape(vectors.shape[0], m, sub)
    cols = [
        torch.cdist(chunks[:, j, :].float(), codebooks[j].float(), p=2).argmin(dim=1)
        for j in range(m)
    ]
    return torch.stack(cols, dim=1)


def pq_lut(query: torch.Tensor, codebooks: torch.Tensor) -> torch.Tensor:
    """lut[b, m, c] = <q_b restricted to subspace m, codebooks[m, c]>
    (pq_hsa/index/pq.py:190-217)."""
    m, _, sub = codebooks.shape
    q = query.reshape(query.shape[0], m, sub)
    return torch.bmm(q.permute(1, 0, 2), codebooks.transpose(1, 2)).permute(1, 0, 2)


def scan_packed_lut(packed: torch.Tensor, lut: torch.Tensor, m: int) -> torch.Tensor:
    """score[b, n] = sum over subspaces, in subspace order 0..m-1, of
    lut[b, s, nibble_s(n)] (pq_hsa/kernels/lut_scan.py:101-114)."""
    out = torch.zeros(lut.shape[0], packed.shape[0], dtype=lut.dtype)
    for s in range(m):
        byte = packed[:, s // 2]
        nib = ((byte >> 4) if (s % 2) else (byte & 0x0F)).long()
        out += lut[:, s, :].gather(1, nib.unsqueeze(0).expand(lut.shape[0], -1))
    return out


# --------------------------------------------------------------------------
# IVF-PQ index                                  pq_hsa/index/ivfpq.py:84-1213
# --------------------------------------------------------------------------


@dataclass
class OracleIndexConfig:
    """The fields of ``IVFPQConfig`` that the decode path reads
    (pq_hsa/index/ivfpq.py:84-101); defaults are the production values of
    ``paper_index_config`` (benchmarks/vllm_backend/pq_hsa_decode_runtime.py:140-155)."""

    num_lists: int = 512
    num_subspaces: int = 8
    num_bits: int = 4
    coarse_max_iter: int = 1
    pq_max_iter: int = 2
    seed: int = 0
    eps: float = 1e-12
    online_codebook_lr: float = 0.05


@dataclass
class OracleIndex:
    """Residual IVF-PQ over unit key directions with the key norm kept beside
    the code (``residual=True``, ``direction_normalize=True``, no rotation)."""

    cfg: OracleIndexConfig
    coarse: torch.Tensor = None        # [L, D]   means of unit directions (not re-normalised)
    codebooks: torch.Tensor = None     # [M, 16, D/M]   residual space
    list_ids: torch.Tensor = None      # [N] int64 (the reference stores uint16)
    packed: torch.Tensor = None        # [N, M/2] uint8
    norms: torch.Tensor = None         # [N]  key dtype, clamped at eps

    @property
    def num_vectors(self) -> int:
        return 0 if self.list_ids is None else int(self.list_ids.shape[0])

    # pq_hsa/index/ivfpq.py:1052-1059
    def split_direction(self, keys: torch.Tensor):
        nrm = torch.linalg.vector_norm(keys.float(), dim=-1).to(keys.dtype).clamp_min(self.cfg.eps)
        return keys / nrm.unsqueeze(-1), nrm

    # pq_hsa/index/ivfpq.py:1001-1005
    def assign(self, unit_keys: torch.Tensor) -> torch.Tensor:
        return torch.cdist(unit_keys.float(), self.coarse.float(), p=2).argmin(dim=1)

    # pq_hsa/index/ivfpq.py:275-348
    def build(self, keys: torch.Tensor) -> "OracleIndex":
        c = self.cfg
        unit, self.norms = self.split_direction(keys)
        lists = min(c.num_lists, unit.shape[0])
        self.coarse, self.list_ids = kmeans_l2(unit, lists, max_iter=c.coarse_max_iter, seed=c.seed, eps=c.eps)
        resid = unit - self.coarse[self.list_ids]
        self.codebooks = pq_train(
            resid, c.num_subspaces, c.num_bits, max_iter=c.pq_max_iter, seed=c.seed + 10_000, eps=c.eps
        )
        self.packed = pack_nibbles(pq_encode(resid, self.codebooks))
        return self

    # pq_hsa/index/ivfpq.py:598-645
    def add(self, keys: torch.Tensor) -> torch.Tensor:
        """Encode new keys against the fixed codebooks and append them."""
        if keys.shape[0] == 0:
            return torch.empty(0, dtype=torch.long)
        unit, nrm = self.split_direction(keys)
        lid = self.assign(unit)
        resid = unit - self.coarse[lid]
        new_packed = pack_nibbles(pq_encode(resid, self.codebooks))
        self.list_ids = torch.cat([self.list_ids, lid])
        self.norms = torch.cat([self.norms, nrm])
        self.packed = torch.cat([self.packed, new_packed])
        return lid

    # pq_hsa/index/ivfpq.py:864-882
    def inverted_lists(self):
        """CSR form: offsets [L+1] and the stable argsort of the list ids."""
        lists = self.coarse.shape[0]
        cnt = torch.bincount(self.list_ids, minlength=lists)
        off = torch.zeros(lists + 1, dtype=torch.int64)
        off[1:] = torch.cumsum(cnt, dim=0)
        return off, torch.argsort(self.list_ids, stable=True)

    # pq_hsa/index/ivfpq.py:709-727, :1061-1070, :1084-1118, :1179-1190
    def approximate_scores(self, queries: torch.Tensor) -> torch.Tensor:
        """[Q, D] -> [Q, N] estimates of q.k: unit-query LUT scan, plus the
        unit query's dot with the key's list centroid, times |q| |k|."""
        qn = torch.linalg.vector_norm(queries.float(), dim=-1).to(queries.dtype).clamp_min(self.cfg.eps)
        qu = queries / qn.unsqueeze(-1)
        s = scan_packed_lut(self.packed, pq_lut(qu, self.codebooks), self.cfg.num_subspaces)
        s = s + qu.matmul(self.coarse.T)[:, self.list_ids]
        return s * qn.unsqueeze(-1) * self.norms.unsqueeze(0)

    # pq_hsa/index/ivfpq.py:647-707, :1160-1177 and pq_hsa/index/pq.py:117-173
    def online_refresh(self, keys: torch.Tensor, update_keys: torch.Tensor) -> "OracleIndex":
        """EMA-move the coarse centroids and the code words towards the
        mini-batch, then re-assign and re-encode every key."""
        lr = self.cfg.online_codebook_lr
        unit, self.norms = self.split_direction(keys)
        uu, _ = self.split_direction(update_keys)
        lid = self.assign(uu)
        lists = self.coarse.shape[0]
        sums = torch.zeros_like(self.coarse)
        cnt = torch.bincount(lid, minlength=lists).to(uu.dtype)
        sums.index_add_(0, lid, uu)
        live = cnt > 0
        means = sums[live] / cnt[live].unsqueeze(1).clamp_min(self.cfg.eps)
        self.coarse[live] = (1.0 - lr) * self.coarse[live] + lr * means
        lid = self.assign(uu)
        ures = uu - self.coarse[lid]
        m, ncodes, sub = self.codebooks.shape
        chunks = ures.reshape(ures.shape[0], m, sub)
        newbooks = self.codebooks.clone()
        for j in range(m):
            a = torch.cdist(chunks[:, j, :].float(), self.codebooks[j].float(), p=2).argmin(dim=1)
            s = torch.zeros_like(self.codebooks[j])
            n = torch.bincount(a, minlength=ncodes).to(ures.dtype)
            s.index_add_(0, a, chunks[:, j, :])
            ok = n > 0
            mu = s[ok] / n[ok].unsqueeze(1).clamp_min(self.cfg.eps)
            newbooks[j, ok] = (1.0 - lr) * self.codebooks[j, ok] + lr * mu
        self.codebooks = newbooks
        self.list_ids = self.assign(unit)
        self.packed = pack_nibbles(pq_encode(unit - self.coarse[self.list_ids], self.codebooks))
        return self


# --------------------------------------------------------------------------
# regions, value means, top-k count
# --------------------------------------------------------------------------


def region_bounds(length: int, indexed_length: int, sink: int, local: int):
    """(sink_end, retrieval_end): sink = [0, sink_end), retrieval =
    [sink_end, retrieval_end), local = [retrieval_end, length)
    (pq_hsa/attention/kv_cache.py:1160-1170)."""
    sink_end = min(sink, length)
    indexed_length = min(indexed_length, length)
    if local > 0:
        retrieval_end = max(sink_end, indexed_length - local)
    else:
        retrieval_end = max(sink_end, indexed_length)
    return sink_end, retrieval_end


def list_value_means(list_ids: torch.Tensor, values: torch.Tensor, lists: int):
    """Per-list mean of the value rows, accumulated in the value dtype; empty
    lists get a zero row (pq_hsa/attention/kv_cache.py:688-728, :766-776).
    Returns (means, sums, counts)."""
    sums = torch.zeros(lists, values.shape[1], dtype=values.dtype)
    sums.index_add_(0, list_ids, values)
    cnt = torch.bincount(list_ids, minlength=lists).to(values.dtype)
    means = torch.zeros_like(sums)
    live = cnt > 0
    means[live] = sums[live] / cnt[live].unsqueeze(1)
    return means, sums, cnt


def resolve_topk(retrieval_len: int, top_fraction: float | None, topk: int = 100) -> int:
    """min(max(ceil(N * fraction), 0), N) in Python double precision
    (pq_hsa/attention/sparse_attention.py:1756-1783)."""
    if retrieval_len == 0:
        return 0
    k = ceil(retrieval_len * top_fraction) if top_fraction is not None else topk
    return min(max(k, 0), retrieval_len)


# --------------------------------------------------------------------------
# hybrid softmax with per-list background
# --------------------------------------------------------------------------


@dataclass
class HybridDetail:
    output: torch.Tensor                # [Q, Dv]
    approx_logits: torch.Tensor         # [Q, N]   scale * approximate q.k
    topk_local: torch.Tensor            # [Q, K]   retrieval-local indices, best first
    topk_approx: torch.Tensor           # [Q, K]
    exact_logits: torch.Tensor          # [Q, K]
    full_logits: torch.Tensor           # [Q, F]
    list_mass: torch.Tensor             # [Q, L]  exp mass per list after removing the selected keys
    denom: torch.Tensor                 # [Q]
    row_max: torch.Tensor               # [Q]


def hybrid_centroid_attention(
    queries: torch.Tensor,
    approx_raw: torch.Tensor,
    list_ids: torch.Tensor,
    value_means: torch.Tensor,
    keys: torch.Tensor,
    values: torch.Tensor,
    full_positions: torch.Tensor,
    retrieval_start: int,
    k: int,
    scale: float,
) -> HybridDetail:
    """One softmax over three sources: exact logits of the sink and local
    rows, exact logits of the k best-scoring retrieval rows, and for every
    other retrieval row its approximate logit paired with the mean value of
    its list (pq_hsa/attention/sparse_attention.py:633-666 for the selection,
    :807-857 for the exact logits, :887-1012 for the merge)."""
    nq = queries.shape[0]
    approx = approx_raw * scale
    if k > 0:
        top_val, top_idx = torch.topk(approx, k=k, dim=1, sorted=True)
    else:
        top_val = torch.empty(nq, 0, dtype=approx.dtype)
        top_idx = torch.empty(nq, 0, dtype=torch.long)
    full_k = keys[full_positions]
    full_v = values[full_positions]
    full_logits = queries.matmul(full_k.T) * scale
    sel_pos = top_idx + retrieval_start
    sel_k = keys[sel_pos.reshape(-1)].reshape(nq, k, -1)
    sel_v = values[sel_pos.reshape(-1)].reshape(nq, k, -1)
    exact = torch.bmm(sel_k, queries.unsqueeze(-1)).squeeze(-1) * scale

    row_max = None
    if full_positions.numel() > 0:
        row_max = full_logits.max(dim=1).values
    if approx.shape[1] > 0:
        amax = top_val[:, 0] if k > 0 else approx.max(dim=1).values
        row_max = amax if row_max is None else torch.maximum(row_max, amax)
    if k > 0:
        emax = exact.max(dim=1).values
        row_max = emax if row_max is None else torch.maximum(row_max, emax)

    full_exp = torch.exp(full_logits - row_max[:, None])
    retr_exp = torch.exp(approx - row_max[:, None])
    old_exp = retr_exp.gather(1, top_idx)
    exact_exp = torch.exp(exact - row_max[:, None])
    denom = full_exp.sum(dim=1) + retr_exp.sum(dim=1) - old_exp.sum(dim=1) + exact_exp.sum(dim=1)
    denom = denom.clamp_min(torch.finfo(denom.dtype).tiny)

    out_full = (full_exp / denom[:, None]).matmul(full_v)
    if k > 0:
        out_exact = torch.bmm((exact_exp / denom[:, None]).unsqueeze(1), sel_v).squeeze(1)
    else:
        out_exact = torch.zeros(nq, values.shape[-1], dtype=values.dtype)
    lists = value_means.shape[0]
    mass = torch.zeros(nq, lists, dtype=approx.dtype)
    mass.scatter_add_(1, list_ids.unsqueeze(0).expand(nq, -1), retr_exp)
    if k > 0:
        mass.scatter_add_(1, list_ids[top_idx], -old_exp)
    out_bg = (mass / denom[:, None]).matmul(value_means)
    return HybridDetail(
        output=out_full + out_exact + out_bg,
        approx_logits=approx,
        topk_local=top_idx,
        topk_approx=top_val,
        exact_logits=exact,
        full_logits=full_logits,
        list_mass=mass,
        denom=denom,
        row_max=row_max,
    )


# --------------------------------------------------------------------------
# one stream = one (request, KV head): cache + index + operator
# --------------------------------------------------------------------------


@dataclass
class OracleAttentionConfig:
    """The fields of ``SparseAttentionConfig`` used by the production hybrid
    path (pq_hsa/attention/sparse_attention.py:15-37; production values:
    benchmarks/vllm_backend/pq_hsa_decode_runtime.py:158-177)."""

    sink_tokens: int = 4
    local_window: int = 128
    retrieval_top_fraction: float | None = 0.02
    retrieval_topk: int = 100
    scale: float | None = None
    index_update_interval: int = 256
    index_update_strategy: str = "deferred"


class OracleStream:
    """Mirror of ``IVFPQSparseAttention`` + ``SparseKVCache`` in hybrid /
    centroid / all_pq mode with exact re-rank and no attention details."""

    def __init__(self, index_cfg: OracleIndexConfig, attn_cfg: OracleAttentionConfig):
        self.icfg = index_cfg
        self.acfg = attn_cfg
        self.keys = None
        self.values = None
        self.index: OracleIndex | None = None
        self.value_means = None
        self._vsum = None
        self._vcnt = None
        self.length = 0
        self.indexed_length = 0
        self.pending = 0
        self.deferred_pending = False

    # ---- regions --------------------------------------------------------
    def bounds(self):
        return region_bounds(self.length, self.indexed_length, self.acfg.sink_tokens, self.acfg.local_window)

    def full_positions(self) -> torch.Tensor:
        s, r = self.bounds()
        return torch.cat([torch.arange(0, s), torch.arange(r, self.length)])

    # ---- build (pq_hsa/attention/kv_cache.py:72-193, :633-664) ----------
    def build_cache(self, keys: torch.Tensor, values: torch.Tensor) -> "OracleStream":
        self.keys = keys.clone()
        self.values = values.clone()
        self.length = self.indexed_length = keys.shape[0]
        self.pending = 0
        self._rebuild()
        return self

    def _rebuild(self):
        s, r = self.bounds()
        if r - s == 0:
            self.index = None
            self.value_means = None
            return
        self.index = OracleIndex(self.icfg).build(self.keys[s:r])
        self.value_means, _, _ = list_value_means(
            self.index.list_ids, self.values[s:r], self.index.coarse.shape[0]
        )
        self._vsum = self._vcnt = None

    # ---- append (pq_hsa/attention/kv_cache.py:195-226, :259-314) --------
    def append(self, key: torch.Tensor, value: torch.Tensor) -> None:
        self.keys = torch.cat([self.keys, key[None]])
        self.values = torch.cat([self.values, value[None]])
        self.length += 1
        self.pending += 1
        if self.pending >= self.acfg.index_update_interval:
            if self.acfg.index_update_strategy == "deferred":
                self.deferred_pending = True
            else:
                self._refresh_now()

    def apply_pending_index_update(self) -> bool:
        if not self.deferred_pending:
            return False
        self._refresh_now()
        self.deferred_pending = False
        return True

    def _refresh_now(self):
        if self.index is None or self.acfg.index_update_strategy == "rebuild":
            self.indexed_length = self.length
            self.pending = 0
            self._rebuild()
            return
        s, old_r = self.bounds()
        self.indexed_length = self.length
        self.pending = 0
        s, r = self.bounds()
        if r == old_r:
            return
        if self.acfg.index_update_strategy in ("online", "deferred"):
            # pq_hsa/attention/kv_cache.py:666-676
            rk = self.keys[s:r]
            self.index.online_refresh(rk, rk[old_r - s:])
            self.value_means, _, _ = list_value_means(
                self.index.list_ids, self.values[s:r], self.index.coarse.shape[0]
            )
            self._vsum = self._vcnt = None
            return
        # incremental: pq_hsa/attention/kv_cache.py:308-312, :730-764
        lid = self.index.add(self.keys[old_r:r])
        lists = self.index.coarse.shape[0]
        if self._vsum is None:
            self.value_means, self._vsum, self._vcnt = list_value_means(
                self.index.list_ids, self.values[s:r], lists
            )
        else:
            new_v = self.values[old_r:r]
            self._vsum.index_add_(0, lid, new_v)
            self._vcnt += torch.bincount(lid, minlength=lists).to(new_v.dtype)
            self.value_means = torch.zeros_like(self._vsum)
            live = self._vcnt > 0
            self.value_means[live] = self._vsum[live] / self._vcnt[live].unsqueeze(1)

    # ---- production deferred flush (benchmarks/e2e_pq_param_sweep.py:3021-3344, incremental branch) ----
    def apply_pending_incremental_flush(self) -> bool:
        """The head-batched flush of the production adapter with PQ_HSA_INCREMENTAL_FLUSH=1 (its default),
        restated for one stream: the keys that left the local window since the last update move the coarse
        centroids and the code words by one EMA step (benchmarks/e2e_pq_param_sweep.py:3173-3220, PQ part
        :2454-2513), then ONLY those keys are assigned and encoded against the moved codebooks (:3222-3256) -
        old list ids and codes stay - and the value means are merged count-weighted (:3259-3281).
        Pinned by tests/golden/golden_flush_incremental.npz: the reference's own method run on CPU tensors
        (tests/golden/make_golden.py, ``production_flush``), which this reproduces bit for bit."""
        if not self.deferred_pending:
            return False
        self.deferred_pending = False
        if self.index is None:
            self._refresh_now()
            return True
        s, old_r = self.bounds()
        self.indexed_length = self.length
        self.pending = 0
        s, r = self.bounds()
        if r <= old_r:
            return True
        ix, lr, eps = self.index, self.icfg.online_codebook_lr, self.icfg.eps
        new_keys, new_vals = self.keys[old_r:r], self.values[old_r:r]
        uu, nrm = ix.split_direction(new_keys)
        lists = ix.coarse.shape[0]
        # coarse EMA on the update batch (:3173-3190), then re-assignment and residuals (:3191-3195)
        lid = ix.assign(uu)
        sums = torch.zeros_like(ix.coarse)
        sums.index_add_(0, lid, uu)
        cnt = torch.bincount(lid, minlength=lists).to(uu.dtype)
        means = sums / cnt.unsqueeze(1).clamp_min(eps)
        ix.coarse = torch.where((cnt > 0).unsqueeze(1), (1.0 - lr) * ix.coarse + lr * means, ix.coarse)
        lid = ix.assign(uu)
        ures = uu - ix.coarse[lid]
        # code-word EMA on the update residuals (:3197-3220 = :2454-2513)
        m, ncodes, sub = ix.codebooks.shape
        chunks = ures.reshape(ures.shape[0], m, sub)
        newbooks = ix.codebooks.clone()
        for j in range(m):
            a = torch.cdist(chunks[:, j, :].float(), ix.codebooks[j].float(), p=2).argmin(dim=1)
            sj = torch.zeros_like(ix.codebooks[j])
            sj.index_add_(0, a, chunks[:, j, :])
            nj = torch.bincount(a, minlength=ncodes).to(ures.dtype)
            mu = sj / nj.unsqueeze(1).clamp_min(eps)
            newbooks[j] = torch.where((nj > 0).unsqueeze(1), (1.0 - lr) * ix.codebooks[j] + lr * mu, ix.codebooks[j])
        ix.codebooks = newbooks
        # only the update batch is encoded, against the moved codebooks (:3222-3256)
        old_counts = torch.bincount(ix.list_ids, minlength=lists).to(new_vals.dtype)
        ix.list_ids = torch.cat([ix.list_ids, lid])
        ix.norms = torch.cat([ix.norms, nrm])
        ix.packed = torch.cat([ix.packed, pack_nibbles(pq_encode(ures, ix.codebooks))])
        # value means: count-weighted merge (:3259-3281)
        vs = torch.zeros_like(self.value_means)
        vs.index_add_(0, lid, new_vals)
        new_counts = old_counts + torch.bincount(lid, minlength=lists).to(new_vals.dtype)
        self.value_means = torch.where(
            (new_counts > 0).unsqueeze(1),
            (self.value_means * old_counts.unsqueeze(1) + vs) / new_counts.unsqueeze(1).clamp_min(eps),
            torch.zeros_like(self.value_means))
        self._vsum = self._vcnt = None
        return True

    # ---- forward (pq_hsa/attention/sparse_attention.py:245-345) ---------
    def forward_detail(self, queries: torch.Tensor) -> HybridDetail:
        scale = (1.0 / sqrt(queries.shape[-1])) if self.acfg.scale is None else self.acfg.scale
        s, r = self.bounds()
        fullpos = self.full_positions()
        if self.index is None or r - s == 0:
            # dense softmax over sink + local: sparse_attention.py:1388-1407
            logits = queries.matmul(self.keys[fullpos].T) * scale
            w = torch.softmax(logits, dim=-1)
            out = w.matmul(self.values[fullpos])
            z = torch.empty(queries.shape[0], 0)
            return HybridDetail(out, z, z.long(), z, z, logits, z, logits.exp().sum(1), logits.max(1).values)
        raw = self.index.approximate_scores(queries)
        k = resolve_topk(r - s, self.acfg.retrieval_top_fraction, self.acfg.retrieval_topk)
        return hybrid_centroid_attention(
            queries, raw, self.index.list_ids, self.value_means, self.keys, self.values, fullpos, s, k, scale
        )

    def forward_many(self, queries: torch.Tensor) -> torch.Tensor:
        return self.forward_detail(queries).output
