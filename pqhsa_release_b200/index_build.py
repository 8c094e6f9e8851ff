"""IVF-PQ index construction after prefill, batched over streams, on the GPU.

Follows ``IVFPQIndex.build`` (pq_hsa/index/ivfpq.py:275-348) step for step:
direction / norm split (:1052-1059), one seeded coarse k-means with
``coarse_max_iter`` Lloyd steps (pq_hsa/index/kmeans.py:134-227), residuals,
one seeded k-means per subspace (pq_hsa/index/pq.py:81-94, seed + 10000 + m),
nearest-code-word encoding (:97-115) and the per-list value means
(pq_hsa/attention/kv_cache.py:688-728).  The random initial rows come from a
CPU generator with the reference's seeds, so the same rows are drawn as in the
reference's CPU build.

This is set-up work outside the per-step path.  With the tensors on a GPU every pass
over the keys is a CUDA kernel: the assignment against the coarse centroids and the
final encoding (``encode_bulk`` -> ``pqhsa_encode_bulk``), the assignment of the
code-word training (``pqhsa_subspace_assign``) and the sums of the Lloyd steps and of
the values per list (``cluster_sums`` -> ``pqhsa_cluster_order`` + ``pqhsa_cluster_sums``:
rows added in the order of the keys, so a build gives the same bits every time it runs).
What stays in torch works on [streams, clusters, width] tensors: dividing by the counts,
re-seeding empty clusters, rounding to the storage type.
"""

from __future__ import annotations

import torch

from .config import IVFPQConfig, validate_index_config
from .device_index import StreamIndexTensors, codes_to_words, words_to_codes  # noqa: F401


def encode_bulk(keys: torch.Tensor, coarse: torch.Tensor, codebooks: torch.Tensor, raw: bool = False,
                lists: torch.Tensor | None = None):
    """Assign and encode every key on the GPU with fixed codebooks (``pqhsa_encode_bulk``).

    keys [S, N, 128] (rows contiguous; streams may be strided views of a cache), coarse
    [S, L, 128], codebooks [S, 8, 16, 16], all of the keys' dtype.  Returns
    ``(words int64 [S, N], list ids int64 [S, N], norms [S, N] in the keys' dtype)``: what
    ``IVFPQIndex.add`` (pq_hsa/index/ivfpq.py:598-645) computes for the batch, in the
    incremental encoder's arithmetic.  ``raw``: words and list ids as the kernel wrote them
    (int32 / int16 holding unsigned bit patterns).  ``lists`` (int16 [S, N], raw ids of an
    earlier call with the same ``coarse``): the nearest-list search is skipped
    (``pqhsa_encode_bulk_assigned``)."""
    from . import _lib
    from .device_index import _DTYPE_CODE

    if not keys.is_cuda:
        raise RuntimeError("encode_bulk needs CUDA tensors: there is no CPU path")
    if keys.dim() != 3 or keys.shape[-1] != 128:
        raise ValueError("keys must be [streams, N, 128]")
    if keys.dtype not in _DTYPE_CODE:
        raise ValueError(f"unsupported dtype {keys.dtype}")
    s, n, _ = keys.shape
    if n and (keys.stride(2) != 1 or keys.stride(1) != 128 or (s > 1 and keys.stride(0) < n * 128)):
        keys = keys.contiguous()
    coarse = coarse.to(keys.dtype).contiguous()
    codebooks = codebooks.to(keys.dtype).contiguous()
    if coarse.dim() != 3 or coarse.shape[0] != s or coarse.shape[2] != 128:
        raise ValueError("coarse must be [streams, lists, 128]")
    if tuple(codebooks.shape) != (s, 8, 16, 16):
        raise ValueError("codebooks must be [streams, 8, 16, 16]")
    words = torch.empty(s, n, dtype=torch.int32, device=keys.device)
    norms = torch.empty(s, n, dtype=keys.dtype, device=keys.device)
    if lists is not None:
        if lists.dtype != torch.int16 or tuple(lists.shape) != (s, n) or lists.device != keys.device:
            raise ValueError("lists must be int16 [streams, N] on the keys' device")
        lids = lists.contiguous()
    else:
        lids = torch.empty(s, n, dtype=torch.int16, device=keys.device)  # u16 bit patterns
    if n == 0:
        return (words, lids, norms) if raw else (words.long(), lids.long(), norms)
    stride = keys.stride(0) if s > 1 else max(n * 128, 1)
    with torch.cuda.device(keys.device):
        st = torch.cuda.current_stream(keys.device).cuda_stream
        if lists is None:
            _lib.call("pqhsa_encode_bulk", keys.data_ptr(), stride, s, n, _DTYPE_CODE[keys.dtype], coarse.data_ptr(),
                      coarse.shape[1], codebooks.data_ptr(), words.data_ptr(), norms.data_ptr(), lids.data_ptr(), st)
        else:
            _lib.call("pqhsa_encode_bulk_assigned", keys.data_ptr(), stride, s, n, _DTYPE_CODE[keys.dtype],
                      coarse.data_ptr(), coarse.shape[1], codebooks.data_ptr(), lids.data_ptr(), words.data_ptr(),
                      norms.data_ptr(), st)
    if raw:
        return words, lids, norms
    return words.long() & 0xFFFFFFFF, _u16(lids), norms


def _u16(t: torch.Tensor) -> torch.Tensor:
    """int16 tensor holding u16 bit patterns -> int64 values."""
    return t.long() & 0xFFFF


def cluster_sums(rows: torch.Tensor, ids: torch.Tensor, k: int, width: int = 128, groups: int = 1):
    """Per-cluster sums of rows, added in the order of the keys (``index_add_`` on one CPU thread, bit for bit).

    rows [S, N, R] (fp32 / bf16 / fp16; rows contiguous, streams may be strided), ids int16 [groups * S, N] with
    u16 cluster ids below k: key set g * S + s sums columns [g * width, (g + 1) * width) of stream s.  Returns
    ``(sums fp32 [groups * S, k, width], counts int32 [groups * S, k])``."""
    from . import _lib
    from .device_index import _DTYPE_CODE

    if not rows.is_cuda:
        raise RuntimeError("cluster_sums needs CUDA tensors: there is no CPU path")
    s, n, r = rows.shape
    if n and (rows.stride(2) != 1 or rows.stride(1) != r or (s > 1 and rows.stride(0) < n * r)):
        rows = rows.contiguous()
    ids = ids.contiguous()
    if ids.dtype != torch.int16 or tuple(ids.shape) != (groups * s, n):
        raise ValueError("ids must be int16 [groups * streams, N]")
    sets = groups * s
    if n == 0:
        return (torch.zeros(sets, k, width, dtype=torch.float32, device=rows.device),
                torch.zeros(sets, k, dtype=torch.int32, device=rows.device))
    order = torch.empty(sets, n, dtype=torch.int32, device=rows.device)
    start = torch.empty(sets, k + 1, dtype=torch.int32, device=rows.device)
    sums = torch.empty(sets, k, width, dtype=torch.float32, device=rows.device)
    stride = rows.stride(0) if s > 1 else max(n * r, 1)
    with torch.cuda.device(rows.device):
        st = torch.cuda.current_stream(rows.device).cuda_stream
        _lib.call("pqhsa_cluster_order", ids.data_ptr(), sets, n, k, order.data_ptr(), start.data_ptr(), st)
        _lib.call("pqhsa_cluster_sums", rows.data_ptr(), _DTYPE_CODE[rows.dtype], stride, r, width, s, groups, n, k,
                  order.data_ptr(), start.data_ptr(), sums.data_ptr(), st)
    return sums, start[:, 1:] - start[:, :-1]


def subspace_assign(resid: torch.Tensor, books: torch.Tensor) -> torch.Tensor:
    """Nearest code word of every residual in every subspace (``pqhsa_subspace_assign``): resid fp32 [S, N, 128],
    books fp32 [S, 8, 16, 16] -> int16 [8, S, N]."""
    from . import _lib

    if not resid.is_cuda or resid.dtype != torch.float32 or not resid.is_contiguous():
        raise ValueError("resid must be a contiguous fp32 CUDA tensor")
    s, n, _ = resid.shape
    books = books.float().contiguous()
    ids = torch.empty(8, s, n, dtype=torch.int16, device=resid.device)
    with torch.cuda.device(resid.device):
        _lib.call("pqhsa_subspace_assign", resid.data_ptr(), max(n * 128, 4), books.data_ptr(), s, n, ids.data_ptr(),
                  torch.cuda.current_stream(resid.device).cuda_stream)
    return ids


def _assign(x: torch.Tensor, cent: torch.Tensor, chunk: int = 16384) -> torch.Tensor:
    """x [S, N, d], cent [S, K, d] -> argmin_k (|c|^2 - 2 x.c) [S, N]
    (pq_hsa/index/kmeans.py:108-131)."""
    csq = (cent * cent).sum(-1)  # [S, K]
    out = torch.empty(x.shape[0], x.shape[1], dtype=torch.long, device=x.device)
    for lo in range(0, x.shape[1], chunk):
        hi = min(x.shape[1], lo + chunk)
        sc = csq.unsqueeze(1) - 2.0 * torch.bmm(x[:, lo:hi], cent.transpose(1, 2))
        out[:, lo:hi] = sc.argmin(dim=-1)
    return out


def _kmeans(x: torch.Tensor, k: int, iters: int, seed: int, store_dtype: torch.dtype, eps: float,
            final_assign: bool = True, step_fn=None, after_launch=None):
    """Batched seeded Lloyd iterations.  x [S, N, d] fp32 -> (centroids [S, k, d]
    holding values representable in ``store_dtype``, assignments [S, N]; None when
    ``final_assign`` is off and the caller assigns with the finished centroids itself).
    ``step_fn(centroids) -> (sums [S, k, d], counts [S, k])`` replaces the torch assignment
    and scatter of a Lloyd step (the kernels, on a GPU); ``after_launch()`` runs once, behind the
    first step's launches and before the host waits for them (host work that can overlap)."""
    s, n, d = x.shape
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    if n >= k:
        rows = torch.randperm(n, generator=gen)[:k]
    else:
        rows = torch.cat([torch.arange(n), torch.randint(0, n, (k - n,), generator=gen)])
    cent = x[:, rows.to(x.device)].to(store_dtype).float()
    for _ in range(iters):
        if step_fn is None:
            a = _assign(x, cent)
            sums = torch.zeros(s, k, d, dtype=torch.float32, device=x.device)
            sums.scatter_add_(1, a.unsqueeze(-1).expand(-1, -1, d), x)
            cnt = torch.zeros(s, k, dtype=torch.float32, device=x.device)
            cnt.scatter_add_(1, a, torch.ones_like(a, dtype=torch.float32))
        else:
            sums, cnt = step_fn(cent)
            cnt = cnt.float()
            if after_launch is not None:
                after_launch()
                after_launch = None
        live = cnt > 0
        new = sums / cnt.clamp_min(eps).unsqueeze(-1)
        dead = (~live).sum(dim=1).tolist()
        if any(dead):
            # the reference draws one batch of replacement rows per stream from the same generator
            for i, nd in enumerate(dead):
                if nd:
                    repl = torch.randint(0, n, (nd,), generator=gen).to(x.device)
                    new[i, ~live[i]] = x[i, repl]
        cent = new.to(store_dtype).float()
    return cent, (_assign(x, cent) if final_assign else None)


def _draw_code_word_rows(n: int, seed: int):
    """The initial rows of the 8 code-word trainings (subspace m: a CPU generator seeded seed + 10000 + m, as
    pq_hsa/index/pq.py:81-94 seeds them) and the generators, which later draw the replacements of empty clusters.
    About a millisecond of host time per subspace at 128K keys."""
    gens, rows = [], []
    for j in range(8):
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed + 10_000 + j)
        if n >= 16:
            rows.append(torch.randperm(n, generator=gen)[:16])
        else:
            rows.append(torch.cat([torch.arange(n), torch.randint(0, n, (16 - n,), generator=gen)]))
        gens.append(gen)
    return gens, rows


def _train_code_words(resid: torch.Tensor, iters: int, seed: int, store_dtype: torch.dtype, eps: float, drawn=None):
    """The 8 seeded code-word trainings of pq_hsa/index/pq.py:81-94 as one batch on the GPU.  resid fp32
    [S, N, 128] -> code words fp32 [S, 8, 16, 16] holding values representable in ``store_dtype``.  Every
    subspace keeps its own generator, so the rows it draws are those of its own sequential run.  ``drawn``: the
    result of :func:`_draw_code_word_rows` when the caller made it earlier."""
    s, n, d = resid.shape
    m, k, sub = 8, 16, 16
    gens, rows = drawn if drawn is not None else _draw_code_word_rows(n, seed)
    first = [resid[:, rows[j].to(resid.device), j * sub : (j + 1) * sub] for j in range(m)]
    cent = torch.stack(first, dim=1).to(store_dtype).float()  # [S, 8, 16, 16]
    for _ in range(iters):
        ids = subspace_assign(resid, cent)
        sums, cnt = cluster_sums(resid, ids.view(m * s, n), k, width=sub, groups=m)
        sums = sums.view(m, s, k, sub).transpose(0, 1)
        cnt = cnt.view(m, s, k).transpose(0, 1).float()
        live = cnt > 0
        new = sums / cnt.clamp_min(eps).unsqueeze(-1)
        dead = (~live).sum(dim=2).tolist()  # [S][8]
        for j in range(m):
            for i in range(s):
                if dead[i][j]:
                    repl = torch.randint(0, n, (dead[i][j],), generator=gens[j]).to(resid.device)
                    new[i, j, ~live[i, j]] = resid[i, repl, j * sub : (j + 1) * sub]
        cent = new.to(store_dtype).float()
    return cent


def _per_stream(words, lid, norms, coarse, books, vmean, vsum, vcnt, dtype) -> list[StreamIndexTensors]:
    """The batch's results as one record per stream; the conversions run once on the batch, the records hold views."""
    codes = words_to_codes(words)
    coarse, books, vmean, vcnt = coarse.to(dtype), books.to(dtype), vmean.to(dtype), vcnt.to(torch.int32)
    return [
        StreamIndexTensors(
            packed_codes=codes[i], list_ids=lid[i], key_norms=norms[i], coarse_centroids=coarse[i], codebooks=books[i],
            value_means=vmean[i], value_sums=vsum[i], value_counts=vcnt[i],
        )
        for i in range(words.shape[0])
    ]


def _value_summaries(values: torch.Tensor, lid: torch.Tensor, lid_raw, lists: int):
    """Per-list value sums, counts and means (pq_hsa/attention/kv_cache.py:688-728): the kernels on a GPU (the
    values are read in their own dtype and widened on the way), torch scatters elsewhere."""
    s, n, d = values.shape
    if lid_raw is not None:
        vsum, cnt = cluster_sums(values, lid_raw, lists)
        vcnt = cnt.float()
    else:
        vsum = torch.zeros(s, lists, d, dtype=torch.float32, device=values.device)
        vsum.scatter_add_(1, lid.unsqueeze(-1).expand(-1, -1, d), values.float())
        vcnt = torch.zeros(s, lists, dtype=torch.float32, device=values.device)
        vcnt.scatter_add_(1, lid, torch.ones_like(lid, dtype=torch.float32))
    vmean = torch.where(vcnt.unsqueeze(-1) > 0, vsum / vcnt.clamp_min(1).unsqueeze(-1), torch.zeros_like(vsum))
    return vsum, vcnt, vmean


@torch.no_grad()
def build_index_batch(keys: torch.Tensor, values: torch.Tensor, cfg: IVFPQConfig) -> list[StreamIndexTensors]:
    """keys/values: [S, N, 128] rows of the retrieval region of S streams that share
    N.  Returns one :class:`StreamIndexTensors` per stream (tensors stay on the
    device of ``keys``)."""
    validate_index_config(cfg)
    if keys.dim() != 3 or keys.shape != values.shape:
        raise ValueError("keys and values must both be [streams, N, dim]")
    s, n, d = keys.shape
    if n == 0:
        raise ValueError("cannot build IVF-PQ index with zero keys")
    dtype = keys.dtype
    # fp32 working copies are made one at a time and reused in place (directions, then residuals; the values only
    # at the end): three of them alive at once at the most, against [S, N, 128] inputs
    unit = keys.to(torch.float32, copy=True)  # a copy also for fp32 keys: it is overwritten below
    norms = torch.linalg.vector_norm(unit, dim=-1).to(dtype).clamp_min(cfg.eps)
    unit.div_(norms.float().unsqueeze(-1))
    lists = min(cfg.num_lists, n)
    on_gpu = keys.is_cuda and d == 128 and cfg.num_subspaces == 8 and cfg.num_bits == 4
    m, sub, ncodes = cfg.num_subspaces, d // cfg.num_subspaces, 1 << cfg.num_bits
    lid_raw = None
    if on_gpu:
        # every assignment against the coarse centroids - the Lloyd steps' and the final one - by the bulk
        # encode kernel (the code words are not known yet: their half of the result is ignored), the sums of
        # a step by the ordered-sum kernels
        no_books = torch.zeros(s, 8, 16, 16, dtype=dtype, device=keys.device)
        drawn = []  # the code-word trainings' random rows are drawn on the host while the first step runs on the device
        coarse, _ = _kmeans(unit, lists, cfg.coarse_max_iter, cfg.seed, dtype, cfg.eps, final_assign=False,
                            step_fn=lambda cent: cluster_sums(unit, encode_bulk(keys, cent, no_books, raw=True)[1], lists),
                            after_launch=lambda: drawn.append(_draw_code_word_rows(n, cfg.seed)))
        _, lid_raw, norms = encode_bulk(keys, coarse, no_books, raw=True)
        lid = _u16(lid_raw)
    else:
        coarse, lid = _kmeans(unit, lists, cfg.coarse_max_iter, cfg.seed, dtype, cfg.eps)
    resid = unit.sub_(torch.gather(coarse, 1, lid.unsqueeze(-1).expand(-1, -1, d)))  # the directions are not needed again
    del unit
    if on_gpu:
        books = _train_code_words(resid, cfg.pq_max_iter, cfg.seed, dtype, cfg.eps, drawn[0] if drawn else None)
        words, _, _ = encode_bulk(keys, coarse, books, lists=lid_raw)  # the lists found above: no second search
    else:
        books = torch.empty(s, m, ncodes, sub, dtype=torch.float32, device=keys.device)
        words = torch.zeros(s, n, dtype=torch.int64, device=keys.device)
        for j in range(m):
            chunk = resid[:, :, j * sub : (j + 1) * sub].contiguous()
            books[:, j], _ = _kmeans(chunk, ncodes, cfg.pq_max_iter, cfg.seed + 10_000 + j, dtype, cfg.eps,
                                     final_assign=False)
            # encode with true squared distances (torch.cdist's small-size path)
            d2 = ((chunk.unsqueeze(2) - books[:, j].unsqueeze(1)) ** 2).sum(-1)
            words |= d2.argmin(dim=-1) << (4 * j)
    del resid
    vsum, vcnt, vmean = _value_summaries(values, lid, lid_raw, lists)
    return _per_stream(words, lid, norms, coarse, books, vmean, vsum, vcnt, dtype)


@torch.no_grad()
def online_refresh_batch(keys: torch.Tensor, values: torch.Tensor, current: list[dict], new_count: int,
                         cfg: IVFPQConfig) -> list[StreamIndexTensors]:
    """Codebook-moving refresh of S streams that share N (pq_hsa/index/ivfpq.py:647-707):
    the last ``new_count`` keys pull the coarse centroids and the code words towards
    their mini-batch means (EMA with ``online_codebook_lr``), then every key is
    re-assigned and re-encoded and the value means are rebuilt.  ``current[i]`` holds
    stream i's ``coarse`` [L, 128] and ``codebooks`` [8, 16, 16]."""
    s, n, d = keys.shape
    dtype = keys.dtype
    lr = cfg.online_codebook_lr
    kf = keys.float()
    norms = torch.linalg.vector_norm(kf, dim=-1).to(dtype).clamp_min(cfg.eps)
    unit = kf / norms.float().unsqueeze(-1)
    coarse = torch.stack([c["coarse"].float() for c in current])        # [S, L, D]
    books = torch.stack([c["codebooks"].float() for c in current])      # [S, M, 16, sub]
    lists = coarse.shape[1]
    upd = unit[:, n - new_count:]
    ones = torch.ones(s, new_count, dtype=torch.float32, device=keys.device)

    def ema(cent, x, assign):
        k = cent.shape[1]
        sums = torch.zeros_like(cent)
        sums.scatter_add_(1, assign.unsqueeze(-1).expand(-1, -1, x.shape[-1]), x)
        cnt = torch.zeros(s, k, dtype=torch.float32, device=x.device)
        cnt.scatter_add_(1, assign, ones)
        live = (cnt > 0).unsqueeze(-1)
        means = sums / cnt.clamp_min(cfg.eps).unsqueeze(-1)
        return torch.where(live, (1.0 - lr) * cent + lr * means, cent)

    coarse = ema(coarse, upd, _assign(upd, coarse)).to(dtype).float()
    ures = upd - torch.gather(coarse, 1, _assign(upd, coarse).unsqueeze(-1).expand(-1, -1, d))
    m, sub = cfg.num_subspaces, d // cfg.num_subspaces
    for j in range(m):
        chunk = ures[:, :, j * sub : (j + 1) * sub].contiguous()
        books[:, j] = ema(books[:, j], chunk, _assign(chunk, books[:, j]))
    books = books.to(dtype).float()
    lid_raw = None
    if keys.is_cuda and d == 128 and m == 8 and cfg.num_bits == 4:
        words, lid_raw, norms = encode_bulk(keys, coarse, books, raw=True)
        words, lid = words.long() & 0xFFFFFFFF, _u16(lid_raw)
    else:
        lid = _assign(unit, coarse)
        resid = unit - torch.gather(coarse, 1, lid.unsqueeze(-1).expand(-1, -1, d))
        words = torch.zeros(s, n, dtype=torch.int64, device=keys.device)
        for j in range(m):
            chunk = resid[:, :, j * sub : (j + 1) * sub]
            d2 = ((chunk.unsqueeze(2) - books[:, j].unsqueeze(1)) ** 2).sum(-1)
            words |= d2.argmin(dim=-1) << (4 * j)
    vsum, vcnt, vmean = _value_summaries(values, lid, lid_raw, lists)
    return _per_stream(words, lid, norms, coarse, books, vmean, vsum, vcnt, dtype)
