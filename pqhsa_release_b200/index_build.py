"""IVF-PQ index construction after prefill, batched over streams, on the GPU.

Follows ``IVFPQIndex.build`` (pq_hsa/index/ivfpq.py:275-348) step for step:
direction / norm split (:1052-1059), one seeded coarse k-means with
``coarse_max_iter`` Lloyd steps (pq_hsa/index/kmeans.py:134-227), residuals,
one seeded k-means per subspace (pq_hsa/index/pq.py:81-94, seed + 10000 + m),
nearest-code-word encoding (:97-115) and the per-list value means
(pq_hsa/attention/kv_cache.py:688-728).  The random initial rows come from a
CPU generator with the reference's seeds, so the same rows are drawn as in the
reference's CPU build.

This is set-up work outside the per-step path.  The k-means training steps are
torch tensor operations on the device; the pass that assigns and encodes every key
against the finished centroids and code words - the bulk of the arithmetic - is one
CUDA kernel (``encode_bulk`` -> ``pqhsa_encode_bulk``) when the tensors are on a GPU.
"""

from __future__ import annotations

import torch

from .config import IVFPQConfig, validate_index_config
from .device_index import StreamIndexTensors, codes_to_words, words_to_codes  # noqa: F401


def encode_bulk(keys: torch.Tensor, coarse: torch.Tensor, codebooks: torch.Tensor):
    """Assign and encode every key on the GPU with fixed codebooks (``pqhsa_encode_bulk``).

    keys [S, N, 128] (rows contiguous; streams may be strided views of a cache), coarse
    [S, L, 128], codebooks [S, 8, 16, 16], all of the keys' dtype.  Returns
    ``(words int64 [S, N], list ids int64 [S, N], norms [S, N] in the keys' dtype)``: what
    ``IVFPQIndex.add`` (pq_hsa/index/ivfpq.py:598-645) computes for the batch, in the
    incremental encoder's arithmetic."""
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
    if n == 0:
        return words.long(), torch.empty(s, 0, dtype=torch.long, device=keys.device), norms
    lids = torch.empty(s, n, dtype=torch.int16, device=keys.device)  # u16 bit patterns
    stride = keys.stride(0) if s > 1 else max(n * 128, 1)
    with torch.cuda.device(keys.device):
        _lib.call(
            "pqhsa_encode_bulk", keys.data_ptr(), stride, s, n, _DTYPE_CODE[keys.dtype], coarse.data_ptr(),
            coarse.shape[1], codebooks.data_ptr(), words.data_ptr(), norms.data_ptr(), lids.data_ptr(),
            torch.cuda.current_stream(keys.device).cuda_stream,
        )
    return words.long() & 0xFFFFFFFF, lids.long() & 0xFFFF, norms


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
            final_assign: bool = True, assign_fn=None):
    """Batched seeded Lloyd iterations.  x [S, N, d] fp32 -> (centroids [S, k, d]
    holding values representable in ``store_dtype``, assignments [S, N]; None when
    ``final_assign`` is off and the caller assigns with the finished centroids itself).
    ``assign_fn(centroids) -> [S, N]`` replaces the torch assignment of the Lloyd steps."""
    s, n, d = x.shape
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    if n >= k:
        rows = torch.randperm(n, generator=gen)[:k]
    else:
        rows = torch.cat([torch.arange(n), torch.randint(0, n, (k - n,), generator=gen)])
    cent = x[:, rows.to(x.device)].to(store_dtype).float()
    for _ in range(iters):
        a = _assign(x, cent) if assign_fn is None else assign_fn(cent)
        sums = torch.zeros(s, k, d, dtype=torch.float32, device=x.device)
        sums.scatter_add_(1, a.unsqueeze(-1).expand(-1, -1, d), x)
        cnt = torch.zeros(s, k, dtype=torch.float32, device=x.device)
        cnt.scatter_add_(1, a, torch.ones_like(a, dtype=torch.float32))
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
    if on_gpu:
        # every assignment against the coarse centroids - the Lloyd steps' and the final one - by the
        # kernel (the code words are not known yet: their half of the result is ignored)
        no_books = torch.zeros(s, 8, 16, 16, dtype=dtype, device=keys.device)
        coarse, _ = _kmeans(unit, lists, cfg.coarse_max_iter, cfg.seed, dtype, cfg.eps, final_assign=False,
                            assign_fn=lambda cent: encode_bulk(keys, cent, no_books)[1])
        _, lid, norms = encode_bulk(keys, coarse, no_books)
    else:
        coarse, lid = _kmeans(unit, lists, cfg.coarse_max_iter, cfg.seed, dtype, cfg.eps)
    resid = unit.sub_(torch.gather(coarse, 1, lid.unsqueeze(-1).expand(-1, -1, d)))  # the directions are not needed again
    del unit
    m, sub, ncodes = cfg.num_subspaces, d // cfg.num_subspaces, 1 << cfg.num_bits
    books = torch.empty(s, m, ncodes, sub, dtype=torch.float32, device=keys.device)
    words = torch.zeros(s, n, dtype=torch.int64, device=keys.device)
    for j in range(m):
        chunk = resid[:, :, j * sub : (j + 1) * sub].contiguous()
        books[:, j], _ = _kmeans(chunk, ncodes, cfg.pq_max_iter, cfg.seed + 10_000 + j, dtype, cfg.eps,
                                 final_assign=False)
        if not on_gpu:
            # encode with true squared distances (torch.cdist's small-size path)
            d2 = ((chunk.unsqueeze(2) - books[:, j].unsqueeze(1)) ** 2).sum(-1)
            words |= d2.argmin(dim=-1) << (4 * j)
    if on_gpu:
        words, _, _ = encode_bulk(keys, coarse, books)  # same lists as above: the kernel is deterministic
    del resid
    vf = values.float()
    vsum = torch.zeros(s, lists, d, dtype=torch.float32, device=keys.device)
    vsum.scatter_add_(1, lid.unsqueeze(-1).expand(-1, -1, d), vf)
    vcnt = torch.zeros(s, lists, dtype=torch.float32, device=keys.device)
    vcnt.scatter_add_(1, lid, torch.ones_like(lid, dtype=torch.float32))
    vmean = torch.where(vcnt.unsqueeze(-1) > 0, vsum / vcnt.clamp_min(1).unsqueeze(-1), torch.zeros_like(vsum))
    out = []
    for i in range(s):
        out.append(
            StreamIndexTensors(
                packed_codes=words_to_codes(words[i]),
                list_ids=lid[i],
                key_norms=norms[i],
                coarse_centroids=coarse[i].to(dtype),
                codebooks=books[i].to(dtype),
                value_means=vmean[i].to(dtype),
                value_sums=vsum[i],
                value_counts=vcnt[i].to(torch.int32),
            )
        )
    return out


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
    if keys.is_cuda and d == 128 and m == 8 and cfg.num_bits == 4:
        words, lid, norms = encode_bulk(keys, coarse, books)
    else:
        lid = _assign(unit, coarse)
        resid = unit - torch.gather(coarse, 1, lid.unsqueeze(-1).expand(-1, -1, d))
        words = torch.zeros(s, n, dtype=torch.int64, device=keys.device)
        for j in range(m):
            chunk = resid[:, :, j * sub : (j + 1) * sub]
            d2 = ((chunk.unsqueeze(2) - books[:, j].unsqueeze(1)) ** 2).sum(-1)
            words |= d2.argmin(dim=-1) << (4 * j)
    vf = values.float()
    vsum = torch.zeros(s, lists, d, dtype=torch.float32, device=keys.device)
    vsum.scatter_add_(1, lid.unsqueeze(-1).expand(-1, -1, d), vf)
    vcnt = torch.zeros(s, lists, dtype=torch.float32, device=keys.device)
    vcnt.scatter_add_(1, lid, torch.ones_like(lid, dtype=torch.float32))
    vmean = torch.where(vcnt.unsqueeze(-1) > 0, vsum / vcnt.clamp_min(1).unsqueeze(-1), torch.zeros_like(vsum))
    return [
        StreamIndexTensors(
            packed_codes=words_to_codes(words[i]), list_ids=lid[i], key_norms=norms[i],
            coarse_centroids=coarse[i].to(dtype), codebooks=books[i].to(dtype), value_means=vmean[i].to(dtype),
            value_sums=vsum[i], value_counts=vcnt[i].to(torch.int32),
        )
        for i in range(s)
    ]
