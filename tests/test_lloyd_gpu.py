"""The Lloyd-step kernels of the device-side index build (pqhsa_cluster_order, pqhsa_cluster_sums,
pqhsa_subspace_assign): the stable order by cluster, sums that equal a CPU ``index_add_`` bit for bit, the
code-word assignment against a double-precision argmin, and a build that gives the same bits twice."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ids(sets: int, n: int, k: int, seed: int, empty=()):
    gen = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, k, (sets, n), generator=gen)
    for c in empty:  # clusters without a key
        ids[ids == c] = (c + 1) % k
    return ids


@pytest.mark.parametrize("sets,n,k", [(3, 5000, 48), (2, 31, 512), (1, 1024, 1), (4, 33333, 512), (5, 7, 16)])
def test_cluster_order_is_the_stable_sort(sets, n, k):
    from pqhsa_release_b200 import _lib

    ids = _ids(sets, n, k, seed=n + k, empty=(3, k - 1) if k > 4 else ())
    dev = ids.to(torch.int16).cuda()
    order = torch.full((sets, n), -1, dtype=torch.int32, device="cuda")
    start = torch.full((sets, k + 1), -1, dtype=torch.int32, device="cuda")
    _lib.call("pqhsa_cluster_order", dev.data_ptr(), sets, n, k, order.data_ptr(), start.data_ptr(),
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    want = torch.sort(ids, dim=1, stable=True).indices
    assert torch.equal(order.cpu().long(), want)
    counts = torch.stack([torch.bincount(r, minlength=k) for r in ids])
    want_start = torch.cat([torch.zeros(sets, 1, dtype=torch.long), counts.cumsum(1)], dim=1)
    assert torch.equal(start.cpu().long(), want_start)


@pytest.mark.parametrize("dtype,groups,width,k,n", [(torch.float32, 1, 128, 48, 3001), (torch.bfloat16, 1, 128, 512, 2500),
                                                   (torch.float32, 8, 16, 16, 4097), (torch.float16, 2, 64, 5, 100)])
def test_cluster_sums_equal_index_add_in_key_order(dtype, groups, width, k, n):
    """Same assignments -> the sums of ``index_add_`` on the CPU (one addition per key, in the order of the keys),
    bit for bit; streams read in place from a strided view."""
    from pqhsa_release_b200.index_build import cluster_sums

    s = 3
    gen = torch.Generator().manual_seed(11)
    cache = (torch.randn(s, n + 40, 128, generator=gen) * 3).to(dtype)
    rows = cache[:, 17 : 17 + n]  # stream stride larger than n * 128
    ids = _ids(groups * s, n, k, seed=5, empty=(1,) if k > 4 else ())
    sums, cnt = cluster_sums(cache.cuda()[:, 17 : 17 + n], ids.to(torch.int16).cuda(), k, width=width, groups=groups)
    torch.cuda.synchronize()
    assert sums.shape == (groups * s, k, width) and cnt.shape == (groups * s, k)
    for g in range(groups):
        for i in range(s):
            t = g * s + i
            want = torch.zeros(k, width).index_add_(0, ids[t], rows[i, :, g * width : (g + 1) * width].float())
            assert torch.equal(sums[t].cpu(), want), (g, i)
            assert torch.equal(cnt[t].cpu().long(), torch.bincount(ids[t], minlength=k))
    # nothing to sum
    z, c = cluster_sums(cache.cuda()[:, :0], torch.zeros(groups * s, 0, dtype=torch.int16, device="cuda"), k,
                        width=width, groups=groups)
    assert float(z.abs().sum()) == 0.0 and int(c.sum()) == 0


def test_subspace_assign_matches_the_argmin():
    """The code word the kernel picks is the double-precision argmin of |c|^2 - 2 x.c, or ties with it to fp32
    rounding; the tile edges (N not a multiple of 256) and per-stream code words are covered."""
    from pqhsa_release_b200.index_build import subspace_assign

    s, n = 2, 1000
    gen = torch.Generator().manual_seed(2)
    resid = torch.randn(s, n, 128, generator=gen) * 0.3
    books = torch.randn(s, 8, 16, 16, generator=gen) * 0.3
    books[1, 3, 5] = books[1, 3, 2]  # two equal code words: the first one wins
    got = subspace_assign(resid.cuda(), books.cuda()).cpu().long()  # [8, S, N]
    assert got.shape == (8, s, n) and int(got.min()) >= 0 and int(got.max()) < 16
    x = resid.double().view(s, n, 8, 16).permute(2, 0, 1, 3)  # [8, S, N, 16]
    c = books.double().permute(1, 0, 2, 3)  # [8, S, 16, 16]
    score = (c * c).sum(-1).unsqueeze(2) - 2.0 * torch.einsum("msnd,mscd->msnc", x, c)
    best = score.argmin(-1)
    picked = score.gather(-1, got.unsqueeze(-1)).squeeze(-1)
    assert bool(((picked - score.min(-1).values) <= 1e-5).all())
    assert float((got == best).float().mean()) >= 0.999
    assert not bool((got[3, 1] == 5).any())


def test_device_build_gives_the_same_bits_twice():
    """No atomics on floats anywhere in the device-side build: two builds of the same keys are equal bit for
    bit (centroids, code words, lists, codes, value sums)."""
    from pqhsa_release_b200.config import paper_index_config
    from pqhsa_release_b200.index_build import build_index_batch

    gen = torch.Generator().manual_seed(9)
    keys = torch.randn(3, 6000, 128, generator=gen).to(torch.bfloat16).cuda()
    vals = torch.randn(3, 6000, 128, generator=gen).to(torch.bfloat16).cuda()
    cfg = paper_index_config(num_lists=128)
    a = build_index_batch(keys, vals, cfg)
    b = build_index_batch(keys, vals, cfg)
    for x, y in zip(a, b):
        for name in ("coarse_centroids", "codebooks", "list_ids", "packed_codes", "key_norms", "value_sums",
                     "value_means", "value_counts"):
            assert torch.equal(getattr(x, name), getattr(y, name)), name
    assert int(a[0].value_counts.sum()) == 6000


def test_lloyd_argument_errors():
    from pqhsa_release_b200 import _lib

    ids = torch.zeros(1, 8, dtype=torch.int16, device="cuda")
    order = torch.zeros(1, 8, dtype=torch.int32, device="cuda")
    start = torch.zeros(1, 600, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    with pytest.raises(_lib.PqhsaError):  # more clusters than the sort's shared-memory table holds
        _lib.call("pqhsa_cluster_order", ids.data_ptr(), 1, 8, _lib.MAX_LISTS + 1, order.data_ptr(), start.data_ptr(), st)
    rows = torch.zeros(1, 8, 128, device="cuda")
    sums = torch.zeros(1, 4, 48, device="cuda")
    with pytest.raises(_lib.PqhsaError):  # a width that does not divide 128
        _lib.call("pqhsa_cluster_sums", rows.data_ptr(), 0, 1024, 128, 48, 1, 1, 8, 4, order.data_ptr(), start.data_ptr(),
                  sums.data_ptr(), st)
