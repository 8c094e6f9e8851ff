"""Bulk encode (pqhsa_encode_bulk) on the GPU: against the oracle's IVFPQIndex.add, against the
incremental encoder of the decode step, and inside the device-side index build and refresh."""

import pytest
import torch

from helpers import make_case, pool_from_case, round_to

pytestmark = pytest.mark.gpu


def _oracle_index(keys: torch.Tensor, lists: int):
    from oracle.pqhsa_oracle import OracleIndex, OracleIndexConfig

    return OracleIndex(OracleIndexConfig(num_lists=lists)).build(keys)


def _true_distances(unit: torch.Tensor, cent: torch.Tensor) -> torch.Tensor:
    return ((unit.double().unsqueeze(1) - cent.double().unsqueeze(0)) ** 2).sum(-1)


@pytest.mark.parametrize("dtype,lists,n_new", [(torch.float32, 100, 1999), (torch.bfloat16, 512, 2500),
                                              (torch.float16, 37, 63)])
def test_bulk_encode_matches_the_oracle_add(dtype, lists, n_new):
    """Three streams with their own codebooks, key counts that are not multiples of the 64-key tile,
    list counts that are not multiples of the 64-list tile: list ids and codes equal the oracle's
    ``add`` except where the two best candidates are a numerical tie in double precision; norms to
    storage precision."""
    from oracle.pqhsa_oracle import unpack_nibbles
    from pqhsa_release_b200.index_build import encode_bulk

    gen = torch.Generator().manual_seed(11)
    S, n_old = 3, 1400
    old = round_to(torch.randn(S, n_old, 128, generator=gen) * torch.rand(S, n_old, 1, generator=gen).add(0.5), dtype)
    new = round_to(old[:, torch.randint(0, n_old, (n_new,), generator=gen)]
                   + 0.4 * torch.randn(S, n_new, 128, generator=gen), dtype)
    idx = [_oracle_index(old[s], lists) for s in range(S)]
    coarse = torch.stack([round_to(i.coarse, dtype) for i in idx])
    books = torch.stack([round_to(i.codebooks, dtype) for i in idx])
    for s, i in enumerate(idx):  # the oracle encodes against exactly the stored code words
        i.coarse, i.codebooks = coarse[s].clone(), books[s].clone()
    words, lids, norms = encode_bulk(new.to(dtype).cuda(), coarse.to(dtype).cuda(), books.to(dtype).cuda())
    torch.cuda.synchronize()
    words, lids, norms = words.cpu(), lids.cpu(), norms.float().cpu()
    list_ties = code_ties = 0
    for s, i in enumerate(idx):
        before = i.num_vectors
        want_lid = i.add(new[s])
        want_codes = unpack_nibbles(i.packed[before:], 8).long()
        want_norm = i.norms[before:].float()
        got_codes = torch.stack([(words[s] >> (4 * m)) & 15 for m in range(8)], dim=1)
        tol = 1e-6 if dtype == torch.float32 else 4e-3 if dtype == torch.bfloat16 else 1e-3
        assert float(((norms[s] - want_norm).abs() / want_norm).max()) <= tol
        unit = new[s] / torch.linalg.vector_norm(new[s], dim=-1, keepdim=True)
        bad = (lids[s] != want_lid).nonzero().flatten()
        if len(bad):
            d = _true_distances(unit[bad], i.coarse)
            gap = (d.gather(1, lids[s][bad, None]) - d.gather(1, want_lid[bad, None])).abs().flatten()
            assert float(gap.max()) <= 5e-6, f"stream {s}: list assignment differs beyond a tie ({float(gap.max())})"
            list_ties += len(bad)
        same_list = lids[s] == want_lid
        resid = unit - i.coarse[lids[s]]
        for m in range(8):
            diff = ((got_codes[:, m] != want_codes[:, m]) & same_list).nonzero().flatten()
            if len(diff):
                d = _true_distances(resid[diff, 16 * m : 16 * m + 16], i.codebooks[m])
                gap = (d.gather(1, got_codes[diff, m, None]) - d.gather(1, want_codes[diff, m, None])).abs().flatten()
                assert float(gap.max()) <= 5e-6, f"stream {s} subspace {m}: code differs beyond a tie"
                code_ties += len(diff)
    assert list_ties <= max(2, S * n_new // 500) and code_ties <= max(4, S * n_new // 100), (list_ties, code_ties)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bulk_encode_equals_the_incremental_encoder(dtype):
    """The same keys through append_kv + append_encode (one at a time, inside the pool) and through
    one bulk call: identical list ids, codes and norms, bit for bit."""
    from pqhsa_release_b200.index_build import encode_bulk

    case = make_case(B=1, Hkv=2, G=2, S=900, L=32, dtype=dtype, seed=29, interval=1, strategy="incremental")
    pool, kc, vc = pool_from_case(case)
    gen = torch.Generator().manual_seed(6)
    steps = 48
    n0 = int(pool.h_sorted[0])
    for step in range(steps):
        nk = (case.keys[0, :, step * 5 + 1].float() + 0.5 * torch.randn(2, 128, generator=gen)).to(dtype)
        nv = torch.randn(2, 128, generator=gen).to(dtype)
        pool.append_kv(nk.cuda().contiguous(), nv.cuda().contiguous())
        pool.append_encode(1)
    torch.cuda.synchronize()
    for s in range(2):
        dev = pool.export_stream(s)
        pos = dev["positions"][n0:]
        assert len(pos) == steps
        keys = kc[0, s, pos.to(kc.device)].unsqueeze(0).contiguous()  # the rows the encoder read from the cache
        words, lids, norms = encode_bulk(keys, pool.coarse[s : s + 1, : case.streams[s].index.coarse.shape[0]],
                                         pool.codebooks[s : s + 1])
        got = torch.stack([(words[0] >> (8 * b)) & 255 for b in range(4)], dim=1).to(torch.uint8)
        assert torch.equal(lids[0], dev["list_ids"][n0:])
        assert torch.equal(got, dev["packed_codes"][n0:])
        assert torch.equal(norms[0], dev["key_norms"][n0:])


def test_device_build_and_refresh_use_the_kernel_and_stay_close_to_the_cpu_build():
    """build_index_batch / online_refresh_batch on the GPU (training in torch, the final assign+encode
    in the kernel, streams read in place from a strided cache view) against the same functions on the
    CPU: a key that sits on a numerical tie may change lists during training and move its two
    centroids a little, so centroids and code words agree on average and nearly all keys get the
    same list and code."""
    from pqhsa_release_b200.config import paper_index_config
    from pqhsa_release_b200.index_build import build_index_batch, online_refresh_batch

    gen = torch.Generator().manual_seed(3)
    cache = torch.randn(2, 2300, 128, generator=gen)
    vals = torch.randn(2, 2300, 128, generator=gen)
    cfg = paper_index_config(num_lists=48)
    k, v = cache[:, 4:2004], vals[:, 4:2004]  # a view with a stream stride larger than N * 128
    cpu = build_index_batch(k, v, cfg)
    gpu = build_index_batch(cache.cuda()[:, 4:2004], vals.cuda()[:, 4:2004], cfg)
    for a, b in zip(cpu, gpu):
        assert float((a.coarse_centroids - b.coarse_centroids.cpu()).abs().mean()) <= 1e-4
        assert float((a.codebooks - b.codebooks.cpu()).abs().mean()) <= 1e-3
        assert float((a.list_ids != b.list_ids.cpu()).float().mean()) <= 0.01
        assert float((a.packed_codes != b.packed_codes.cpu()).any(dim=1).float().mean()) <= 0.05
        assert int(b.value_counts.sum()) == 2000
    k2, v2 = cache[:, 4:2204], vals[:, 4:2204]
    cur = [{"coarse": a.coarse_centroids, "codebooks": a.codebooks} for a in cpu]
    r_cpu = online_refresh_batch(k2, v2, cur, 200, cfg)
    cur_gpu = [{"coarse": a.coarse_centroids.cuda(), "codebooks": a.codebooks.cuda()} for a in cpu]
    r_gpu = online_refresh_batch(cache.cuda()[:, 4:2204], vals.cuda()[:, 4:2204], cur_gpu, 200, cfg)
    for a, b in zip(r_cpu, r_gpu):
        assert float((a.coarse_centroids - b.coarse_centroids.cpu()).abs().mean()) <= 1e-4
        assert float((a.list_ids != b.list_ids.cpu()).float().mean()) <= 0.01
        assert float((a.packed_codes != b.packed_codes.cpu()).any(dim=1).float().mean()) <= 0.05


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bulk_encode_with_given_lists_equals_the_full_pass(dtype):
    """pqhsa_encode_bulk_assigned: with the lists of an earlier pass as an input the codes and norms are those of
    the full pass, bit for bit (the index build's last pass skips the nearest-list search this way)."""
    from pqhsa_release_b200.index_build import encode_bulk

    gen = torch.Generator().manual_seed(21)
    keys = torch.randn(2, 1500, 128, generator=gen).to(dtype).cuda()
    coarse = torch.nn.functional.normalize(torch.randn(2, 77, 128, generator=gen), dim=-1).to(dtype).cuda()
    books = (0.1 * torch.randn(2, 8, 16, 16, generator=gen)).to(dtype).cuda()
    words, lids, norms = encode_bulk(keys, coarse, books, raw=True)
    w2, l2, n2 = encode_bulk(keys, coarse, books, raw=True, lists=lids.clone())
    assert torch.equal(w2, words) and torch.equal(l2, lids) and torch.equal(n2, norms)
    with pytest.raises(ValueError):
        encode_bulk(keys, coarse, books, lists=lids[:, :10])


def test_bulk_encode_argument_errors():
    from pqhsa_release_b200 import _lib
    from pqhsa_release_b200.index_build import encode_bulk

    k = torch.zeros(1, 8, 128, device="cuda")
    with pytest.raises(ValueError):
        encode_bulk(k, torch.zeros(1, 4, 128, device="cuda"), torch.zeros(1, 8, 16, 8, device="cuda"))
    with pytest.raises(_lib.PqhsaError):  # more lists than the library's maximum
        encode_bulk(k, torch.zeros(1, _lib.MAX_LISTS + 1, 128, device="cuda"), torch.zeros(1, 8, 16, 16, device="cuda"))
    words, lids, norms = encode_bulk(k[:, :0], torch.zeros(1, 4, 128, device="cuda"), torch.zeros(1, 8, 16, 16, device="cuda"))
    assert words.shape == (1, 0) and lids.shape == (1, 0) and norms.shape == (1, 0)
