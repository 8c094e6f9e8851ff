"""The adapters with the reference's call signatures, on the GPU: contracts the reference
tests for its own adapters (tests/test_decode_adapter.py, tests/test_kv_cache_growth.py
there) plus parity with the oracle holding the same index."""

from types import SimpleNamespace

import pytest
import torch

from helpers import assert_output_close
from oracle.pqhsa_oracle import OracleAttentionConfig, OracleIndex, OracleIndexConfig, OracleStream
from pqhsa_release_b200 import workloads
from pqhsa_release_b200.config import paper_attention_config, paper_index_config

pytestmark = pytest.mark.gpu


def _inputs(B, H, S, G=1, dtype=torch.bfloat16, seed=0):
    ks, vs, qs = [], [], []
    for b in range(B):
        k, v = workloads.mixture_kv(seed * 100 + b, H, S, dtype=dtype, components=16)
        ks.append(k); vs.append(v); qs.append(workloads.planted_queries(seed * 100 + 50 + b, k, G))
    return torch.stack(ks), torch.stack(vs), torch.stack(qs)


def _oracle_of(engine, s, frac, interval=256, strategy="deferred"):
    """Oracle stream holding exactly the index the device holds for stream ``s``."""
    b, h = divmod(s, engine.H)
    n = engine.length
    keys = engine.keys[b, h, :n].float().cpu()
    values = engine.values[b, h, :n].float().cpu()
    st = OracleStream(OracleIndexConfig(num_lists=engine.icfg.num_lists),
                      OracleAttentionConfig(sink_tokens=engine.acfg.sink_tokens, local_window=engine.acfg.local_window,
                                            retrieval_top_fraction=frac, index_update_interval=interval,
                                            index_update_strategy=strategy))
    st.keys, st.values, st.length = keys, values, n
    st.indexed_length = engine.indexed_length
    e = engine.pool.export_stream_state(s)
    if e is not None:
        ix = OracleIndex(st.icfg)
        ix.packed, ix.list_ids = e.packed_codes.cpu(), e.list_ids.cpu()
        ix.norms, ix.coarse, ix.codebooks = e.key_norms.float().cpu(), e.coarse_centroids.float().cpu(), e.codebooks.float().cpu()
        st.index, st.value_means = ix, e.value_means.float().cpu()
    return st


def test_all_tokens_selected_equals_dense_attention():
    # reference contract: tests/test_decode_adapter.py:11-47
    from pqhsa_release_b200 import IVFPQDecodeAttentionAdapter

    k, v, q = _inputs(2, 2, 700, dtype=torch.float32, seed=1)
    ad = IVFPQDecodeAttentionAdapter(paper_index_config(num_lists=32),
                                     paper_attention_config(retrieval_top_fraction=1.0, sink_tokens=2, local_window=8))
    ad.build_cache(k.cuda(), v.cuda())
    assert ad.leading_shape == (2, 2) and len(ad.streams) == 4
    out = ad.forward(q.cuda()).context.cpu()
    logits = torch.einsum("bhd,bhsd->bhs", q, k) / 128 ** 0.5
    dense = torch.einsum("bhs,bhsd->bhd", torch.softmax(logits, -1), v)
    assert float((out - dense).abs().max()) <= 5e-4 * float(dense.abs().max())


def test_shape_and_state_errors():
    from pqhsa_release_b200 import IVFPQDecodeAttentionAdapter

    ad = IVFPQDecodeAttentionAdapter(paper_index_config(num_lists=16), paper_attention_config())
    with pytest.raises(RuntimeError):
        ad.forward(torch.zeros(1, 1, 128, device="cuda"))
    with pytest.raises(ValueError):
        ad.build_cache(torch.zeros(4, 128, device="cuda"), torch.zeros(4, 128, device="cuda"))
    with pytest.raises(RuntimeError):
        ad.build_cache(torch.zeros(1, 1, 300, 128), torch.zeros(1, 1, 300, 128))   # CPU tensors: no fallback
    k, v, q = _inputs(1, 2, 400, seed=2)
    ad.build_cache(k.cuda(), v.cuda())
    with pytest.raises(ValueError):
        ad.forward(torch.zeros(1, 3, 128, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        ad.decode_step(q.cuda())
    with pytest.raises(ValueError):
        ad.append(torch.zeros(1, 2, 2, 128, device="cuda"), torch.zeros(1, 2, 2, 128, device="cuda"))


@pytest.mark.parametrize("strategy, interval", [("incremental", 1), ("incremental", 5), ("deferred", 6)])
def test_decode_steps_follow_the_oracle(strategy, interval):
    """decode_step appends before attending (reference tests/test_decode_adapter.py:91-145); recent
    tokens stay exact until the update interval (tests/test_acceptance_contracts.py:78-128)."""
    from pqhsa_release_b200 import IVFPQDecodeAttentionAdapter

    dtype = torch.bfloat16
    k, v, q = _inputs(1, 2, 1200, dtype=dtype, seed=3)
    ac = paper_attention_config(retrieval_top_fraction=0.03, index_update_interval=interval,
                                index_update_strategy=strategy)
    ad = IVFPQDecodeAttentionAdapter(paper_index_config(num_lists=48), ac).build_cache(k.cuda(), v.cuda())
    gen = torch.Generator().manual_seed(9)
    for step in range(14):
        nk = (k[:, :, 11 * step + 5].float() + 0.3 * torch.randn(1, 2, 128, generator=gen)).to(dtype)
        nv = torch.randn(1, 2, 128, generator=gen).to(dtype)
        qq = (q.float() + 0.02 * step).to(dtype)
        out = ad.decode_step(qq.cuda(), nk.cuda().unsqueeze(2), nv.cuda().unsqueeze(2)).context.float().cpu()
        eng = ad.attention
        assert eng.length == 1201 + step
        if strategy == "deferred" and step == 9:
            assert ad.apply_pending_index_update() == 2 and ad.apply_pending_index_update() == 0
            out = ad.forward(qq.cuda()).context.float().cpu()
        s_end, r_end = eng.bounds()
        for s in range(2):
            st = _oracle_of(eng, s, 0.03)
            assert st.index.num_vectors == r_end - s_end
            det = st.forward_detail(qq[0, s : s + 1].float())
            assert_output_close(out[0, s], det.output[0], dtype, f"step {step} stream {s}")


def test_state_dict_round_trip():
    from pqhsa_release_b200 import IVFPQDecodeAttentionAdapter

    k, v, q = _inputs(1, 2, 900, seed=4)
    ac = paper_attention_config(retrieval_top_fraction=0.05, index_update_interval=1, index_update_strategy="incremental")
    ad = IVFPQDecodeAttentionAdapter(paper_index_config(num_lists=32), ac).build_cache(k.cuda(), v.cuda())
    for i in range(3):
        ad.append(k[:, :, i].cuda(), v[:, :, i].cuda())
    want = ad.forward(q.cuda()).context
    state = ad.state_dict()
    again = IVFPQDecodeAttentionAdapter.from_state_dict(state)
    got = again.forward(q.cuda()).context
    assert again.attention.length == 903 and again.leading_shape == (1, 2)
    assert float((got.float() - want.float()).abs().max()) <= 1e-2 * float(want.float().abs().max())
    with pytest.raises(ValueError):
        IVFPQDecodeAttentionAdapter(paper_index_config(num_lists=16), ac).load_state_dict(state)


@pytest.mark.parametrize("layout", ["5d", "4d"])
def test_gqa_sidecar_reads_vllm_pages_in_place(layout):
    """Both FLASH_ATTN page layouts, 16-token blocks, a permuted block table: the sidecar on the
    pages equals the sidecar on a contiguous copy and the oracle."""
    from pqhsa_release_b200 import GQASidecar
    from pqhsa_release_b200.paged_kv import gather_paged_kv, write_paged_token

    dtype, Hkv, G, S, bs = torch.bfloat16, 2, 4, 1000, 16
    k, v, q = _inputs(1, Hkv, S, G=G, dtype=dtype, seed=5)
    nblk = 80
    gen = torch.Generator().manual_seed(1)
    table = torch.randperm(nblk, generator=gen)[: (S + 64 + bs - 1) // bs].to(torch.int32).reshape(1, -1).cuda()
    if layout == "5d":
        kv_cache = torch.zeros(2, nblk, bs, Hkv, 128, dtype=dtype, device="cuda")
    else:
        kv_cache = torch.zeros(nblk, Hkv, bs, 256, dtype=dtype, device="cuda")
    for t in range(S):
        write_paged_token(kv_cache, table, 0, t, k[0, :, t].cuda(), v[0, :, t].cuda())
    kk, vv = gather_paged_kv(kv_cache, table, 0, S)
    assert torch.equal(kk.cpu(), k) and torch.equal(vv.cpu(), v)
    md = SimpleNamespace(block_table=table)
    ic = paper_index_config(num_lists=32)
    ac = paper_attention_config(retrieval_top_fraction=0.04, index_update_interval=1, index_update_strategy="incremental")
    paged = GQASidecar(ic, ac, num_query_heads=Hkv * G, num_kv_heads=Hkv)
    paged.set_paged_kv_context(kv_cache, md, 0)
    paged.build_cache(kk, vv)
    assert paged.engine.keys is None, "the paged sidecar must not hold a K/V copy"
    flat = GQASidecar(ic, ac, num_query_heads=Hkv * G, num_kv_heads=Hkv).build_cache(k.cuda(), v.cuda())
    gen = torch.Generator().manual_seed(2)
    for step in range(4):
        qq = (q.float() + 0.03 * step).to(dtype).cuda()
        a, b = paged.forward(qq).float().cpu(), flat.forward(qq).float().cpu()
        assert float((a - b).abs().max()) <= 1e-2 * float(b.abs().max())
        for s in range(Hkv):
            st = _oracle_of(flat.engine, s, 0.04)
            det = st.forward_detail(qq[0, s * G : (s + 1) * G].float().cpu())
            for g in range(G):
                assert_output_close(a[0, s * G + g], det.output[g], dtype, f"step {step} head {s * G + g}")
        nk, nv = torch.randn(1, Hkv, 128, generator=gen).to(dtype), torch.randn(1, Hkv, 128, generator=gen).to(dtype)
        write_paged_token(kv_cache, table, 0, S + step, nk[0].cuda(), nv[0].cuda())   # vLLM writes the page
        assert paged.lean_append(nk.cuda(), nv.cuda())
        flat.append(nk.cuda(), nv.cuda())
    with pytest.raises(ValueError):
        paged.forward(torch.zeros(2, Hkv * G, 128, dtype=dtype, device="cuda"))


def test_deferred_fixture_of_the_reference_through_the_engine():
    """The reference's own run with deferred index updates (tests/golden/golden_mix_deferred.npz: 20 appends,
    the pending update applied after the 11th) replayed on the GPU: the engine starts from the index tensors
    the reference built, appends the same rows, applies the update at the same step (EMA of centroids and code
    words, every key re-encoded: pq_hsa/index/ivfpq.py:647-707) and must give the reference's outputs at every
    step, and the reference's codes, list ids and codebooks at the end."""
    import sys
    from pathlib import Path

    import numpy as np

    here = Path(__file__).resolve().parent
    sys.path.insert(0, str(here / "golden"))
    from make_golden import CASES, case_inputs

    from pqhsa_release_b200.device_index import StreamIndexTensors
    from pqhsa_release_b200.engine import PoolAttention

    name = "mix_deferred"
    kind, seed, ctx, lists, group, dtype, strategy, interval, appends = CASES[name]
    g = np.load(here / "golden" / f"golden_{name}.npz")
    k, v, q, nk, nv = case_inputs(name)
    eng = PoolAttention(paper_index_config(num_lists=lists),
                        paper_attention_config(retrieval_top_fraction=0.02, index_update_interval=interval,
                                               index_update_strategy=strategy), group=group)
    idx = StreamIndexTensors(torch.from_numpy(g["packed_codes"]), torch.from_numpy(g["list_ids"]).long(),
                             torch.from_numpy(g["key_norms"]), torch.from_numpy(g["coarse"]),
                             torch.from_numpy(g["codebooks"]), torch.from_numpy(g["value_means"]))
    eng.restore({"keys": k.cuda()[None, None], "values": v.cuda()[None, None], "indexed_length": ctx, "pending": 0,
                 "deferred_pending": False, "streams": (idx,)})
    out0 = eng.forward(q.cuda()[None]).cpu()[0]
    for r in range(group):
        assert_output_close(out0[r], torch.from_numpy(g["output0"][r]), torch.float32, f"row {r} before any append")
    flushed = False
    for i in range(appends):
        eng.append(nk[i].cuda()[None, None], nv[i].cuda()[None, None])
        if i == appends // 2:
            assert eng.apply_pending_index_update()
            flushed = True
        out = eng.forward((q + 0.01 * i).cuda()[None]).cpu()[0]
        want = torch.from_numpy(g["outputs_after_appends"][i])
        for r in range(group):
            if not flushed:
                assert_output_close(out[r], want[r], torch.float32, f"append {i} row {r}")
            else:
                # after the update a handful of keys may sit in another list or carry another code than in the
                # reference's CPU run (ties of the re-encode): the bar is the 2e-3 of the output tolerance
                err = float((out[r] - want[r]).norm() / want[r].norm())
                assert err <= 2e-3, f"append {i} row {r}: {err:.2e}"
    e = eng.pool.export_stream_state(0)
    n = g["list_ids_end"].shape[0]
    assert e.list_ids.numel() == n
    lid_same = (e.list_ids.cpu().numpy() == g["list_ids_end"].astype(np.int64))
    code_same = (e.packed_codes.cpu().numpy() == g["packed_codes_end"]).all(axis=1)
    assert lid_same.mean() >= 0.99 and (code_same | ~lid_same).mean() >= 0.95, (lid_same.mean(), code_same.mean())
    np.testing.assert_allclose(e.coarse_centroids.float().cpu().numpy(), g["coarse_end"], rtol=0, atol=2e-6)
    np.testing.assert_allclose(e.codebooks.float().cpu().numpy(), g["codebooks_end"], rtol=0, atol=2e-6)
    np.testing.assert_allclose(e.key_norms.float().cpu().numpy(), g["key_norms_end"], rtol=1e-6)


@pytest.mark.parametrize("strategy, interval", [("incremental", 1), ("deferred", 4)])
def test_sidecar_fast_path_replays_a_validated_cuda_graph(strategy, interval):
    """lean_append + forward = one fused library call; with the graph on it is captured on the first step,
    validates itself (NaN poison, replay, compare with the eager call: benchmarks/e2e_pq_param_sweep.py:6170-6201)
    and is replayed from then on.  Graph and eager sidecars must agree step for step and follow the oracle,
    also across a deferred flush and for two requests that advance together."""
    from pqhsa_release_b200 import GQASidecar

    dtype, B, Hkv, G, S = torch.bfloat16, 2, 2, 4, 5300
    k, v, q = _inputs(B, Hkv, S, G=G, dtype=dtype, seed=6)
    ic = paper_index_config(num_lists=64)
    ac = paper_attention_config(retrieval_top_fraction=0.03, index_update_interval=interval, index_update_strategy=strategy)
    fast = GQASidecar(ic, ac, num_query_heads=Hkv * G, num_kv_heads=Hkv, cuda_graph=True).build_cache(k.cuda(), v.cuda())
    slow = GQASidecar(ic, ac, num_query_heads=Hkv * G, num_kv_heads=Hkv, cuda_graph=False).build_cache(k.cuda(), v.cuda())
    assert not fast.cuda_graph_active and fast.batched_heads_active
    gen = torch.Generator().manual_seed(4)
    for step in range(10):
        nk = (k[:, :, 13 * step + 7].float() + 0.3 * torch.randn(B, Hkv, 128, generator=gen)).to(dtype).cuda()
        nv = torch.randn(B, Hkv, 128, generator=gen).to(dtype).cuda()
        qq = (q.float() + 0.02 * step).to(dtype).cuda()
        assert fast.lean_append(nk, nv, qq) and slow.lean_append(nk, nv, qq)
        a = fast.forward(qq).clone()
        b = slow.forward(qq)
        torch.cuda.synchronize()
        assert fast.cuda_graph_active and not slow.cuda_graph_active
        assert fast.length == slow.length == S + step + 1 and fast.engine.length == slow.engine.length
        assert float((a.float() - b.float()).abs().max()) <= 1e-2 * float(b.float().abs().max()), f"step {step}"
        assert torch.equal(fast.engine.pool.state, slow.engine.pool.state)
        if strategy == "deferred" and step == 5:
            assert fast.apply_pending_index_update() == B * Hkv and slow.apply_pending_index_update() == B * Hkv
        if step in (0, 6, 9):
            out = a.float().cpu()
            for s in range(B * Hkv):
                st = _oracle_of(fast.engine, s, 0.03, interval, strategy)
                b_, h_ = divmod(s, Hkv)
                det = st.forward_detail(qq[b_, h_ * G : (h_ + 1) * G].float().cpu())
                for g in range(G):
                    assert_output_close(out[b_, h_ * G + g], det.output[g], dtype, f"step {step} stream {s} row {g}")
    assert fast._step_graph.attempts == 1, "the first capture must validate"
    # the static input buffer filled by the caller: the same step without the copies into it
    if strategy == "incremental":
        sq, sk, sv, flat = fast.static_inputs()
        assert flat.numel() == sq.numel() + sk.numel() + sv.numel() and sq.data_ptr() == flat.data_ptr()
        nk = (k[:, :, 999].float() + 0.1).to(dtype).cuda()
        nv = torch.randn(B, Hkv, 128, generator=gen).to(dtype).cuda()
        qq = (q.float() - 0.05).to(dtype).cuda()
        flat.copy_(torch.cat([qq.reshape(-1), nk.reshape(-1), nv.reshape(-1)]))
        assert fast.lean_append(sk, sv, sq) and slow.lean_append(nk, nv, qq)
        a = fast.forward(sq).clone()
        b = slow.forward(qq)
        torch.cuda.synchronize()
        assert fast.cuda_graph_active and torch.equal(fast.engine.pool.state, slow.engine.pool.state)
        assert float((a.float() - b.float()).abs().max()) <= 1e-2 * float(b.float().abs().max())


def test_prefix_checkpoint_restores_the_index_without_a_rebuild():
    """checkpoint_prefix / restore_prefix (benchmarks/e2e_pq_param_sweep.py:3358-3432, :3735-3899): after decoding past
    the prompt the sidecar goes back to the checkpointed prefix - same index, same counters, same output as right
    after the build - and decodes again as if freshly built."""
    from pqhsa_release_b200 import GQASidecar

    dtype, Hkv, G, S = torch.bfloat16, 2, 4, 4800
    k, v, q = _inputs(1, Hkv, S, G=G, dtype=dtype, seed=8)
    ic = paper_index_config(num_lists=64)
    ac = paper_attention_config(retrieval_top_fraction=0.03, index_update_interval=1, index_update_strategy="incremental")
    side = GQASidecar(ic, ac, num_query_heads=Hkv * G, num_kv_heads=Hkv).build_cache(k.cuda(), v.cuda())
    assert side.prefix_checkpoint_length is None and not side.restore_prefix()
    first = side.forward(q.cuda()).clone()
    side.checkpoint_prefix()
    assert side.prefix_checkpoint_length == S
    state0 = side.engine.pool.state.clone()
    gen = torch.Generator().manual_seed(3)
    rows = [(torch.randn(1, Hkv, 128, generator=gen).to(dtype).cuda(), torch.randn(1, Hkv, 128, generator=gen).to(dtype).cuda())
            for _ in range(6)]
    outs = []
    for nk, nv in rows:
        side.lean_append(nk, nv)
        outs.append(side.forward(q.cuda()).clone())
    rebuilds = side.engine.index_rebuilds
    assert side.length == S + 6 and side.restore_prefix()
    assert side.length == S and side.engine.length == S and side.engine.index_rebuilds == rebuilds
    assert torch.equal(side.engine.pool.state, state0)
    again = side.forward(q.cuda())
    assert float((again.float() - first.float()).abs().max()) <= 1e-2 * float(first.float().abs().max())
    for (nk, nv), want in zip(rows, outs):   # the same continuation gives the same outputs
        side.lean_append(nk, nv)
        got = side.forward(q.cuda())
        assert float((got.float() - want.float()).abs().max()) <= 1e-2 * float(want.float().abs().max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_incremental_deferred_flush_follows_the_production_update(dtype):
    """The sidecar's deferred flush (PQ_HSA_INCREMENTAL_FLUSH=1: EMA of centroids and code words on the keys that
    left the local window, only those keys encoded, count-weighted value means -
    benchmarks/e2e_pq_param_sweep.py:3021-3344) against the CPU restatement of those lines: moved codebooks to
    rounding, list ids and codes of the new keys bit for bit (a differing assignment must be a rare tie), old
    entries untouched, value means and the attention output to tolerance."""
    from helpers import round_to
    from pqhsa_release_b200 import GQASidecar

    Hkv, G, S, L = 2, 2, 3000, 48
    k, v, q = _inputs(1, Hkv, S, G=G, dtype=dtype, seed=12)
    ic = paper_index_config(num_lists=L)
    ac = paper_attention_config(retrieval_top_fraction=0.03, index_update_interval=8, index_update_strategy="deferred")
    side = GQASidecar(ic, ac, num_query_heads=Hkv * G, num_kv_heads=Hkv, cuda_graph=False).build_cache(k.cuda(), v.cuda())
    oracles = [_oracle_of(side.engine, s, 0.03, 8, "deferred") for s in range(Hkv)]
    before = [side.engine.pool.export_stream(s) for s in range(Hkv)]
    gen = torch.Generator().manual_seed(5)
    for step in range(11):
        nk = (k[:, :, 17 * step + 3].float() + 0.4 * torch.randn(1, Hkv, 128, generator=gen)).to(dtype)
        nv = torch.randn(1, Hkv, 128, generator=gen).to(dtype)
        side.lean_append(nk.cuda(), nv.cuda())
        side.forward(q.cuda())
        for s, st in enumerate(oracles):
            st.append(nk[0, s].float(), nv[0, s].float())
    assert side.apply_pending_index_update() == Hkv and side.apply_pending_index_update() == 0
    out = side.forward(q.cuda()).float().cpu()
    mism = total = 0
    for s, st in enumerate(oracles):
        assert st.apply_pending_incremental_flush()
        e = side.engine.pool.export_stream_state(s)
        n_old, n_new = before[s]["list_ids"].numel(), 11
        assert e.list_ids.numel() == st.index.num_vectors == n_old + n_new
        tol = 2e-6 if dtype == torch.float32 else 1e-2
        assert float((e.coarse_centroids.float().cpu() - st.index.coarse).abs().max()) <= tol
        assert float((e.codebooks.float().cpu() - st.index.codebooks).abs().max()) <= tol
        # old entries stay as they were
        assert torch.equal(e.list_ids[:n_old].cpu(), before[s]["list_ids"].cpu())
        assert torch.equal(e.packed_codes[:n_old].cpu(), before[s]["packed_codes"].cpu())
        same = (e.list_ids[n_old:].cpu() == st.index.list_ids[n_old:]) & (
            e.packed_codes[n_old:].cpu() == st.index.packed[n_old:]).all(dim=1)
        total += n_new
        mism += int((~same).sum())
        if dtype == torch.float32 and bool(same.all()):
            assert float((e.value_means.float().cpu() - st.value_means).abs().max()) <= 1e-5
            st.index.coarse, st.index.codebooks = e.coarse_centroids.float().cpu(), e.codebooks.float().cpu()
            st.index.norms = round_to(st.index.norms, dtype)
            det = st.forward_detail(q[0, s * G : (s + 1) * G].float())
            for g in range(G):
                assert_output_close(out[0, s * G + g], det.output[g], dtype, f"stream {s} row {g} after the flush")
    assert mism <= (1 if dtype == torch.float32 else 3), f"{mism} of {total} new keys differ from the restatement"


def test_reference_adapter_checkpoint_loads_and_round_trips():
    """A checkpoint written by the reference's own IVFPQDecodeAttentionAdapter.state_dict
    (tests/golden/golden_adapter_state.pt, made by tests/golden/make_golden.py) loads here without a rebuild and
    answers the stored queries as the reference did; what this adapter writes has the same layout, field for field,
    holds the same index, and loads again."""
    from pathlib import Path

    from pqhsa_release_b200 import IVFPQDecodeAttentionAdapter

    d = torch.load(Path(__file__).resolve().parent / "golden" / "golden_adapter_state.pt")
    state, q, want = d["state"], d["queries"], d["context"]
    for st in state["attention"]["streams"]:
        st["keys"], st["values"] = st["keys"].float(), st["values"].float()
    ad = IVFPQDecodeAttentionAdapter.from_state_dict(state)
    assert ad.leading_shape == (1, 2) and ad.attention.length == 523 and ad.attention.index_rebuilds == 0
    out = ad.forward(q.cuda()).context.cpu()
    for h in range(2):
        assert_output_close(out[0, h], want[0, h], torch.float32, f"head {h}")
    mine, ref = ad.state_dict()["attention"], state["attention"]
    assert list(mine) == list(ref) and mine["leading_shape"] == ref["leading_shape"] and mine["key_dim"] == 128
    for a, b in zip(mine["streams"], ref["streams"]):
        assert list(a) == list(b) and list(a["metadata"]) == list(b["metadata"]) and list(a["index"]) == list(b["index"])
        assert a["metadata"]["indexed_length"] == b["metadata"]["indexed_length"] == 523
        for name in ("coarse_centroids", "packed_codes", "pq_codebooks", "key_norms"):
            assert a["index"][name].dtype == b["index"][name].dtype, name
            assert torch.equal(a["index"][name].cpu(), b["index"][name]), name
        assert a["index"]["list_ids"].dtype == torch.uint16
        assert torch.equal(a["index"]["list_ids"].cpu().to(torch.int64), b["index"]["list_ids"].to(torch.int64))
        assert torch.equal(a["keys"].cpu(), b["keys"]) and torch.equal(a["values"].cpu(), b["values"])
        assert torch.allclose(a["retrieval_value_centroids"].cpu(), b["retrieval_value_centroids"], atol=1e-6)
        assert torch.allclose(a["retrieval_value_sums"].cpu(), b["retrieval_value_sums"], atol=1e-4)
    again = IVFPQDecodeAttentionAdapter.from_state_dict(ad.state_dict())
    out2 = again.forward(q.cuda()).context.cpu()
    assert float((out2 - out).abs().max()) <= 1e-5 * float(out.abs().max())
    with pytest.raises(ValueError):
        IVFPQDecodeAttentionAdapter(paper_index_config(num_lists=16), paper_attention_config()).load_state_dict(state)
