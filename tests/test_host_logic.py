"""CPU tests of the host side: configuration, list-sorted layout, the batched index
build against the oracle, workload byte counts, the plugin surface and KV-head
sharding over two gloo ranks."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from oracle.pqhsa_oracle import OracleIndex, OracleIndexConfig, list_value_means  # noqa: E402
from pqhsa_release_b200 import config as cfgmod  # noqa: E402
from pqhsa_release_b200 import workloads  # noqa: E402
from pqhsa_release_b200.device_index import codes_to_words, list_sorted_layout, words_to_codes  # noqa: E402
from pqhsa_release_b200.index_build import build_index_batch, online_refresh_batch  # noqa: E402


def test_config_defaults_match_the_reference_dataclasses():
    ic, ac = cfgmod.IVFPQConfig(), cfgmod.SparseAttentionConfig()
    assert (ic.num_lists, ic.num_subspaces, ic.num_bits, ic.coarse_max_iter, ic.pq_max_iter) == (256, 16, 8, 30, 25)
    assert (ac.sink_tokens, ac.local_window, ac.retrieval_topk, ac.mode, ac.index_update_strategy) == (
        0, 0, 100, "sparse", "incremental")
    pic, pac = cfgmod.paper_index_config(), cfgmod.paper_attention_config()
    cfgmod.validate_index_config(pic)
    cfgmod.validate_attention_config(pac)
    assert (pic.num_lists, pic.num_subspaces, pic.num_bits, pic.direction_normalize) == (512, 8, 4, True)
    assert (pac.sink_tokens, pac.local_window, pac.index_update_strategy, pac.index_update_interval) == (
        4, 128, "deferred", 256)


@pytest.mark.parametrize("field, value", [("num_subspaces", 16), ("num_bits", 8), ("residual", False),
                                          ("direction_normalize", False), ("rotation", "random_orthogonal"),
                                          ("num_lists", 1024), ("kernel_backend", "cuda")])
def test_unsupported_index_settings_are_rejected(field, value):
    with pytest.raises(ValueError):
        cfgmod.validate_index_config(cfgmod.paper_index_config(**{field: value}))


@pytest.mark.parametrize("field, value", [("mode", "sparse"), ("hybrid_value_mode", "denominator"),
                                          ("exact_rerank", False), ("retrieval_top_p", 0.9),
                                          ("collect_attention_details", True), ("kv_storage", "cpu"),
                                          ("index_update_strategy", "never"), ("index_update_interval", 0)])
def test_unsupported_attention_settings_are_rejected(field, value):
    with pytest.raises(ValueError):
        cfgmod.validate_attention_config(cfgmod.paper_attention_config(**{field: value}))


def test_topk_resolution():
    ac = cfgmod.paper_attention_config(retrieval_top_fraction=0.02)
    assert cfgmod.resolve_topk(130940, ac) == 2619 and cfgmod.resolve_topk(0, ac) == 0
    assert cfgmod.resolve_topk(50, cfgmod.paper_attention_config(retrieval_top_fraction=None)) == 50


def test_code_word_round_trip_and_list_sorted_layout():
    g = torch.Generator().manual_seed(0)
    packed = torch.randint(0, 256, (1000, 4), generator=g, dtype=torch.int64).to(torch.uint8)
    assert torch.equal(words_to_codes(codes_to_words(packed)), packed)
    ids = torch.randint(0, 37, (1000,), generator=g)
    ids[ids == 5] = 6  # an empty list
    perm, unit_off, unit_list = list_sorted_layout(ids, 37)
    assert torch.equal(perm, torch.argsort(ids, stable=True))
    assert int(unit_off[0]) == 0 and int(unit_off[-1]) == 1000
    lens = unit_off[1:] - unit_off[:-1]
    assert int(lens.min()) >= 1 and int(lens.max()) <= 128
    sorted_ids = ids[perm]
    for u in range(unit_list.numel()):  # every unit lies inside one list
        seg = sorted_ids[int(unit_off[u]): int(unit_off[u + 1])]
        assert bool((seg == unit_list[u]).all())
    assert 5 not in unit_list.tolist()


def test_batched_index_build_equals_the_oracle_build():
    g = torch.Generator().manual_seed(1)
    k = torch.randn(2, 2500, 128, generator=g)
    v = torch.randn(2, 2500, 128, generator=g)
    res = build_index_batch(k, v, cfgmod.paper_index_config(num_lists=48))
    for i in range(2):
        o = OracleIndex(OracleIndexConfig(num_lists=48)).build(k[i])
        assert torch.equal(res[i].list_ids, o.list_ids)
        assert torch.equal(res[i].packed_codes, o.packed)
        assert torch.equal(res[i].coarse_centroids, o.coarse)
        assert torch.equal(res[i].codebooks, o.codebooks)
        assert torch.equal(res[i].key_norms, o.norms)
        vm, vs, vc = list_value_means(o.list_ids, v[i], 48)
        assert torch.allclose(res[i].value_means, vm, atol=1e-6)
        assert torch.equal(res[i].value_counts.float(), vc)


def test_device_build_draws_the_rows_of_the_sequential_trainings():
    """The batched code-word training of the device-side build seeds subspace m like the per-subspace k-means of
    the CPU build (seed + 10000 + m, pq_hsa/index/pq.py:81-94): same initial rows, and a generator per subspace
    that continues where that k-means' generator would."""
    from pqhsa_release_b200.index_build import _draw_code_word_rows

    gens, rows = _draw_code_word_rows(300, 7)
    assert len(gens) == 8 and len(rows) == 8
    for m in range(8):
        ref = torch.Generator().manual_seed(7 + 10_000 + m)
        assert torch.equal(rows[m], torch.randperm(300, generator=ref)[:16])
        assert torch.equal(torch.randint(0, 300, (5,), generator=gens[m]), torch.randint(0, 300, (5,), generator=ref))
    _, few = _draw_code_word_rows(9, 7)  # fewer keys than code words: every key, then random repeats
    for m in range(8):
        ref = torch.Generator().manual_seed(7 + 10_000 + m)
        assert torch.equal(few[m], torch.cat([torch.arange(9), torch.randint(0, 9, (7,), generator=ref)]))


def test_online_refresh_equals_the_oracle_refresh():
    g = torch.Generator().manual_seed(2)
    k = torch.randn(1, 1800, 128, generator=g)
    v = torch.randn(1, 1800, 128, generator=g)
    cfg = cfgmod.paper_index_config(num_lists=32)
    n0 = 1700
    first = build_index_batch(k[:, :n0], v[:, :n0], cfg)[0]
    o = OracleIndex(OracleIndexConfig(num_lists=32)).build(k[0, :n0])
    cur = [{"coarse": first.coarse_centroids, "codebooks": first.codebooks}]
    got = online_refresh_batch(k, v, cur, 1800 - n0, cfg)[0]
    o.online_refresh(k[0], k[0, n0:])
    assert torch.allclose(got.coarse_centroids, o.coarse, atol=1e-6)
    assert torch.allclose(got.codebooks, o.codebooks, atol=1e-6)
    assert float((got.list_ids == o.list_ids).float().mean()) > 0.999
    assert float((got.packed_codes == o.packed).float().mean()) > 0.999


def test_workload_shapes_and_algorithmic_bytes():
    c2 = workloads.WORKLOADS["c2"]
    assert (c2.batch, c2.kv_heads, c2.group, c2.context) == (4, 8, 4, 131072)
    assert c2.retrieval_len() == 130940 and c2.topk() == 2619
    assert abs(c2.algorithmic_bytes() / 1e6 - 215.9) < 0.2   # the step's byte count at 128K, batch 4
    c0 = workloads.WORKLOADS["c0"]
    assert c0.retrieval_len() == 8060 and c0.topk() == 162
    k, v, q = workloads.config0_stream(0, 512)
    assert k.shape == (512, 128) and q.shape == (128,)
    k2, _, _ = workloads.config0_stream(0, 512)
    assert torch.equal(k, k2)


def test_plugin_is_cheap_inert_by_default_and_idempotent(monkeypatch):
    code = ("import sys; import pqhsa_release_b200.pq_hsa_vllm as m; "
            "assert 'torch' not in sys.modules and 'vllm' not in sys.modules; m.vllm_general_plugin(); "
            "print(m.install()['installed'])")
    env = {k: v for k, v in os.environ.items() if not k.startswith("PQ_HSA")}
    out = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "False", out.stderr

    from pqhsa_release_b200.pq_hsa_vllm import plugin
    from pqhsa_release_b200.pq_hsa_vllm.config import PQHSAConfig

    class Impl:
        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None):
            return "dense"

    for k in list(os.environ):
        if k.startswith("PQ_HSA"):
            monkeypatch.delenv(k)
    monkeypatch.setenv("PQ_HSA_TOP_FRAC", "0.05")
    r = plugin.install(force=True, impl_cls=Impl)
    assert r["installed"] and not r["already"] and r["config"]["top_fraction"] == 0.05
    assert os.environ["PQ_HSA_TOP_FRAC"] == "0.05" and os.environ["PQ_HSA_SINK"] == "4"   # explicit env wins
    assert plugin.install(force=True, impl_cls=Impl)["already"]
    assert Impl().forward(None, None, None, None, None, None) == "dense"                # no metadata: dense path
    cfg = PQHSAConfig()
    assert cfg.as_env()["PQ_HSA_NUM_LISTS"] == "512" and cfg.asdict()["flush_interval"] == 256
    for k in list(os.environ):
        if k.startswith("PQ_HSA") or k.startswith("PQ_USE"):
            monkeypatch.delenv(k, raising=False)


def test_admission_rules_of_the_decode_runtime(monkeypatch):
    from types import SimpleNamespace as NS

    from pqhsa_release_b200.pq_hsa_vllm import runtime

    monkeypatch.delenv("PQ_HSA_BATCH", raising=False)
    md = NS(use_cascade=False, max_query_len=1, num_actual_tokens=1, seq_lens=torch.tensor([5000]), max_seq_len=5000)
    assert runtime.should_pq_decode(md)
    assert not runtime.should_pq_decode(None)
    assert not runtime.should_pq_decode(NS(**{**md.__dict__, "max_query_len": 7}))
    assert not runtime.should_pq_decode(NS(**{**md.__dict__, "max_seq_len": 100}))
    assert not runtime.should_pq_decode(NS(**{**md.__dict__, "use_cascade": True}))
    two = NS(**{**md.__dict__, "seq_lens": torch.tensor([5000, 6000]), "num_actual_tokens": 2,
                "seq_lens_cpu": torch.tensor([5000, 6000])})
    assert not runtime.should_pq_decode(two)
    monkeypatch.setenv("PQ_HSA_BATCH", "1")
    assert not runtime.should_pq_decode(two) and runtime.rejects()["no_req_ids"] == 1   # slots alone do not tell requests apart
    runner = NS(input_batch=NS(req_ids=["a", "b"]), requests={})
    two._pq_runner = runner
    assert runtime.should_pq_decode(two)
    assert runtime.batch_req_keys(two, 2) == ["a", "b"] and runtime.batch_seq_lens(two) == [5000, 6000]
    short = NS(**{**two.__dict__, "seq_lens_cpu": torch.tensor([5000, 100]), "_pq_batch_seq_lens": None})
    assert not runtime.should_pq_decode(short)
    assert runtime.rejects()["seq_too_short"] >= 2
    # the metadata builder wrap hands the runner to the metadata (pq_hsa_decode_runtime.py:874-902)
    class Builder:
        def build(self, *a, **k):
            return NS(max_query_len=1)

    Builder.runner = runner
    assert runtime.attach_runner(Builder) == {"attached": True, "already": False}
    assert Builder().build()._pq_runner is runner and runtime.attach_runner(Builder)["already"]
    # prefix keys: (context length, digest of the prompt ids)
    runner.requests = {"a": NS(prompt_token_ids=[1, 2, 3]), "b": NS(prompt_token_ids=None)}
    keys = runtime.prefix_keys(two, [5000, 6000])
    assert keys[0][0] == 4999 and len(keys[0][1]) == 16 and keys[1] is None


def test_kv_head_sharding_and_gather_over_two_gloo_ranks(tmp_path):
    from pqhsa_release_b200.parallel import kv_head_shard, query_head_shard

    assert list(kv_head_shard(8, 1, 4)) == [2, 3] and list(query_head_shard(8, 4, 1, 4)) == list(range(8, 16))
    with pytest.raises(ValueError):
        kv_head_shard(8, 0, 3)
    script = tmp_path / "w.py"
    script.write_text(
        "import os, sys, torch, torch.distributed as dist\n"
        f"sys.path.insert(0, {str(ROOT)!r})\n"
        "from pqhsa_release_b200.parallel import gather_context, query_head_shard\n"
        "dist.init_process_group('gloo')\n"
        "r, w = dist.get_rank(), dist.get_world_size()\n"
        "full = torch.arange(2 * 8 * 4, dtype=torch.float32).reshape(2, 8, 4)\n"
        "mine = full[:, list(query_head_shard(4, 2, r, w))]\n"
        "got = gather_context(mine)\n"
        "assert torch.equal(got, full), (r, got)\n"
        "dist.destroy_process_group()\n"
    )
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29731")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29731", str(script)],
                         env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]


def test_reference_checkpoint_layout_is_understood_on_the_host():
    """The reference adapter's state_dict (a fixture written by the reference itself) parses into what the engine
    restores from: stacked K/V, the shared counters, one index per stream.  No GPU needed for the parsing."""
    from pathlib import Path

    from pqhsa_release_b200.decode_adapter import reference_attention_state

    d = torch.load(Path(__file__).resolve().parent / "golden" / "golden_adapter_state.pt")
    att = d["state"]["attention"]
    r = reference_attention_state(att, device="cpu")
    assert tuple(r["keys"].shape) == (1, 2, 523, 128) and r["indexed_length"] == 523 and r["pending"] == 0
    ix = r["streams"][0]
    assert ix.list_ids.dtype == torch.int64 and ix.packed_codes.dtype == torch.uint8 and ix.list_ids.numel() == 391
    assert int(ix.value_counts.sum()) == 391
    bad = dict(att, leading_shape=(2, 2))
    with pytest.raises(ValueError):
        reference_attention_state(bad, device="cpu")


def test_multi_query_admission(monkeypatch):
    """benchmarks/vllm_backend/pq_hsa_multi_query.py:112-160: a step with several query tokens is taken only with
    PQ_HSA_MULTI_QUERY=1, for one request, within PQ_HSA_MQ_MAX, when it starts after the prompt."""
    from types import SimpleNamespace as NS

    import torch

    from pqhsa_release_b200.pq_hsa_vllm import runtime

    runtime.reset()
    monkeypatch.setenv("PQ_HSA_ENABLE", "1")
    monkeypatch.delenv("PQ_HSA_BATCH", raising=False)
    runner = NS(input_batch=NS(req_ids=["r"]), requests={"r": NS(prompt_token_ids=[0] * 900, num_prompt_tokens=900)})

    def md(total, T, n=1):
        lens = torch.tensor([total] * n, dtype=torch.int32)
        return NS(use_cascade=False, max_query_len=T, num_actual_tokens=T * n, seq_lens=lens, seq_lens_cpu=lens,
                  max_seq_len=total, _pq_runner=runner)

    monkeypatch.delenv("PQ_HSA_MULTI_QUERY", raising=False)
    assert not runtime.should_pq_decode(md(1000, 3))
    monkeypatch.setenv("PQ_HSA_MULTI_QUERY", "1")
    assert runtime.should_pq_decode(md(1000, 3))
    assert not runtime.should_pq_decode(md(1000, 9)), "more query tokens than PQ_HSA_MQ_MAX"
    assert not runtime.should_pq_decode(md(902, 3)), "the step starts inside the prompt: a prefill chunk"
    assert not runtime.should_pq_decode(md(1000, 3, n=2)), "one request only"
    runner.requests.clear()
    assert not runtime.should_pq_decode(md(1000, 3)), "no request object: a chunk cannot be told from a speculative step"
    assert runtime.rejects()["mq_prefill_chunk"] == 1 and runtime.rejects()["mq_no_request"] == 1
