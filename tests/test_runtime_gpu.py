"""The vLLM decode hook on the GPU: ``pq_or_dense_forward`` driven with stand-in metadata / impl objects over
both FLASH_ATTN page layouts for 44 decode steps of a changing batch - first-call builds, steady state, a
request joining, one leaving (vLLM moves the tail request into the freed row), a jump in length that forces
a rebuild, deferred flushes, a repeated prompt restored from its prefix checkpoint - with the in-place
``output`` checked against the oracle that holds the same index."""

from types import SimpleNamespace as NS

import pytest
import torch

from helpers import assert_output_close
from oracle.pqhsa_oracle import OracleAttentionConfig, OracleIndex, OracleIndexConfig, OracleStream
from pqhsa_release_b200 import workloads

pytestmark = pytest.mark.gpu

HKV, G, BS, D = 2, 4, 16, 128
HQ = HKV * G
FRAC = 0.03


class Pages:
    """A paged KV cache in either vLLM layout with a block allocator and per-request token streams."""

    def __init__(self, layout, nblk=1400, max_blocks=400, dtype=torch.bfloat16):
        self.layout, self.dtype = layout, dtype
        if layout == "5d":
            self.kv = torch.zeros(2, nblk, BS, HKV, D, dtype=dtype, device="cuda")
        else:
            self.kv = torch.zeros(nblk, HKV, BS, 2 * D, dtype=dtype, device="cuda")
        self.free = torch.randperm(nblk, generator=torch.Generator().manual_seed(7)).tolist()
        self.max_blocks = max_blocks
        self.blocks: dict[str, list[int]] = {}
        self.len: dict[str, int] = {}
        self.k: dict[str, torch.Tensor] = {}   # host copies [Hkv, n, D] for the oracle
        self.v: dict[str, torch.Tensor] = {}

    def _store(self, rid, pos, k, v):  # k, v [n, Hkv, D] on the device
        n = k.shape[0]
        t = torch.arange(pos, pos + n, device="cuda")
        blk = torch.tensor(self.blocks[rid], device="cuda")[t // BS]
        if self.layout == "5d":
            self.kv[0, blk, t % BS] = k
            self.kv[1, blk, t % BS] = v
        else:
            self.kv[blk, :, t % BS, :D] = k
            self.kv[blk, :, t % BS, D:] = v

    def add_request(self, rid, keys, values):  # [Hkv, n, D]
        n = keys.shape[1]
        self.blocks[rid] = [self.free.pop() for _ in range((n + 200 + BS - 1) // BS)]
        self.len[rid] = n
        self.k[rid], self.v[rid] = keys.clone(), values.clone()
        self._store(rid, 0, keys.cuda().permute(1, 0, 2), values.cuda().permute(1, 0, 2))

    def append(self, rid, k, v, write):  # k, v [Hkv, D]; write=False: the hook stores the row itself
        pos = self.len[rid]
        if write:
            self._store(rid, pos, k.cuda()[None], v.cuda()[None])
        self.k[rid] = torch.cat([self.k[rid], k[:, None]], 1)
        self.v[rid] = torch.cat([self.v[rid], v[:, None]], 1)
        self.len[rid] = pos + 1

    def release(self, rid):
        self.free.extend(self.blocks.pop(rid))
        del self.len[rid], self.k[rid], self.v[rid]

    def metadata(self, batch, runner):
        table = torch.zeros(len(batch), self.max_blocks, dtype=torch.int32)
        slots = []
        for i, rid in enumerate(batch):
            b = self.blocks[rid]
            table[i, : len(b)] = torch.tensor(b, dtype=torch.int32)
            pos = self.len[rid] - 1            # the step's token
            slots.append(b[pos // BS] * BS + pos % BS)
        lens = torch.tensor([self.len[r] for r in batch], dtype=torch.int32)
        runner.input_batch.req_ids = list(batch)
        return NS(use_cascade=False, max_query_len=1, num_actual_tokens=len(batch), seq_lens=lens.cuda(),
                  seq_lens_cpu=lens, max_seq_len=int(lens.max()), block_table=table.cuda(),
                  slot_mapping=torch.tensor(slots, dtype=torch.long, device="cuda"), _pq_runner=runner)


def _oracle(eng, pages, rid, head):
    slot = eng.slots[rid]
    sidx = slot * HKV + head
    n = pages.len[rid]
    st = OracleStream(OracleIndexConfig(num_lists=eng.icfg.num_lists),
                      OracleAttentionConfig(sink_tokens=4, local_window=128, retrieval_top_fraction=FRAC,
                                            index_update_interval=10 ** 6, index_update_strategy="deferred"))
    st.keys, st.values, st.length = pages.k[rid][head].float(), pages.v[rid][head].float(), n
    st.indexed_length = int(eng.indexed_length[slot])
    e = eng.pool.export_stream_state(sidx)
    ix = OracleIndex(st.icfg)
    ix.packed, ix.list_ids = e.packed_codes.cpu(), e.list_ids.cpu()
    ix.norms, ix.coarse, ix.codebooks = e.key_norms.float().cpu(), e.coarse_centroids.float().cpu(), e.codebooks.float().cpu()
    st.index, st.value_means = ix, e.value_means.float().cpu()
    s, r = st.bounds()
    assert ix.num_vectors == r - s, (rid, head, ix.num_vectors, r - s)
    return st


@pytest.mark.parametrize("layout", ["5d", "4d"])
def test_hook_runs_a_changing_batch_for_44_steps(layout, monkeypatch):
    from pqhsa_release_b200.pq_hsa_vllm import runtime

    for k, v in {"PQ_HSA_BATCH": "1", "PQ_HSA_TOP_FRAC": str(FRAC), "PQ_HSA_NUM_LISTS": "64", "PQ_HSA_FLUSH_INTERVAL": "16",
                 "PQ_HSA_MAX_REQUESTS": "4", "PQ_HSA_MAX_CONTEXT": "8192", "PQ_HSA_ENABLE": "1",
                 "PQ_HSA_UPD_STRATEGY": "deferred", "PQ_HSA_FALLBACK": "0"}.items():
        monkeypatch.setenv(k, v)
    runtime.reset()
    dtype = torch.bfloat16
    pages = Pages(layout)
    ctx = {"A": 3000, "B": 5100, "C": 4000}
    data = {}
    for j, (rid, n) in enumerate(ctx.items()):
        k, v = workloads.mixture_kv(300 + j, HKV, n, dtype=dtype, components=16)
        data[rid] = (k, v, workloads.planted_queries(900 + j, k, G))
    data["D"] = data["C"]                      # the same prompt again
    prompts = {"A": [1, 2, 3], "B": [4, 5], "C": [6, 7, 8, 9], "D": [6, 7, 8, 9]}
    runner = NS(input_batch=NS(req_ids=[]), requests={r: NS(prompt_token_ids=p) for r, p in prompts.items()})
    impl = NS(scale=1.0 / D ** 0.5, num_heads=HQ, num_kv_heads=HKV, kv_cache_dtype="auto")
    layer = object()
    dense_calls = []

    def original(impl_, layer_, q, k, v, kv, md, output=None, **kw):
        dense_calls.append(q.shape[0])
        return output

    gen = torch.Generator().manual_seed(11)
    batch = []
    first_out = {}
    for step in range(44):
        if step == 0:
            for rid in ("A", "B"):
                pages.add_request(rid, data[rid][0], data[rid][1]); batch.append(rid)
        if step == 10:
            pages.add_request("C", data["C"][0], data["C"][1]); batch.append("C")
        if step == 20:                       # A ends: vLLM moves the tail request into its row
            pages.release("A"); batch = ["C", "B"]
        if step == 30:
            pages.add_request("D", data["D"][0], data["D"][1]); batch.append("D")
        jump = step == 25
        T = len(batch)
        nk = torch.randn(T, HKV, D, generator=gen).to(dtype)
        nv = torch.randn(T, HKV, D, generator=gen).to(dtype)
        if step == 30:                       # D's first decode token equals C's, so that its pages equal C's then
            nk[2], nv[2] = first_out["C_tok"]
        for i, rid in enumerate(batch):
            if jump and rid == "B":          # five tokens arrive outside the PQ path (a chunked prefill)
                for _ in range(5):
                    pages.append("B", torch.randn(HKV, D, generator=gen).to(dtype), torch.randn(HKV, D, generator=gen).to(dtype), True)
            pages.append(rid, nk[i], nv[i], write=(layout == "4d"))   # the 5-D layout is stored by the hook
        if step == 10:
            first_out["C_tok"] = (nk[2].clone(), nv[2].clone())
        q = torch.stack([(data[r][2].float() * (1 + 0.01 * step)).to(dtype) for r in batch]).cuda()   # [T, Hq, D]
        md = pages.metadata(batch, runner)
        out = torch.zeros(T, HQ * D, dtype=dtype, device="cuda")      # vLLM hands a [T, Hq * D] buffer
        res = runtime.pq_or_dense_forward(original, impl, layer, q, nk.cuda(), nv.cuda(), pages.kv, md, output=out)
        torch.cuda.synchronize()
        assert res is out and not dense_calls
        eng = runtime._LAYERS[id(layer)]
        o = out.view(T, HQ, D).float().cpu()
        assert bool(torch.isfinite(o).all())
        if step in (10, 30):
            key = "C" if step == 10 else "D"
            first_out[key] = o[2].clone()
        # (a request's deferred flush runs after the step's call, at steps 16, 26, 41 and 42: the state exported
        # after those steps is no longer the one their outputs were computed with)
        if step in (0, 5, 10, 15, 17, 20, 25, 27, 30, 31, 43):
            for i, rid in enumerate(batch):
                for h in range(HKV):
                    st = _oracle(eng, pages, rid, h)
                    det = st.forward_detail(q[i, h * G : (h + 1) * G].float().cpu())
                    for g in range(G):
                        # every element within its bf16 rounding + 5e-4 of the row's scale, as everywhere; the L2 bar over
                        # the ROUNDED rows is 3e-3 here: right after a flush a row whose fp32 value sits 3e-4 of the scale
                        # off the oracle's flips enough roundings to read 2.4e-3 (seen at step 27), without any element
                        # leaving its bound
                        assert_output_close(o[i, h * G + g], det.output[g], dtype, f"step {step} request {rid} head {h * G + g}",
                                            l2_bar=3e-3)
    s = runtime.STATS
    assert s["pq_steps"] == 44 and s["dense_steps"] == 0 and s["fallbacks"] == 0
    assert s["builds"] == 4, "A, B, C once each, B again after its jump"
    assert s["restores"] == 1, "D arrives with C's prompt and length: its index comes from the checkpoint"
    assert s["evictions"] == 1 and s["flushes"] >= 4
    assert s["kv_writes"] == (44 if layout == "5d" else 0)
    assert eng.stats["launch_calls"] == 44, "one library call per layer-step whatever the batch looks like"


def test_steps_the_pq_path_does_not_take_go_to_the_original_forward(monkeypatch):
    from pqhsa_release_b200.pq_hsa_vllm import runtime

    runtime.reset()
    monkeypatch.setenv("PQ_HSA_ENABLE", "1")
    monkeypatch.delenv("PQ_HSA_BATCH", raising=False)
    calls = []

    def original(impl_, layer_, q, k, v, kv, md, output=None, **kw):
        calls.append("dense")
        return output

    out = torch.zeros(1, HQ * D, device="cuda")
    prefill = NS(use_cascade=False, max_query_len=7, num_actual_tokens=7, seq_lens=torch.tensor([700]), max_seq_len=700)
    assert runtime.pq_or_dense_forward(original, None, object(), None, None, None, None, prefill, output=out) is out
    short = NS(use_cascade=False, max_query_len=1, num_actual_tokens=1, seq_lens=torch.tensor([60]), max_seq_len=60)
    runtime.pq_or_dense_forward(original, None, object(), None, None, None, None, short, output=out)
    assert calls == ["dense", "dense"] and runtime.STATS["dense_steps"] == 2
    # an error on the PQ path re-raises unless PQ_HSA_FALLBACK=1
    bad = NS(use_cascade=False, max_query_len=1, num_actual_tokens=1, seq_lens=torch.tensor([5000]), max_seq_len=5000)
    with pytest.raises(Exception):
        runtime.pq_or_dense_forward(original, NS(scale=1.0, num_heads=HQ, num_kv_heads=HKV), object(), None, None, None,
                                    None, bad, output=out)
    monkeypatch.setenv("PQ_HSA_FALLBACK", "1")
    runtime.pq_or_dense_forward(original, NS(scale=1.0, num_heads=HQ, num_kv_heads=HKV), object(), None, None, None, None,
                                bad, output=out)
    assert calls[-1] == "dense" and runtime.STATS["fallbacks"] == 1


@pytest.mark.parametrize("layout", ["5d", "4d"])
def test_speculative_steps_replay_in_order_and_roll_back(layout, monkeypatch):
    """PQ_HSA_MULTI_QUERY=1: a step of one request carries T = 3 query tokens at consecutive positions (the token
    the last step committed + two drafts).  Query j must see the prefix and the step's tokens up to its own
    (benchmarks/vllm_backend/pq_hsa_multi_query.py:14-60) - checked against the oracle holding the engine's index
    at every length - and after verification only 1 + a tokens survive: the next step starts at a lower position,
    overwrites the rejected rows in the pages, and the engine takes the length back without rebuilding anything.
    Single-token steps in between follow the same rule.  Deferred flushes run on committed tokens only."""
    from pqhsa_release_b200.pq_hsa_vllm import runtime

    for k, v in {"PQ_HSA_MULTI_QUERY": "1", "PQ_HSA_TOP_FRAC": str(FRAC), "PQ_HSA_NUM_LISTS": "64",
                 "PQ_HSA_FLUSH_INTERVAL": "8", "PQ_HSA_MAX_REQUESTS": "1", "PQ_HSA_MAX_CONTEXT": "8192",
                 "PQ_HSA_ENABLE": "1", "PQ_HSA_UPD_STRATEGY": "deferred", "PQ_HSA_FALLBACK": "0"}.items():
        monkeypatch.setenv(k, v)
    monkeypatch.delenv("PQ_HSA_BATCH", raising=False)
    runtime.reset()
    dtype = torch.bfloat16
    pages = Pages(layout)
    k0, v0 = workloads.mixture_kv(411, HKV, 3000, dtype=dtype, components=16)
    qbase = workloads.planted_queries(977, k0, G)
    pages.add_request("A", k0, v0)
    runner = NS(input_batch=NS(req_ids=["A"]), requests={"A": NS(prompt_token_ids=[1, 2, 3], num_prompt_tokens=2990)})
    impl = NS(scale=1.0 / D ** 0.5, num_heads=HQ, num_kv_heads=HKV, kv_cache_dtype="auto")
    layer = object()

    def original(*a, **kw):
        raise AssertionError("the step fell through to the dense path: " + str(runtime.rejects()))

    gen = torch.Generator().manual_seed(5)

    def run_step(T):
        """Append T tokens at the request's current length and run the hook; returns (queries, outputs, C)."""
        C = pages.len["A"]
        nk = torch.randn(T, HKV, D, generator=gen).to(dtype)
        nv = torch.randn(T, HKV, D, generator=gen).to(dtype)
        for j in range(T):
            pages.append("A", nk[j], nv[j], write=(layout == "4d"))
        b = pages.blocks["A"]
        table = torch.zeros(1, pages.max_blocks, dtype=torch.int32)
        table[0, : len(b)] = torch.tensor(b, dtype=torch.int32)
        slots = [b[(C + j) // BS] * BS + (C + j) % BS for j in range(T)]
        lens = torch.tensor([C + T], dtype=torch.int32)
        md = NS(use_cascade=False, max_query_len=T, num_actual_tokens=T, seq_lens=lens.cuda(), seq_lens_cpu=lens,
                max_seq_len=C + T, block_table=table.cuda(), slot_mapping=torch.tensor(slots, dtype=torch.long, device="cuda"),
                _pq_runner=runner)
        q = torch.stack([(qbase.float() * (1 + 0.01 * ((C + j) % 7))).to(dtype) for j in range(T)]).cuda()   # [T, Hq, D]
        out = torch.zeros(T, HQ * D, dtype=dtype, device="cuda")
        res = runtime.pq_or_dense_forward(original, impl, layer, q, nk.cuda(), nv.cuda(), pages.kv, md, output=out)
        torch.cuda.synchronize()
        assert res is out
        return q, out.view(T, HQ, D).float().cpu(), C

    def check(q, o, C, T):
        eng = runtime._LAYERS[id(layer)]
        full_len = pages.len["A"]
        for j in range(T):
            pages.len["A"] = C + j + 1                     # the oracle of query j sees the tokens up to its own
            for h in range(HKV):
                st = _oracle(eng, pages, "A", h)
                st.keys, st.values = st.keys[: C + j + 1], st.values[: C + j + 1]
                det = st.forward_detail(q[j, h * G : (h + 1) * G].float().cpu())
                for g in range(G):
                    assert_output_close(o[j, h * G + g], det.output[g], dtype, f"context {C} token {j} head {h * G + g}", l2_bar=3e-3)
        pages.len["A"] = full_len

    def keep(C, kept):
        """Verification keeps `kept` of the step's tokens: the request is C + kept tokens long."""
        pages.len["A"] = C + kept
        pages.k["A"], pages.v["A"] = pages.k["A"][:, : C + kept], pages.v["A"][:, : C + kept]

    q, o, C = run_step(1)                                  # a plain decode step installs the request
    check(q, o, C, 1)
    eng = runtime._LAYERS[id(layer)]
    compared = 0
    for it, kept in enumerate([3, 1, 2, 1, 3, 2, 1, 1, 2, 3, 1, 2]):
        T = 1 if it in (4, 9) else 3                       # single-token steps in between
        flushes = eng.stats["flushes"]
        q, o, C = run_step(T)
        assert bool(torch.isfinite(o).all())
        if eng.stats["flushes"] == flushes:                # a flush inside the step changes the index under the later queries
            check(q, o, C, T)
            compared += 1
        keep(C, min(kept, T))
    s = runtime.STATS
    assert s["dense_steps"] == 0 and s["fallbacks"] == 0 and s["builds"] == 1, "rejections never rebuild the index"
    assert s["mq_steps"] == 10 and s["mq_tokens"] == 30
    assert eng.stats["rollbacks"] >= 10 and eng.stats["flushes"] >= 1 and compared >= 6
    assert s["kv_writes"] == (13 if layout == "5d" else 0)
