"""Pool-level GPU parity through the C ABI: golden fixtures of the reference, ragged
batches, the unsorted tail with incremental encoding, and the stand-alone top-k."""

import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import assert_output_close, make_case, pool_from_case, topk_sets_match

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE / "golden"))
from make_golden import CASES, case_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["c0_fp32", "mix_bf16"])
def test_cuda_path_reproduces_the_reference_fixture(name):
    """Index tensors exactly as the reference built them -> scores, top-k set and output of
    the reference's own forward_many."""
    from pqhsa_release_b200.device_index import DeviceIndexPool, StreamIndexTensors

    kind, seed, ctx, lists, group, dtype, strategy, interval, appends = CASES[name]
    g = np.load(HERE / "golden" / f"golden_{name}.npz")
    k, v, q, nk, nv = case_inputs(name)
    # the fixture is fp32 throughout (the reference ran in fp32 on values representable in `dtype`)
    dt = torch.float32
    G = 4 if group == 4 else 1
    rows = q[:G] if group >= G else q
    pool = DeviceIndexPool(num_streams=1, group=G, dtype=dt, device="cuda", slot_capacity=ctx + 64,
                           num_lists=lists, sink_tokens=4, local_window=128, scale=128 ** -0.5, top_fraction=0.02)
    kc = torch.zeros(1, 1, ctx + 64, 128, dtype=dt, device="cuda")
    vc = torch.zeros_like(kc)
    kc[0, 0, :ctx], vc[0, 0, :ctx] = k.cuda(), v.cuda()
    pool.bind_kv_contiguous(kc, vc)
    idx = StreamIndexTensors(torch.from_numpy(g["packed_codes"]), torch.from_numpy(g["list_ids"]).long(),
                             torch.from_numpy(g["key_norms"]), torch.from_numpy(g["coarse"]),
                             torch.from_numpy(g["codebooks"]), torch.from_numpy(g["value_means"]))
    pool.load_stream(0, idx, seq_len=ctx, req=0, kv_head=0)
    qd = rows.cuda().reshape(1, G, 128).contiguous()
    out = pool.decode_step(qd)
    torch.cuda.synchronize()
    n = g["approx_logits"].shape[1]
    pos = pool.slot_pos[0, :n].long().cpu() - 4
    scores = pool.scan_scores(qd).cpu()
    for r in range(G):
        want = torch.from_numpy(g["approx_logits"][r])
        got = torch.empty_like(want)
        got[pos] = scores[r, :n]
        assert float((got - want).abs().max()) <= 1e-3 * float(want.abs().max())
        sel = pool.selected_positions(r).cpu()
        ok, nd = topk_sets_match(torch.cat([torch.zeros(4), want]), sel, torch.sort(torch.from_numpy(g["topk"][r]) + 4).values,
                                 rtol=1e-5)
        assert ok, f"{nd} members differ beyond boundary ties"
        assert_output_close(out[0, r].cpu(), torch.from_numpy(g["output0"][r]), dt, f"row {r}")


def test_ragged_batch_of_requests():
    """Requests of different context lengths in one launch (one index per stream, per-stream counts)."""
    ctxs = [700, 2600, 1500, 140]
    case = make_case(B=4, Hkv=2, G=4, S=2600, L=64, dtype=torch.bfloat16, seed=21, contexts=ctxs)
    pool, _, _ = pool_from_case(case)
    q = case.queries.cuda().reshape(case.num_streams, 4, 128).contiguous()
    out = pool.decode_step(q).float().cpu()
    info = pool.ws_view("row_info").cpu()
    for s, st in enumerate(case.streams):
        det = st.forward_detail(case.queries.reshape(case.num_streams, 4, 128)[s].float())
        for g in range(4):
            assert int(info[s * 4 + g, 0]) == det.topk_local.shape[1]
            assert_output_close(out[s, g], det.output[g], case.dtype, f"stream {s} row {g}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_incremental_encode_matches_the_oracle(dtype):
    """append_kv + append_encode against IVFPQIndex.add semantics: list ids and codes bit for bit
    (a differing assignment must be a numerical tie), norms and value means to storage precision,
    and the step after each append against the oracle that holds the same index."""
    from helpers import round_to

    case = make_case(B=1, Hkv=2, G=2, S=900, L=32, dtype=dtype, seed=23, interval=1, strategy="incremental")
    pool, kc, vc = pool_from_case(case)
    gen = torch.Generator().manual_seed(5)
    mism = total = 0
    for step in range(12):
        nk = (case.keys[0, :, step * 7 + 3].float() + 0.3 * torch.randn(2, 128, generator=gen)).to(dtype)
        nv = torch.randn(2, 128, generator=gen).to(dtype)
        pool.append_kv(nk.cuda().contiguous(), nv.cuda().contiguous())
        pool.append_encode(1)
        torch.cuda.synchronize()
        for s, st in enumerate(case.streams):
            n_before = st.index.num_vectors
            st.append(nk[s].float(), nv[s].float())      # the oracle encodes the key that left the window
            assert st.index.num_vectors == n_before + 1
            # storage rounding of what the oracle appended, as the device stores it
            st.index.norms[-1] = round_to(st.index.norms[-1:], dtype)[0]
            dev = pool.export_stream(s)
            total += 1
            same = int(dev["list_ids"][-1]) == int(st.index.list_ids[-1]) and torch.equal(
                dev["packed_codes"][-1].cpu(), st.index.packed[-1])
            if not same:
                mism += 1
                # adopt the device's assignment so that later steps compare like with like
                st.index.list_ids[-1] = int(dev["list_ids"][-1])
                st.index.packed[-1] = dev["packed_codes"][-1].cpu()
            assert abs(float(dev["key_norms"][-1]) - float(st.index.norms[-1])) <= 1e-6 * float(st.index.norms[-1]) + (
                0 if dtype == torch.float32 else 1e-2 * float(st.index.norms[-1]))
            assert int(dev["positions"][-1]) == 4 + st.index.num_vectors - 1
            # value means: device keeps fp32 running sums and stores the mean in `dtype`
            lists = st.index.coarse.shape[0]
            vm_dev = pool.vmeans[s, :lists].float().cpu()
            from oracle.pqhsa_oracle import list_value_means

            s0, r0 = st.bounds()
            vm, _, _ = list_value_means(st.index.list_ids, st.values[s0:r0], lists)
            assert float((vm_dev - vm).abs().max()) <= (1e-5 if dtype == torch.float32 else 2e-2)
            st.value_means = vm_dev.clone()
        q = (case.queries.float() + 0.05 * step).to(dtype)
        out = pool.decode_step(q.cuda().reshape(2, 2, 128).contiguous()).float().cpu()
        for s, st in enumerate(case.streams):
            det = st.forward_detail(q.reshape(2, 2, 128)[s].float())
            for g in range(2):
                assert_output_close(out[s, g], det.output[g], dtype, f"step {step} stream {s} row {g}")
    assert mism <= max(1, total // 20), f"{mism} of {total} encodes differ from the oracle"
    # folding the tail into the sorted region changes nothing
    q = case.queries.cuda().reshape(2, 2, 128).contiguous()
    before = pool.decode_step(q).float().cpu()
    pool.compact()
    assert int(pool.h_tail.max()) == 0
    after = pool.decode_step(q).float().cpu()
    assert float((before - after).abs().max()) <= 2e-2 * float(before.abs().max())


def test_standalone_topk_radix_against_torch_topk():
    from pqhsa_release_b200 import _lib

    gen = torch.Generator().manual_seed(3)
    for n, k in [(5000, 100), (131, 131), (4096, 1), (70000, 1400)]:
        x = torch.randn(3, n, generator=gen)
        x[1, : n // 2] = x[1, : n // 2].round()          # many exact ties
        xd = x.cuda()
        idx = torch.full((3, k), -1, dtype=torch.int32, device="cuda")
        val = torch.zeros(3, k, device="cuda")
        _lib.call("pqhsa_topk_radix", xd.data_ptr(), 3, n, n, k, idx.data_ptr(), val.data_ptr(),
                  torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        ref = torch.topk(x, k, dim=1)
        for r in range(3):
            got = idx[r].cpu().long()
            assert len(set(got.tolist())) == k and int(got.min()) >= 0
            # same multiset of values (ties may pick different members), values match the indices
            assert torch.equal(torch.sort(x[r][got]).values, torch.sort(ref.values[r]).values)
            assert torch.equal(val[r].cpu(), x[r][got])
            # ties at the k-th value go to the lower index
            kth = ref.values[r].min()
            tied = torch.nonzero(x[r] == kth).flatten()
            chosen = sorted(i for i in got.tolist() if x[r, i] == kth)
            assert chosen == tied[: len(chosen)].tolist()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_step_equals_the_three_calls(dtype):
    """pqhsa_decode_step_append (append, encode and tables in one kernel) leaves the same index,
    counters and cache rows as append_kv + append_encode + decode_step, and the same output."""
    case = make_case(B=2, Hkv=2, G=4, S=5000, L=96, dtype=dtype, seed=21, interval=1, strategy="incremental")
    a, ka, va = pool_from_case(case)
    b, kb, vb = pool_from_case(case)
    gen = torch.Generator().manual_seed(5)
    q0 = case.queries.cuda().reshape(case.num_streams, case.G, 128).contiguous()
    for step in range(3):
        nk = torch.randn(case.num_streams, 128, generator=gen).to(dtype).cuda()
        nv = torch.randn(case.num_streams, 128, generator=gen).to(dtype).cuda()
        q = (q0.float() * (1 + 0.1 * step)).to(dtype).contiguous()
        a.append_kv(nk, nv)
        a.append_encode(1)
        want = a.decode_step(q)
        got = b.decode_step_append(q, nk, nv, encode=1)
        torch.cuda.synchronize()
        assert torch.equal(a.state, b.state)
        n = int(a.h_sorted[0] + a.h_tail[0])
        for name in ("codes", "norms", "list_ids", "slot_pos", "vmeans", "vsum", "vcnt", "norm_max"):
            assert torch.equal(getattr(a, name), getattr(b, name)), name
        assert torch.equal(ka, kb) and torch.equal(va, vb)
        ia, ib = a.ws_view("row_info"), b.ws_view("row_info")
        assert torch.equal(ia[:, :2], ib[:, :2]) and int(ib[:, 4].sum()) == 0
        for row in range(case.num_streams * case.G):
            assert torch.equal(a.selected_positions(row), b.selected_positions(row))
        assert float((got.float() - want.float()).abs().max()) <= 2e-3 * float(want.float().abs().max())
        assert n == 5000 - 4 - 128 + step + 1


def test_paged_ragged_batch_64_decode_steps():
    """The shape of the plugin workload (16-token pages, permuted block table, requests of different
    lengths, 64 consecutive decode steps each appending one K/V row per head and encoding the key
    that leaves the local window), contexts scaled down so that the CPU oracle can follow every step.
    The library writes the new rows into the pages itself (fused step).  Codes and list ids of every
    encoded key bit for bit (a differing assignment must be a rare numerical tie), outputs against
    the oracle every 8 steps and at the end."""
    from helpers import round_to
    from pqhsa_release_b200.device_index import DeviceIndexPool, StreamIndexTensors
    from oracle.pqhsa_oracle import list_value_means

    dtype, Hkv, G, bs, steps = torch.bfloat16, 2, 4, 16, 64
    ctxs = [5200, 6900, 4700]
    B, smax = len(ctxs), max(ctxs)
    case = make_case(B=B, Hkv=Hkv, G=G, S=smax, L=128, dtype=dtype, seed=41, interval=1, strategy="incremental",
                     contexts=ctxs)
    dev = "cuda"
    blocks_per_req = (smax + steps + bs - 1) // bs
    nblk = B * blocks_per_req + 7
    gen = torch.Generator().manual_seed(3)
    table = torch.randperm(nblk, generator=gen)[: B * blocks_per_req].to(torch.int32).reshape(B, blocks_per_req).to(dev)
    kv_cache = torch.zeros(2, nblk, bs, Hkv, 128, dtype=dtype, device=dev)
    for b, n in enumerate(ctxs):
        t = torch.arange(n, device=dev)
        blk, off = table[b, t // bs].long(), t % bs
        kv_cache[0, blk, off] = case.keys[b, :, :n].to(dev).permute(1, 0, 2)
        kv_cache[1, blk, off] = case.values[b, :, :n].to(dev).permute(1, 0, 2)
    pool = DeviceIndexPool(num_streams=B * Hkv, group=G, dtype=dtype, device=dev, slot_capacity=smax + steps + 64,
                           num_lists=case.L, sink_tokens=case.sink, local_window=case.local, scale=1.0 / 128 ** 0.5,
                           top_fraction=case.frac, tail_capacity=steps + 8)
    pool.bind_kv_paged(kv_cache, table)
    for b in range(B):
        for h in range(Hkv):
            st = case.streams[b * Hkv + h]
            ix = st.index
            s0, r0 = st.bounds()
            _, vsum, vcnt = list_value_means(ix.list_ids, st.values[s0:r0], ix.coarse.shape[0])
            pool.load_stream(b * Hkv + h, StreamIndexTensors(ix.packed, ix.list_ids, ix.norms, ix.coarse, ix.codebooks,
                                                              st.value_means, vsum, vcnt),
                             seq_len=st.length, req=b, kv_head=h)
    S = B * Hkv
    q0 = case.queries.reshape(S, G, 128)
    mism = total = 0
    for step in range(steps):
        nk = (torch.randn(S, 128, generator=gen) * 1.5).to(dtype)
        nv = torch.randn(S, 128, generator=gen).to(dtype)
        q = (q0.float() * (1.0 + 0.01 * step) + 0.02 * torch.randn(S, G, 128, generator=gen)).to(dtype)
        out = pool.decode_step_append(q.to(dev).contiguous(), nk.to(dev).contiguous(), nv.to(dev).contiguous(), encode=1)
        torch.cuda.synchronize()
        for s, st in enumerate(case.streams):
            st.append(nk[s].float(), nv[s].float())
            st.index.norms[-1] = round_to(st.index.norms[-1:], dtype)[0]
            d = pool.export_stream(s)
            total += 1
            if int(d["list_ids"][-1]) != int(st.index.list_ids[-1]) or not torch.equal(d["packed_codes"][-1].cpu(), st.index.packed[-1]):
                mism += 1
                st.index.list_ids[-1] = int(d["list_ids"][-1])
                st.index.packed[-1] = d["packed_codes"][-1].cpu()
            lists = st.index.coarse.shape[0]
            st.value_means = pool.vmeans[s, :lists].float().cpu().clone()
            assert int(pool.state[s, 2]) == st.length  # SEQ_LEN on the device
        if step % 8 == 7 or step == steps - 1:
            o = out.float().cpu()
            for s, st in enumerate(case.streams):
                det = st.forward_detail(q[s].float())
                for g in range(G):
                    assert_output_close(o[s, g], det.output[g], dtype, f"step {step} stream {s} row {g}")
    assert mism <= max(1, total // 20), f"{mism} of {total} encodes differ from the oracle"
    # the rows the library wrote are in the pages
    b, n = 1, ctxs[1] + steps
    t = torch.arange(ctxs[1], n, device=dev)
    assert bool((kv_cache[0, table[b, t // bs].long(), t % bs].float().abs().sum(-1) > 0).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_compact_kernel_equals_the_stable_sort(dtype):
    """pqhsa_compact folds the tails of all streams into their sorted regions in place, without a sort; the
    layout must be the one a stable sort by (list, token position) gives - every index array, the scan units,
    the slots' unit ids, the sample records and the counters, bit for bit - for ragged streams, a stream with
    an empty tail, and tails of different lengths (one longer than a chunk of 1024)."""
    import copy

    from pqhsa_release_b200 import _lib

    case = make_case(B=3, Hkv=2, G=2, S=6200, L=48, dtype=dtype, seed=37, interval=1, strategy="incremental",
                     contexts=[6200, 4300, 5000])
    pool, kc, vc = pool_from_case(case, tail_capacity=2048, extra_slots=2200)
    gen = torch.Generator().manual_seed(9)
    S = pool.S
    # tails of 1500, 700, 0, 40, 1100 and 1 keys: append rows for everybody, encode per-stream counts
    want = [1500, 700, 0, 40, 1100, 1]
    steps = max(want)
    for t in range(steps):
        nk = torch.randn(S, 128, generator=gen).to(dtype).cuda()
        nv = torch.randn(S, 128, generator=gen).to(dtype).cuda()
        pool.append_kv(nk, nv)
    for s0 in range(0, steps, 500):
        pool.append_encode([max(0, min(500, w - s0)) for w in want])
    torch.cuda.synchronize()
    assert pool.h_tail.tolist() == want
    # the same pool compacted by the sort
    ref = copy.copy(pool)
    for name in ("codes", "norms", "list_ids", "slot_pos", "slot_unit", "unit_off", "unit_list", "state", "sample"):
        setattr(ref, name, getattr(pool, name).clone())
    ref.h_sorted, ref.h_tail = pool.h_sorted.copy(), pool.h_tail.copy()
    ref._compact_by_sort()
    pool.compact()
    torch.cuda.synchronize()
    assert not pool.compact_failed()
    assert pool.h_tail.tolist() == [0] * S and pool.h_sorted.tolist() == ref.h_sorted.tolist()
    assert torch.equal(pool.state, ref.state)
    for s in range(S):
        n = int(pool.h_sorted[s])
        u = int(pool.state[s, _lib.ST_N_UNITS])
        for name in ("codes", "norms", "list_ids", "slot_pos", "slot_unit"):
            assert torch.equal(getattr(pool, name)[s, :n], getattr(ref, name)[s, :n]), f"stream {s}: {name}"
        assert torch.equal(pool.unit_off[s, : u + 1], ref.unit_off[s, : u + 1]), f"stream {s}: unit_off"
        assert torch.equal(pool.unit_list[s, :u], ref.unit_list[s, :u]), f"stream {s}: unit_list"
        if n > _lib.SAMPLE_KEYS:
            assert torch.equal(pool.sample[s], ref.sample[s]), f"stream {s}: sample records"
    # the rest of the appended keys, a second compaction, and the step on the compacted pool against the
    # same pool before the compaction (the selection is exact either way)
    for s0 in range(0, steps, 500):
        pool.append_encode([max(0, min(500, (steps - w) - s0)) for w in want])
    q = case.queries.cuda().reshape(S, case.G, 128).contiguous()
    before = pool.decode_step(q).float().cpu()
    pool.compact()
    after = pool.decode_step(q).float().cpu()
    torch.cuda.synchronize()
    assert not pool.compact_failed() and int(pool.h_tail.max()) == 0
    assert float((before - after).abs().max()) <= 2e-2 * float(before.abs().max())
