"""CUDA decode step against the CPU oracle on the same seeded inputs (through the C ABI)."""

import pytest
import torch

from helpers import assert_output_close, make_case, pool_from_case, topk_sets_match

pytestmark = pytest.mark.gpu

SCORE_RTOL = 1e-3   # approximate logits: relative to the row's largest magnitude


def _check_case(case, pool, check_scores=True):
    dev = "cuda"
    q = case.queries.to(dev).reshape(case.num_streams, case.G, 128).contiguous()
    out = pool.decode_step(q)
    torch.cuda.synchronize()
    out = out.float().cpu()
    # row_info of the step (the scoring call below starts a new step and clears the counters)
    info = pool.ws_view("row_info").cpu().clone()
    scores = pool.scan_scores(q).cpu() if check_scores else None
    worst_out = 0.0
    for s, st in enumerate(case.streams):
        qs = case.queries.reshape(case.num_streams, case.G, 128)[s].float()
        det = st.forward_detail(qs)
        n = det.approx_logits.shape[1]
        if n:
            pos = pool.slot_pos[s, :n].long().cpu()
            sink_end, _ = st.bounds()
            local = pos - sink_end
        for g in range(case.G):
            row = s * case.G + g
            if n and check_scores:
                want = det.approx_logits[g]
                got = torch.empty_like(want)
                got[local] = scores[row, :n]
                tol = SCORE_RTOL * float(want.abs().max())
                assert float((got - want).abs().max()) <= tol
            k = det.topk_local.shape[1]
            assert int(info[row, 0]) == k
            if k:
                got_pos = pool.selected_positions(row).cpu()
                want_pos = torch.sort(det.topk_local[g] + sink_end).values
                ok, ndiff = topk_sets_match(
                    torch.cat([torch.zeros(sink_end), det.approx_logits[g]]), got_pos, want_pos, rtol=1e-5)
                assert ok, f"row {row}: {ndiff} members differ beyond boundary ties"
            err = assert_output_close(out[s, g], det.output[g], case.dtype, f"row {row}")
            worst_out = max(worst_out, err)
    return info


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("G", [1, 4, 8])
def test_decode_step_matches_oracle(dtype, G):
    case = make_case(B=1, Hkv=2, G=G, S=1800, L=64, dtype=dtype, seed=3)
    pool, _, _ = pool_from_case(case)
    _check_case(case, pool)


def test_batch_of_requests_and_group2():
    case = make_case(B=3, Hkv=2, G=2, S=1300, L=32, dtype=torch.bfloat16, seed=5)
    pool, _, _ = pool_from_case(case)
    _check_case(case, pool)


def test_config0_like_fp32_single_head():
    case = make_case(B=1, Hkv=1, G=1, S=4096, L=128, dtype=torch.float32, seed=0, kind="config0")
    pool, _, _ = pool_from_case(case)
    _check_case(case, pool)


def test_short_context_without_index_is_dense():
    # context <= sink + local: no retrieval region, the step is plain attention over all rows
    case = make_case(B=1, Hkv=2, G=4, S=100, L=16, dtype=torch.bfloat16, seed=7)
    assert all(st.index is None for st in case.streams)
    pool, _, _ = pool_from_case(case)
    _check_case(case, pool, check_scores=False)


def test_full_lists_512():
    case = make_case(B=1, Hkv=1, G=4, S=6000, L=512, dtype=torch.bfloat16, seed=11)
    pool, _, _ = pool_from_case(case)
    _check_case(case, pool)


def test_sampled_threshold_path_long_context():
    # more than 4096 indexed keys: the candidate threshold comes from the sample histogram
    case = make_case(B=1, Hkv=2, G=4, S=14000, L=256, dtype=torch.bfloat16, seed=13)
    pool, _, _ = pool_from_case(case)
    info = _check_case(case, pool)
    assert int(info[:, 4].sum()) == 0, "the exact fallback should not be needed at the default margin"
    k = int(info[0, 0])
    assert (info[:, 2] >= k).all() and (info[:, 2] < 8 * k + 4096).all(), "candidate count out of the expected range"


def test_forced_fallback_is_still_exact():
    # a negative margin puts the threshold above the K-th logit: too few candidates, so the
    # selection kernel must fall back to all keys and still return the exact top-K
    case = make_case(B=1, Hkv=1, G=4, S=9000, L=128, dtype=torch.bfloat16, seed=17)
    pool, _, _ = pool_from_case(case, select_margin=-9.0)
    info = _check_case(case, pool)
    assert int(info[:, 4].sum()) >= 1, "expected at least one row to take the fallback"
