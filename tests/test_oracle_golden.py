"""The CPU oracle against the fixtures produced by the reference itself
(tests/golden/make_golden.py): index tensors and top-k sets bit for bit, floating
point results to 1e-6.  This is what pins the oracle."""

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE / "golden"))
sys.path.insert(0, str(HERE.parent))

from make_golden import CASES, case_inputs, checksum  # noqa: E402
from oracle.pqhsa_oracle import OracleAttentionConfig, OracleIndexConfig, OracleStream  # noqa: E402


def _load(name):
    return np.load(HERE / "golden" / f"golden_{name}.npz")


def _stream(name):
    kind, seed, ctx, lists, group, dtype, strategy, interval, appends = CASES[name]
    k, v, q, nk, nv = case_inputs(name)
    st = OracleStream(
        OracleIndexConfig(num_lists=lists),
        OracleAttentionConfig(sink_tokens=4, local_window=128, retrieval_top_fraction=0.02,
                              index_update_interval=interval, index_update_strategy=strategy),
    ).build_cache(k, v)
    return st, (k, v, q, nk, nv)


@pytest.mark.parametrize("name", sorted(CASES))
def test_inputs_are_the_ones_the_fixture_was_made_from(name):
    g = _load(name)
    assert checksum(*case_inputs(name)) == pytest.approx(float(g["input_checksum"]), rel=1e-12)


@pytest.mark.parametrize("name", sorted(CASES))
def test_index_build_is_bit_exact(name):
    g = _load(name)
    st, _ = _stream(name)
    ix = st.index
    assert np.array_equal(ix.packed.numpy(), g["packed_codes"])
    assert np.array_equal(ix.list_ids.numpy(), g["list_ids"])
    assert np.array_equal(ix.norms.numpy(), g["key_norms"])
    assert np.array_equal(ix.coarse.numpy(), g["coarse"])
    assert np.array_equal(ix.codebooks.numpy(), g["codebooks"])
    assert np.array_equal(st.value_means.numpy(), g["value_means"])


@pytest.mark.parametrize("name", sorted(CASES))
def test_scores_topk_and_output(name):
    g = _load(name)
    st, (k, v, q, nk, nv) = _stream(name)
    det = st.forward_detail(q)
    np.testing.assert_allclose(det.approx_logits.numpy(), g["approx_logits"], rtol=1e-6, atol=1e-6)
    assert np.array_equal(det.topk_local.numpy(), g["topk"])
    np.testing.assert_allclose(det.output.numpy(), g["output0"], rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("name", sorted(CASES))
def test_decode_steps_with_appends(name):
    kind, seed, ctx, lists, group, dtype, strategy, interval, appends = CASES[name]
    g = _load(name)
    st, (k, v, q, nk, nv) = _stream(name)
    for i in range(appends):
        st.append(nk[i], nv[i])
        if strategy == "deferred" and i == appends // 2:
            assert st.apply_pending_index_update()
        out = st.forward_many(q + 0.01 * i)
        np.testing.assert_allclose(out.numpy(), g["outputs_after_appends"][i], rtol=1e-6, atol=1e-6)
    ix = st.index
    assert np.array_equal(ix.packed.numpy(), g["packed_codes_end"])
    assert np.array_equal(ix.list_ids.numpy(), g["list_ids_end"])
    assert np.array_equal(ix.norms.numpy(), g["key_norms_end"])
    np.testing.assert_allclose(st.value_means.numpy(), g["value_means_end"], rtol=1e-6, atol=1e-7)
    assert np.array_equal(ix.coarse.numpy(), g["coarse_end"])
    assert np.array_equal(ix.codebooks.numpy(), g["codebooks_end"])


def test_packing_round_trip_and_word_layout():
    # nibble layout contract of the reference (tests/test_packing.py:7-43 there)
    from oracle.pqhsa_oracle import codes_as_u32, pack_nibbles, unpack_nibbles

    gen = torch.Generator().manual_seed(0)
    codes = torch.randint(0, 16, (257, 8), generator=gen)
    packed = pack_nibbles(codes)
    assert packed.dtype == torch.uint8 and packed.shape == (257, 4)
    assert torch.equal(unpack_nibbles(packed, 8), codes)
    w = codes_as_u32(packed)
    for s in range(8):
        assert torch.equal((w >> (4 * s)) & 15, codes[:, s])
    with pytest.raises(ValueError):
        pack_nibbles(torch.full((2, 8), 16))


def test_topk_count_is_ceil_in_double():
    # pq_hsa/attention/sparse_attention.py:1779-1783 (reference tests/test_sparse_attention.py:219-250)
    from oracle.pqhsa_oracle import resolve_topk

    assert resolve_topk(0, 0.02) == 0
    assert resolve_topk(8060, 0.02) == 162
    assert resolve_topk(130940, 0.02) == 2619
    assert resolve_topk(100, 1.0) == 100
    assert resolve_topk(5, None, 100) == 5


def test_production_flush_is_bit_exact():
    """The oracle's restatement of the production deferred flush (codebook EMA over the keys that left the
    local window, only those keys encoded, count-weighted value means: benchmarks/e2e_pq_param_sweep.py:3021-3344)
    against what the reference's own method produced on the same inputs (tests/golden/make_golden.py,
    ``production_flush``): every index tensor of every head, bit for bit."""
    from make_golden import FLUSH_CASE, flush_inputs

    from oracle.pqhsa_oracle import OracleAttentionConfig, OracleIndexConfig, OracleStream

    g = np.load(HERE / "golden" / "golden_flush_incremental.npz")
    K, V = flush_inputs()
    assert checksum(K, V) == pytest.approx(float(g["input_checksum"]), rel=1e-12)
    c = FLUSH_CASE
    S, U = c["context"], c["appends"]
    for h in range(c["heads"]):
        st = OracleStream(
            OracleIndexConfig(num_lists=c["lists"]),
            OracleAttentionConfig(sink_tokens=4, local_window=128, retrieval_top_fraction=0.05,
                                  index_update_interval=c["interval"], index_update_strategy="deferred"),
        ).build_cache(K[h, :S], V[h, :S])
        assert st.index.list_ids.numel() == int(g["old_indexed"])
        for t in range(U):
            st.append(K[h, S + t], V[h, S + t])
        assert st.deferred_pending and st.apply_pending_incremental_flush()
        ix = st.index
        assert ix.list_ids.numel() == int(g["old_indexed"]) + U
        assert np.array_equal(ix.packed.numpy(), g[f"packed_codes_{h}"])
        assert np.array_equal(ix.list_ids.numpy(), g[f"list_ids_{h}"])
        assert np.array_equal(ix.norms.numpy(), g[f"key_norms_{h}"])
        assert np.array_equal(ix.coarse.numpy(), g[f"coarse_{h}"])
        assert np.array_equal(ix.codebooks.numpy(), g[f"codebooks_{h}"])
        assert np.array_equal(st.value_means.numpy(), g[f"value_means_{h}"])
