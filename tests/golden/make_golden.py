"""Generate the golden fixtures of this directory by running the REFERENCE itself.

    python tests/golden/make_golden.py /path/to/reference

The reference package (pq_hsa) is imported from the given path and driven through
its own public API (IVFPQSparseAttention: build_cache / forward_many / append /
apply_pending_index_update) on small seeded inputs; what it computes is stored in
``golden_*.npz`` beside this script.  The inputs are not stored: they come from
``pqhsa_release_b200.workloads`` with the seeds recorded in ``CASES`` and are
guarded by a checksum, so a drifting generator fails the tests loudly instead of
silently comparing different data.

The fixtures pin the CPU oracle (tests/test_oracle_golden.py) and, through the
stored index tensors, the CUDA path (tests/test_pool_gpu.py, tests/test_adapters_gpu.py).  Nothing here is
needed at test time except the .npz files.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
sys.path.insert(0, str(ROOT))

from pqhsa_release_b200 import workloads  # noqa: E402

# name -> (kind, seed, context, lists, group, dtype, strategy, interval, appends)
CASES = {
    "c0_fp32": ("config0", 0, 1700, 64, 3, "float32", "incremental", 1, 24),
    "mix_bf16": ("mixture", 1, 2300, 96, 4, "bfloat16", "incremental", 4, 24),
    "mix_deferred": ("mixture", 2, 1500, 48, 2, "bfloat16", "deferred", 8, 20),
}


def case_inputs(name: str):
    """(keys [S, D], values [S, D], queries [G, D], new_keys [A, D], new_values [A, D]) in fp32,
    holding values representable in the case dtype."""
    kind, seed, ctx, lists, group, dtype, strategy, interval, appends = CASES[name]
    dt = getattr(torch, dtype)
    if kind == "config0":
        k, v, q1 = workloads.config0_stream(seed, ctx)
        g = torch.Generator().manual_seed(seed + 99)
        q = torch.stack([q1 + 0.3 * torch.randn(128, generator=g) for _ in range(group)])
    else:
        kk, vv = workloads.mixture_kv(seed, 1, ctx, dtype=dt, components=16)
        k, v = kk[0].float(), vv[0].float()
        q = workloads.planted_queries(seed + 500, kk, group).float()
    g = torch.Generator().manual_seed(seed + 7)
    nk = (k[torch.randint(0, ctx, (appends,), generator=g)] + 0.5 * torch.randn(appends, 128, generator=g))
    nv = torch.randn(appends, 128, generator=g)
    rd = lambda t: t.to(dt).float()
    return rd(k), rd(v), rd(q), rd(nk), rd(nv)


def checksum(*tensors) -> float:
    return float(sum(t.double().abs().sum() for t in tensors))


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from pq_hsa.attention.sparse_attention import IVFPQSparseAttention, SparseAttentionConfig
    from pq_hsa.index.ivfpq import IVFPQConfig

    for name, (kind, seed, ctx, lists, group, dtype, strategy, interval, appends) in CASES.items():
        k, v, q, nk, nv = case_inputs(name)
        ic = IVFPQConfig(num_lists=lists, nprobe=64, num_subspaces=8, num_bits=4, residual=True, coarse_max_iter=1,
                         pq_max_iter=2, pack_codes=True, topk_block_size=1024, kernel_backend="torch",
                         rotation="none", direction_normalize=True, seed=0)
        ac = SparseAttentionConfig(sink_tokens=4, local_window=128, retrieval_top_fraction=0.02, exact_rerank=True,
                                   mode="hybrid", hybrid_value_mode="centroid", hybrid_topk_source="all_pq",
                                   hybrid_denominator_source="all_pq", index_update_interval=interval,
                                   index_update_strategy=strategy, collect_attention_details=False)
        att = IVFPQSparseAttention(ic, ac).build_cache(k, v)
        idx = att.cache.index
        scale = 1.0 / 128 ** 0.5
        out = {
            "input_checksum": np.float64(checksum(k, v, q, nk, nv)),
            "packed_codes": idx.packed_codes.numpy().copy(),
            "list_ids": idx.list_ids.to(torch.int32).numpy().copy(),
            "key_norms": idx.key_norms.numpy().copy(),
            "coarse": idx.coarse_centroids.numpy().copy(),
            "codebooks": idx.pq.codebooks.numpy().copy(),
            "value_means": att.cache.retrieval_value_centroids.numpy().copy(),
        }
        approx = idx.approximate_scores(q) * scale
        out["approx_logits"] = approx.numpy().copy()
        kk = int(np.ceil(approx.shape[1] * 0.02))
        out["topk"] = torch.topk(approx, k=kk, dim=1, sorted=True).indices.numpy().copy()
        out["output0"] = torch.stack([o.output for o in att.forward_many(q)]).numpy().copy()
        # decode steps: append one token, attend with a rotating query
        outs = []
        for i in range(appends):
            att.append(nk[i], nv[i])
            if strategy == "deferred" and i == appends // 2:
                att.apply_pending_index_update()
            outs.append(torch.stack([o.output for o in att.forward_many(q + 0.01 * i)]))
        idx = att.cache.index
        out["outputs_after_appends"] = torch.stack(outs).numpy().copy()
        out["packed_codes_end"] = idx.packed_codes.numpy().copy()
        out["list_ids_end"] = idx.list_ids.to(torch.int32).numpy().copy()
        out["key_norms_end"] = idx.key_norms.numpy().copy()
        out["value_means_end"] = att.cache.retrieval_value_centroids.numpy().copy()
        out["coarse_end"] = idx.coarse_centroids.numpy().copy()
        out["codebooks_end"] = idx.pq.codebooks.numpy().copy()
        np.savez_compressed(HERE / f"golden_{name}.npz", **out)
        print(name, "indexed", idx.num_vectors, "bytes", (HERE / f"golden_{name}.npz").stat().st_size)


def adapter_state(ref_root: str) -> None:
    """``golden_adapter_state.pt``: a checkpoint written by the reference's own decode adapter
    (``IVFPQDecodeAttentionAdapter.state_dict``, two heads, three appended tokens) with the queries it was then
    asked and the contexts it answered - the wire format the B200 adapter must load and emit."""
    sys.path.insert(0, ref_root)
    from pq_hsa.attention.decode_adapter import IVFPQDecodeAttentionAdapter
    from pq_hsa.attention.sparse_attention import SparseAttentionConfig
    from pq_hsa.index.ivfpq import IVFPQConfig

    dt = torch.bfloat16
    kk, vv = workloads.mixture_kv(77, 2, 520, dtype=dt, components=16)
    q = workloads.planted_queries(78, kk, 1).float()[None]            # [1, 2, 128]
    ic = IVFPQConfig(num_lists=32, nprobe=64, num_subspaces=8, num_bits=4, residual=True, coarse_max_iter=1, pq_max_iter=2,
                     pack_codes=True, topk_block_size=1024, kernel_backend="torch", rotation="none",
                     direction_normalize=True, seed=0)
    ac = SparseAttentionConfig(sink_tokens=4, local_window=128, retrieval_top_fraction=0.05, exact_rerank=True, mode="hybrid",
                               hybrid_value_mode="centroid", hybrid_topk_source="all_pq", hybrid_denominator_source="all_pq",
                               index_update_interval=1, index_update_strategy="incremental", collect_attention_details=False)
    ad = IVFPQDecodeAttentionAdapter(ic, ac).build_cache(kk.float()[None], vv.float()[None])
    g = torch.Generator().manual_seed(79)
    for _ in range(3):
        ad.append(torch.randn(1, 2, 128, generator=g).to(dt).float(), torch.randn(1, 2, 128, generator=g).to(dt).float())
    out = ad.forward(q).context
    state = ad.state_dict()
    for st in state["attention"]["streams"]:
        # the K/V rows hold bf16-representable values: stored as bf16 (lossless) to keep the fixture small;
        # the test widens them to the float32 the reference wrote
        st["keys"], st["values"] = st["keys"].to(dt), st["values"].to(dt)
    torch.save({"state": state, "queries": q, "context": out}, HERE / "golden_adapter_state.pt")
    print("adapter state bytes", (HERE / "golden_adapter_state.pt").stat().st_size)


FLUSH_CASE = dict(seed=91, heads=2, context=1400, appends=37, lists=48, interval=32)


def flush_inputs():
    """(keys [H, S + U, D], values) in fp32 holding bf16-representable values."""
    c = FLUSH_CASE
    kk, vv = workloads.mixture_kv(c["seed"], c["heads"], c["context"] + c["appends"], dtype=torch.bfloat16, components=16)
    return kk.float(), vv.float()


def production_flush(ref_root: str) -> None:
    """``golden_flush_incremental.npz``: the PRODUCTION deferred flush of the reference
    (``GQAIVFPQDecodeAttentionAdapter._apply_pending_batched`` with PQ_HSA_INCREMENTAL_FLUSH=1,
    benchmarks/e2e_pq_param_sweep.py:3021-3344) run on CPU tensors.  The method itself has no device test;
    what keeps it off the CPU in the reference is that only the CUDA decode path fills the shared K/V
    buffers it reads.  Here the adapter is built by the reference's own CPU path (one stream per head),
    tokens are appended until the deferred update is pending, and the shared buffers are then set to the
    very K/V rows the streams hold - after which the unmodified method runs.  ``datasets`` is not
    installed in the build container and is stubbed for the import of the benchmark module (nothing on
    this path calls it)."""
    import types

    sys.path.insert(0, ref_root)
    if "datasets" not in sys.modules:
        stub = types.ModuleType("datasets")
        stub.load_dataset = lambda *a, **k: None
        sys.modules["datasets"] = stub
    os.environ["PQ_HSA_INCREMENTAL_FLUSH"] = "1"
    from benchmarks.e2e_pq_param_sweep import GQAIVFPQDecodeAttentionAdapter
    from pq_hsa.attention.sparse_attention import SparseAttentionConfig
    from pq_hsa.index.ivfpq import IVFPQConfig

    c = FLUSH_CASE
    H, S, U = c["heads"], c["context"], c["appends"]
    K, V = flush_inputs()
    ic = IVFPQConfig(num_lists=c["lists"], nprobe=64, num_subspaces=8, num_bits=4, residual=True, coarse_max_iter=1,
                     pq_max_iter=2, pack_codes=True, topk_block_size=1024, kernel_backend="torch", rotation="none",
                     direction_normalize=True, seed=0)
    ac = SparseAttentionConfig(sink_tokens=4, local_window=128, retrieval_top_fraction=0.05, exact_rerank=True,
                               mode="hybrid", hybrid_value_mode="centroid", hybrid_topk_source="all_pq",
                               hybrid_denominator_source="all_pq", index_update_interval=c["interval"],
                               index_update_strategy="deferred", collect_attention_details=False)
    ad = GQAIVFPQDecodeAttentionAdapter(ic, ac, num_query_heads=2 * H, num_key_value_heads=H)
    ad.build_cache(K[None, :, :S], V[None, :, :S])
    for t in range(U):
        ad.append(K[None, :, S + t], V[None, :, S + t])
    caches = [s.cache for s in ad._streams]
    assert all(bool(x._deferred_index_update_pending) for x in caches)
    ad._shared_base_keys, ad._shared_base_vals, ad._shared_base_fallback = K.clone(), V.clone(), False
    for h, x in enumerate(caches):
        x._key_buf, x._val_buf = ad._shared_base_keys[h], ad._shared_base_vals[h]
    old_n = int(caches[0].index.num_vectors)
    assert ad._apply_pending_batched() == H, "the batched flush refused its preconditions"
    out = {"input_checksum": np.float64(checksum(K, V)), "old_indexed": np.int64(old_n)}
    for h, x in enumerate(caches):
        ix = x.index
        out[f"packed_codes_{h}"] = ix.packed_codes.numpy().copy()
        out[f"list_ids_{h}"] = ix.list_ids.to(torch.int32).numpy().copy()
        out[f"key_norms_{h}"] = ix.key_norms.numpy().copy()
        out[f"coarse_{h}"] = ix.coarse_centroids.numpy().copy()
        out[f"codebooks_{h}"] = ix.pq.codebooks.numpy().copy()
        out[f"value_means_{h}"] = x.retrieval_value_centroids.numpy().copy()
    np.savez_compressed(HERE / "golden_flush_incremental.npz", **out)
    print("production flush: indexed", old_n, "->", int(caches[0].index.num_vectors), "bytes",
          (HERE / "golden_flush_incremental.npz").stat().st_size)


if __name__ == "__main__":
    adapter_state(sys.argv[1] if len(sys.argv) > 1 else os.environ["PQHSA_REFERENCE"])
    production_flush(sys.argv[1] if len(sys.argv) > 1 else os.environ["PQHSA_REFERENCE"])
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["PQHSA_REFERENCE"])  # a checkout of the reference
