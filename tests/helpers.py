"""Shared builders for the parity tests: the same seeded inputs go to the CPU
oracle (fp32 arithmetic on the stored element values) and to the CUDA path."""

from __future__ import annotations

import sys
from dataclasses import dataclass
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from oracle.pqhsa_oracle import OracleAttentionConfig, OracleIndexConfig, OracleStream  # noqa: E402
from pqhsa_release_b200 import workloads  # noqa: E402


def round_to(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Value of ``t`` after storage in ``dtype``, back in fp32."""
    return t.to(dtype).float()


@dataclass
class Case:
    B: int
    Hkv: int
    G: int
    S: int
    L: int
    dtype: torch.dtype
    frac: float
    sink: int
    local: int
    keys: torch.Tensor      # [B, Hkv, S, D] dtype
    values: torch.Tensor
    queries: torch.Tensor   # [B, Hkv*G, D] dtype
    streams: list           # OracleStream per (b, h), fp32 on stored values

    @property
    def num_streams(self) -> int:
        return self.B * self.Hkv


def make_case(B=1, Hkv=2, G=4, S=1500, L=64, dtype=torch.bfloat16, frac=0.02, sink=4, local=128, seed=0,
              interval=256, strategy="deferred", contexts=None, kind="mixture", components=16) -> Case:
    """Build inputs + one oracle stream per (request, KV head).  The oracle's index
    float tensors are rounded to ``dtype`` after the build: both sides then see the
    identical stored index."""
    D = 128
    keys = torch.empty(B, Hkv, S, D, dtype=dtype)
    values = torch.empty(B, Hkv, S, D, dtype=dtype)
    queries = torch.empty(B, Hkv * G, D, dtype=dtype)
    for b in range(B):
        if kind == "mixture":
            k, v = workloads.mixture_kv(seed * 1000 + b, Hkv, S, dtype=dtype, components=components)
            q = workloads.planted_queries(seed * 1000 + 500 + b, k, G)
        else:
            ks, vs, qs = [], [], []
            for h in range(Hkv):
                k1, v1, q1 = workloads.config0_stream(seed * 1000 + b * 17 + h, S)
                ks.append(k1.to(dtype)); vs.append(v1.to(dtype))
                g = torch.Generator().manual_seed(seed + 99 + h)
                qs.append(torch.stack([q1 + 0.3 * torch.randn(D, generator=g) for _ in range(G)]).to(dtype))
            k, v, q = torch.stack(ks), torch.stack(vs), torch.cat(qs)
        keys[b], values[b], queries[b] = k, v, q
    streams = []
    for b in range(B):
        for h in range(Hkv):
            n_ctx = S if contexts is None else contexts[b]
            st = OracleStream(
                OracleIndexConfig(num_lists=L),
                OracleAttentionConfig(sink_tokens=sink, local_window=local, retrieval_top_fraction=frac,
                                      index_update_interval=interval, index_update_strategy=strategy),
            ).build_cache(keys[b, h, :n_ctx].float(), values[b, h, :n_ctx].float())
            if st.index is not None:
                ix = st.index
                ix.coarse = round_to(ix.coarse, dtype)
                ix.codebooks = round_to(ix.codebooks, dtype)
                ix.norms = round_to(ix.norms, dtype)
                st.value_means = round_to(st.value_means, dtype)
            streams.append(st)
    return Case(B, Hkv, G, S, L, dtype, frac, sink, local, keys, values, queries, streams)


def pool_from_case(case: Case, device="cuda", tail_capacity=256, extra_slots=512, contexts=None, **kw):
    """DeviceIndexPool + contiguous KV cache holding ``case``."""
    from pqhsa_release_b200.device_index import DeviceIndexPool, StreamIndexTensors

    margin = extra_slots + 64
    pool = DeviceIndexPool(
        num_streams=case.num_streams, group=case.G, dtype=case.dtype, device=device,
        slot_capacity=case.S + extra_slots, num_lists=case.L, sink_tokens=case.sink, local_window=case.local,
        scale=1.0 / 128 ** 0.5, top_fraction=case.frac, tail_capacity=tail_capacity, **kw,
    )
    kc = torch.zeros(case.B, case.Hkv, case.S + margin, 128, dtype=case.dtype, device=device)
    vc = torch.zeros_like(kc)
    kc[:, :, : case.S] = case.keys.to(device)
    vc[:, :, : case.S] = case.values.to(device)
    pool.bind_kv_contiguous(kc, vc)
    for b in range(case.B):
        for h in range(case.Hkv):
            s = b * case.Hkv + h
            st = case.streams[s]
            idx = None
            if st.index is not None:
                from oracle.pqhsa_oracle import list_value_means

                ix = st.index
                s0, r0 = st.bounds()
                _, vsum, vcnt = list_value_means(ix.list_ids, st.values[s0:r0], ix.coarse.shape[0])
                idx = StreamIndexTensors(ix.packed, ix.list_ids, ix.norms, ix.coarse, ix.codebooks, st.value_means,
                                         vsum, vcnt)
            pool.load_stream(s, idx, seq_len=st.length, req=b, kv_head=h)
    return pool, kc, vc


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a - b| over max |b| (per tensor)."""
    a, b = a.float().cpu(), b.float().cpu()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


def topk_sets_match(approx_row: torch.Tensor, got: torch.Tensor, want: torch.Tensor, rtol: float = 0.0):
    """True if the index sets are equal, or differ only in members whose score is
    within ``rtol`` (relative to the row's spread) of the k-th value (ties / rounding
    at the boundary)."""
    g, w = set(got.tolist()), set(want.tolist())
    if g == w:
        return True, 0
    diff = (g ^ w)
    kth = approx_row[want].min()
    span = float(approx_row.max() - approx_row.min()) + 1e-30
    bad = [i for i in diff if abs(float(approx_row[i] - kth)) > rtol * span]
    return len(bad) == 0 and len(g) == len(w), len(diff)


# Output tolerance.  The stated bar is 2e-3 relative for a bf16 result.  A bf16
# (fp16) element carries a rounding error of up to 2^-8 (2^-11) of its own
# magnitude, so the check is: relative L2 error of the row <= 2e-3, and every
# element within its storage rounding plus 5e-4 of the row's largest magnitude.
# fp32 rows are held to 5e-4 of the largest magnitude (the merge removes the
# selected keys' approximate mass from the list sums, which leaves both sides with
# a cancellation error of that order on rows dominated by one key).
_HALF_ULP = {torch.float32: 0.0, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


L2_LOG: list = []   # (what, relative L2 error) of every checked row, for a look at the margins


def assert_output_close(got: torch.Tensor, want: torch.Tensor, dtype: torch.dtype, what: str = "", l2_bar: float = 2e-3) -> float:
    got, want = got.float().cpu(), want.float().cpu()
    scale = float(want.abs().max().clamp_min(1e-30))
    bound = _HALF_ULP[dtype] * want.abs() * 1.01 + 5e-4 * scale
    diff = (got - want).abs()
    assert bool((diff <= bound).all()), f"{what}: max excess {float((diff - bound).max())} (scale {scale})"
    # the reference's own result would be stored in `dtype` too: the L2 bar is taken
    # against the oracle rounded to the output type
    stored = want.to(dtype).float()
    l2 = float((got - stored).norm() / stored.norm().clamp_min(1e-30))
    L2_LOG.append((what, l2, float((got - want).norm() / want.norm().clamp_min(1e-30))))
    assert l2 <= l2_bar, f"{what}: relative L2 error {l2}"
    return l2
