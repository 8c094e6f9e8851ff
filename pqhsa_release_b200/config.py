"""Configuration types with the reference's field names and defaults.

``IVFPQConfig`` mirrors pq_hsa/index/ivfpq.py:84-101 and
``SparseAttentionConfig`` mirrors pq_hsa/attention/sparse_attention.py:15-37,
so that code written against the reference constructs them unchanged.  The
B200 path implements the production operating point
(benchmarks/vllm_backend/pq_hsa_decode_runtime.py:140-177): residual IVF-PQ over
unit directions, 8 subspaces x 4 bits, hybrid mode with per-list value means.
Anything else is rejected with a ``ValueError`` naming the field; there is no
silent fallback.
"""

from __future__ import annotations

from dataclasses import dataclass
from math import ceil, sqrt

ALLOWED_KERNEL_BACKENDS = {"auto", "torch", "triton", "h20", "b200"}


@dataclass(slots=True)
class IVFPQConfig:
    num_lists: int = 256
    nprobe: int = 8
    num_subspaces: int = 16
    num_bits: int = 8
    residual: bool = True
    coarse_max_iter: int = 30
    pq_max_iter: int = 25
    pack_codes: bool = True
    topk_block_size: int | None = None
    kernel_backend: str = "auto"   # accepted for compatibility; there is one backend
    rotation: str = "none"
    direction_normalize: bool = False
    online_codebook_lr: float = 0.05
    seed: int = 0
    eps: float = 1e-12


@dataclass(slots=True)
class SparseAttentionConfig:
    sink_tokens: int = 0
    local_window: int = 0
    retrieval_topk: int = 100
    retrieval_top_fraction: float | None = None
    retrieval_top_p: float | None = None
    retrieval_top_p_scope: str = "retrieval"
    nprobe: int | None = None
    candidate_budget: int | None = None
    exact_rerank: bool = True
    scale: float | None = None
    mode: str = "sparse"
    hybrid_value_mode: str = "denominator"
    hybrid_topk_source: str = "all_pq"
    hybrid_denominator_source: str = "all_pq"
    index_update_interval: int = 1
    index_update_strategy: str = "incremental"
    codebook_refresh_interval: int | None = None
    kv_storage: str = "device"
    pin_offloaded_kv: bool = False
    prefetch_full_kv: bool = False
    collect_attention_details: bool = True
    profile_attention_components: bool = False


def paper_index_config(**overrides) -> IVFPQConfig:
    """Production index settings (benchmarks/vllm_backend/pq_hsa_decode_runtime.py:140-155)."""
    cfg = IVFPQConfig(
        num_lists=512, nprobe=64, num_subspaces=8, num_bits=4, residual=True, coarse_max_iter=1,
        pq_max_iter=2, pack_codes=True, topk_block_size=1024, kernel_backend="b200", rotation="none",
        direction_normalize=True, seed=0,
    )
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def paper_attention_config(scale: float | None = None, **overrides) -> SparseAttentionConfig:
    """Production operator settings (benchmarks/vllm_backend/pq_hsa_decode_runtime.py:158-177)."""
    cfg = SparseAttentionConfig(
        sink_tokens=4, local_window=128, retrieval_topk=100, retrieval_top_fraction=0.01, nprobe=64,
        candidate_budget=4096, exact_rerank=True, scale=scale, mode="hybrid", hybrid_value_mode="centroid",
        hybrid_topk_source="all_pq", hybrid_denominator_source="all_pq", index_update_interval=256,
        index_update_strategy="deferred", kv_storage="device", collect_attention_details=False,
        profile_attention_components=False,
    )
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def validate_index_config(cfg: IVFPQConfig) -> None:
    """Same checks as IVFPQIndex.__init__ (pq_hsa/index/ivfpq.py:151-160) plus the
    shape this library is built for."""
    if cfg.topk_block_size is not None and cfg.topk_block_size <= 0:
        raise ValueError("topk_block_size must be positive when provided")
    if cfg.kernel_backend not in ALLOWED_KERNEL_BACKENDS:
        raise ValueError("kernel_backend must be 'auto', 'torch', 'triton', 'h20' or 'b200'")
    if cfg.rotation not in {"none", "random_orthogonal"}:
        raise ValueError("rotation must be 'none' or 'random_orthogonal'")
    if not (0.0 < cfg.online_codebook_lr <= 1.0):
        raise ValueError("online_codebook_lr must be in (0, 1]")
    if cfg.num_subspaces != 8 or cfg.num_bits != 4:
        raise ValueError("the B200 kernels are built for num_subspaces=8, num_bits=4")
    if not (1 <= cfg.num_lists <= 512):
        raise ValueError("num_lists must be in 1..512")
    if not cfg.residual or not cfg.direction_normalize or cfg.rotation != "none" or not cfg.pack_codes:
        raise ValueError(
            "the B200 kernels implement residual=True, direction_normalize=True, rotation='none', pack_codes=True"
        )


def validate_attention_config(cfg: SparseAttentionConfig) -> None:
    """Checks of IVFPQSparseAttention.__init__ (pq_hsa/attention/sparse_attention.py:103-140)
    restricted to the production mode."""
    if cfg.mode not in {"sparse", "hybrid"}:
        raise ValueError("mode must be 'sparse' or 'hybrid'")
    if cfg.index_update_strategy not in {"incremental", "online", "rebuild", "deferred"}:
        raise ValueError("index_update_strategy must be 'incremental', 'online', 'rebuild', or 'deferred'")
    if cfg.index_update_interval <= 0:
        raise ValueError("index_update_interval must be positive")
    if cfg.sink_tokens < 0 or cfg.local_window < 0:
        raise ValueError("sink_tokens and local_window must be non-negative")
    if (
        cfg.mode != "hybrid"
        or cfg.hybrid_value_mode != "centroid"
        or cfg.hybrid_topk_source != "all_pq"
        or cfg.hybrid_denominator_source != "all_pq"
        or not cfg.exact_rerank
        or cfg.retrieval_top_p is not None
        or cfg.collect_attention_details
    ):
        raise ValueError(
            "the B200 kernels implement mode='hybrid', hybrid_value_mode='centroid', all_pq top-k and "
            "denominator, exact_rerank=True, no top-p, collect_attention_details=False"
        )
    if cfg.kv_storage != "device":
        raise ValueError("kv_storage must be 'device': there is no CPU path")
    if getattr(cfg, "codebook_refresh_interval", None) is not None:
        raise ValueError("codebook_refresh_interval is not supported: the B200 path has no warm-start retrain "
                         "(pq_hsa/attention/kv_cache.py:276-314); leave it None")


def resolve_topk(retrieval_len: int, cfg: SparseAttentionConfig) -> int:
    """min(max(ceil(N * fraction), 0), N) in Python floats
    (pq_hsa/attention/sparse_attention.py:1756-1783)."""
    if retrieval_len == 0:
        return 0
    if cfg.retrieval_top_fraction is not None:
        k = ceil(retrieval_len * cfg.retrieval_top_fraction)
    else:
        k = cfg.retrieval_topk
    return min(max(k, 0), retrieval_len)


def softmax_scale(cfg: SparseAttentionConfig, head_dim: int) -> float:
    return (1.0 / sqrt(head_dim)) if cfg.scale is None else float(cfg.scale)
