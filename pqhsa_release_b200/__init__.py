"""B200-native (sm_100a) PQ-HSA per-step decode operator.

Host-side mirror of the reference's ``pq_hsa`` adapters and ``pq_hsa_vllm`` plugin
surface over ``libpqhsa_b200.so``.  Submodules are imported lazily so that
``import pqhsa_release_b200`` stays cheap and does not touch torch or CUDA.
"""

from __future__ import annotations

from typing import Any

__version__ = "0.1.0"

_LAZY = {
    "IVFPQConfig": "config",
    "SparseAttentionConfig": "config",
    "paper_index_config": "config",
    "paper_attention_config": "config",
    "DeviceIndexPool": "device_index",
    "StreamIndexTensors": "device_index",
    "IVFPQDecodeAttentionAdapter": "decode_adapter",
    "DecodeAttentionOutput": "decode_adapter",
    "GQASidecar": "gqa_sidecar",
}

__all__ = ["__version__", *_LAZY]


def __getattr__(name: str) -> Any:
    if name in _LAZY:
        from importlib import import_module

        return getattr(import_module(f"{__name__}.{_LAZY[name]}"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
