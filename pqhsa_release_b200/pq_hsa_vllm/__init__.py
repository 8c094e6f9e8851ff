"""vLLM general plugin for the B200 PQ-HSA decode operator: the entry point, the
``PQHSAConfig`` knobs and the worker class of the reference's ``pq_hsa_vllm``
package (pq_hsa_vllm/src/pq_hsa_vllm/__init__.py:35-48), over the CUDA library.

Imports are lazy: ``import pqhsa_release_b200.pq_hsa_vllm`` touches neither torch,
vLLM nor CUDA, so plugin discovery stays cheap.
"""

from __future__ import annotations

from typing import Any

__version__ = "0.1.0"

__all__ = ["__version__", "PQHSAConfig", "PQHSAWorker", "vllm_general_plugin", "install", "enabled"]


def __getattr__(name: str) -> Any:
    if name == "PQHSAConfig":
        from .config import PQHSAConfig

        return PQHSAConfig
    if name == "PQHSAWorker":
        from .worker import PQHSAWorker

        return PQHSAWorker
    if name in {"vllm_general_plugin", "install", "enabled"}:
        from . import plugin

        return getattr(plugin, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
