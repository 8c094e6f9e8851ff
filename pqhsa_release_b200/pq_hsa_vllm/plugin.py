"""``vllm.general_plugins`` entry point and installer
(pq_hsa_vllm/src/pq_hsa_vllm/plugin.py:57-97 in the reference).

Register it in the packaging metadata as

    [project.entry-points."vllm.general_plugins"]
    pq_hsa_vllm = "pqhsa_release_b200.pq_hsa_vllm.plugin:vllm_general_plugin"

vLLM calls the entry point once per process (driver and every tensor-parallel worker).
It is a no-op unless ``PQ_HSA_VLLM=1``; ``install`` is idempotent.
"""

from __future__ import annotations

import os
from typing import Any, Optional

from .config import PQHSAConfig

_INSTALLED = False


def enabled() -> bool:
    return os.environ.get("PQ_HSA_VLLM", "0") == "1"


def install(rank: Optional[int] = None, *, force: bool = False, config: Optional[PQHSAConfig] = None,
            impl_cls=None) -> dict[str, Any]:
    """Apply the :class:`PQHSAConfig` defaults to the environment and wrap the
    FLASH_ATTN decode forward.  ``impl_cls`` lets a test pass a stand-in class."""
    global _INSTALLED
    if not force and not enabled():
        return {"installed": False, "reason": "PQ_HSA_VLLM!=1"}
    cfg = config or PQHSAConfig.from_env()
    written = cfg.apply_env_defaults()
    from .runtime import install_flashattn_backend

    result = install_flashattn_backend(impl_cls)
    result["rank"] = rank
    result["config"] = cfg.asdict()
    result["env_defaults_written"] = sorted(written)
    _INSTALLED = True
    return result


def vllm_general_plugin() -> None:
    if not enabled():
        return
    install()


__all__ = ["vllm_general_plugin", "install", "enabled", "PQHSAConfig"]
