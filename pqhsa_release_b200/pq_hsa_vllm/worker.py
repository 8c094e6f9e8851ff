"""Worker class for ``--worker-cls`` (pq_hsa_vllm/src/pq_hsa_vllm/worker.py:30-66 in the
reference): choosing it is the opt-in, so ``init_device`` installs unconditionally.
vLLM is imported only when the class is first used."""

from __future__ import annotations

from typing import Any


def _base():
    from vllm.v1.worker.gpu_worker import Worker  # type: ignore

    return Worker


class _Lazy(type):
    def __call__(cls, *args: Any, **kwargs: Any):
        base = _base()
        real = type("PQHSAWorker", (base,), {"init_device": _init_device})
        return real(*args, **kwargs)


def _init_device(self, *args: Any, **kwargs: Any):
    from .plugin import install

    install(rank=getattr(self, "rank", None), force=True)
    return super(type(self), self).init_device(*args, **kwargs)


class PQHSAWorker(metaclass=_Lazy):
    """``--worker-cls pqhsa_release_b200.pq_hsa_vllm.PQHSAWorker``"""
