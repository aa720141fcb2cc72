"""streamep_b200: streaming expert-parallel MoE for NVIDIA B200 (sm_100a).

Public names mirror the reference package (stream_ep/__init__.py:1-20):
``Buffer``, ``Config``, ``EventHandle``, ``topk_idx_t``.  ``Config`` and
``EventHandle`` come from the native extension and are resolved lazily so that
the pure-Python parts (oracles, tile config) import on machines without the
built extension.
"""
from .errors import StreamEPError, StreamEPTimeout  # noqa: F401
from .buffer import Buffer, LocalWorld, StreamingHandle, topk_idx_t  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Config", "EventHandle"):
        from . import _ext
        return getattr(_ext.load(), name)
    raise AttributeError(f"module 'streamep_b200' has no attribute {name!r}")
