"""Drop-in import name of the reference package (stream_ep/__init__.py:1-20): everything is
re-exported from ``streamep_b200``."""
from streamep_b200 import Buffer, LocalWorld, StreamEPError, StreamEPTimeout, StreamingHandle, topk_idx_t  # noqa: F401


def __getattr__(name):
    if name in ("Config", "EventHandle"):
        import streamep_b200
        return getattr(streamep_b200, name)
    raise AttributeError(f"module 'stream_ep' has no attribute {name!r}")
