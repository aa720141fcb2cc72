"""``stream_ep.buffer`` of the reference: same names, implemented in ``streamep_b200.buffer``."""
from streamep_b200.buffer import Buffer, StreamingHandle, topk_idx_t  # noqa: F401
