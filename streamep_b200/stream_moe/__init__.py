"""The streaming MoE layer (reference: stream_ep/stream_moe/__init__.py)."""
from .tile_config import TileConfig, default_tile_config, _resolve_tile_config  # noqa: F401
from .stream_moe import (  # noqa: F401
    StreamHolder,
    StreamMoEFunc,
    make_streams,
    moe_backward,
    moe_forward,
    stream_moe_func,
)
from ..ops.grouped_gemm import (  # noqa: F401
    compress_pool_to_recv,
    fire_tiles_with_delay,
    grouped_gemm_dw,
    grouped_gemm_preact,
    reexpand_recv_to_pool,
    streaming_moe_a,
    streaming_moe_a_bwd,
    streaming_moe_y,
    streaming_moe_y_bwd,
)
