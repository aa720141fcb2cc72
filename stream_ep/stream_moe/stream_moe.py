"""``stream_ep.stream_moe.stream_moe`` of the reference: same public names."""
from streamep_b200.stream_moe.stream_moe import (  # noqa: F401
    StreamHolder, StreamMoEFunc, make_streams, stream_moe_func)
from streamep_b200.stream_moe.tile_config import TileConfig, _resolve_tile_config, default_tile_config  # noqa: F401
