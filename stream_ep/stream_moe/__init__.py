from streamep_b200.stream_moe import *  # noqa: F401,F403
from streamep_b200.stream_moe import _resolve_tile_config  # noqa: F401
