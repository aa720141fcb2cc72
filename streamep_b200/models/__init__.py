"""Model-side pieces: the ``StreamMoE`` module and the pure-PyTorch oracles."""
import importlib


def __getattr__(name):
    if name in ("StreamMoE", "make_buffer"):
        return getattr(importlib.import_module(__name__ + ".moe_layer"), name)
    raise AttributeError(name)
