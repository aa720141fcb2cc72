"""Python entry points of the native kernels (lazy: importing the package does not load the extension)."""
import importlib


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    mod = importlib.import_module(__name__ + ".grouped_gemm")
    if name == "grouped_gemm":
        return mod
    if hasattr(mod, name):
        return getattr(mod, name)
    raise AttributeError(name)
