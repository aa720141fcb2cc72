"""Build and load the native extension ``streamep_b200._C`` (CUDA for sm_100a only).

The shared object is built IN-TREE (``streamep_b200/_C*.so``) so that a source
checkout carries its own binary; nothing is installed into site-packages and no
JIT cache outside the tree is used.  ``build()`` compiles with ninja through
``torch.utils.cpp_extension`` using an explicit ``-gencode
arch=compute_100a,code=sm_100a`` (it works on a machine without a GPU);
``load()`` imports the prebuilt object and fails loudly when it is missing.

Reference counterpart: setup.py:1-113 (extension build) and
stream_ep/__init__.py:1-20 (package init).
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import os
import sys
import threading
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
_CSRC = _PKG_DIR / "csrc"
_BUILD_DIR = _PKG_DIR / "build"
_NAME = "_C"
_lock = threading.Lock()
_module = None

SOURCES = ["runtime.cpp", "comm_kernels.cu", "gemm_kernels.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
]


def _so_path() -> Path:
    return _PKG_DIR / f"{_NAME}.so"


def _sources():
    missing = [s for s in SOURCES if not (_CSRC / s).exists()]
    if missing:
        raise FileNotFoundError(f"extension sources missing from {_CSRC}: {missing}")
    return [str(_CSRC / s) for s in SOURCES]


def _stale() -> bool:
    so = _so_path()
    if not so.exists():
        return True
    newest = max(p.stat().st_mtime for p in _CSRC.iterdir() if p.suffix in (".cu", ".cuh", ".cpp", ".h"))
    return newest > so.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA/C++ source of the package for sm_100a into ``_C.so``."""
    with _lock:
        if not force and not _stale():
            return _so_path()
        from torch.utils import cpp_extension

        _BUILD_DIR.mkdir(exist_ok=True)
        # torch appends its own -gencode list from TORCH_CUDA_ARCH_LIST; pin it to the one
        # architecture this library is written for.
        os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
        # A host compiler whose libstdc++.so link is dangling silently links libstdc++ statically;
        # a second copy of the C++ runtime inside the extension makes every C++ exception crash the
        # process.  Use the system compiler and name the shared runtime explicitly.
        if os.path.exists("/usr/bin/g++"):
            os.environ["CXX"] = "/usr/bin/g++"
            os.environ["CC"] = "/usr/bin/gcc"
        os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 1)))
        cpp_extension.load(
            name=_NAME,
            sources=_sources(),
            extra_cflags=["-O3", "-std=c++17"],
            extra_cuda_cflags=NVCC_FLAGS + os.environ.get("STREAMEP_EXTRA_NVCC_FLAGS", "").split(),
            extra_ldflags=["-l:libstdc++.so.6"],
            build_directory=str(_BUILD_DIR),
            verbose=verbose,
            is_python_module=False,
        )
        built = _BUILD_DIR / f"{_NAME}.so"
        if not built.exists():
            raise RuntimeError(f"extension build produced no {built}")
        tmp = _PKG_DIR / f".{_NAME}.so.tmp{os.getpid()}"
        tmp.write_bytes(built.read_bytes())
        os.replace(tmp, _so_path())
        _self_test()
        return _so_path()


def _self_test() -> None:
    """Import the fresh object in a child process and make it throw once: a build whose C++
    exceptions do not reach Python (see the note on libstdc++ above) must not go unnoticed."""
    import subprocess

    code = ("import sys; sys.path.insert(0, %r)\n"
            "from streamep_b200 import _ext\n"
            "m = _ext.load()\n"
            "try:\n    m.Config(-1, 6, 256, 6, 128)\nexcept ValueError:\n    print('ok')\n" % str(_PKG_DIR.parent))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    if out.returncode != 0 or "ok" not in out.stdout:
        raise RuntimeError("the built extension failed its exception self-test "
                           f"(exit {out.returncode}): {out.stderr[-2000:]}")


def load():
    """Import the prebuilt extension.  Raises ``ImportError`` with build
    instructions when the shared object is absent; never falls back to Python."""
    global _module
    if _module is not None:
        return _module
    with _lock:
        if _module is not None:
            return _module
        so = _so_path()
        if not so.exists():
            raise ImportError(
                f"{so} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "or `python -m streamep_b200._ext` (needs nvcc; no GPU required)")
        import torch  # noqa: F401  (libtorch must be loaded before the extension)

        full = f"streamep_b200.{_NAME}"
        loader = importlib.machinery.ExtensionFileLoader(full, str(so))
        spec = importlib.util.spec_from_file_location(full, str(so), loader=loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        sys.modules[full] = mod
        _module = mod
        return mod


def available() -> bool:
    return _so_path().exists()


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
