"""In-tree build of the sm_100a extension (``deliverance_b200/ops/_build/_dlv_C.so``).

The shared object is compiled with ``-gencode arch=compute_100a,code=sm_100a`` only; nvcc cross-compiles without a GPU.
``load_extension()`` imports an already built ``.so`` directly (no JIT rebuild, no cache outside the tree).
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
BUILD_DIR = os.path.join(_HERE, "_build")
NAME = "_dlv_C"
SOURCES = ["bindings.cpp", "gemm.cu", "gemm_persist.cu", "elementwise.cu", "attention.cu", "sampling.cu", "quant.cu", "moe.cu", "mamba.cu",
           "comm.cu", "noalloc.cu", "chain.cu", "aux.cu", "a2a.cu", "attention_tc.cu", "lz4_block.cpp"]

CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def so_path() -> str:
    return os.path.join(BUILD_DIR, NAME + ".so")


def _stale() -> bool:
    so = so_path()
    if not os.path.exists(so):
        return True
    t = os.path.getmtime(so)
    for f in os.listdir(CSRC):
        if os.path.getmtime(os.path.join(CSRC, f)) > t:
            return True
    return False


def build_extension(verbose: bool = False, force: bool = False):
    """Compile (if sources changed) and import the extension."""
    if force or _stale():
        os.makedirs(BUILD_DIR, exist_ok=True)
        # torch derives -gencode flags from TORCH_CUDA_ARCH_LIST; the explicit flag above is the one that matters and
        # an empty list would make torch probe a GPU, so pin it to the same target.
        os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
        os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
        from torch.utils.cpp_extension import load

        return load(
            name=NAME,
            sources=_sources(),
            extra_cflags=["-O3", "-std=c++17"],
            extra_cuda_cflags=CUDA_FLAGS,
            extra_include_paths=[CSRC],
            build_directory=BUILD_DIR,
            verbose=verbose,
        )
    return load_extension()


def load_extension():
    """Import the built ``.so`` without invoking the JIT builder. Returns ``None`` when it has not been built."""
    if NAME in sys.modules:
        return sys.modules[NAME]
    so = so_path()
    if not os.path.exists(so):
        return None
    import torch  # noqa: F401  (libtorch symbols must be loaded first)

    loader = importlib.machinery.ExtensionFileLoader(NAME, so)
    spec = importlib.util.spec_from_loader(NAME, loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules[NAME] = mod
    return mod


if __name__ == "__main__":
    build_extension(verbose=True, force="--force" in sys.argv)
    print("built", so_path())
