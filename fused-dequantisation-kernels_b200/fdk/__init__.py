"""fdk -- drop-in for the LUT hot path of graphcore-research/fused-dequantisation-kernels,
running on hand-written sm_100a CUDA kernels (libfdk_b200.so) instead of Triton.

Sub-modules are imported lazily, as in the reference package (src/fdk/__init__.py):
`fdk.models`, `fdk.kernels`, `fdk.bench`.
"""

import importlib
from typing import Any

__all__ = ["bench", "kernels", "models", "llama", "native"]

_LAZY = {"bench", "kernels", "models", "llama", "native"}


def __getattr__(name: str) -> Any:
    if name in _LAZY:
        module = importlib.import_module(f".{name}", __name__)
        globals()[name] = module
        return module
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__() -> list[str]:
    return sorted(set(globals()) | _LAZY)
