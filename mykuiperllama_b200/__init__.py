"""B200-native (sm_100a) decode hot path behind the MyKuiperLLama operator API.

The product is native: hand-written CUDA kernels behind a C ABI
(``include/kuiper_b200.h``) and a C++ host side that mirrors the reference's
``base`` / ``tensor`` / ``op`` / ``model`` interfaces (``include/kuiper_llama.h``).
This Python package only builds and loads those libraries for tests and benchmarks.
"""
from . import _build  # noqa: F401

__all__ = ["_build"]
