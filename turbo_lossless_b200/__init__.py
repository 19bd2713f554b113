"""split12 decode + GEMV/GEMM for NVIDIA B200 (sm_100a).

A drop-in for the kernel entry points of the Turbo-Lossless engine: the shared
library ``libsplit12_b200.so`` exports the engine's own ``extern "C"`` names
(see ``include/split12_b200.h``).  The Python layer only mirrors the engine's
host-side structures so that tests and benchmarks read like the engine's call
sites; all arithmetic of the path runs in the CUDA library.
"""
from .capi import S12Error, S12Tensor, load  # noqa: F401
from .engine import CompressedWeight, Split12Engine, TPComm  # noqa: F401
from .decoder import Decoder, DecoderConfig  # noqa: F401
from .loader import load_model, read_config  # noqa: F401

__all__ = ["S12Error", "S12Tensor", "load", "CompressedWeight", "Split12Engine", "TPComm", "Decoder", "DecoderConfig", "load_model", "read_config"]
