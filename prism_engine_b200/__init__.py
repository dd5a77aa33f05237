"""B200 (sm_100a) backend for Prism Engine's palettized-LUT matmul path.

``CudaBackend`` is the drop-in peer of the reference's ``MetalBackend``;
``PrismEngine`` mirrors the reference engine's load/generate.  Everything
executes in ``libprism_cuda.so`` (C ABI: ``include/prism_cuda.h``).
"""
from ._lib import ModelConfig, PrismCudaError  # noqa: F401
from .backend import (QWEN25_0P5B, QWEN25_7B, QWEN25_72B, CudaBackend, PrismEngine,  # noqa: F401
                      model_config)
from .cimage import CImageReader, CImageWriter  # noqa: F401
from .graph import ModelGraph, UnifiedConfig, generate_plan  # noqa: F401
