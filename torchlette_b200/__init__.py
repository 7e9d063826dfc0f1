"""torchlette_b200 — sm_100a kernels for torchlette's quantized-weight matmul
path behind a C ABI (``include/tlcuda.h``), plus the host-side mirror of the
reference backend interface (``backend.py``)."""
from .backend import (CudaBackend, CudaTensor, EpilogueConfig, QuantPacking, StorageFormat, TlError,  # noqa: F401
                      destroyCuda, detectMatmulEpilogue, getBackend, getCudaInitError, initCuda,
                      perChannelFormat, resolveWeightFormat)

__all__ = ["CudaBackend", "CudaTensor", "EpilogueConfig", "QuantPacking", "StorageFormat", "TlError",
           "destroyCuda", "detectMatmulEpilogue", "getBackend", "getCudaInitError", "initCuda",
           "perChannelFormat", "resolveWeightFormat"]
