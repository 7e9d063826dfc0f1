"""Quantize-at-load for the cuda backend: the weight-loading half of the path.

Mirrors what the reference's Qwen3 loader does with ``weightFormat``
(examples/qwen3/loader.ts:228-253): every projection weight ``[N, K]`` with
``K % 4 == 0`` and ``K % groupSize == 0`` is quantized when it is loaded and the
module's parameter is replaced by a packed-int operand; everything else (norms,
embeddings, shapes that do not divide) stays a plain tensor.  Two differences, both
on purpose:

* the quantizer runs on the GPU (``tl_quantize_linear_weight_device``, bit-identical
  to the host quantizer), so an f32 checkpoint tensor is uploaded once and its packed
  form never visits the host;
* packed weights can be cached on disk, keyed like the reference's browser cache
  (``${url}#${tensor}#${scheme}g${G}``, docs/quantization-design.md:397-401): a second
  load reads ``packed`` + ``scales`` and skips the quantizer.

No checkpoint format is parsed here: the caller hands over ``name -> numpy array``
(the reference's safetensors reader is application code, outside the path).
"""
from __future__ import annotations

import hashlib
import os
from typing import Callable, Dict, Iterable, Optional, Tuple

import numpy as np

from .backend import CudaBackend, CudaTensor, StorageFormat, resolveWeightFormat

# names the reference treats as projection weights (loader.ts resolveProjModule: q/k/v/o, gate/up/down)
PROJECTION_SUFFIXES = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight",
                       "gate_proj.weight", "up_proj.weight", "down_proj.weight")


def is_projection(name: str) -> bool:
    return name.endswith(PROJECTION_SUFFIXES)


def cache_key(source: str, tensor: str, fmt: StorageFormat) -> str:
    """``${source}#${tensor}#${scheme}g${G}`` (docs/quantization-design.md:397-401)."""
    p = fmt.packing
    scheme = "int8" if p.scheme == "int8-grouped" else p.scheme
    return f"{source}#{tensor}#{scheme}g{p.groupSize}"


def _cache_path(cache_dir: str, key: str) -> str:
    return os.path.join(cache_dir, hashlib.sha256(key.encode()).hexdigest()[:32] + ".npz")


def load_weights(be: CudaBackend, tensors: Iterable[Tuple[str, np.ndarray]], weightFormat: Optional[str] = None,
                 cache_dir: Optional[str] = None, source: str = "local",
                 select: Callable[[str], bool] = is_projection) -> Dict[str, CudaTensor]:
    """Uploads ``(name, array)`` pairs; with ``weightFormat`` ("int8-64" | "int8-128") the selected
    2-D weights become quantized operands (``tensor.format`` / ``tensor.scales`` set, as
    ``createQuantizedWeight`` leaves them).  Returns ``name -> CudaTensor``."""
    fmt = resolveWeightFormat(weightFormat, "f16") if weightFormat else None
    out: Dict[str, CudaTensor] = {}
    for name, data in tensors:
        arr = np.asarray(data)
        if fmt is not None and select(name) and arr.ndim == 2:
            n, k = arr.shape
            g = fmt.packing.groupSize
            if k % 4 == 0 and k % g == 0:  # loader.ts:236-241: otherwise the weight stays as it is
                path = _cache_path(cache_dir, cache_key(source, name, fmt)) if cache_dir else None
                if path and os.path.exists(path):
                    with np.load(path) as z:
                        if tuple(z["shape"]) == (n, k):
                            out[name] = be.createQuantizedWeight(z["packed"], z["scales"], n, k, fmt)
                            continue
                w32 = be.ops.tensorFromArray(np.ascontiguousarray(arr, dtype=np.float32), [n, k], "f32")
                qw = be.quantizeLinearWeightOnDevice(w32, fmt)
                w32.destroy()
                if path:
                    os.makedirs(cache_dir, exist_ok=True)
                    qw_view = CudaTensor(be, [n, k // 4], "u32", qw.buffer, n * (k // 4) * 4, ownsBuffer=False)
                    np.savez(path, packed=be.ops.read(qw_view), scales=be.ops.read(qw.scales), shape=np.array([n, k]))
                out[name] = qw
                continue
        dtype = {np.dtype(np.float32): "f32", np.dtype(np.float16): "f16", np.dtype(np.uint32): "u32",
                 np.dtype(np.uint16): "u16"}.get(arr.dtype)
        if dtype is None:
            arr, dtype = arr.astype(np.float32), "f32"
        src = arr.view(np.uint16) if dtype == "f16" else arr
        out[name] = be.ops.tensorFromArray(np.ascontiguousarray(src), list(arr.shape), dtype)
    return out
