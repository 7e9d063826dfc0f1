"""Host-side mirror of torchlette's backend interface for the quantized-weight
matmul path, over the C ABI in ``include/tlcuda.h``.

Names, argument meaning and error behaviour follow the reference (paths relative
to the torchlette repository root):

  Backend / BackendOps.matmul        src/backend/types.ts:340-745
  StorageFormat / resolveWeightFormat src/backend/types.ts:38-67
  createQuantizedWeight              src/runtime/engine.ts:2041-2149
  api.linear                         src/frontend/torchlette.ts:878-894
  matmul seam / matmulQuantizedB     src/backend/webgpu/ops/matmul-ops.ts:42-182
  dispatchQuantizedGemvNT            src/backend/webgpu/matmul/dispatch.ts:875-931
  dispatchDequantizeInt8Grouped      src/backend/webgpu/matmul/dispatch.ts:949-1037
  route counters                     src/backend/webgpu/matmul/dispatch.ts:833-864, 943-947
  epilogue-fusion decision           src/compiler/matmul-epilogue.ts:131-262
  autotune surface                   src/backend/webgpu/matmul/dispatch.ts:79-141, 405-578

Python stands in for the TypeScript frontend because no node toolchain exists
where this was built; every function here is a thin call into the C ABI, which
is what an N-API addon would bind.  There is no CPU or WebGPU fallback: without
the CUDA library and an sm_100 GPU, ``initCuda`` raises.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

from . import binding as B
from .binding import TlError

# ---------------------------------------------------------------------------
# StorageFormat (src/backend/types.ts:38-67), widened with the scale convention
# ---------------------------------------------------------------------------


@dataclass(frozen=True)
class QuantPacking:
    scheme: str = "int8-grouped"
    groupSize: int = 64
    scalesDtype: str = "f16"
    scaleConvention: str = "snorm127"  # "snorm127": w=(q/127)*s ; "direct": w=q*s


_VALUES_PER_WORD = {"int8-grouped": 4, "int4-grouped": 8}


@dataclass(frozen=True)
class StorageFormat:
    elementType: str = "f16"
    packing: Optional[QuantPacking] = None


def resolveWeightFormat(name: str, elementType: str = "f16") -> StorageFormat:
    """"int8-64" | "int8-128" -> StorageFormat (types.ts:57-67); "int4-32" | "int4-128" name the
    scheme the reference plans next (docs/quantization-design.md:69-75)."""
    if name in ("int4-32", "int4-128"):
        return StorageFormat(elementType, QuantPacking("int4-grouped", int(name.split("-")[1]), "f16"))
    if name not in ("int8-64", "int8-128"):
        raise ValueError(f"unknown weight format {name}")
    return StorageFormat(elementType, QuantPacking("int8-grouped", 64 if name == "int8-64" else 128, "f16"))


def perChannelFormat(k: int, elementType: str = "f16") -> StorageFormat:
    """Per-output-channel f32 scales, w = q*s (the benchmark configurations)."""
    return StorageFormat(elementType, QuantPacking("int8-grouped", k, "f32", "direct"))


# ---------------------------------------------------------------------------
# EpilogueConfig (src/backend/webgpu/matmul/types.ts:13-24)
# ---------------------------------------------------------------------------


@dataclass
class EpilogueConfig:
    ops: list = field(default_factory=list)  # dicts: {"kind": "bias", "inputIndex": 0} ...
    additionalInputCount: int = 0
    outputDtype: str = "f32"


_FUSIBLE_UNARY = {"relu", "silu", "sigmoid", "tanh", "gelu", "gelu_tanh", "gelu_erf"}


def detectMatmulEpilogue(chain: Sequence[tuple], matmulDtype: str = "f32"):
    """The lazy graph's epilogue-fusion decision for the ops that follow a matmul
    (matmul-epilogue.ts:131-262), applied to a linear chain description.

    The decision itself is ``epilogue_fusion.detectMatmulEpilogueCore`` (consumer counts, outside
    references, reshape skips); this adapter feeds it a straight chain.  In a chain the name "gelu"
    means the tanh form unless the operand says {"approximate": "none"}.

    ``chain`` is a list of (opName, operand) where operand is a CudaTensor for
    add/sub/mul, a dtype name for cast, a dict of options for gelu
    ({"approximate": "none"} selects gelu_erf, matmul-epilogue.ts:52-56) and
    None otherwise.  Returns (EpilogueConfig, inputs, consumed) claiming at most
    four ops, or None when nothing fuses.  Unlike the reference
    (graph-compiler.ts:150-152) a quantized B operand does not veto the fusion.
    """
    from .epilogue_fusion import PlanNode, detectMatmulEpilogueCore

    # the chain as a plan: every op consumes the one before it
    nodes = [PlanNode(0, "matmul", [], [], matmulDtype)]
    for i, (name, operand) in enumerate(chain):
        prev = nodes[-1]
        if name == "cast":
            nodes.append(PlanNode(i + 1, "cast", [prev], [], operand, {"dtype": operand}))
        elif name in ("add", "mul", "sub"):
            nodes.append(PlanNode(i + 1, name, [prev, operand]))
        elif name in ("gelu", "gelu_tanh", "gelu_erf"):
            erf = name == "gelu_erf" or (isinstance(operand, dict) and operand.get("approximate") == "none")
            nodes.append(PlanNode(i + 1, "gelu", [prev], [], None, None if erf else {"approximate": "tanh"}))
        else:
            nodes.append(PlanNode(i + 1, name, [prev]))
    plan = detectMatmulEpilogueCore(nodes, 0)
    if plan is None:
        return None
    return EpilogueConfig(plan.epilogueOps, len(plan.epilogueInputs), plan.outputDtype), plan.epilogueInputs, plan.consumedCount - 1


# ---------------------------------------------------------------------------
# Tensors
# ---------------------------------------------------------------------------


class CudaTensor:
    """BackendTensor (types.ts:5-27): shape, dtype, ownsBuffer, format, scales.
    ``buffer`` is a raw device pointer.  ``transposed`` marks the [K,N] view of a
    contiguous [N,K] buffer produced by ``transpose`` (the only view the path
    needs; src/backend/webgpu/ops/views.ts:925-933 propagates format/scales)."""

    def __init__(self, backend, shape, dtype, buffer, nbytes, ownsBuffer=True, format=None, scales=None,
                 transposed=False):
        self.backend = backend
        self.shape = list(shape)
        self.dtype = dtype
        self.buffer = buffer
        self.nbytes = nbytes
        self.ownsBuffer = ownsBuffer
        self.format = format
        self.scales = scales
        self.transposed = transposed

    def destroy(self):
        if self.ownsBuffer and self.buffer:
            self.backend._free(self.buffer)
        self.buffer = None

    def toArray(self):
        return self.backend.ops.read(self)


_NP_OF = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16, "u32": np.uint32, "u16": np.uint16,
          "i8": np.int8}


class CudaOps:
    """BackendOps subset the path needs (types.ts:340-680)."""

    def __init__(self, backend):
        self._b = backend

    # tensorFromArray: f32 uploads verbatim; "f16" takes np.float16 values or raw
    # uint16 bit patterns; "bf16" takes raw uint16 bit patterns; u32/u16 verbatim.
    def tensorFromArray(self, values, shape, dtype="f32") -> CudaTensor:
        arr = np.asarray(values)
        if dtype == "f16" and arr.dtype == np.uint16:
            host = np.ascontiguousarray(arr)
        elif dtype == "bf16":
            if arr.dtype != np.uint16:
                raise TypeError("bf16 tensors are created from uint16 bit patterns")
            host = np.ascontiguousarray(arr)
        else:
            host = np.ascontiguousarray(arr, dtype=_NP_OF[dtype])
        n = int(np.prod(shape)) if len(shape) else 1
        if host.size != n:
            raise ValueError(f"tensorFromArray: expected {n} elements, got {host.size}")
        buf = self._b._alloc(host.nbytes)
        self._b._upload(buf, host)
        return CudaTensor(self._b, shape, dtype, buf, host.nbytes)

    def empty(self, shape, dtype="f32") -> CudaTensor:
        n = int(np.prod(shape)) if len(shape) else 1
        nbytes = n * np.dtype(_NP_OF[dtype]).itemsize
        return CudaTensor(self._b, shape, dtype, self._b._alloc(nbytes), nbytes)

    def read(self, t: CudaTensor) -> np.ndarray:
        if t.transposed:
            raise ValueError("read: materialize the transposed view first")
        host = np.empty(int(np.prod(t.shape)) if t.shape else 1, dtype=_NP_OF[t.dtype])
        self._b._download(host, t.buffer)
        if t.dtype == "f16":
            host = host.view(np.float16)
        return host.reshape(t.shape)

    def reshape(self, t: CudaTensor, shape) -> CudaTensor:
        """A view of a contiguous tensor under another shape (no copy; the buffer stays the owner's)."""
        if t.transposed or int(np.prod(shape)) != int(np.prod(t.shape)):
            raise ValueError("reshape: needs a contiguous tensor and the same element count")
        return CudaTensor(self._b, list(shape), t.dtype, t.buffer, t.nbytes, ownsBuffer=False, format=t.format, scales=t.scales)

    def transpose(self, t: CudaTensor, dim0: int = -2, dim1: int = -1) -> CudaTensor:
        nd = len(t.shape)
        if nd < 2 or {dim0 % nd, dim1 % nd} != {nd - 2, nd - 1}:
            raise ValueError("transpose: only the last two dims can be swapped on this path")
        shape = t.shape[:-2] + [t.shape[-1], t.shape[-2]]
        return CudaTensor(self._b, shape, t.dtype, t.buffer, t.nbytes, ownsBuffer=False, format=t.format,
                          scales=t.scales, transposed=not t.transposed)

    # -- companion ops: the unfused forms of the epilogue (types.ts:340-680) ----------
    def _unary(self, op: int, t: CudaTensor, out_dtype: Optional[str] = None) -> CudaTensor:
        src = self.contiguous(t) if t.transposed else t
        out = self.empty(src.shape, out_dtype or src.dtype)
        n = int(np.prod(src.shape)) if src.shape else 1
        B.check(self._b._ctx, self._b._lib.tl_unary_op(self._b._ctx, op, src.buffer, B.DTYPE_ID[src.dtype], out.buffer,
                                                       B.DTYPE_ID[out.dtype], n))
        if src is not t:
            src.destroy()
        return out

    def relu(self, t): return self._unary(B.TL_UNARY["relu"], t)
    def silu(self, t): return self._unary(B.TL_UNARY["silu"], t)
    def sigmoid(self, t): return self._unary(B.TL_UNARY["sigmoid"], t)
    def tanh(self, t): return self._unary(B.TL_UNARY["tanh"], t)
    def gelu(self, t, approximate: str = "tanh"): return self._unary(B.TL_UNARY["gelu_tanh" if approximate == "tanh" else "gelu_erf"], t)

    def cast(self, t: CudaTensor, dtype: str) -> CudaTensor:
        return self._unary(0, t, dtype)

    def _binary(self, name: str, a: CudaTensor, b: CudaTensor) -> CudaTensor:
        """a [..., N] (op) b of the same shape, or b [N] broadcast over the rows (a bias)."""
        if a.transposed or b.transposed:
            raise TlError(B.TL_ERR_UNSUPPORTED, f"{name}: materialize transposed views first (contiguous)")
        cols = a.shape[-1]
        rows = int(np.prod(a.shape[:-1])) if len(a.shape) > 1 else 1
        is_row = list(b.shape) == [cols] and len(a.shape) > 1
        if not is_row and list(b.shape) != list(a.shape):
            raise TlError(B.TL_ERR_UNSUPPORTED, f"{name}: b must match a or be its last dim")
        out = self.empty(a.shape, a.dtype)
        B.check(self._b._ctx, self._b._lib.tl_binary_op(self._b._ctx, B.TL_BINARY[name], a.buffer, B.DTYPE_ID[a.dtype], b.buffer,
                                                        B.DTYPE_ID[b.dtype], out.buffer, B.DTYPE_ID[out.dtype], rows, cols,
                                                        1 if is_row else 0))
        return out

    def add(self, a, b): return self._binary("add", a, b)
    def sub(self, a, b): return self._binary("sub", a, b)
    def mul(self, a, b): return self._binary("mul", a, b)

    def contiguous(self, t: CudaTensor) -> CudaTensor:
        """Materializes a transposed view (a packed weight cannot be: its bytes are not elements)."""
        if t.format is not None and t.format.packing is not None:
            raise TlError(B.TL_ERR_UNSUPPORTED, "contiguous: a packed weight has no element-wise transposition")
        itemsize = np.dtype(_NP_OF[t.dtype]).itemsize
        if not t.transposed:
            return self._unary(0, t)  # a plain copy
        out = self.empty(t.shape, t.dtype)
        rows, cols = t.shape[-1], t.shape[-2]  # of the stored buffer
        B.check(self._b._ctx, self._b._lib.tl_transpose2d(self._b._ctx, t.buffer, out.buffer, 1, rows, cols, itemsize))
        return out

    # -- the other ops of a decode step (packages/qwen3-browser/src/model.ts:220-420) ----------
    def rmsnorm(self, x: CudaTensor, weight: CudaTensor, eps: float = 1e-5, outputDtype: Optional[str] = None) -> CudaTensor:
        """x * rsqrt(mean(x^2) + eps) * weight over the last dim (src/frontend/tensor.ts:363-367)."""
        cols = x.shape[-1]
        if list(weight.shape) != [cols]:
            raise TlError(B.TL_ERR_INVALID_ARG, "rmsnorm: weight must be [lastDim]")
        rows = int(np.prod(x.shape[:-1])) if len(x.shape) > 1 else 1
        out = self.empty(x.shape, outputDtype or x.dtype)
        B.check(self._b._ctx, self._b._lib.tl_rmsnorm(self._b._ctx, x.buffer, B.DTYPE_ID[x.dtype], weight.buffer, B.DTYPE_ID[weight.dtype],
                                                      out.buffer, B.DTYPE_ID[out.dtype], rows, cols, float(eps)))
        return out

    def fusedRoPE(self, qk: CudaTensor, cos: CudaTensor, sin: CudaTensor, config: Optional[dict] = None) -> CudaTensor:
        """fusedRoPE (src/backend/types.ts:593-598): qk [*, S, D], cos / sin f32 [S, D/2]; config may carry
        sinScale (-1: the inverse rotation), cosOffset / sinOffset (element offsets into larger tables)."""
        config = config or {}
        seq, hd = qk.shape[-2], qk.shape[-1]
        outer = int(np.prod(qk.shape[:-2])) if len(qk.shape) > 2 else 1
        if cos.dtype != "f32" or sin.dtype != "f32":
            raise TlError(B.TL_ERR_UNSUPPORTED, "fusedRoPE: cos / sin tables are f32")
        out = self.empty(qk.shape, qk.dtype)
        B.check(self._b._ctx, self._b._lib.tl_rope(self._b._ctx, qk.buffer, B.DTYPE_ID[qk.dtype], cos.buffer, sin.buffer, out.buffer, outer, seq, hd,
                                                   float(config.get("sinScale", 1.0)), int(config.get("cosOffset", 0)), int(config.get("sinOffset", 0))))
        return out

    def decodeAttention(self, q: CudaTensor, kCache: CudaTensor, vCache: CudaTensor, kvLen: int, scale: float,
                        mask: Optional[CudaTensor] = None) -> CudaTensor:
        """softmax(q k^T * scale + mask) v for one query token per sequence (model.ts:292-312): q [B, H, 1, D]
        (or [B, H, D]), caches [B, kvH, capacity, D]; returns [B, 1, H * D], the layout o_proj reads."""
        b, h, d = q.shape[0], q.shape[1], q.shape[-1]
        kvh, cap = kCache.shape[1], kCache.shape[2]
        out = self.empty([b, 1, h * d], q.dtype)
        B.check(self._b._ctx, self._b._lib.tl_decode_attention(self._b._ctx, q.buffer, kCache.buffer, vCache.buffer, out.buffer, B.DTYPE_ID[q.dtype], b, h,
                                                               kvh, d, kvLen, cap, float(scale), mask.buffer if mask is not None else None))
        return out

    def attention(self, q: CudaTensor, kCache: CudaTensor, vCache: CudaTensor, kvLen: int, scale: float, causal: bool = True,
                  mask: Optional[CudaTensor] = None) -> CudaTensor:
        """scaledDotProductAttention over (a prefix of) a KV cache for S query positions (model.ts:284-318):
        q [B, H, S, D], caches [B, kvH, capacity, D]; returns [B, S, H * D].  With ``causal`` query s sees
        keys up to kvLen - S + s (prefill: kvLen == S)."""
        b, h, sq, d = q.shape
        out = self.empty([b, sq, h * d], q.dtype)
        B.check(self._b._ctx, self._b._lib.tl_attention(self._b._ctx, q.buffer, kCache.buffer, vCache.buffer, out.buffer, B.DTYPE_ID[q.dtype], b, h,
                                                        kCache.shape[1], sq, d, kvLen, kCache.shape[2], float(scale),
                                                        mask.buffer if mask is not None else None, 1 if causal else 0))
        return out

    def kvAppend(self, cache: CudaTensor, new: CudaTensor, position: int):
        """cache[:, :, position, :] = new ([B, kvH, 1, D] or [B, kvH, D]): one strided copy (model.ts:240-262)."""
        b, kvh, cap, d = cache.shape
        esz = np.dtype(_NP_OF[cache.dtype]).itemsize
        B.check(self._b._ctx, self._b._lib.tl_copy2d(self._b._ctx, cache.buffer + position * d * esz, cap * d * esz, new.buffer, d * esz, d * esz, b * kvh))

    def matmul(self, a: CudaTensor, b: CudaTensor, options: Optional[dict] = None) -> CudaTensor:
        """Backend matmul; the storage-format seam (matmul-ops.ts:42-59)."""
        if b.format is not None and b.format.packing is not None:
            return self._b._matmulQuantizedB(a, b, options or {})
        return self._b.dispatchMatmul(a, b, options or {})


class CudaBackend:
    """``Backend`` named "cuda" (types.ts:681-696)."""

    name = "cuda"

    def __init__(self, device: int = 0):
        self._lib = B.load()
        ctx = C.c_void_p()
        B.check(None, self._lib.tl_ctx_create(device, C.byref(ctx)))
        self._ctx = ctx
        self.device = device
        self.ops = CudaOps(self)

    # -- lifetime -----------------------------------------------------------
    def destroy(self):
        if self._ctx:
            self._lib.tl_ctx_destroy(self._ctx)
            self._ctx = None

    def sync(self):
        B.check(self._ctx, self._lib.tl_sync(self._ctx))

    def getGpuUncapturedErrorCount(self) -> int:
        return int(self._lib.tl_async_error_count(self._ctx))

    def stream(self) -> int:
        s = C.c_void_p()
        B.check(self._ctx, self._lib.tl_ctx_stream(self._ctx, C.byref(s)))
        return s.value or 0

    def smCount(self) -> int:
        v = C.c_int32()
        B.check(self._ctx, self._lib.tl_device_sm_count(self._ctx, C.byref(v)))
        return v.value

    # -- raw memory ---------------------------------------------------------
    def _alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        B.check(self._ctx, self._lib.tl_alloc(self._ctx, nbytes, C.byref(p)))
        return p.value

    def _free(self, ptr: int):
        B.check(self._ctx, self._lib.tl_free(self._ctx, C.c_void_p(ptr)))

    def _upload(self, ptr: int, host: np.ndarray):
        B.check(self._ctx, self._lib.tl_upload(self._ctx, C.c_void_p(ptr), host.ctypes.data_as(C.c_void_p),
                                               host.nbytes))
        self.sync()

    def _download(self, host: np.ndarray, ptr: int):
        B.check(self._ctx, self._lib.tl_download(self._ctx, host.ctypes.data_as(C.c_void_p), C.c_void_p(ptr),
                                                 host.nbytes))
        self.sync()

    # -- quantized weights --------------------------------------------------
    def quantizeLinearWeight(self, weight: np.ndarray, groupSize: int = 64, scheme: str = "int8-grouped"):
        """quantizeLinearWeight (quantize.ts:77-131) through the library's host
        quantizer.  Returns (packed u32 [N,K/4], scales u16 [N,K/G]); with
        ``scheme="int4-grouped"`` the packed words are [N,K/8]."""
        w = np.ascontiguousarray(weight, dtype=np.float32)
        if w.ndim != 2:
            raise ValueError("quantize: weight must be [N, K]")
        n, k = w.shape
        per_word = _VALUES_PER_WORD[scheme]
        if k % per_word != 0:
            raise TlError(B.TL_ERR_INVALID_ARG, f"quantize: K={k} must be divisible by {per_word}")
        if groupSize <= 0 or k % groupSize != 0:
            raise TlError(B.TL_ERR_INVALID_ARG, f"quantize: K={k} must be divisible by groupSize={groupSize}")
        packed = np.zeros((n, k // per_word), dtype=np.uint32)
        scales = np.zeros((n, k // groupSize), dtype=np.uint16)
        fn = self._lib.tl_quantize_linear_weight if per_word == 4 else self._lib.tl_quantize_linear_weight_int4
        B.check(None, fn(w.ctypes.data_as(C.c_void_p), n, k, groupSize, packed.ctypes.data_as(C.c_void_p),
                         scales.ctypes.data_as(C.c_void_p)))
        return packed, scales

    def quantizeLinearWeightOnDevice(self, weight: CudaTensor, format: StorageFormat) -> CudaTensor:
        """quantizeLinearWeight (quantize.ts:77-131) + createQuantizedWeight (engine.ts:2041-2149) with
        the f32 [N, K] weight already on the GPU: one kernel writes the packed words and the f16 scale
        bits, bit-identical to the host quantizer; nothing travels back to the host."""
        packing = format.packing
        if packing is None or packing.scheme != "int8-grouped" or packing.scalesDtype != "f16":
            raise TlError(B.TL_ERR_UNSUPPORTED, "quantizeLinearWeightOnDevice: the reference quantizer emits int8-grouped with f16 scales")
        if weight.dtype != "f32" or len(weight.shape) != 2:
            raise TlError(B.TL_ERR_INVALID_ARG, "quantize: weight must be f32 [N, K]")
        n, k = weight.shape
        if k % 4 != 0:
            raise TlError(B.TL_ERR_INVALID_ARG, f"quantize: K={k} must be divisible by 4")
        g = packing.groupSize
        if g <= 0 or k % g != 0:
            raise TlError(B.TL_ERR_INVALID_ARG, f"quantize: K={k} must be divisible by groupSize={g}")
        wt = self.ops.empty([n, k // 4], "u32")
        st = self.ops.empty([n, k // g], "u16")
        B.check(self._ctx, self._lib.tl_quantize_linear_weight_device(self._ctx, weight.buffer, n, k, g, wt.buffer, st.buffer))
        wt.shape = [n, k]
        wt.dtype = format.elementType
        wt.format = format
        wt.scales = st
        return wt

    def createQuantizedWeight(self, packed, scales, n: int, k: int, format: StorageFormat) -> CudaTensor:
        """engine.ts:2041-2149: validate lengths, upload the packed words and the
        scales, return the logical [N,K] tensor carrying format + scales."""
        packing = format.packing
        if packing is None:
            raise TlError(B.TL_ERR_INVALID_ARG, "createQuantizedWeight: format.packing is required")
        per_word = _VALUES_PER_WORD.get(packing.scheme)
        if per_word is None:
            raise TlError(B.TL_ERR_UNSUPPORTED, f"createQuantizedWeight: unsupported scheme {packing.scheme}")
        if k % per_word != 0:
            raise TlError(B.TL_ERR_INVALID_ARG, f"createQuantizedWeight: K={k} must be divisible by {per_word}")
        packed = np.ascontiguousarray(packed, dtype=np.uint32)
        if packed.size != n * (k // per_word):
            raise TlError(B.TL_ERR_INVALID_ARG, f"createQuantizedWeight: packed length {packed.size} != {n * (k // per_word)}")
        if packing.groupSize <= 0 or k % packing.groupSize != 0:
            raise TlError(B.TL_ERR_INVALID_ARG,
                          f"createQuantizedWeight: K={k} must be divisible by groupSize={packing.groupSize}")
        groups = k // packing.groupSize
        sdt = np.uint16 if packing.scalesDtype == "f16" else np.float32
        scales = np.asarray(scales)
        if packing.scalesDtype == "f16" and scales.dtype == np.float16:
            scales = scales.view(np.uint16)
        scales = np.ascontiguousarray(scales, dtype=sdt)
        if scales.size != n * groups:
            raise TlError(B.TL_ERR_INVALID_ARG, f"createQuantizedWeight: scales length {scales.size} != {n * groups}")
        st = self.ops.tensorFromArray(scales, [n, groups], "u16" if packing.scalesDtype == "f16" else "f32")
        wt = self.ops.tensorFromArray(packed, [n, k // per_word], "u32")
        wt.shape = [n, k]  # logical shape; the buffer stays u32 [N, K/4] (int8) or [N, K/8] (int4)
        wt.dtype = format.elementType
        wt.format = format
        wt.scales = st
        return wt

    # -- descriptors ----------------------------------------------------------
    @staticmethod
    def _qdesc(packing: QuantPacking) -> B.QuantDesc:
        if packing.scheme not in _VALUES_PER_WORD:
            raise TlError(B.TL_ERR_UNSUPPORTED, f"matmulQuantizedB: unsupported scheme {packing.scheme}")
        return B.QuantDesc(B.TL_SCHEME_INT8_GROUPED if packing.scheme == "int8-grouped" else B.TL_SCHEME_INT4_GROUPED, packing.groupSize, B.DTYPE_ID[packing.scalesDtype],
                           B.TL_SCALE_SNORM127 if packing.scaleConvention == "snorm127" else B.TL_SCALE_DIRECT)

    @staticmethod
    def _epilogue(epilogue: Optional[EpilogueConfig], epilogueInputs: Sequence[CudaTensor]):
        if epilogue is None:
            return None
        e = B.Epilogue()
        if len(epilogue.ops) > B.TL_EPI_MAX_OPS:
            raise TlError(B.TL_ERR_INVALID_ARG, "epilogue: too many ops")
        if len(epilogueInputs) > B.TL_EPI_MAX_INPUTS:
            raise TlError(B.TL_ERR_INVALID_ARG, "epilogue: at most 4 extra inputs")
        e.n_ops = len(epilogue.ops)
        for i, op in enumerate(epilogue.ops):
            kind = op["kind"]
            if kind == "none":
                e.ops[i] = B.EpilogueOp(B.TL_EPI_NONE, 0, 0, 0)
            elif kind == "bias":
                e.ops[i] = B.EpilogueOp(B.TL_EPI_BIAS, 0, op["inputIndex"], 0)
            elif kind == "unary":
                if op["op"] not in B.TL_UNARY:
                    raise TlError(B.TL_ERR_UNSUPPORTED, f"epilogue: unsupported unary op {op['op']}")
                e.ops[i] = B.EpilogueOp(B.TL_EPI_UNARY, B.TL_UNARY[op["op"]], 0, 0)
            elif kind == "binary":
                if op["op"] not in B.TL_BINARY:
                    raise TlError(B.TL_ERR_UNSUPPORTED, f"epilogue: unsupported binary op {op['op']}")
                e.ops[i] = B.EpilogueOp(B.TL_EPI_BINARY, B.TL_BINARY[op["op"]], op["inputIndex"], 0)
            elif kind == "cast":
                e.ops[i] = B.EpilogueOp(B.TL_EPI_CAST, 0, 0, B.DTYPE_ID[op["toDtype"]])
            else:
                raise TlError(B.TL_ERR_INVALID_ARG, f"epilogue: unknown op kind {kind}")
        e.n_inputs = len(epilogueInputs)
        for i, t in enumerate(epilogueInputs):
            if t.dtype != "f32":
                raise TlError(B.TL_ERR_UNSUPPORTED, "epilogue inputs must be f32")
            e.inputs[i] = t.buffer
        return e

    # -- the hot path ---------------------------------------------------------
    def dispatchQuantizedGemvNT(self, aBuffer: CudaTensor, packedWeight: CudaTensor, scales: CudaTensor,
                                outBuffer: CudaTensor, n: int, k: int, groupSize: int, outputDtype: str = "f32",
                                alpha: float = 1.0, *, m: int = 1, epilogue: Optional[EpilogueConfig] = None,
                                epilogueInputs: Sequence[CudaTensor] = (), packing: Optional[QuantPacking] = None):
        """dispatch.ts:875-931.  ``m``, ``epilogue`` and ``packing`` are the
        widenings; with the defaults the call is the reference's."""
        if packing is None:
            packing = QuantPacking("int8-grouped", groupSize, "f16" if scales.dtype == "u16" else "f32")
        q = self._qdesc(packing)
        e = self._epilogue(epilogue, epilogueInputs)
        B.check(self._ctx, self._lib.tl_qgemv_nt(
            self._ctx, aBuffer.buffer, B.DTYPE_ID[aBuffer.dtype], packedWeight.buffer, scales.buffer,
            outBuffer.buffer, B.DTYPE_ID[outputDtype], m, n, k, C.byref(q), alpha,
            C.byref(e) if e is not None else None))

    def createQuantizedGemvChain(self, phases: Sequence[dict], m: int, scaleConvention: str = "direct"):
        """Vertical fusion (no counterpart in the reference): describe a sequence of dependent
        small-batch quantized products once, then run it as ONE persistent launch with
        ``runQuantizedGemvChain``.  Each phase is a dict
        ``{"a": CudaTensor [m,k], "k": int, "groupSize": int, "outputDtype": str, "items": [...]}``
        whose items are dicts ``{"packed", "scales", "out", "n", "alpha", "epilogue", "epilogueInputs"}``
        with the meaning of ``dispatchQuantizedGemvNT``'s arguments (1..4 items share the
        phase's activations)."""
        arr = (B.ChainPhase * len(phases))()
        keep = []
        scales_dtype = None
        for pi, ph in enumerate(phases):
            c = arr[pi]
            c.a, c.k, c.group_size = ph["a"].buffer, ph["k"], ph["groupSize"]
            c.out_dtype, c.n_items = B.DTYPE_ID[ph.get("outputDtype", "f32")], len(ph["items"])
            if len(ph["items"]) > 4:
                raise TlError(B.TL_ERR_INVALID_ARG, "chain: at most 4 items per phase")
            for ii, it in enumerate(ph["items"]):
                e = self._epilogue(it.get("epilogue"), it.get("epilogueInputs", ()))
                if e is not None:
                    keep.append(e)
                sd = "f16" if it["scales"].dtype == "u16" else "f32"
                if scales_dtype not in (None, sd):
                    raise TlError(B.TL_ERR_INVALID_ARG, "chain: all scales must share one dtype")
                scales_dtype = sd
                c.items[ii] = B.QGemvItem(it["packed"].buffer, it["scales"].buffer, it["out"].buffer, it["n"],
                                          it.get("alpha", 1.0), C.pointer(e) if e is not None else None)
        convention = B.TL_SCALE_SNORM127 if scaleConvention == "snorm127" else B.TL_SCALE_DIRECT
        handle = C.c_void_p()
        a_dtype = B.DTYPE_ID[phases[0]["a"].dtype]
        B.check(self._ctx, self._lib.tl_qgemv_chain_create(self._ctx, arr, len(phases), a_dtype, m,
                                                           B.DTYPE_ID[scales_dtype or "f32"], convention,
                                                           C.byref(handle)))
        return handle

    def runQuantizedGemvChain(self, chain):
        B.check(self._ctx, self._lib.tl_qgemv_chain_launch(self._ctx, chain))

    def destroyQuantizedGemvChain(self, chain):
        B.check(self._ctx, self._lib.tl_qgemv_chain_destroy(self._ctx, chain))

    def dispatchDequantizeInt8Grouped(self, packedWeight: CudaTensor, scales: CudaTensor, outBuffer: CudaTensor,
                                      n: int, k: int, groupSize: int, *, packing: Optional[QuantPacking] = None):
        """dispatch.ts:949-1037: explicit dequant to [N,K] of outBuffer.dtype."""
        if packing is None:
            packing = QuantPacking("int8-grouped", groupSize, "f16" if scales.dtype == "u16" else "f32")
        q = self._qdesc(packing)
        B.check(self._ctx, self._lib.tl_dequant_int8(self._ctx, packedWeight.buffer, scales.buffer, outBuffer.buffer,
                                                     B.DTYPE_ID[outBuffer.dtype], n, k, C.byref(q)))

    def dequantize(self, weight: CudaTensor, outDtype: str = "f32") -> CudaTensor:
        """Explicit dequant of a packed weight of either scheme to [N, K] (dispatch.ts:949-1037)."""
        packing = weight.format.packing
        n, k = weight.shape
        out = self.ops.empty([n, k], outDtype)
        q = self._qdesc(packing)
        fn = self._lib.tl_dequant_int8 if packing.scheme == "int8-grouped" else self._lib.tl_dequant_int4
        B.check(self._ctx, fn(self._ctx, weight.buffer, weight.scales.buffer, out.buffer, B.DTYPE_ID[outDtype], n, k, C.byref(q)))
        return out

    def unpackInt4(self, packedWeight: CudaTensor, n: int, k: int) -> np.ndarray:
        out = self.ops.empty([n, k], "i8")
        B.check(self._ctx, self._lib.tl_unpack_int4(self._ctx, packedWeight.buffer, out.buffer, n, k))
        r = self.ops.read(out)
        out.destroy()
        return r

    def unpackInt8(self, packedWeight: CudaTensor, n: int, k: int) -> np.ndarray:
        out = self.ops.empty([n, k], "i8")
        B.check(self._ctx, self._lib.tl_unpack_int8(self._ctx, packedWeight.buffer, out.buffer, n, k))
        r = self.ops.read(out)
        out.destroy()
        return r

    def _matmulQuantizedB(self, a: CudaTensor, b: CudaTensor, options: dict) -> CudaTensor:
        """matmul-ops.ts:113-182.  B is the transposed [K,N] view of a packed
        [N,K] weight.  Every M goes to a fused-dequant kernel (small-batch GEMV
        for M <= 16, tensor-core GEMM above), so no dequantized weight is ever
        materialized; the reference falls back to explicit dequant for M > 1."""
        packing = b.format.packing if b.format else None
        scales = b.scales
        if packing is None or scales is None:
            raise TlError(B.TL_ERR_INVALID_ARG, "matmulQuantizedB: missing packing/scales on B operand")
        if not b.transposed:
            raise TlError(B.TL_ERR_UNSUPPORTED, "matmulQuantizedB: B must be the transposed view of the [N,K] weight")
        k, n = b.shape[-2], b.shape[-1]
        if a.shape[-1] != k:
            raise TlError(B.TL_ERR_INVALID_ARG, "matmul dimension mismatch")
        m = int(np.prod(a.shape[:-1])) if len(a.shape) > 1 else 1
        epilogue: Optional[EpilogueConfig] = options.get("epilogue")
        epilogueInputs = options.get("epilogueInputs", ())
        out_dtype = epilogue.outputDtype if epilogue is not None else options.get("outputDtype", "f32")
        out_shape = (a.shape[:-1] if len(a.shape) > 1 else [1]) + [n]
        out = options.get("outBuffer") or self.ops.empty(out_shape, out_dtype)
        q = self._qdesc(packing)
        e = self._epilogue(epilogue, epilogueInputs)
        B.check(self._ctx, self._lib.tl_qmatmul_nt(
            self._ctx, a.buffer, B.DTYPE_ID[a.dtype], b.buffer, scales.buffer, out.buffer, B.DTYPE_ID[out_dtype],
            m, n, k, C.byref(q), float(options.get("alpha", 1.0)), C.byref(e) if e is not None else None))
        return out

    def dispatchMatmul(self, a: CudaTensor, b: CudaTensor, options: dict) -> CudaTensor:
        """dispatchMatmul for dense operands (src/backend/webgpu/matmul/dispatch.ts:1331-1700).
        ``a`` is [..., M, K] and ``b`` [..., K, N] (either may be the transposed view of a
        contiguous buffer); leading dims are the batch, and an operand without them is
        broadcast over the batch (dispatch.ts:1411-1510).  Options: ``epilogue`` /
        ``epilogueInputs`` / ``outputDtype`` / ``alpha`` / ``outBuffer`` as for the quantized
        product, ``inputCastA`` / ``inputCastB`` ("f16" | "bf16") for the cast-on-load
        prologue (variants.ts:170-175)."""
        for t in (a, b):
            if t.dtype not in ("f32", "f16", "bf16"):
                raise TlError(B.TL_ERR_UNSUPPORTED, f"matmul: unsupported operand dtype {t.dtype}")
        a_shape = list(a.shape) if len(a.shape) > 1 else [1] + list(a.shape)
        b_shape = list(b.shape)
        if len(b_shape) < 2:
            raise TlError(B.TL_ERR_INVALID_ARG, "matmul: B needs at least two dims")
        m, k = a_shape[-2], a_shape[-1]
        n = b_shape[-1]
        if b_shape[-2] != k:
            raise TlError(B.TL_ERR_INVALID_ARG, "matmul dimension mismatch")
        batch_a, batch_b = a_shape[:-2], b_shape[:-2]
        if batch_a and batch_b and batch_a != batch_b:
            raise TlError(B.TL_ERR_UNSUPPORTED, "matmul: batch dims must match or be absent on one operand")
        batch_dims = batch_a or batch_b
        batch = int(np.prod(batch_dims)) if batch_dims else 1
        if (a.transposed and batch_a) or (b.transposed and batch_b):
            raise TlError(B.TL_ERR_UNSUPPORTED, "matmul: a transposed view must be a single matrix")
        epilogue: Optional[EpilogueConfig] = options.get("epilogue")
        epilogueInputs = options.get("epilogueInputs", ())
        out_dtype = epilogue.outputDtype if epilogue is not None else options.get("outputDtype", "f32")
        # a flattened [rows, K] x [K, N] product (no batch on B) runs as ONE matrix of batch*M rows
        if batch > 1 and not batch_b and not a.transposed:
            m, batch = m * batch, 1
        out = options.get("outBuffer") or self.ops.empty(list(batch_dims) + [a_shape[-2], n], out_dtype)
        e = self._epilogue(epilogue, epilogueInputs)
        cast = {None: -1, "f16": B.TL_F16, "bf16": B.TL_BF16}
        B.check(self._ctx, self._lib.tl_matmul(
            self._ctx, a.buffer, b.buffer, out.buffer, m, n, k, batch,
            m * k if (batch_a and batch > 1) else 0, k * n if (batch_b and batch > 1) else 0, m * n,
            1 if a.transposed else 0, 1 if b.transposed else 0, float(options.get("alpha", 1.0)),
            B.DTYPE_ID[a.dtype], B.DTYPE_ID[b.dtype], B.DTYPE_ID[out_dtype],
            cast[options.get("inputCastA")], cast[options.get("inputCastB")],
            C.byref(e) if e is not None else None, None))
        return out

    def planMatmul(self, m, n, k, aDtype, bDtype, *, batch=1, transA=False, transB=False,
                   inputCastA=None, inputCastB=None):
        """planTiledMatmul for dense operands: which kernel a call of this geometry runs."""
        cast = {None: -1, "f16": B.TL_F16, "bf16": B.TL_BF16}
        r = B.PlanReceipt()
        B.check(self._ctx, self._lib.tl_matmul(
            self._ctx, None, None, None, m, n, k, batch, 0, 0, m * n, 1 if transA else 0, 1 if transB else 0, 1.0,
            B.DTYPE_ID[aDtype], B.DTYPE_ID[bDtype], B.TL_F32, cast[inputCastA], cast[inputCastB], None, C.byref(r)))
        return {"variant": self._lib.tl_variant_name(C.byref(r.choice)).decode(), "choice": r.choice.as_tuple(),
                "grid": list(r.grid), "block": r.block}

    def getGemvDispatchCount(self) -> int:
        return int(self._lib.tl_counter_get(self._ctx, B.TL_COUNTER_GEMV))

    def getTiledMatmulDispatchCount(self) -> int:
        return int(self._lib.tl_counter_get(self._ctx, B.TL_COUNTER_MATMUL))

    def linear(self, x: CudaTensor, weight: CudaTensor, bias: Optional[CudaTensor] = None,
               activation: Optional[str] = None, outputDtype: str = "f32") -> CudaTensor:
        """api.linear (torchlette.ts:878-894): transpose(weight) -> matmul -> add
        bias, with the following bias/activation/cast chain fused by the
        epilogue decision (matmul-epilogue.ts:131-262)."""
        chain = []
        if bias is not None:
            chain.append(("add", bias))
        if activation is not None:
            chain.append((activation, None))
        if outputDtype != "f32":
            chain.append(("cast", outputDtype))
        plan = detectMatmulEpilogue(chain)
        wT = self.ops.transpose(weight)
        opts: dict = {"outputDtype": outputDtype}
        if plan is not None:
            opts["epilogue"], opts["epilogueInputs"], _ = plan
        return self.ops.matmul(x, wT, opts)

    def swiglu(self, x: CudaTensor, gate: CudaTensor, up: CudaTensor, outputDtype: str = "f16") -> CudaTensor:
        """h = silu(x @ gate^T) * (x @ up^T), the gated MLP's first half
        (packages/qwen3-browser/src/model.ts:360-364), as two launches with NO element-wise kernel:
        the up projection stores f32, and the gate projection's epilogue is [silu, mul by that
        result, cast] -- the multiply rides in the second product's store loop.  Both weights may be
        packed (either scheme) or dense."""
        u = self.linear(x, up, None, None, "f32")
        chain = [("silu", None), ("mul", u)] + ([("cast", outputDtype)] if outputDtype != "f32" else [])
        plan = detectMatmulEpilogue(chain)
        h = self.ops.matmul(x, self.ops.transpose(gate), {"epilogue": plan[0], "epilogueInputs": plan[1], "outputDtype": outputDtype})
        u.destroy()
        return h

    # -- selection / counters / autotune --------------------------------------
    def planQuantizedMatmul(self, m, n, k, aDtype, outDtype, packing: QuantPacking,
                            epilogue: Optional[EpilogueConfig] = None):
        q = self._qdesc(packing)
        r = B.PlanReceipt()
        e = None
        if epilogue is not None:
            e = B.Epilogue()
            e.n_ops = 0  # geometry only; presence is reported through epilogue_engaged below
        B.check(self._ctx, self._lib.tl_plan_qmatmul(self._ctx, m, n, k, B.DTYPE_ID[aDtype], B.DTYPE_ID[outDtype],
                                                     C.byref(q), C.byref(e) if e is not None else None, C.byref(r)))
        name = self._lib.tl_variant_name(C.byref(r.choice)).decode()
        return {"family": "gemv" if r.choice.family == B.TL_FAMILY_QGEMV else "gemm", "variant": name,
                "choice": r.choice.as_tuple(), "grid": list(r.grid), "block": r.block, "splitK": r.split_k,
                "fromTuningCache": bool(r.from_tuning_cache),
                "tuningCacheLevel": {0: None, 1: "shape", 2: "shapeClass"}[r.from_tuning_cache]}

    def classifyShape(self, m: int, n: int, k: int, batchSize: int = 1) -> str:
        """classifyShape (src/backend/webgpu/matmul/types.ts:146-200)."""
        return self._lib.tl_shape_class_name(self._lib.tl_classify_shape(m, n, k, batchSize)).decode()

    def forceVariant(self, choice: Optional[tuple]):
        if choice is None:
            B.check(self._ctx, self._lib.tl_force_variant(self._ctx, None))
        else:
            v = B.Variant(*choice)
            B.check(self._ctx, self._lib.tl_force_variant(self._ctx, C.byref(v)))

    def setOption(self, name: str, value: int):
        """Per-context setting by name (tl_set_option); the counterpart of the
        reference's ENV accessor (src/core/env.ts:14-26)."""
        B.check(self._ctx, self._lib.tl_set_option(self._ctx, name.encode(), int(value)))

    def getOption(self, name: str) -> int:
        v = C.c_int64()
        B.check(self._ctx, self._lib.tl_get_option(self._ctx, name.encode(), C.byref(v)))
        return int(v.value)

    def getQuantGemvDispatchCount(self) -> int:
        return int(self._lib.tl_counter_get(self._ctx, B.TL_COUNTER_QGEMV))

    def getDequantI8DispatchCount(self) -> int:
        return int(self._lib.tl_counter_get(self._ctx, B.TL_COUNTER_DEQUANT))

    def getGemvEpilogueDispatchCount(self) -> int:
        return int(self._lib.tl_counter_get(self._ctx, B.TL_COUNTER_QGEMV_EPILOGUE))

    def getQuantGemmDispatchCount(self) -> int:
        return int(self._lib.tl_counter_get(self._ctx, B.TL_COUNTER_QGEMM))

    def getKernelLaunchCount(self) -> int:
        return int(self._lib.tl_counter_get(self._ctx, B.TL_COUNTER_KERNEL_LAUNCHES))

    def resetCounters(self):
        B.check(self._ctx, self._lib.tl_counters_reset(self._ctx))

    def setAutotuneEnabled(self, enabled: bool):
        B.check(self._ctx, self._lib.tl_autotune_set_enabled(self._ctx, 1 if enabled else 0))

    def isAutotuneEnabled(self) -> bool:
        return bool(self._lib.tl_autotune_is_enabled(self._ctx))

    def pretuneMatmulShapes(self, shapes, aDtype: str, outDtype: str, packing: QuantPacking):
        arr = (B.Shape * len(shapes))(*[B.Shape(*s) for s in shapes])
        q = self._qdesc(packing)
        B.check(self._ctx, self._lib.tl_pretune(self._ctx, arr, len(shapes), B.DTYPE_ID[aDtype],
                                                B.DTYPE_ID[outDtype], C.byref(q)))

    def seedPerShapeMatmulChoice(self, m, n, k, aDtype, packing: QuantPacking, choice: tuple):
        q = self._qdesc(packing)
        v = B.Variant(*choice)
        B.check(self._ctx, self._lib.tl_tune_seed(self._ctx, m, n, k, B.DTYPE_ID[aDtype], C.byref(q), C.byref(v)))

    def getPerShapeMatmulChoice(self, m, n, k, aDtype, packing: QuantPacking):
        q = self._qdesc(packing)
        v = B.Variant()
        found = self._lib.tl_tune_get(self._ctx, m, n, k, B.DTYPE_ID[aDtype], C.byref(q), C.byref(v))
        if found < 0:
            B.check(self._ctx, found)
        return v.as_tuple() if found == 1 else None

    def clearPerShapeMatmulChoices(self):
        B.check(self._ctx, self._lib.tl_tune_clear(self._ctx))

    def getAutotuneRunCount(self) -> int:
        return int(self._lib.tl_tune_run_count(self._ctx))

    def exportTuningCache(self) -> str:
        need = C.c_size_t()
        B.check(self._ctx, self._lib.tl_tune_export_json(self._ctx, None, 0, C.byref(need)))
        buf = C.create_string_buffer(need.value)
        B.check(self._ctx, self._lib.tl_tune_export_json(self._ctx, buf, need.value, C.byref(need)))
        return buf.value.decode()

    def importTuningCache(self, text: str):
        B.check(self._ctx, self._lib.tl_tune_import_json(self._ctx, text.encode()))

    # -- replay ---------------------------------------------------------------
    def beginCapture(self):
        B.check(self._ctx, self._lib.tl_graph_begin(self._ctx))

    def endCapture(self) -> int:
        g = C.c_void_p()
        B.check(self._ctx, self._lib.tl_graph_end(self._ctx, C.byref(g)))
        return g.value

    def replay(self, graph: int):
        B.check(self._ctx, self._lib.tl_graph_launch(self._ctx, C.c_void_p(graph)))

    def destroyGraph(self, graph: int):
        B.check(self._ctx, self._lib.tl_graph_destroy(self._ctx, C.c_void_p(graph)))


_backend: Optional[CudaBackend] = None
_init_error: Optional[str] = None


def initCuda(device: int = 0) -> bool:
    """initWebGPU's counterpart (src/backend/webgpu/index.ts:39-70): returns
    False and records the error when no usable device/library exists."""
    global _backend, _init_error
    if _backend is not None:
        return True
    try:
        _backend = CudaBackend(device)
        return True
    except (TlError, ImportError, OSError) as e:  # no GPU, or library not built
        _init_error = str(e)
        return False


def getCudaInitError() -> Optional[str]:
    return _init_error


def getBackend() -> CudaBackend:
    if _backend is None and not initCuda():
        raise RuntimeError(f"cuda backend unavailable: {_init_error}")
    return _backend


def destroyCuda():
    global _backend
    if _backend is not None:
        _backend.destroy()
        _backend = None
