"""CPU oracle for the quantized-weight matmul path — TEST INFRASTRUCTURE ONLY.

Loads ``libtloracle.so`` (built from ``tl_oracle.c`` by the Makefile beside it)
and exposes the restated torchlette CPU arithmetic as numpy-in / numpy-out
functions.  Only the tests, the smoke check and the CPU-baseline leg of the
benchmark import this module; the shipped library never does.

PARITY UNPINNED: the reference holds no golden vectors for this path and cannot
be executed where this was written, so the restatement is pinned procedurally
(IEEE facts, an independent numpy restatement in this file, the reference
probes' seeds / shapes / tolerances).

The ``np_*`` functions are a second, independent restatement in vectorised
numpy used to cross-check the C code.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtloracle.so")

RELU, SILU, SIGMOID, TANH, GELU_TANH, GELU_ERF = 1, 2, 3, 4, 5, 6
UNARY_BY_NAME = {
    "relu": RELU, "silu": SILU, "sigmoid": SIGMOID, "tanh": TANH,
    "gelu": GELU_TANH, "gelu_tanh": GELU_TANH, "gelu_erf": GELU_ERF,
}


def build(force: bool = False) -> str:
    """Compile the C restatement if the shared object is missing or stale."""
    src = os.path.join(_HERE, "tl_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libtloracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        p = C.c_void_p
        i64 = C.c_int64
        L.orc_f32_to_f16_bits.argtypes = [C.c_float]
        L.orc_f32_to_f16_bits.restype = C.c_uint32
        L.orc_f16_bits_to_f32.argtypes = [C.c_uint32]
        L.orc_f16_bits_to_f32.restype = C.c_float
        L.orc_quantize_linear_weight.argtypes = [p, i64, i64, i64, p, p]
        L.orc_quantize_linear_weight.restype = C.c_int
        L.orc_unpack_int8.argtypes = [p, i64, i64, p]
        L.orc_quantize_linear_weight_int4.argtypes = [p, i64, i64, i64, p, p]
        L.orc_quantize_linear_weight_int4.restype = C.c_int
        L.orc_unpack_int4.argtypes = [p, i64, i64, p]
        L.orc_dequantize_int4_to_f32.argtypes = [p, p, i64, i64, i64, p]
        L.orc_dequantize_to_f32.argtypes = [p, p, i64, i64, i64, p]
        L.orc_dequantize_direct_f32.argtypes = [p, p, i64, i64, i64, p]
        L.orc_matmul_nt.argtypes = [p, p, p, i64, i64, i64, C.c_int]
        L.orc_unary_f64.argtypes = [C.c_int, C.c_double]
        L.orc_unary_f64.restype = C.c_double
        L.orc_unary.argtypes = [C.c_int, p, p, i64]
        L.orc_add_bias.argtypes = [p, p, p, i64, i64]
        L.orc_lcg_fill.argtypes = [C.c_uint32, C.c_double, p, i64]
        L.orc_lcg_fill.restype = C.c_uint32
        L.orc_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


# --------------------------------------------------------------------------
# C-backed restatement
# --------------------------------------------------------------------------

def f32_to_f16_bits(values) -> np.ndarray:
    """quantize.ts:22-47, elementwise."""
    v = _c(values, np.float32).ravel()
    L = lib()
    return np.array([L.orc_f32_to_f16_bits(float(x)) for x in v], dtype=np.uint16).reshape(np.shape(values))


def f16_bits_to_f32(bits) -> np.ndarray:
    """quantize.ts:50-60, elementwise."""
    b = _c(bits, np.uint16).ravel()
    L = lib()
    return np.array([L.orc_f16_bits_to_f32(int(x)) for x in b], dtype=np.float32).reshape(np.shape(bits))


def quantize_linear_weight(weight: np.ndarray, group: int = 64):
    """quantize.ts:77-131 -> (packed u32 [N,K/4], scales u16 [N,K/G])."""
    w = _c(weight, np.float32)
    n, k = w.shape
    packed = np.zeros((n, k // 4), dtype=np.uint32)
    scales = np.zeros((n, k // group), dtype=np.uint16)
    rc = lib().orc_quantize_linear_weight(_ptr(w), n, k, group, _ptr(packed), _ptr(scales))
    if rc != 0:
        raise ValueError(f"quantize: K={k} must be divisible by 4 and by groupSize={group}")
    return packed, scales


def quantize_linear_weight_int4(weight: np.ndarray, group: int = 32):
    """The planned int4-grouped scheme (docs/quantization-design.md:69-75), by analogy with
    quantize.ts:77-131 -> (packed u32 [N,K/8], scales u16 [N,K/G])."""
    w = _c(weight, np.float32)
    n, k = w.shape
    packed = np.zeros((n, k // 8), dtype=np.uint32)
    scales = np.zeros((n, k // group), dtype=np.uint16)
    rc = lib().orc_quantize_linear_weight_int4(_ptr(w), n, k, group, _ptr(packed), _ptr(scales))
    if rc != 0:
        raise ValueError(f"quantize int4: K={k} must be divisible by 8 and by groupSize={group}")
    return packed, scales


def unpack_int4(packed: np.ndarray, k: int) -> np.ndarray:
    pk = _c(packed, np.uint32)
    n = pk.size * 8 // k
    out = np.empty((n, k), dtype=np.int8)
    lib().orc_unpack_int4(_ptr(pk), n, k, _ptr(out))
    return out


def dequantize_int4_to_f32(packed, scales_f16_bits, k: int, group: int) -> np.ndarray:
    pk = _c(packed, np.uint32)
    sc = _c(scales_f16_bits, np.uint16)
    n = pk.size * 8 // k
    out = np.empty((n, k), dtype=np.float32)
    lib().orc_dequantize_int4_to_f32(_ptr(pk), _ptr(sc), n, k, group, _ptr(out))
    return out


def unpack_int8(packed: np.ndarray, k: int) -> np.ndarray:
    pk = _c(packed, np.uint32)
    n = pk.shape[0]
    out = np.empty((n, k), dtype=np.int8)
    lib().orc_unpack_int8(_ptr(pk), n, k, _ptr(out))
    return out


def dequantize_to_f32(packed, scales_f16_bits, k: int, group: int) -> np.ndarray:
    """quantize.ts:138-156 (snorm127 convention, f16 scales)."""
    pk = _c(packed, np.uint32)
    sc = _c(scales_f16_bits, np.uint16)
    n = pk.shape[0]
    out = np.empty((n, k), dtype=np.float32)
    lib().orc_dequantize_to_f32(_ptr(pk), _ptr(sc), n, k, group, _ptr(out))
    return out


def dequantize_direct_f32(packed, scales_f32, k: int, group: int) -> np.ndarray:
    """Benchmark-config convention: w = f32(q * s), f32 scales [N, K/G]."""
    pk = _c(packed, np.uint32)
    sc = _c(scales_f32, np.float32)
    n = pk.shape[0]
    out = np.empty((n, k), dtype=np.float32)
    lib().orc_dequantize_direct_f32(_ptr(pk), _ptr(sc), n, k, group, _ptr(out))
    return out


def matmul_nt(a: np.ndarray, w: np.ndarray, threads: int = 0) -> np.ndarray:
    """numeric.ts:510-595 with B = transposed view of w [N,K]; a is [M,K] f32."""
    a32 = _c(a, np.float32)
    w32 = _c(w, np.float32)
    m, k = a32.shape
    n, k2 = w32.shape
    assert k == k2
    out = np.empty((m, n), dtype=np.float32)
    lib().orc_matmul_nt(_ptr(a32), _ptr(w32), _ptr(out), m, n, k, threads)
    return out


def unary(name_or_op, x: np.ndarray) -> np.ndarray:
    op = UNARY_BY_NAME[name_or_op] if isinstance(name_or_op, str) else int(name_or_op)
    x32 = _c(x, np.float32)
    out = np.empty_like(x32)
    lib().orc_unary(op, _ptr(x32), _ptr(out), x32.size)
    return out


def add_bias(x: np.ndarray, bias: np.ndarray) -> np.ndarray:
    x32 = _c(x, np.float32)
    b32 = _c(bias, np.float32)
    m, n = x32.shape
    out = np.empty_like(x32)
    lib().orc_add_bias(_ptr(x32), _ptr(b32), _ptr(out), m, n)
    return out


def lcg_fill(state: int, count: int, mul: float = 1.0):
    """probe-quant-gemv.ts:44-50 stream; returns (values f32, next state)."""
    out = np.empty(count, dtype=np.float32)
    nxt = lib().orc_lcg_fill(state & 0xFFFFFFFF, mul, _ptr(out), count)
    return out, int(nxt)


def max_threads() -> int:
    return int(lib().orc_max_threads())


def linear_reference(a_f32, w_f32, bias=None, act=None, alpha: float = 1.0, threads: int = 0):
    """The reference's unfused CPU sequence for ``act(linear(a, w) + bias)``:
    matmul (f32 store) -> optional alpha multiply -> bias add (f32 store) ->
    activation (f32 store).  numeric.ts:510-595, 448-466, 436-447."""
    y = matmul_nt(a_f32, w_f32, threads)
    if alpha != 1.0:
        y = (y.astype(np.float64) * alpha).astype(np.float32)
    if bias is not None:
        y = add_bias(y, bias)
    if act:
        y = unary(act, y)
    return y


# --------------------------------------------------------------------------
# Independent numpy restatement (cross-check of the C code)
# --------------------------------------------------------------------------

def np_unpack_int8(packed: np.ndarray, k: int) -> np.ndarray:
    pk = _c(packed, np.uint32)
    return pk.view(np.uint8).reshape(pk.shape[0], -1)[:, :k].view(np.int8) if np.little_endian else None


def np_dequantize_to_f32(packed, scales_f16_bits, k: int, group: int) -> np.ndarray:
    q = np_unpack_int8(packed, k).astype(np.float64)
    s = _c(scales_f16_bits, np.uint16).view(np.float16).astype(np.float64)
    return ((q / 127.0) * np.repeat(s, group, axis=1)).astype(np.float32)


def np_dequantize_direct_f32(packed, scales_f32, k: int, group: int) -> np.ndarray:
    q = np_unpack_int8(packed, k).astype(np.float64)
    s = _c(scales_f32, np.float32).astype(np.float64)
    return (q * np.repeat(s, group, axis=1)).astype(np.float32)


def np_matmul_nt_small(a, w) -> np.ndarray:
    """Sequential-k f64 accumulation with python loops over k (small cases)."""
    a64 = _c(a, np.float32).astype(np.float64)
    w64 = _c(w, np.float32).astype(np.float64)
    acc = np.zeros((a64.shape[0], w64.shape[0]), dtype=np.float64)
    for kk in range(a64.shape[1]):
        acc += np.outer(a64[:, kk], w64[:, kk])
    return acc.astype(np.float32)


def np_unary(name: str, x) -> np.ndarray:
    v = _c(x, np.float32).astype(np.float64)
    if name == "relu":
        r = np.where(v > 0, v, 0.0)
    elif name == "silu":
        r = v / (1.0 + np.exp(-v))
    elif name == "sigmoid":
        r = 1.0 / (1.0 + np.exp(-v))
    elif name == "tanh":
        r = np.tanh(v)
    elif name in ("gelu", "gelu_tanh"):
        r = (0.5 * v) * (1.0 + np.tanh(0.7978845608 * (v + 0.044715 * (v * (v * v)))))
    elif name == "gelu_erf":
        a = [0.254829592, -0.284496736, 1.421413741, -1.453152027, 1.061405429]
        u = v * 0.7071067811865476
        ax = np.abs(u)
        t = 1.0 / (1.0 + 0.3275911 * ax)
        poly = ((((a[4] * t + a[3]) * t + a[2]) * t + a[1]) * t + a[0]) * t
        r = (0.5 * v) * (1.0 + np.where(u < 0, -1.0, 1.0) * (1.0 - poly * np.exp(-ax * ax)))
    else:
        raise KeyError(name)
    return r.astype(np.float32)


def np_lcg(state: int, count: int, mul: float = 1.0):
    out = np.empty(count, dtype=np.float32)
    s = state & 0xFFFFFFFF
    for i in range(count):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32((s / 2 ** 31 - 1) * mul)
    return out, s


# --------------------------------------------------------------------------
# bit-pattern helpers shared by tests and bench (exact widenings)
# --------------------------------------------------------------------------

def bf16_bits_rne(x_f32: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns, round-to-nearest-even (finite inputs)."""
    u = _c(x_f32, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (_c(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)
