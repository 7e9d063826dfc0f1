"""ctypes binding of libtlcuda.so — a 1:1 map of ``include/tlcuda.h``.

The library is built in-tree (``torchlette_b200/csrc/libtlcuda.so``).  There is
no CPU fallback: if the shared object is missing, or no sm_100 GPU is present
when a context is created, the call raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TLCUDA_LIB") or os.path.join(_HERE, "csrc", "libtlcuda.so")

TL_OK = 0
TL_ERR_INVALID_ARG, TL_ERR_UNSUPPORTED, TL_ERR_CUDA, TL_ERR_NCCL = -1, -2, -3, -4
TL_ERR_TIMEOUT, TL_ERR_OOM, TL_ERR_UNIMPLEMENTED = -5, -6, -7
TL_F32, TL_F16, TL_BF16 = 0, 1, 2
TL_SCHEME_INT8_GROUPED, TL_SCHEME_INT4_GROUPED = 1, 2
TL_SCALE_SNORM127, TL_SCALE_DIRECT = 0, 1
TL_EPI_NONE, TL_EPI_BIAS, TL_EPI_UNARY, TL_EPI_BINARY, TL_EPI_CAST = 0, 1, 2, 3, 4
TL_UNARY = {"relu": 1, "silu": 2, "sigmoid": 3, "tanh": 4, "gelu": 5, "gelu_tanh": 5, "gelu_erf": 6}
TL_BINARY = {"add": 1, "sub": 2, "mul": 3}
TL_FAMILY_QGEMV, TL_FAMILY_QGEMM, TL_FAMILY_MATMUL = 1, 2, 3
TL_COUNTER_QGEMV, TL_COUNTER_DEQUANT, TL_COUNTER_QGEMV_EPILOGUE = 0, 1, 2
TL_COUNTER_QGEMM, TL_COUNTER_KERNEL_LAUNCHES, TL_COUNTER_GEMV, TL_COUNTER_MATMUL = 3, 4, 5, 6
TL_EPI_MAX_OPS, TL_EPI_MAX_INPUTS = 8, 4
TL_COMM_ID_BYTES = 128

DTYPE_ID = {"f32": TL_F32, "f16": TL_F16, "bf16": TL_BF16}
DTYPE_NAME = {v: k for k, v in DTYPE_ID.items()}
DTYPE_SIZE = {"f32": 4, "f16": 2, "bf16": 2}


class QuantDesc(C.Structure):
    _fields_ = [("scheme", C.c_int32), ("group_size", C.c_int32), ("scales_dtype", C.c_int32),
                ("scale_convention", C.c_int32)]


class EpilogueOp(C.Structure):
    _fields_ = [("kind", C.c_int32), ("op", C.c_int32), ("input_index", C.c_int32), ("to_dtype", C.c_int32)]


class Epilogue(C.Structure):
    _fields_ = [("n_ops", C.c_int32), ("ops", EpilogueOp * TL_EPI_MAX_OPS), ("n_inputs", C.c_int32),
                ("inputs", C.c_void_p * TL_EPI_MAX_INPUTS)]


class QGemvItem(C.Structure):
    _fields_ = [("packed", C.c_void_p), ("scales", C.c_void_p), ("out", C.c_void_p), ("n", C.c_int64),
                ("alpha", C.c_float), ("epilogue", C.POINTER(Epilogue))]


class ChainPhase(C.Structure):
    _fields_ = [("a", C.c_void_p), ("k", C.c_int64), ("group_size", C.c_int32), ("out_dtype", C.c_int32),
                ("n_items", C.c_int32), ("reserved", C.c_int32), ("items", QGemvItem * 4)]


class Variant(C.Structure):
    _fields_ = [("family", C.c_int32), ("kernel", C.c_int32), ("p0", C.c_int32), ("p1", C.c_int32),
                ("p2", C.c_int32), ("p3", C.c_int32)]

    def as_tuple(self):
        return (self.family, self.kernel, self.p0, self.p1, self.p2, self.p3)


class PlanReceipt(C.Structure):
    _fields_ = [("choice", Variant), ("grid", C.c_int32 * 3), ("block", C.c_int32), ("split_k", C.c_int32),
                ("from_tuning_cache", C.c_int32), ("epilogue_engaged", C.c_int32)]


class Shape(C.Structure):
    _fields_ = [("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64)]


# name -> (restype, argtypes); every symbol include/tlcuda.h declares
_P, _I32, _I64, _SZ, _F = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float
_QARGS = [_P, _P, _I32, _P, _P, _P, _I32]
SIGNATURES = {
    "tl_ctx_create": (_I32, [_I32, C.POINTER(_P)]),
    "tl_ctx_destroy": (_I32, [_P]),
    "tl_sync": (_I32, [_P]),
    "tl_async_error_count": (_I64, [_P]),
    "tl_last_error": (C.c_char_p, [_P]),
    "tl_ctx_stream": (_I32, [_P, C.POINTER(_P)]),
    "tl_device_sm_count": (_I32, [_P, C.POINTER(_I32)]),
    "tl_set_option": (_I32, [_P, C.c_char_p, _I64]),
    "tl_get_option": (_I32, [_P, C.c_char_p, C.POINTER(_I64)]),
    "tl_alloc": (_I32, [_P, _SZ, C.POINTER(_P)]),
    "tl_free": (_I32, [_P, _P]),
    "tl_upload": (_I32, [_P, _P, _P, _SZ]),
    "tl_download": (_I32, [_P, _P, _P, _SZ]),
    "tl_host_alloc_pinned": (_I32, [_P, _SZ, C.POINTER(_P)]),
    "tl_host_free_pinned": (_I32, [_P, _P]),
    "tl_memset": (_I32, [_P, _P, _I32, _SZ]),
    "tl_copy2d": (_I32, [_P, _P, _SZ, _P, _SZ, _SZ, _SZ]),
    "tl_quantize_linear_weight": (_I32, [_P, _I64, _I64, _I32, _P, _P]),
    "tl_quantize_linear_weight_device": (_I32, [_P, _P, _I64, _I64, _I32, _P, _P]),
    "tl_f32_to_f16_bits": (C.c_uint32, [_F]),
    "tl_f16_bits_to_f32": (_F, [C.c_uint32]),
    "tl_qgemv_nt": (_I32, _QARGS + [_I32, _I64, _I64, C.POINTER(QuantDesc), _F, C.POINTER(Epilogue)]),
    "tl_qgemv_nt_static_scratch": (_I32, _QARGS + [_I32, _I64, _I64, C.POINTER(QuantDesc), _F, C.POINTER(Epilogue)]),
    "tl_qgemv_nt_batched": (_I32, [_P, _P, _I32, C.POINTER(QGemvItem), _I32, _I32, _I32, _I64, C.POINTER(QuantDesc)]),
    "tl_qgemv_nt_allreduce": (_I32, _QARGS + [_I32, _I64, _I64, C.POINTER(QuantDesc), _F]),
    "tl_qgemv_chain_create": (_I32, [_P, C.POINTER(ChainPhase), _I32, _I32, _I32, _I32, _I32, C.POINTER(C.c_void_p)]),
    "tl_qgemv_chain_launch": (_I32, [_P, _P]),
    "tl_qgemv_chain_destroy": (_I32, [_P, _P]),
    "tl_qgemm_nt": (_I32, _QARGS + [_I64, _I64, _I64, C.POINTER(QuantDesc), _F, C.POINTER(Epilogue)]),
    "tl_qmatmul_nt": (_I32, _QARGS + [_I64, _I64, _I64, C.POINTER(QuantDesc), _F, C.POINTER(Epilogue)]),
    "tl_matmul": (_I32, [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _I32, _I32, _F, _I32, _I32, _I32,
                         _I32, _I32, C.POINTER(Epilogue), C.POINTER(PlanReceipt)]),
    "tl_quantize_linear_weight_int4": (_I32, [_P, _I64, _I64, _I32, _P, _P]),
    "tl_dequant_int4": (_I32, [_P, _P, _P, _P, _I32, _I64, _I64, C.POINTER(QuantDesc)]),
    "tl_unpack_int4": (_I32, [_P, _P, _P, _I64, _I64]),
    "tl_unary_op": (_I32, [_P, _I32, _P, _I32, _P, _I32, _I64]),
    "tl_binary_op": (_I32, [_P, _I32, _P, _I32, _P, _I32, _P, _I32, _I64, _I64, _I32]),
    "tl_transpose2d": (_I32, [_P, _P, _P, _I64, _I64, _I64, _I32]),
    "tl_rmsnorm": (_I32, [_P, _P, _I32, _P, _I32, _P, _I32, _I64, _I64, _F]),
    "tl_rope": (_I32, [_P, _P, _I32, _P, _P, _P, _I64, _I64, _I64, _F, _I64, _I64]),
    "tl_attention": (_I32, [_P, _P, _P, _P, _P, _I32, _I64, _I64, _I64, _I64, _I64, _I64, _I64, _F, _P, _I32]),
    "tl_decode_attention": (_I32, [_P, _P, _P, _P, _P, _I32, _I64, _I64, _I64, _I64, _I64, _I64, _F, _P]),
    "tl_dequant_int8": (_I32, [_P, _P, _P, _P, _I32, _I64, _I64, C.POINTER(QuantDesc)]),
    "tl_unpack_int8": (_I32, [_P, _P, _P, _I64, _I64]),
    "tl_plan_qmatmul": (_I32, [_P, _I64, _I64, _I64, _I32, _I32, C.POINTER(QuantDesc), C.POINTER(Epilogue),
                               C.POINTER(PlanReceipt)]),
    "tl_variant_name": (C.c_char_p, [C.POINTER(Variant)]),
    "tl_force_variant": (_I32, [_P, C.POINTER(Variant)]),
    "tl_counter_get": (_I64, [_P, _I32]),
    "tl_counters_reset": (_I32, [_P]),
    "tl_classify_shape": (_I32, [_I64, _I64, _I64, _I64]),
    "tl_shape_class_name": (C.c_char_p, [_I32]),
    "tl_autotune_set_enabled": (_I32, [_P, _I32]),
    "tl_autotune_is_enabled": (_I32, [_P]),
    "tl_pretune": (_I32, [_P, C.POINTER(Shape), _I32, _I32, _I32, C.POINTER(QuantDesc)]),
    "tl_tune_seed": (_I32, [_P, _I64, _I64, _I64, _I32, C.POINTER(QuantDesc), C.POINTER(Variant)]),
    "tl_tune_get": (_I32, [_P, _I64, _I64, _I64, _I32, C.POINTER(QuantDesc), C.POINTER(Variant)]),
    "tl_tune_clear": (_I32, [_P]),
    "tl_tune_run_count": (_I64, [_P]),
    "tl_tune_export_json": (_I32, [_P, C.c_char_p, _SZ, C.POINTER(_SZ)]),
    "tl_tune_import_json": (_I32, [_P, C.c_char_p]),
    "tl_graph_begin": (_I32, [_P]),
    "tl_graph_end": (_I32, [_P, C.POINTER(_P)]),
    "tl_graph_launch": (_I32, [_P, _P]),
    "tl_graph_destroy": (_I32, [_P, _P]),
    "tl_event_create": (_I32, [_P, C.POINTER(_P)]),
    "tl_event_record": (_I32, [_P, _P]),
    "tl_event_elapsed_ms": (_I32, [_P, _P, _P, C.POINTER(_F)]),
    "tl_event_synchronize": (_I32, [_P, _P]),
    "tl_event_destroy": (_I32, [_P, _P]),
    "tl_comm_unique_id": (_I32, [_P]),
    "tl_comm_init": (_I32, [_P, _I32, _I32, _P]),
    "tl_comm_destroy": (_I32, [_P]),
    "tl_allgather_cols": (_I32, [_P, _P, _P, _I64, _I64, _I32]),
    "tl_allreduce_sum": (_I32, [_P, _P, _I64, _I32]),
    "tl_p2p_create": (_I32, [_P, _SZ, _P]),
    "tl_p2p_attach": (_I32, [_P, _P]),
    "tl_allreduce_sum_p2p": (_I32, [_P, _P, _P, _I64, _I32]),
    "tl_allreduce_sum_p2p_f32_to": (_I32, [_P, _P, _P, _I32, _I64]),
    "tl_p2p_reset": (_I32, [_P]),
    "tl_qgemv_nt_push": (_I32, _QARGS + [_I32, _I64, _I64, C.POINTER(QuantDesc), _F]),
    "tl_reduce_pending": (_I32, [_P]),
    "tl_p2p_attach_loopback": (_I32, [_P, _I32]),
}


class TlError(RuntimeError):
    """A non-zero status from the library, carrying tl_last_error()'s message
    (the reference throws a JS Error with a descriptive message in the same
    situations)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[tl status {status}] {message}")
        self.status = status
        self.message = message


_lib = None


def load():
    """Load libtlcuda.so; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m torchlette_b200._build` "
            "(there is no CPU or WebGPU fallback on this path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header/library mismatch
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(ctx, status: int):
    if status != TL_OK:
        msg = load().tl_last_error(ctx)
        raise TlError(status, msg.decode() if msg else "")
    return status


def preload_nccl():
    """Make the NCCL that ships with torch visible to dlopen("libnccl.so.2")."""
    try:
        import nvidia.nccl  # type: ignore

        for base in list(nvidia.nccl.__path__):
            p = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(p):
                C.CDLL(p, mode=C.RTLD_GLOBAL)
                os.environ.setdefault("TL_NCCL_LIB", p)
                return p
    except Exception:
        pass
    return None
