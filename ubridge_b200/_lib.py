"""ctypes binding of ``libubridge_b200.so`` (the C-ABI declared in ``include/ubridge_b200.h``).

The library is the only compute path: if it is missing or fails to load, importing a symbol from
here raises; there is no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_size_t, c_uint32, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libubridge_b200.so")

UB_OK = 0
UB_ERR_INVALID_ARG = 1
UB_ERR_UNSUPPORTED = 2
UB_ERR_WORKSPACE = 3
UB_ERR_CUDA = 4
UB_ERR_BAD_INDEX = 5
UB_ERR_TIMEOUT = 6
UB_ERR_NCCL = 7
UB_ERR_TOO_LARGE = 8
UB_ERR_NOT_READY = 9

# element type codes (the reference's DATATYPE enum, src/lib.rs:87-106)
DTYPE_I8, DTYPE_U8, DTYPE_F16, DTYPE_BF16, DTYPE_I32, DTYPE_F32 = 0, 1, 4, 5, 6, 8
# OR into out_dtype of ub_qmatmul_*: the weight bytes were written by the kernel launched just before on the stream
UB_QMATMUL_WEIGHTS_FRESH = 0x100
# GGML type tags of the GGUF formats the library takes
GGML_Q4_0, GGML_Q8_0, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K = 2, 8, 12, 13, 14


class UbridgeError(RuntimeError):
    def __init__(self, status: int, what: str = ""):
        self.status = status
        msg = "ubridge_b200: %s (status %d)" % (status_string(status), status)
        if what:
            msg = "%s in %s" % (msg, what)
        if status == UB_ERR_CUDA:
            msg += " [cudaError %d]" % lib().ub_last_cuda_error()
        super().__init__(msg)


class LaunchConfig(ctypes.Structure):
    """ub_launch_config: mirrors GcuLaunchConfig (src/gcu_launch.rs:40-90)."""

    _fields_ = [("grid_dim", ctypes.c_uint * 3), ("block_dim", ctypes.c_uint * 3),
                ("shared_mem_bytes", ctypes.c_uint), ("is_cooperative_launch", c_int)]


class EcclUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * 128)]


_lib = None

_P = c_void_p
_SIGS = {
    "ub_version": (c_int, []),
    "ub_status_string": (c_char_p, [c_int]),
    "ub_last_status": (c_int, []),
    "ub_last_cuda_error": (c_int, []),
    "ub_device_status": (c_int, [_P]),
    "ub_device_count": (c_int, []),
    "ub_device_new": (c_int, [c_int, POINTER(_P)]),
    "ub_device_free": (None, [_P]),
    "ub_device_ordinal": (c_int, [_P]),
    "ub_device_stream": (_P, [_P]),
    "ub_device_bind": (c_int, [_P]),
    "ub_alloc": (c_int, [_P, c_size_t, POINTER(_P)]),
    "ub_alloc_zeros": (c_int, [_P, c_size_t, POINTER(_P)]),
    "ub_free": (c_int, [_P, _P]),
    "ub_memcpy_htod": (c_int, [_P, _P, _P, c_size_t]),
    "ub_memcpy_dtoh": (c_int, [_P, _P, _P, c_size_t]),
    "ub_memcpy_dtod": (c_int, [_P, _P, _P, c_size_t]),
    "ub_memcpy_dtod_2d": (c_int, [_P, _P, c_size_t, _P, c_size_t, c_size_t, c_size_t]),
    "ub_p2p_alloc": (c_int, [c_size_t, ctypes.POINTER(_P)]),
    "ub_p2p_free": (c_int, [_P]),
    "ub_ipc_get_handle": (c_int, [_P, _P]),
    "ub_ipc_open_handle": (c_int, [_P, ctypes.POINTER(_P)]),
    "ub_ipc_close_handle": (c_int, [_P]),
    "ub_enable_peer_access": (c_int, [c_int]),
    "ub_allreduce_oneshot_staging_bytes": (c_size_t, [c_int, c_size_t]),
    "ub_allreduce_oneshot_bf16": (c_int, [_P, c_size_t, ctypes.POINTER(_P), c_int, c_int, c_size_t, _P]),
    "ub_allreduce_oneshot_set_spin_limit": (ctypes.c_uint, [ctypes.c_uint]),
    "ub_synchronize": (c_int, [_P]),
    "ub_stream_query": (c_int, [_P]),
    "ub_mem_info": (c_int, [_P, POINTER(c_size_t), POINTER(c_size_t)]),
    "ub_get_function": (_P, [c_char_p, c_char_p]),
    "ub_has_function": (c_int, [c_char_p, c_char_p]),
    "ub_function_count": (c_int, []),
    "ub_function_name": (c_char_p, [c_int]),
    "ub_function_opcode": (c_int, [_P]),
    "ub_launch": (c_int, [_P, POINTER(LaunchConfig), POINTER(_P), _P]),
    "ub_dequant_q8_0": (c_int, [_P, _P, c_size_t, c_int, _P]),
    "ub_dequant_q4k": (c_int, [_P, _P, c_size_t, c_int, _P]),
    "ub_quantize_q8_0": (c_int, [_P, _P, c_size_t, c_int, _P]),
    "ub_repack_to_split": (c_int, [_P, _P, c_size_t, c_int, _P]),
    "ub_repack_to_interleaved": (c_int, [_P, _P, c_size_t, c_int, _P]),
    "ub_gguf_block_values": (c_int, [c_int]),
    "ub_gguf_block_bytes": (c_int, [c_int]),
    "ub_gguf_tensor_bytes": (c_size_t, [c_int, c_size_t]),
    "ub_dequant_gguf": (c_int, [_P, _P, c_int, c_size_t, c_int, _P]),
    "ub_qmatmul_gguf_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "ub_qmatmul_gguf": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "ub_dequant_q6k": (c_int, [_P, _P, c_size_t, c_int, _P]),
    "ub_qmatmul_q6k_f32": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "ub_qmatmul_q6k_bf16": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "ub_qmatmul_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "ub_qmatmul_q8_0_f32": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "ub_qmatmul_q8_0_bf16": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "ub_qmatmul_q4k_f32": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "ub_qmatmul_q4k_bf16": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "ub_qmatmul_q4k_gate_up_workspace_bytes": (c_size_t, [c_int, c_int, c_int]),
    "ub_qmatmul_q4k_gate_up_bf16": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "ub_qmatmul_q4k_allreduce_bf16": (c_int, [_P, _P, _P, c_int, c_int, c_int, ctypes.POINTER(_P), c_int, c_int,
                                              c_size_t, _P]),
    "ub_qmatmul_q4k_allreduce_residual_bf16": (c_int, [_P, _P, _P, _P, c_int, c_int, c_int, ctypes.POINTER(_P), c_int,
                                                       c_int, c_size_t, _P]),
    "topsaten_rms_norm": (c_int, [_P, _P, _P, c_int, c_int, ctypes.c_float, c_int, _P]),
    "ub_qmatmul_q4k_rmsnorm_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "ub_qmatmul_q4k_rmsnorm_bf16": (c_int, [_P, _P, _P, ctypes.c_float, _P, c_int, c_int, c_int, c_int, c_int, _P,
                                            c_size_t, _P]),
    "ub_qmatmul_q4k_f32_static": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "topk_softmax_f32": (None, [_P, _P, _P, c_int32, c_int32, c_int32, c_int32, _P]),
    "topk_softmax_f16": (None, [_P, _P, _P, c_int32, c_int32, c_int32, c_int32, _P]),
    "topk_softmax_bf16": (None, [_P, _P, _P, c_int32, c_int32, c_int32, c_int32, _P]),
    "moe_align_block_size": (None, [_P, _P, _P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, _P]),
    "invoke_fused_moe_f16": (None, [_P] * 8 + [c_int32] * 9 + [_P]),
    "invoke_fused_moe_bf16": (None, [_P] * 8 + [c_int32] * 9 + [_P]),
    "moe_f16": (None, [_P] * 5 + [c_int] * 4 + [_P]),
    "moe_bf16": (None, [_P] * 5 + [c_int] * 4 + [_P]),
    "indexed_moe_f16": (None, [_P] * 4 + [c_int] * 6 + [_P]),
    "indexed_moe_bf16": (None, [_P] * 4 + [c_int] * 6 + [_P]),
    "dequant_f16": (None, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "dequant_bf16": (None, [_P, _P, _P, _P, c_int, c_int, c_int, c_int, _P]),
    "topsaten_topk_softmax_f32": (c_int, [_P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, _P]),
    "topsaten_moe_align_block_size": (c_int, [_P, _P, _P, _P, c_int32, c_int32, c_int32, c_int32, _P]),
    "topsaten_fused_moe_gemm": (c_int, [_P] * 8 + [c_int32] * 8 + [_P]),
    "topsaten_release_graph_workspace_pool": (None, [_P]),
    "ub_silu_and_mul": (c_int, [_P, _P, c_int, c_int, c_int, _P]),
    "ub_topk_sum": (c_int, [_P, _P, c_int, c_int, c_int, c_int, _P]),
    "ub_fused_moe_q4k_gemm": (c_int, [_P] * 7 + [c_int] * 9 + [_P, c_size_t, _P]),
    "ub_indexed_moe_q4k": (c_int, [_P, _P, _P, _P] + [c_int] * 7 + [_P]),
    "ub_moe_layer_q4k_workspace_bytes": (c_size_t, [c_int] * 6),
    "ub_moe_layer_q4k": (c_int, [_P] * 6 + [c_int] * 7 + [_P, c_size_t, _P]),
    "ecclGetVersion": (c_int, [POINTER(c_int)]),
    "ecclGetUniqueId": (c_int, [POINTER(EcclUniqueId)]),
    "ecclCommInitRank": (c_int, [POINTER(_P), c_int, EcclUniqueId, c_int]),
    "ecclCommInitAll": (c_int, [POINTER(_P), c_int, POINTER(c_int)]),
    "ecclCommDestroy": (c_int, [_P]),
    "ecclCommAbort": (c_int, [_P]),
    "ecclCommCount": (c_int, [_P, POINTER(c_int)]),
    "ecclCommDevice": (c_int, [_P, POINTER(c_int)]),
    "ecclCommUserRank": (c_int, [_P, POINTER(c_int)]),
    "ecclReduce": (c_int, [_P, _P, c_size_t, c_int, c_int, c_int, _P, _P]),
    "ecclBroadcast": (c_int, [_P, _P, c_size_t, c_int, c_int, _P, _P]),
    "ecclAllReduce": (c_int, [_P, _P, c_size_t, c_int, c_int, _P, _P]),
    "ecclReduceScatter": (c_int, [_P, _P, c_size_t, c_int, c_int, _P, _P]),
    "ecclAllGather": (c_int, [_P, _P, c_size_t, c_int, _P, _P]),
    "ecclSend": (c_int, [_P, c_size_t, c_int, c_int, _P, _P]),
    "ecclRecv": (c_int, [_P, c_size_t, c_int, c_int, _P, _P]),
    "ecclGroupStart": (c_int, []),
    "ecclGroupEnd": (c_int, []),
    "ub_eccl_comm_async_error": (c_int, [_P, POINTER(c_int)]),
}

EXPORTED_SYMBOLS = tuple(sorted(_SIGS))


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it has not been built (``python -m ubridge_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "ubridge_b200: %s is missing; build it with `python -m ubridge_b200.build` "
                "(nvcc, sm_100a). There is no fallback path." % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGS.items():
            fn = getattr(handle, name)  # AttributeError if the export is missing
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().ub_status_string(status).decode()


def check(status: int, what: str = "") -> None:
    if status != UB_OK:
        raise UbridgeError(status, what)


def check_last(what: str = "") -> None:
    """For the reference-named `void` exports: raise if the call recorded a failure."""
    check(lib().ub_last_status(), what)
