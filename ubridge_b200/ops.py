"""Python entry points of the quantized-linear + fused-MoE path: one function per C-ABI export.

Buffers are device pointers: a :class:`~ubridge_b200.device.GcuSlice`, an int address (for example
``tensor.data_ptr()``), or None.  ``stream`` is a ``cudaStream_t`` as int / ``c_void_p`` (None = default
stream).  Every call enqueues and returns; nothing here synchronises.
"""
from __future__ import annotations

import ctypes

from . import _lib
from ._lib import DTYPE_BF16, DTYPE_F16, DTYPE_F32, check, check_last, lib

_SUFFIX = {DTYPE_F32: "f32", DTYPE_F16: "f16", DTYPE_BF16: "bf16"}


def _p(buf):
    # every pointer parameter is declared c_void_p, which takes None, an int or a c_void_p as it is: no object is
    # made per call (a decode step makes hundreds of these calls)
    if buf is None or type(buf) is int or isinstance(buf, ctypes.c_void_p):
        return buf
    if hasattr(buf, "ptr"):
        return buf.ptr
    return int(buf)


def _s(stream):
    if stream is None or type(stream) is int or isinstance(stream, ctypes.c_void_p):
        return stream
    return int(stream)


# ----------------------------------------------------------------------------- GGUF blocks
def dequantize_q8_0(out, blocks, numel: int, out_dtype: int, stream=None) -> None:
    check(lib().ub_dequant_q8_0(_p(out), _p(blocks), numel, out_dtype, _s(stream)), "ub_dequant_q8_0")


def dequantize_q4k(out, blocks, numel: int, out_dtype: int, stream=None) -> None:
    check(lib().ub_dequant_q4k(_p(out), _p(blocks), numel, out_dtype, _s(stream)), "ub_dequant_q4k")


def dequantize_q6k(out, blocks, numel: int, out_dtype: int, stream=None) -> None:
    check(lib().ub_dequant_q6k(_p(out), _p(blocks), numel, out_dtype, _s(stream)), "ub_dequant_q6k")


def qmatmul_q6k(y, x, wq, M: int, N: int, K: int, *, x_dtype: int, out_dtype: int, stream=None) -> None:
    """y[M,N] = x[M,K] . dequant(Wq)^T for Q6_K weights (decode kernel, no workspace)."""
    if x_dtype == DTYPE_F32:
        fn, name = lib().ub_qmatmul_q6k_f32, "ub_qmatmul_q6k_f32"
    elif x_dtype == DTYPE_BF16:
        fn, name = lib().ub_qmatmul_q6k_bf16, "ub_qmatmul_q6k_bf16"
    else:
        raise ValueError("activations must be f32 or bf16")
    check(fn(_p(y), _p(x), _p(wq), M, N, K, out_dtype, _s(stream)), name)


def quantize_q8_0(blocks, x, numel: int, in_dtype: int, stream=None) -> None:
    check(lib().ub_quantize_q8_0(_p(blocks), _p(x), numel, in_dtype, _s(stream)), "ub_quantize_q8_0")


def repack_to_split(split, interleaved, nblocks: int, is_q4k: bool, stream=None) -> None:
    check(lib().ub_repack_to_split(_p(split), _p(interleaved), nblocks, int(is_q4k), _s(stream)), "ub_repack_to_split")


def repack_to_interleaved(interleaved, split, nblocks: int, is_q4k: bool, stream=None) -> None:
    check(lib().ub_repack_to_interleaved(_p(interleaved), _p(split), nblocks, int(is_q4k), _s(stream)),
          "ub_repack_to_interleaved")


# ----------------------------------------------------------------------------- GGUF tensor blobs (dispatch on the type tag)
def gguf_tensor_bytes(ggml_type: int, numel: int) -> int:
    return lib().ub_gguf_tensor_bytes(ggml_type, numel)


def dequantize_gguf(out, blob, ggml_type: int, numel: int, out_dtype: int, stream=None) -> None:
    check(lib().ub_dequant_gguf(_p(out), _p(blob), ggml_type, numel, out_dtype, _s(stream)), "ub_dequant_gguf")


def qmatmul_gguf(y, x, blob, ggml_type: int, M: int, N: int, K: int, *, x_dtype: int, out_dtype: int, workspace=None,
                 ws_bytes: int = 0, stream=None) -> None:
    """y[M,N] = x[M,K] . W^T for a GGUF tensor blob of N rows x K values of the given GGML type."""
    check(lib().ub_qmatmul_gguf(_p(y), _p(x), _p(blob), ggml_type, M, N, K, x_dtype, out_dtype, _p(workspace), ws_bytes,
                                _s(stream)), "ub_qmatmul_gguf")


# ----------------------------------------------------------------------------- quantized matmul
_QMATMUL = {}  # (is_q4k, x_dtype) -> (function, name): looked up once


def qmatmul_workspace_bytes(M: int, N: int, K: int, is_q4k: bool) -> int:
    return lib().ub_qmatmul_workspace_bytes(M, N, K, int(is_q4k))


def qmatmul(y, x, wq, M: int, N: int, K: int, *, is_q4k: bool, x_dtype: int, out_dtype: int, workspace=None,
            ws_bytes: int = 0, stream=None) -> None:
    """y[M,N] = x[M,K] . W^T with W given as interleaved GGUF blocks (Q4_K when is_q4k else Q8_0)."""
    if x_dtype not in (DTYPE_F32, DTYPE_BF16):
        raise _lib.UbridgeError(_lib.UB_ERR_INVALID_ARG, "qmatmul: activations must be f32 or bf16")
    fn = _QMATMUL.get((is_q4k, x_dtype))
    if fn is None:
        name = "ub_qmatmul_%s_%s" % ("q4k" if is_q4k else "q8_0", _SUFFIX[x_dtype])
        fn = _QMATMUL[(is_q4k, x_dtype)] = (getattr(lib(), name), name)
    st = fn[0](_p(y), _p(x), _p(wq), M, N, K, out_dtype, _p(workspace), ws_bytes, _s(stream))
    if st:
        check(st, fn[1])


def qmatmul_q4k_gate_up_workspace_bytes(M: int, I: int, K: int) -> int:
    return lib().ub_qmatmul_q4k_gate_up_workspace_bytes(M, I, K)


def qmatmul_q4k_gate_up(y, x, wq, M: int, I: int, K: int, *, out_dtype: int, workspace=None, ws_bytes: int = 0,
                        stream=None) -> None:
    """y[M, I] = silu(x . Wgate^T) * (x . Wup^T), wq = [gate rows; up rows] of Q4_K, x bf16.  One token is one
    launch (SiLU.up in the matmul's epilogue); other shapes run the matmul into the workspace, then SiLU.up."""
    check(lib().ub_qmatmul_q4k_gate_up_bf16(_p(y), _p(x), _p(wq), M, I, K, out_dtype, _p(workspace), ws_bytes,
                                            _s(stream)), "ub_qmatmul_q4k_gate_up_bf16")


def rms_norm(out, inp, gamma, num_tokens: int, hidden_size: int, eps: float, dtype: int, stream=None) -> None:
    """out[t,:] = rmsnorm(inp[t,:]) * gamma (the reference's topsaten_rms_norm, src/ffi.rs:719-728)."""
    check(lib().topsaten_rms_norm(_p(out), _p(inp), _p(gamma), num_tokens, hidden_size, eps, dtype, _s(stream)),
          "topsaten_rms_norm")


def qmatmul_q4k_rmsnorm_workspace_bytes(M: int, N: int, K: int, gate_up: bool) -> int:
    return lib().ub_qmatmul_q4k_rmsnorm_workspace_bytes(M, N, K, int(gate_up))


def qmatmul_q4k_rmsnorm(y, x, gamma, eps: float, wq, M: int, N: int, K: int, *, gate_up: bool = False, out_dtype: int,
                        workspace=None, ws_bytes: int = 0, stream=None) -> None:
    """Q4_K matmul (or gate/up + SiLU.up when gate_up) on rmsnorm(x; gamma, eps); one launch for one token."""
    check(lib().ub_qmatmul_q4k_rmsnorm_bf16(_p(y), _p(x), _p(gamma), eps, _p(wq), M, N, K, int(gate_up), out_dtype,
                                            _p(workspace), ws_bytes, _s(stream)), "ub_qmatmul_q4k_rmsnorm_bf16")


def qmatmul_q4k_f32_static(y, x, wq, M: int, N: int, K: int, out_dtype: int, stream=None) -> None:
    """Q4_K matmul with f32 activations that takes no workspace and allocates nothing: its scratch is a
    fixed 8 MiB array inside the library (so roughly M*(K+N) <= 4M elements, else UB_ERR_TOO_LARGE).
    For hosts that cannot provide device memory themselves.  Calls on one GPU must not overlap."""
    check(lib().ub_qmatmul_q4k_f32_static(_p(y), _p(x), _p(wq), M, N, K, out_dtype, _s(stream)),
          "ub_qmatmul_q4k_f32_static")


# ----------------------------------------------------------------------------- MoE (reference names)
def topk_softmax(logits, weights, indices, num_tokens: int, num_experts: int, topk: int, norm_topk_prob: bool,
                 dtype: int, stream=None) -> None:
    name = "topk_softmax_" + _SUFFIX[dtype]
    getattr(lib(), name)(_p(logits), _p(weights), _p(indices), num_tokens, num_experts, topk, int(norm_topk_prob),
                         _s(stream))
    check_last(name)


def moe_align_block_size(sorted_ids, experts_ids, num_tokens_post_pad, topk_ids, num_experts: int, block_size: int,
                         token_num: int, topk: int, real_token_num=None, expert_map=None, stream=None) -> None:
    lib().moe_align_block_size(_p(sorted_ids), _p(experts_ids), _p(num_tokens_post_pad), _p(topk_ids),
                               _p(real_token_num), _p(expert_map), num_experts, block_size, token_num, topk,
                               _s(stream))
    check_last("moe_align_block_size")


def moe_align_sizes(token_num: int, topk: int, num_experts: int, block_size: int):
    """(len(sorted_ids), len(experts_ids)) the caller must allocate (kernels/moe_align_host.cpp:56-58)."""
    max_padded = token_num * topk + num_experts * (block_size - 1)
    return max_padded, max_padded // block_size


def invoke_fused_moe(C, A, B, bias, topk_weights, sorted_ids, experts_ids, num_tokens_post_pad, M: int, K: int, N: int,
                     E: int, topk_ids_size: int, top_k: int, block_size: int, mul_routed_weight: bool,
                     bias_flag: bool, dtype: int, stream=None) -> None:
    name = "invoke_fused_moe_" + _SUFFIX[dtype]
    getattr(lib(), name)(_p(C), _p(A), _p(B), _p(bias), _p(topk_weights), _p(sorted_ids), _p(experts_ids),
                         _p(num_tokens_post_pad), M, K, N, E, topk_ids_size, top_k, block_size,
                         int(mul_routed_weight), int(bias_flag), _s(stream))
    check_last(name)


def moe_combine(y, e_out, w, idx, top, N: int, K: int, M: int, topk: int, dtype: int, stream=None) -> None:
    name = "moe_" + _SUFFIX[dtype]
    getattr(lib(), name)(_p(y), _p(e_out), _p(w), _p(idx), _p(top), N, K, M, topk, _s(stream))
    check_last(name)


def indexed_moe(inp, w, out, indices, N: int, K: int, M: int, batch: int, topk: int, num_experts: int, dtype: int,
                stream=None) -> None:
    name = "indexed_moe_" + _SUFFIX[dtype]
    getattr(lib(), name)(_p(inp), _p(w), _p(out), _p(indices), N, K, M, batch, topk, num_experts, _s(stream))
    check_last(name)


# ----------------------------------------------------------------------------- MoE (fused Q4_K)
def silu_and_mul(out, inp, rows: int, D: int, dtype: int, stream=None) -> None:
    check(lib().ub_silu_and_mul(_p(out), _p(inp), rows, D, dtype, _s(stream)), "ub_silu_and_mul")


def topk_sum(out, inp, T: int, topk: int, H: int, dtype: int, stream=None) -> None:
    check(lib().ub_topk_sum(_p(out), _p(inp), T, topk, H, dtype, _s(stream)), "ub_topk_sum")


def fused_moe_q4k_gemm(C, A, Bq, topk_weights, sorted_ids, experts_ids, num_tokens_post_pad, M: int, K: int, N: int,
                       E: int, topk_ids_size: int, top_k: int, block_size: int, mul_routed_weight: bool,
                       act_silu_mul: bool, workspace=None, ws_bytes: int = 0, stream=None) -> None:
    check(lib().ub_fused_moe_q4k_gemm(_p(C), _p(A), _p(Bq), _p(topk_weights), _p(sorted_ids), _p(experts_ids),
                                      _p(num_tokens_post_pad), M, K, N, E, topk_ids_size, top_k, block_size,
                                      int(mul_routed_weight), int(act_silu_mul), _p(workspace), ws_bytes, _s(stream)),
          "ub_fused_moe_q4k_gemm")


def indexed_moe_q4k(out, inp, wq, indices, N: int, K: int, M: int, batch: int, topk: int, num_experts: int, dtype: int,
                    stream=None) -> None:
    """out[b,t,:] = inp[b,(M==1?0:t),:] . dequant(wq[indices[b,t]])^T for Q4_K expert matrices."""
    check(lib().ub_indexed_moe_q4k(_p(out), _p(inp), _p(wq), _p(indices), N, K, M, batch, topk, num_experts, dtype,
                                   _s(stream)), "ub_indexed_moe_q4k")


def moe_layer_q4k_workspace_bytes(T: int, H: int, I: int, E: int, top_k: int, block_size: int) -> int:
    return lib().ub_moe_layer_q4k_workspace_bytes(T, H, I, E, top_k, block_size)


def moe_layer_q4k(out, hidden, router_logits, w13q, w2q, T: int, H: int, I: int, E: int, top_k: int, block_size: int,
                  norm_topk_prob: bool, workspace, ws_bytes: int, expert_map=None, stream=None) -> None:
    check(lib().ub_moe_layer_q4k(_p(out), _p(hidden), _p(router_logits), _p(w13q), _p(w2q), _p(expert_map), T, H, I, E,
                                 top_k, block_size, int(norm_topk_prob), _p(workspace), ws_bytes, _s(stream)),
          "ub_moe_layer_q4k")
