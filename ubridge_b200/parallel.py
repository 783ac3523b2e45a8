"""Tensor-parallel and expert-parallel sharding of the quantized path, one rank per GPU.

The reference offers only the pieces: ECCL collectives (src/eccl.rs:298-413) and the expert-parallel
hooks in its kernels (``expert_map`` -> local id or -1 in kernels/moe_align_host.cpp:298,535-543; skip /
zero-fill of non-local experts in kernels/fused_moe_host.cpp:89-93,161-176).  The splits themselves are
done by its caller.  This module holds that caller-side logic for GGUF block matrices:

* column split  - rows of the [N, K] block matrix (output features); any row boundary is legal;
* row split     - the K axis, in whole blocks (256 values for Q4_K, 32 for Q8_0); partial outputs are
                  summed with one all-reduce;
* expert split  - contiguous ranges of experts plus the ``expert_map`` the alignment kernel takes.

The shard arithmetic is plain numpy on the packed bytes and runs anywhere; the two runner classes
drive the C-ABI ops and a communicator and need a GPU.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import numpy as np

from . import ops
from ._lib import DTYPE_BF16

QK = {True: 256, False: 32}
BLOCK_BYTES = {True: 144, False: 34}


# ----------------------------------------------------------------------------- shard arithmetic (host)
def split_range(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous near-even partition of range(n): the first n % world ranks get one extra."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def as_block_matrix(wq: np.ndarray, N: int, K: int, is_q4k: bool) -> np.ndarray:
    """View packed bytes as [N, K/QK, block_bytes]."""
    return np.ascontiguousarray(wq, dtype=np.uint8).reshape(N, K // QK[is_q4k], BLOCK_BYTES[is_q4k])


def column_split(wq: np.ndarray, N: int, K: int, is_q4k: bool, rank: int, world: int,
                 group: int = 1) -> Tuple[np.ndarray, Tuple[int, int]]:
    """Rows [n0, n1) of the block matrix.  `group` keeps that many consecutive rows together
    (an attention head, for instance): N must be a multiple of it."""
    if N % group:
        raise ValueError("N is not a multiple of the row group")
    g0, g1 = split_range(N // group, rank, world)
    n0, n1 = g0 * group, g1 * group
    return np.ascontiguousarray(as_block_matrix(wq, N, K, is_q4k)[n0:n1]), (n0, n1)


def row_split(wq: np.ndarray, N: int, K: int, is_q4k: bool, rank: int, world: int) -> Tuple[np.ndarray, Tuple[int, int]]:
    """K range [k0, k1) in whole blocks, repacked contiguously as an [N, (k1-k0)/QK] block matrix."""
    qk = QK[is_q4k]
    nblk = K // qk
    if nblk % world:
        raise ValueError("K/%d = %d blocks do not divide over %d ranks" % (qk, nblk, world))
    b0, b1 = split_range(nblk, rank, world)
    return np.ascontiguousarray(as_block_matrix(wq, N, K, is_q4k)[:, b0:b1]), (b0 * qk, b1 * qk)


def qkv_column_split(wq: np.ndarray, n_q_heads: int, n_kv_heads: int, head_dim: int, K: int, is_q4k: bool, rank: int,
                     world: int) -> np.ndarray:
    """Fused [q; k; v] projection split on head boundaries: each rank gets its q heads, then its k heads,
    then its v heads."""
    nq, nkv = n_q_heads * head_dim, n_kv_heads * head_dim
    m = as_block_matrix(wq, nq + 2 * nkv, K, is_q4k)
    q0, q1 = split_range(n_q_heads, rank, world)
    k0, k1 = split_range(n_kv_heads, rank, world)
    parts = [m[q0 * head_dim:q1 * head_dim], m[nq + k0 * head_dim:nq + k1 * head_dim],
             m[nq + nkv + k0 * head_dim:nq + nkv + k1 * head_dim]]
    return np.ascontiguousarray(np.concatenate(parts, axis=0))


def gate_up_column_split(w_gate: np.ndarray, w_up: np.ndarray, I: int, K: int, is_q4k: bool, rank: int,
                         world: int) -> np.ndarray:
    """Same row range of gate and up stacked as [gate rows; up rows], so SiLU.up stays local to the rank."""
    g, _ = column_split(w_gate, I, K, is_q4k, rank, world)
    u, _ = column_split(w_up, I, K, is_q4k, rank, world)
    return np.ascontiguousarray(np.concatenate([g, u], axis=0))


def expert_range(E: int, rank: int, world: int) -> Tuple[int, int]:
    return split_range(E, rank, world)


def expert_map(E: int, rank: int, world: int) -> np.ndarray:
    """int32[E]: local index of each expert on this rank, -1 for experts held elsewhere
    (the convention of kernels/moe_align_host.cpp:535-543)."""
    e0, e1 = expert_range(E, rank, world)
    m = np.full((E,), -1, dtype=np.int32)
    m[e0:e1] = np.arange(e1 - e0, dtype=np.int32)
    return m


# ----------------------------------------------------------------------------- runners (GPU)
AllReduce = Callable[[object, int], None]  # (device buffer, element count) -> in-place bf16 sum


def _resident(dev, w):
    """Packed weights as a device buffer: host arrays are uploaded, device buffers are taken as they are."""
    return w if hasattr(w, "ptr") else dev.htod_sync_copy(w)


class TPLinearStack:
    """Llama-style linear stack under tensor parallelism: qkv (column) -> o (row) -> all-reduce ->
    gate/up (column, SiLU.up) -> down (row) -> all-reduce.  Attention itself is not part of this path:
    the first `hidden` columns of this rank's q output feed o, which keeps the data flow and sizes.

    `dev` is a GcuDevice; weights are numpy block arrays (or device buffers) already sharded for this rank; `all_reduce`
    is called with (buffer, count) after each row-split GEMM (None for a single rank)."""

    def __init__(self, dev, hidden: int, inter: int, n_q_heads: int, n_kv_heads: int, head_dim: int, world: int,
                 w_qkv: np.ndarray, w_o: np.ndarray, w_gate_up: np.ndarray, w_down: np.ndarray, max_m: int,
                 all_reduce: Optional[AllReduce] = None, fused=None):
        self.dev, self.H, self.I, self.world = dev, hidden, inter, world
        self.q_local = n_q_heads * head_dim // world
        self.kv_local = n_kv_heads * head_dim // world
        self.qkv_n = self.q_local + 2 * self.kv_local
        self.i_local = inter // world
        self.all_reduce = all_reduce
        # an eccl.OneShotAllReduce: row-split matmuls whose output fits its staging slots run with the exchange
        # in their own epilogue (one launch instead of matmul + all-reduce)
        self.fused = fused
        self.w_qkv, self.w_o = _resident(dev, w_qkv), _resident(dev, w_o)
        self.w_gu, self.w_down = _resident(dev, w_gate_up), _resident(dev, w_down)
        self.max_m = max_m
        self.qkv = dev.alloc(max_m * self.qkv_n * 2)
        self.attn = dev.alloc(max_m * self.q_local * 2)
        self.h1 = dev.alloc(max_m * hidden * 2)
        self.gu = dev.alloc(max_m * 2 * self.i_local * 2)
        self.act = dev.alloc(max_m * self.i_local * 2)
        self.out = dev.alloc(max_m * hidden * 2)
        shapes = [(self.qkv_n, hidden), (hidden, self.q_local), (2 * self.i_local, hidden), (hidden, self.i_local)]
        self.ws_bytes = max(max(ops.qmatmul_workspace_bytes(max_m, n, k, True) for n, k in shapes),
                            ops.qmatmul_q4k_gate_up_workspace_bytes(max_m, self.i_local, hidden))
        self.ws = dev.alloc(max(self.ws_bytes, 256))

    @property
    def launches_per_forward(self) -> int:
        """Kernels of this library per forward() at max_m: one token runs four launches (SiLU.up and the
        exchanges ride in the matmuls' epilogues); otherwise four matmuls, SiLU.up and, beyond one rank, two
        all-reduces (the stand-in copy for attention is a device copy, not a kernel of this library)."""
        if self.max_m == 1:
            return 4 if (self.world == 1 or self.fused is not None) else 6
        return 5 + (2 if self.world > 1 else 0)

    def _mm(self, y, x, w, M, N, K):
        ops.qmatmul(y, x, w, M, N, K, is_q4k=True, x_dtype=DTYPE_BF16, out_dtype=DTYPE_BF16, workspace=self.ws,
                    ws_bytes=self.ws_bytes, stream=self.dev.stream)

    def forward(self, x, M: int):
        """x: device bf16 [M, hidden] (replicated).  Returns the device buffer holding bf16 [M, hidden]."""
        dev = self.dev
        self._mm(self.qkv, x, self.w_qkv, M, self.qkv_n, self.H)
        # stand-in for attention: this rank's q columns.  One token: they already lie contiguously at the start
        # of the row; more tokens: made contiguous by one strided device copy
        attn = self.qkv
        if M > 1:
            ops_copy_cols(dev, self.attn, self.qkv, M, self.qkv_n, self.q_local)
            attn = self.attn
        self._row_split(self.h1, attn, self.w_o, M, self.H, self.q_local)
        ops.qmatmul_q4k_gate_up(self.act, self.h1, self.w_gu, M, self.i_local, self.H, out_dtype=DTYPE_BF16,
                                workspace=self.ws, ws_bytes=self.ws_bytes, stream=dev.stream)
        self._row_split(self.out, self.act, self.w_down, M, self.H, self.i_local)
        return self.out

    def _row_split(self, y, x, w, M, N, K):
        """Row-split matmul + sum over the ranks."""
        if self.world > 1 and self.fused is not None and M * N * 2 <= self.fused.max_bytes and (M * N) % 8 == 0:
            self.fused.matmul_all_reduce(y, x, w, M, N, K, stream=self.dev.stream)
            return
        self._mm(y, x, w, M, N, K)
        if self.all_reduce:
            self.all_reduce(y, M * N)


def ops_copy_cols(dev, dst, src, M: int, src_cols: int, cols: int) -> None:
    """dst[M, cols] = src[M, :cols] for bf16 rows (one strided device copy)."""
    import ctypes

    from ._lib import check, lib
    check(lib().ub_memcpy_dtod_2d(dev._handle, ctypes.c_void_p(dst.ptr), cols * 2, ctypes.c_void_p(src.ptr),
                                  src_cols * 2, cols * 2, M), "dtod_2d")


class EPMoELayer:
    """Mixtral-style expert layer under expert parallelism: hidden states and router logits are
    replicated, each rank holds experts [e0, e1) and runs the whole layer with an expert_map that sends
    the other experts' slots to -1 (their rows come out zero), then one all-reduce sums the partials."""

    def __init__(self, dev, T: int, H: int, I: int, E: int, top_k: int, block: int, rank: int, world: int,
                 w13_local: np.ndarray, w2_local: np.ndarray, all_reduce: Optional[AllReduce] = None):
        self.dev, self.T, self.H, self.I, self.E, self.top_k, self.block = dev, T, H, I, E, top_k, block
        self.all_reduce = all_reduce
        self.w13, self.w2 = _resident(dev, w13_local), _resident(dev, w2_local)
        self.map = dev.htod_sync_copy(expert_map(E, rank, world)) if world > 1 else None
        self.ws_bytes = ops.moe_layer_q4k_workspace_bytes(T, H, I, E, top_k, block)
        self.ws = dev.alloc(self.ws_bytes)
        self.out = dev.alloc(T * H * 2)

    # kernels per forward(): router, weight conversion, alignment, two grouped GEMMs, top-k sum
    launches_per_forward = 6

    def forward(self, hidden, logits, norm_topk_prob: bool = True):
        ops.moe_layer_q4k(self.out, hidden, logits, self.w13, self.w2, self.T, self.H, self.I, self.E, self.top_k,
                          self.block, norm_topk_prob, self.ws, self.ws_bytes, expert_map=self.map,
                          stream=self.dev.stream)
        if self.all_reduce:
            self.all_reduce(self.out, self.T * self.H)
        return self.out
