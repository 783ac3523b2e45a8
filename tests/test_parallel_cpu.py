"""CPU: tensor-parallel and expert-parallel shard arithmetic, checked with two gloo ranks.

Each rank shards the packed weights with ubridge_b200.parallel, computes its part with the oracle
(standing in for the GPU kernels, which this box cannot run) and the partial results meet in a
torch.distributed all-reduce, exactly where the GPU path calls ecclAllReduce."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as o
from ubridge_b200 import parallel as par


def test_split_range_covers_everything():
    for n in (1, 7, 8, 64, 112):
        for world in (1, 2, 3, 4, 8):
            pieces = [par.split_range(n, r, world) for r in range(world)]
            assert pieces[0][0] == 0 and pieces[-1][1] == n
            assert all(pieces[i][1] == pieces[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in pieces]
            assert max(sizes) - min(sizes) <= 1


def test_expert_map_matches_reference_convention():
    m = par.expert_map(8, 1, 4)
    assert m.tolist() == [-1, -1, 0, 1, -1, -1, -1, -1]
    assert par.expert_map(8, 0, 1).tolist() == list(range(8))


def test_row_split_needs_whole_blocks():
    rng = np.random.default_rng(0)
    w = o.gen_q4k_weight(rng, 4, 768)  # 3 super-blocks per row
    with pytest.raises(ValueError):
        par.row_split(w, 4, 768, True, 0, 2)
    shard, (k0, k1) = par.row_split(w, 4, 768, True, 1, 3)
    assert (k0, k1) == (256, 512) and shard.shape == (4, 1, 144)


def test_column_and_row_split_recompose():
    rng = np.random.default_rng(1)
    N, K = 24, 1024
    w = o.gen_q4k_weight(rng, N, K)
    full = o.dequant_q4k(w).reshape(N, K)
    cols = [o.dequant_q4k(par.column_split(w, N, K, True, r, 3)[0]).reshape(-1, K) for r in range(3)]
    assert np.array_equal(np.concatenate(cols, axis=0), full)
    rows = [o.dequant_q4k(par.row_split(w, N, K, True, r, 4)[0]).reshape(N, -1) for r in range(4)]
    assert np.array_equal(np.concatenate(rows, axis=1), full)
    w8 = o.gen_q8_0_weight(rng, N, 256)
    rows8 = [o.dequant_q8_0(par.row_split(w8, N, 256, False, r, 2)[0]).reshape(N, -1) for r in range(2)]
    assert np.array_equal(np.concatenate(rows8, axis=1), o.dequant_q8_0(w8).reshape(N, 256))


def test_qkv_split_keeps_heads_whole():
    rng = np.random.default_rng(2)
    nq, nkv, hd, K = 8, 2, 16, 256
    w = o.gen_q4k_weight(rng, (nq + 2 * nkv) * hd, K)
    full = o.dequant_q4k(w).reshape(-1, K)
    s0 = o.dequant_q4k(par.qkv_column_split(w, nq, nkv, hd, K, True, 0, 2)).reshape(-1, K)
    s1 = o.dequant_q4k(par.qkv_column_split(w, nq, nkv, hd, K, True, 1, 2)).reshape(-1, K)
    assert s0.shape[0] == (4 + 1 + 1) * hd
    assert np.array_equal(s0[:4 * hd], full[:4 * hd]) and np.array_equal(s1[:4 * hd], full[4 * hd:8 * hd])
    assert np.array_equal(s0[4 * hd:5 * hd], full[8 * hd:9 * hd])          # k head 0
    assert np.array_equal(s1[5 * hd:6 * hd], full[(8 + 2 + 1) * hd:(8 + 2 + 2) * hd])  # v head 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _bf16(x):
    return o.bf16_bits_to_f32(o.f32_to_bf16_bits(np.asarray(x, dtype=np.float32)))


def _tp_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(100)  # same seed on every rank: replicated inputs and full weights
        H, I, M = 256, 512, 3
        x = o.gen_activation(rng, M, H, True)
        w_gate, w_up = o.gen_q4k_weight(rng, I, H), o.gen_q4k_weight(rng, I, H)
        w_down = o.gen_q4k_weight(rng, H, I)
        gu = par.gate_up_column_split(w_gate, w_up, I, H, True, rank, world)
        down, (k0, k1) = par.row_split(w_down, H, I, True, rank, world)
        i_local = I // world
        y_gu = _bf16(o.qmatmul_exact(x, o.dequant_q4k(gu).reshape(2 * i_local, H)))
        act = o.silu_and_mul(y_gu, o.UB_BF16)
        part = o.qmatmul_exact(act, o.dequant_q4k(down).reshape(H, i_local))
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t)  # the one exchange of a row-split GEMM
        if rank == 0:
            g = _bf16(o.qmatmul_exact(x, o.dequant_q4k(w_gate).reshape(I, H)))
            u = _bf16(o.qmatmul_exact(x, o.dequant_q4k(w_up).reshape(I, H)))
            full_act = o.silu_and_mul(np.concatenate([g, u], axis=1), o.UB_BF16)
            want = o.qmatmul_exact(full_act, o.dequant_q4k(w_down).reshape(H, I))
            q.put(("tp", o.rel_l2(t.numpy(), want), (k0, k1)))
    finally:
        dist.destroy_process_group()


def _ep_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(200)
        T, H, I, E, k, block = 6, 256, 256, 4, 2, 4
        hidden = o.gen_activation(rng, T, H, True)
        logits = o.gen_activation(rng, T, E, True)
        w13 = o.dequant_q4k(o.gen_q4k_weight(rng, E * 2 * I, H)).reshape(E, 2 * I, H)
        w2 = o.dequant_q4k(o.gen_q4k_weight(rng, E * H, I)).reshape(E, H, I)
        e0, e1 = par.expert_range(E, rank, world)
        emap = par.expert_map(E, rank, world)
        part, _ = o.moe_layer_exact(hidden, logits, w13[e0:e1], w2[e0:e1], k, block, True, expert_map=emap)
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t)
        if rank == 0:
            want, _ = o.moe_layer_exact(hidden, logits, w13, w2, k, block, True)
            q.put(("ep", o.rel_l2(t.numpy(), want), (e0, e1)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("worker", [_tp_worker, _ep_worker])
def test_two_gloo_ranks_reproduce_the_unsharded_result(worker):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    kind, err, rng_ = q.get(timeout=10)
    # each rank rounds its own partial sums; the sum of two bf16-rounded halves differs from one rounding
    assert err < (1e-5 if kind == "tp" else 1e-2), (kind, err)
