"""GPU, two or more devices: the tensor-parallel linear stack and the expert-parallel MoE layer, threads as
ranks (one device each, the pattern of the reference's collective tests, src/eccl.rs:428-492), partial
outputs summed with ecclAllReduce, against the oracle's unsharded result."""
import threading

import numpy as np
import pytest

import ubridge_b200 as ub
from oracle import oracle as o
from ubridge_b200 import eccl, parallel as par

pytestmark = pytest.mark.gpu


def _world():
    n = ub.lib().ub_device_count()
    if n < 2:
        pytest.skip("needs 2+ GPUs")
    return 2


def _bf16(x):
    return o.bf16_bits_to_f32(o.f32_to_bf16_bits(np.asarray(x, dtype=np.float32)))


def _run_ranks(world, rank_main):
    errors, results = [None] * world, [None] * world

    def wrap(r):
        try:
            results[r] = rank_main(r)
        except Exception as e:  # noqa: BLE001 - reported below, in the main thread
            errors[r] = e

    threads = [threading.Thread(target=wrap, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    for e in errors:
        if e is not None:
            raise e
    assert all(r is not None for r in results), "a rank did not finish"
    return results


@pytest.mark.parametrize("M", [1, 40])
def test_tp_stack_matches_the_unsharded_oracle(M):
    world = _world()
    hidden, inter, nq, nkv, hd = 1024, 2048, 8, 2, 128
    rng = np.random.default_rng(300)
    x = o.gen_activation(rng, M, hidden, True)
    w_qkv = o.gen_q4k_weight(rng, (nq + 2 * nkv) * hd, hidden)
    w_o = o.gen_q4k_weight(rng, hidden, nq * hd)
    w_gate, w_up = o.gen_q4k_weight(rng, inter, hidden), o.gen_q4k_weight(rng, inter, hidden)
    w_down = o.gen_q4k_weight(rng, hidden, inter)
    uid = eccl.Id()

    def rank_main(r):
        d = ub.GcuDevice(r)
        d.bind_to_thread()
        comm = eccl.Comm.from_rank(r, world, uid)

        def all_reduce(buf, count):
            comm.all_reduce(buf, buf, count, eccl.Bfloat16, eccl.ReduceOp.Sum, stream=d.stream)

        stack = par.TPLinearStack(
            d, hidden, inter, nq, nkv, hd, world,
            par.qkv_column_split(w_qkv, nq, nkv, hd, hidden, True, r, world),
            par.row_split(w_o, hidden, nq * hd, True, r, world)[0],
            par.gate_up_column_split(w_gate, w_up, inter, hidden, True, r, world),
            par.row_split(w_down, hidden, inter, True, r, world)[0], M, all_reduce)
        d_x = d.htod_sync_copy(o.f32_to_bf16_bits(x).reshape(-1))
        out = stack.forward(d_x, M)
        d.synchronize()
        y = o.bf16_bits_to_f32(d.dtoh_sync_copy(out, np.uint16)[:M * hidden]).reshape(M, hidden)
        comm.destroy()
        return y

    got = _run_ranks(world, rank_main)
    # unsharded restatement with the same roundings to bf16 between the matmuls
    q = _bf16(o.qmatmul_exact(x, o.dequant_q4k(w_qkv).reshape(-1, hidden)))[:, :nq * hd]
    h1 = _bf16(o.qmatmul_exact(q, o.dequant_q4k(w_o).reshape(hidden, nq * hd)))
    g = _bf16(o.qmatmul_exact(h1, o.dequant_q4k(w_gate).reshape(inter, hidden)))
    u = _bf16(o.qmatmul_exact(h1, o.dequant_q4k(w_up).reshape(inter, hidden)))
    act = o.silu_and_mul(np.concatenate([g, u], axis=1), o.UB_BF16)
    want = o.qmatmul_exact(act, o.dequant_q4k(w_down).reshape(hidden, inter))
    for r in range(world):
        # bf16 partial sums are rounded before the all-reduce: 1e-2 is the tensor-core tolerance of the path
        assert o.rel_l2(got[r], want) < 1e-2
    assert np.array_equal(got[0], got[1])  # all ranks hold the same reduced result


def test_ep_layer_matches_the_unsharded_oracle():
    world = _world()
    T, H, I, E, k, block = 48, 512, 768, 4, 2, 16
    rng = np.random.default_rng(400)
    hidden = o.gen_activation(rng, T, H, True)
    logits = o.gen_activation(rng, T, E, True)
    w13_blocks, w2_blocks = o.gen_q4k_weight(rng, E * 2 * I, H), o.gen_q4k_weight(rng, E * H, I)
    w13, w2 = w13_blocks.reshape(E, -1), w2_blocks.reshape(E, -1)  # bytes of each expert
    uid = eccl.Id()

    def rank_main(r):
        d = ub.GcuDevice(r)
        d.bind_to_thread()
        comm = eccl.Comm.from_rank(r, world, uid)

        def all_reduce(buf, count):
            comm.all_reduce(buf, buf, count, eccl.Bfloat16, eccl.ReduceOp.Sum, stream=d.stream)

        e0, e1 = par.expert_range(E, r, world)
        layer = par.EPMoELayer(d, T, H, I, E, k, block, r, world, w13[e0:e1].reshape(-1), w2[e0:e1].reshape(-1),
                               all_reduce)
        d_h = d.htod_sync_copy(o.f32_to_bf16_bits(hidden).reshape(-1))
        d_l = d.htod_sync_copy(o.f32_to_bf16_bits(logits).reshape(-1))
        out = layer.forward(d_h, d_l)
        d.synchronize()
        y = o.bf16_bits_to_f32(d.dtoh_sync_copy(out, np.uint16)[:T * H]).reshape(T, H)
        comm.destroy()
        return y

    got = _run_ranks(world, rank_main)
    want, _ = o.moe_layer_exact(hidden, logits, o.dequant_q4k(w13_blocks).reshape(E, 2 * I, H),
                                o.dequant_q4k(w2_blocks).reshape(E, H, I), k, block, True)
    for r in range(world):
        assert o.rel_l2(got[r], want) < 1e-2
    assert np.array_equal(got[0], got[1])


def test_oneshot_all_reduce_matches_rank_ordered_sum():
    """Peer-memory all-reduce: every rank ends with the f32 sum of the ranks' bf16 vectors in rank order,
    rounded once, over several rounds (both slot sets are reused) and two sizes."""
    world = _world()
    barrier = threading.Barrier(world)
    shared = [None] * world
    rng = np.random.default_rng(500)
    rounds, counts = 5, [8192, 64]
    data = [[[o.gen_activation(rng, 1, c, True).reshape(-1) for _ in range(world)] for c in counts]
            for _ in range(rounds)]

    def rank_main(r):
        d = ub.GcuDevice(r)
        d.bind_to_thread()

        def exchange(obj):
            shared[r] = obj
            barrier.wait()
            out = list(shared)
            barrier.wait()
            return out

        ar = eccl.OneShotAllReduce(d, r, world, 16384, exchange, same_process=True)
        barrier.wait()  # every staging buffer is zeroed and every peer enabled
        outs = []
        for k in range(rounds):
            for ci, c in enumerate(counts):
                buf = d.htod_sync_copy(o.f32_to_bf16_bits(data[k][ci][r]))
                ar.all_reduce(buf, c)
                d.synchronize()
                outs.append(d.dtoh_sync_copy(buf, np.uint16))
        assert d.device_status() == 0
        barrier.wait()
        ar.close()
        return outs

    got = _run_ranks(world, rank_main)
    i = 0
    for k in range(rounds):
        for ci, c in enumerate(counts):
            acc = np.zeros(c, dtype=np.float32)
            for r in range(world):
                acc = acc + _bf16(data[k][ci][r])
            want = o.f32_to_bf16_bits(acc)
            for r in range(world):
                assert np.array_equal(got[r][i][:c], want)
            i += 1


@pytest.mark.parametrize("N,K", [(1024, 4096), (8192, 2048), (512, 8192), (256, 1024), (2048, 3584)])
def test_matmul_with_fused_all_reduce(N, K):
    """Row-split one-token matmul whose CTAs push their rows to the peers and whose last CTA completes the
    exchange: same bits as matmul followed by the one-shot all-reduce, over several rounds and on every kernel
    that carries the epilogue (K = 4096 / 2048: register fragments; 8192: shared-memory fragments; 1024 and 3584:
    the token-pair kernel with and without tensor-map copies)."""
    world = _world()
    barrier = threading.Barrier(world)
    shared = [None] * world
    rng = np.random.default_rng(N + K)
    rounds = 4
    ws = [o.gen_q4k_weight(rng, N, K) for _ in range(world)]
    xs = [[o.gen_activation(rng, 1, K, True) for _ in range(world)] for _ in range(rounds)]

    def rank_main(r):
        d = ub.GcuDevice(r)
        d.bind_to_thread()

        def exchange(obj):
            shared[r] = obj
            barrier.wait()
            out = list(shared)
            barrier.wait()
            return out

        ar = eccl.OneShotAllReduce(d, r, world, 16384, exchange, same_process=True)
        barrier.wait()
        d_w = d.htod_sync_copy(ws[r])
        outs = []
        for k in range(rounds):
            d_x = d.htod_sync_copy(o.f32_to_bf16_bits(xs[k][r]).reshape(-1))
            d_y = d.alloc(N * 2)
            ar.matmul_all_reduce(d_y, d_x, d_w, 1, N, K)
            if k == 1:  # a stand-alone exchange in between shares the staging buffers and the epoch sequence
                ar.all_reduce(d_y, N)
            d.synchronize()
            outs.append(d.dtoh_sync_copy(d_y, np.uint16).copy())
        assert d.device_status() == 0
        barrier.wait()
        ar.close()
        return outs

    got = _run_ranks(world, rank_main)
    for k in range(rounds):
        acc = np.zeros(N, dtype=np.float32)
        exact = np.zeros(N, dtype=np.float64)
        for r in range(world):
            part = o.c_qmatmul(xs[k][r], ws[r], N, K, True).reshape(-1)
            acc = acc + _bf16(part)
            exact += part
        if k == 1:
            acc = _bf16(acc) * world  # the extra stand-alone exchange sums `world` copies of the reduced vector
            exact *= world
        for r in range(world):
            assert np.array_equal(got[r][k], got[0][k])  # every rank holds the same bits
        y = o.bf16_bits_to_f32(got[0][k])
        # partial sums are rounded to bf16 before the exchange (matmul accumulation differs in the last bits
        # from the oracle's, so a bf16 tie may fall the other way: compare values, not bits)
        assert o.rel_l2(y, exact.astype(np.float32)) < 5e-3
        assert o.rel_l2(y, acc) < 2e-3


def test_tp_stack_with_fused_exchanges_matches_the_plain_one():
    """The tensor-parallel stack at one token with SiLU.up and both exchanges inside the matmul launches gives
    the bits of the same stack with separate matmul / SiLU.up / one-shot all-reduce launches."""
    world = _world()
    hidden, inter, nq, nkv, hd = 2048, 4096, 16, 2, 128
    rng = np.random.default_rng(700)
    x = o.gen_activation(rng, 1, hidden, True)
    w_qkv = o.gen_q4k_weight(rng, (nq + 2 * nkv) * hd, hidden)
    w_o = o.gen_q4k_weight(rng, hidden, nq * hd)
    w_gate, w_up = o.gen_q4k_weight(rng, inter, hidden), o.gen_q4k_weight(rng, inter, hidden)
    w_down = o.gen_q4k_weight(rng, hidden, inter)
    barrier = threading.Barrier(world)
    shared = [None] * world

    def rank_main(r):
        d = ub.GcuDevice(r)
        d.bind_to_thread()

        def exchange(obj):
            shared[r] = obj
            barrier.wait()
            out = list(shared)
            barrier.wait()
            return out

        ar = eccl.OneShotAllReduce(d, r, world, 16384, exchange, same_process=True)
        barrier.wait()
        shards = (par.qkv_column_split(w_qkv, nq, nkv, hd, hidden, True, r, world),
                  par.row_split(w_o, hidden, nq * hd, True, r, world)[0],
                  par.gate_up_column_split(w_gate, w_up, inter, hidden, True, r, world),
                  par.row_split(w_down, hidden, inter, True, r, world)[0])
        d_x = d.htod_sync_copy(o.f32_to_bf16_bits(x).reshape(-1))
        outs = []
        for fused in (ar, None):
            stack = par.TPLinearStack(d, hidden, inter, nq, nkv, hd, world, *shards, 1, ar.all_reduce, fused=fused)
            for _ in range(2):
                out = stack.forward(d_x, 1)
                d.synchronize()
                outs.append(d.dtoh_sync_copy(out, np.uint16)[:hidden].copy())
        assert d.device_status() == 0
        barrier.wait()
        ar.close()
        return outs

    got = _run_ranks(world, rank_main)
    for r in range(world):
        for k in range(1, 4):
            assert np.array_equal(got[r][k], got[0][0])


@pytest.mark.parametrize("M", [1, 5])
def test_linear_stack_on_one_gpu_chains_dependent_launches(dev, M):
    """World size 1: four matmuls back to back on one stream, each consuming the previous one's output (the
    decode kernels start early under programmatic dependent launch and must wait before touching activations)."""
    hidden, inter, nq, nkv, hd = 2048, 4096, 16, 2, 128
    rng = np.random.default_rng(600 + M)
    x = o.gen_activation(rng, M, hidden, True)
    w_qkv = o.gen_q4k_weight(rng, (nq + 2 * nkv) * hd, hidden)
    w_o = o.gen_q4k_weight(rng, hidden, nq * hd)
    w_gate, w_up = o.gen_q4k_weight(rng, inter, hidden), o.gen_q4k_weight(rng, inter, hidden)
    w_down = o.gen_q4k_weight(rng, hidden, inter)
    stack = par.TPLinearStack(dev, hidden, inter, nq, nkv, hd, 1, w_qkv.reshape(-1), w_o.reshape(-1),
                              par.gate_up_column_split(w_gate, w_up, inter, hidden, True, 0, 1), w_down.reshape(-1), M)
    d_x = dev.htod_sync_copy(o.f32_to_bf16_bits(x).reshape(-1))
    outs = []
    for _ in range(3):  # repeated: any race between consecutive launches would show as a difference
        out = stack.forward(d_x, M)
        dev.synchronize()
        outs.append(o.bf16_bits_to_f32(dev.dtoh_sync_copy(out, np.uint16)[:M * hidden]).reshape(M, hidden))
    assert dev.device_status() == 0
    q = _bf16(o.qmatmul_exact(x, o.dequant_q4k(w_qkv).reshape(-1, hidden)))[:, :nq * hd]
    h1 = _bf16(o.qmatmul_exact(q, o.dequant_q4k(w_o).reshape(hidden, nq * hd)))
    g = _bf16(o.qmatmul_exact(h1, o.dequant_q4k(w_gate).reshape(inter, hidden)))
    u = _bf16(o.qmatmul_exact(h1, o.dequant_q4k(w_up).reshape(inter, hidden)))
    act = o.silu_and_mul(np.concatenate([g, u], axis=1), o.UB_BF16)
    want = o.qmatmul_exact(act, o.dequant_q4k(w_down).reshape(hidden, inter))
    assert o.rel_l2(outs[0], want) < 1e-2
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])
