"""CPU: the bench's rank rendezvous (barrier, max over ranks, all-gather and broadcast of small objects)
over two gloo ranks, and its single-rank shortcuts."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench  # noqa: E402


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ctl = bench.Control(torch, dist, world)
        ctl.barrier()
        m = ctl.max(1.5 + rank)
        gathered = ctl.all_gather(b"id-%d" % rank)
        b = ctl.broadcast("from-zero" if rank == 0 else None)
        q.put((rank, m, gathered, b))
    finally:
        dist.destroy_process_group()


def test_control_over_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, m, gathered, b in got:
        assert m == 2.5
        assert gathered == [b"id-0", b"id-1"]
        assert b == "from-zero"


def test_control_single_rank_needs_no_process_group():
    ctl = bench.Control(torch, dist, 1)
    ctl.barrier()
    assert ctl.max(3.25) == 3.25
    assert ctl.all_gather("x") == ["x"]
    assert ctl.broadcast({"a": 1}) == {"a": 1}


def test_workload_table_is_consistent():
    for name, wl in bench.WORKLOADS.items():
        assert wl["unit"] in ("GB/s", "TFLOP/s", "tok/s"), name
        assert wl["K"] % 256 == 0 and wl["N"] > 0 and wl["M"] > 0
        if wl.get("kind") == "tp":
            assert wl["hidden"] % 2048 == 0 and wl["inter"] % (8 * 256) == 0  # row splits stay whole blocks at 8 ranks
            assert (wl["q_heads"] % 8, wl["kv_heads"] % 8) == (0, 0)
        if wl.get("kind") == "ep":
            assert wl["E"] % 8 == 0 and wl["flop_per_token"] == 2 * 3 * 2.0 * wl["H"] * wl["I"]


def test_timed_region_sizing_and_profile_lookup():
    # steps x k replays must reach the minimum duration; never fewer than one replay per step
    assert bench.replays_for(2.0, 20, 0.85e-3) == 118
    assert bench.replays_for(2.0, 20, 1.0) == 1
    assert bench.replays_for(2.0, 20, 0.0) == 1
    # roofline.traffic comes from the profile summaries, not from a constant in the script
    for wl, name in bench.PROFILE_OF.items():
        text = open(os.path.join(os.path.dirname(bench.__file__), "profiles", name)).read()
        assert "dram_bytes_per_launch = %d" % bench.profile_traffic(wl) in text, wl
    assert bench.profile_traffic("c1") == 17868032
    assert bench.profile_traffic("c5_m1") is None
