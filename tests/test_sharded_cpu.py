"""The N>1 path without GPUs: routing, displacement tables and the exchange pattern run as
gloo ranks on the CPU, the oracle standing in for the kernels."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from gear_b200.sharded import exchange_plan, route

HERE = Path(__file__).resolve().parent


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_reproduce_single_process_gather(world):
    port = 29400 + world
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(HERE / "sharded_cpu_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert f"SHARDED_CPU_OK {world}" in out.stdout


def test_route_edges():
    totals = np.array([2.0, 0.0, 6.0])                 # a shard without any mass is never chosen
    u = np.array([0.0, 0.2499, 0.25, 0.5, 0.999999, 1.0])
    owner, res, req = route(totals, u, 3)
    assert list(owner) == [0, 0, 2, 2, 2, 2]
    assert res[0] == 0.0 and abs(res[2]) < 1e-12 and np.all(res < totals[owner])
    assert list(req) == [0, 0, 1, 1, 2, 2]
    with pytest.raises(ValueError):
        route(totals, u[:5], 3)


def test_exchange_plan_counts_and_order():
    owner = np.array([0, 0, 1, 1, 1, 2, 2, 2], np.int32)     # sorted batch, world 4 -> slices of 2
    req = np.arange(8) // 2
    p1 = exchange_plan(owner, req, 1, 4)
    assert list(p1.mine) == [2, 3, 4] and list(p1.send_count) == [0, 2, 1, 0] and list(p1.send_first) == [0, 0, 2, 3]
    assert list(p1.slice_owner) == [1, 1] and list(p1.recv_count) == [0, 2, 0, 0]
    p2 = exchange_plan(owner, req, 2, 4)
    assert list(p2.slice_owner) == [1, 2] and list(p2.recv_count) == [0, 1, 1, 0] and list(p2.recv_first) == [0, 0, 1, 2]
    with pytest.raises(ValueError):
        exchange_plan(owner[::-1].copy(), req, 1, 4)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_plan_sorted_equals_route_plus_exchange_plan(world):
    from gear_b200.sharded import plan_sorted
    rng = np.random.default_rng(world)
    for trial in range(20):
        totals = rng.lognormal(3, 1, world)
        if trial % 3 == 0 and world > 1:
            totals[rng.integers(0, world)] = 0.0          # a shard without mass
        if trial % 5 == 0 and world > 2:
            totals[-1] = 0.0
        B = 16 * world
        u = np.sort(rng.random(B))
        if trial == 7:
            u[:] = np.sort(rng.random(B) * 1e-3)          # everything on the first shard
        owner, residual, requester = route(totals, u, world)
        for rank in range(world):
            a = exchange_plan(owner, requester, rank, world)
            b, total, prefix = plan_sorted(totals, u, rank, world)
            assert np.array_equal(a.mine, b.mine), (trial, rank)
            assert np.array_equal(a.send_count, b.send_count) and np.array_equal(a.send_first, b.send_first)
            assert np.array_equal(a.recv_count, b.recv_count) and np.array_equal(a.recv_first, b.recv_first)
            assert np.array_equal(a.slice_owner, b.slice_owner)
            # what the kernel computes from (u, mul=total, sub=prefix[rank]) is route()'s residual
            v = np.minimum(u[b.mine] * total, np.nextafter(total, 0.0)) - prefix[rank]
            assert np.array_equal(np.where(v < totals[rank], v, np.nextafter(totals[rank], 0.0)), residual[b.mine])
