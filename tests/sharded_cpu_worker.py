"""CPU ranks for the sharded path (run by test_sharded_cpu.py under torch.distributed.run, gloo).

Every rank plays both roles with the ORACLE standing in for the GPU kernels: as an owner
it searches its shard's cumulative table and gathers segments into per-requester regions
of a send buffer; as a requester it receives its slice of the sorted global batch, ordered
by owner.  Routing and displacement tables come from the product code
(gear_b200.sharded.route / exchange_plan); messages follow the plan exactly as
gearb_comm_alltoallv does.  The result must equal a single-process gather from the
concatenated table with the concatenated priorities.
"""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from gear_b200.sharded import exchange_plan, route  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, W = dist.get_rank(), dist.get_world_size()
    rows, T, cap, L = [12, 3, 8], 64, 128, 5            # 8192 steps per shard = 2 partitions
    n_local = cap * T
    B = 64 * W
    accu, stride = O.table_layout(rows, T)

    def shard_data(r):
        img = O.philox_u32(100 + r, 0, 0, (stride * cap + 3) // 4).view(np.uint8)[: stride * cap].copy()
        prio = O.synth_lognormal(200 + r, 0, n_local)
        prio[r::7] = 0.0
        return img, prio

    img, prio = shard_data(rank)
    cdf, l1, total, _ = O.scan(prio)
    u01 = np.sort(O.synth_u01(300, 0, B))               # every rank holds the whole sorted batch

    gathered = [torch.zeros(1, dtype=torch.float64) for _ in range(W)]
    dist.all_gather(gathered, torch.tensor([total], dtype=torch.float64))
    totals = np.array([float(t[0]) for t in gathered])

    owner, residual, requester = route(totals, u01, W)
    plan = exchange_plan(owner, requester, rank, W)
    b = B // W

    # owner role
    flat_local = O.search(cdf, l1, residual[plan.mine])
    oi, ot, ol = O.decode(flat_local, T)
    send = [O.fused_subcopy(img, oi, ot, ol, stride, int(accu[c]), T, rows[c], 0, L, False) for c in range(len(rows))]
    send.append(flat_local.astype(np.int64).view(np.uint8))
    units = [L * r for r in rows] + [8]
    recv = [np.zeros(b * u, np.uint8) for u in units]

    # the exchange, message by message as the plan says
    reqs = []
    for k, u in enumerate(units):
        for peer in range(W):
            s0, sc = int(plan.send_first[peer]) * u, int(plan.send_count[peer]) * u
            r0, rc = int(plan.recv_first[peer]) * u, int(plan.recv_count[peer]) * u
            if peer == rank:
                assert sc == rc
                recv[k][r0:r0 + rc] = send[k][s0:s0 + sc]
                continue
            if sc:
                reqs.append(dist.isend(torch.from_numpy(send[k][s0:s0 + sc].copy()), peer, tag=k))
            if rc:
                buf = torch.from_numpy(recv[k][r0:r0 + rc])
                reqs.append(dist.irecv(buf, peer, tag=k))
    for r in reqs:
        r.wait()
    gflat = recv[-1].view(np.int64) + plan.slice_owner.astype(np.int64) * n_local

    # single-process answer on the concatenated table
    imgs, prios = zip(*[shard_data(r) for r in range(W)])
    gimg, gprio = np.concatenate(imgs), np.concatenate(prios)
    gcdf, gl1, gtotal, _ = O.scan(gprio)
    want_flat = O.search(gcdf, gl1, u01, scale=True)[rank * b:(rank + 1) * b]
    assert np.array_equal(gflat, want_flat), (rank, np.nonzero(gflat != want_flat)[0][:5])
    gi, gt, gl = O.decode(want_flat, T)
    for c in range(len(rows)):
        want = O.fused_subcopy(gimg, gi, gt, gl, stride, int(accu[c]), T, rows[c], 0, L, False)
        assert np.array_equal(recv[c], want), (rank, c)
    # the plan is consistent across ranks: what I send to p is what p expects from me
    mat = [torch.zeros(W, dtype=torch.int64) for _ in range(W)]
    dist.all_gather(mat, torch.from_numpy(plan.send_count.copy()))
    for p in range(W):
        assert int(mat[p][rank]) == int(plan.recv_count[p])
    dist.barrier()
    if rank == 0:
        print("SHARDED_CPU_OK", W)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
