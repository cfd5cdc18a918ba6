"""Online ingestion end to end: what simulators commit through the shared-memory index reaches
the device-side cumulative-priority table by the incremental update, and that table stays
equal, bit for bit, to the oracle's full scan of the server's weights; a trajectory that is
being (re)written is never drawn."""
import os

import numpy as np
import pytest
import torch

from gear_b200 import core
from gear_b200._native import GearError
from gear_b200.ingest import IndexClient, IndexServer, OnlineIngest

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("cap,m", [(3 * 4096 + 11, 16), (300, 7)])
def test_committed_trajectories_reach_the_device_table(O, cap, m):
    key = 0x48000000 + (os.getpid() % 50000) * 16 + (1 if cap > 1000 else 2)
    rng = np.random.default_rng(cap)
    srv = IndexServer(key, m, 0, cap)
    cls = [IndexClient(key, i, m) for i in range(m)]
    assert all(c.connect() == 0 for c in cls)
    prio = torch.zeros(cap, dtype=torch.float32, device=DEV)
    sampler = core.PrioritySampler(cap)
    sampler.scan(prio)
    ing = OnlineIngest(srv, sampler, prio)
    flying = [False] * m
    being_written = set()
    for it in range(400):
        for i in range(m):                            # every simulator moves once per trainer step
            if not flying[i]:
                try:
                    being_written.add(cls[i].acquire(0))
                    flying[i] = True
                except GearError:
                    continue
            if cls[i].status()["ownership"] != 0:
                continue
            cls[i].step_inc()
            if rng.random() < 0.3:
                being_written.discard(cls[i].get_index())
                cls[i].writeback(True, bool(rng.random() < 0.8), float(rng.lognormal(0, 1)))
                flying[i] = False
            else:
                cls[i].writeback(False, False)
        slots, _, _ = ing.step()
        srv.callback(slots)
        if it % 50 == 49 or it < 3:
            w = srv.weights.copy()
            ocdf, ol1, ototal, _ = O.scan(w)
            tot, st = sampler.result()
            assert np.array_equal(prio.cpu().numpy(), w)
            assert np.array_equal(sampler.cdf.cpu().numpy(), ocdf)
            assert np.array_equal(sampler.l1.cpu().numpy(), ol1) and tot == ototal and st[0] == 0
            if ototal > 0:
                u = torch.from_numpy(rng.random(2048)).to(DEV)
                got = sampler.search(u, scale=True).cpu().numpy()
                assert np.array_equal(got, O.search(ocdf, ol1, u.cpu().numpy(), scale=True))
                assert (w[got] > 0).all()             # zero-weight (free or in-flight) trajectories are never drawn
                held = {c.get_index() for c, f in zip(cls, flying) if f}
                assert not (set(got.tolist()) & held)
    assert (srv.weights > 0).sum() > 10
    for c in cls:
        c.close()
    srv.close()


def test_committed_bytes_reach_the_device_table_before_they_can_be_drawn(O):
    # Simulators write their trajectory into the shared-memory side of the table; the trainer's
    # step copies a finished trajectory to the device copy and only then gives it weight.  Every
    # drawn segment therefore holds exactly what its simulator wrote.
    from gear_b200 import _native as N
    rows, T, cap, m, L = [12, 4], 50, 200, 6, 5
    key = 0x49000000 + (os.getpid() % 50000) * 16
    table = core.TrajectoryTable(rows, T, cap, residency=N.RES_HOST, key=key + 1)
    table.connect()
    host = table.host_view()
    host[:] = 0xEE                                         # stale bytes everywhere
    table.upload()
    h = core.StorageHandler(table)
    h.set([0, 1], [core.SubscribePattern(0, L, N.PAD_TAIL)] * 2)
    srv = IndexServer(key, m, 0, cap)
    cls = [IndexClient(key, i, m) for i in range(m)]
    assert all(c.connect() == 0 for c in cls)
    n = cap * T
    # one priority per STEP of a trajectory here: weight w of a trajectory -> its T steps share it
    prio = torch.zeros(cap, dtype=torch.float32, device=DEV)
    sampler = core.PrioritySampler(cap)
    sampler.scan(prio)
    ing = OnlineIngest(srv, sampler, prio, table=table)
    rng = np.random.default_rng(8)
    stride = table.trajectory_stride
    written = {}
    flying, epoch = [False] * m, 0
    for it in range(300):
        for i in range(m):
            if not flying[i]:
                try:
                    cls[i].acquire(0)
                    flying[i] = True
                except GearError:
                    continue
            if cls[i].status()["ownership"] != 0:
                continue
            cls[i].step_inc()
            if rng.random() < 0.25:
                idx = cls[i].get_index()
                epoch += 1
                img = rng.integers(0, 256, stride, dtype=np.uint8)
                host[idx * stride:(idx + 1) * stride] = img   # the simulator's finished trajectory
                written[idx] = img
                cls[i].writeback(True, True, float(rng.random() + 0.5))
                flying[i] = False
            else:
                cls[i].writeback(False, False)
        slots, _, _ = ing.step()
        srv.callback(slots)
        if it % 60 == 59:
            w = srv.weights.copy()
            assert (w > 0).sum() > 0
            u = torch.from_numpy(rng.random(64)).to(DEV)
            traj = sampler.search(u, scale=True)
            assert (w[traj.cpu().numpy()] > 0).all()
            ts = torch.from_numpy(rng.integers(0, T - L, 64)).to(DEV)
            ln = torch.full((64,), T, dtype=torch.int64, device=DEV)
            dsts = [torch.empty(64 * L * r, dtype=torch.uint8, device=DEV) for r in rows]
            h.gather([0, 1], traj, ts, ln, dsts, zero_fill=True)
            ti, tt = traj.cpu().numpy(), ts.cpu().numpy()
            for c, r in enumerate(rows):
                got = dsts[c].cpu().numpy().reshape(64, L * r)
                for q in range(64):
                    img = written[int(ti[q])]
                    lo = table.accu[c] * T + int(tt[q]) * r
                    assert np.array_equal(got[q], img[lo:lo + L * r]), (it, c, q)
    for c in cls:
        c.close()
    srv.close()
