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
