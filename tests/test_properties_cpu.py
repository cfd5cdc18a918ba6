"""Property tests (hypothesis) of the host logic and of the oracle's two restatements: whatever the
shapes, offsets, priorities and shard totals, the C restatement and the numpy one agree, the
cumulative table has the properties the search relies on, and the O(world) routing of a sorted
batch equals the request-by-request one."""
import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from gear_b200 import sharded
from oracle import oracle as O

SET = dict(deadline=None, max_examples=60, suppress_health_check=[HealthCheck.too_slow])


@settings(**SET)
@given(st.integers(1, 40), st.integers(1, 30), st.integers(1, 13), st.integers(-12, 12), st.integers(1, 20),
       st.booleans(), st.integers(0, 2**31 - 1))
def test_addressing_c_equals_numpy(n, T, row, offset, length, pad_head, seed):
    rng = np.random.default_rng(seed)
    cap, col_accu = 9, int(rng.integers(0, 50))
    stride = (col_accu + row + int(rng.integers(0, 20))) * T
    idx = rng.integers(0, cap, n)
    ts = rng.integers(0, T, n)
    ln = rng.integers(0, T + 1, n)
    a = O.sub(idx, ts, ln, stride, col_accu, T, row, offset, length, pad_head)
    b = O.np_sub(idx, ts, ln, stride, col_accu, T, row, offset, length, pad_head)
    for x, y in zip(a[:3], b[:3]):
        assert np.array_equal(x, y)
    assert a[3] == b[3] == length * row
    src, dst, nb, slot = a
    assert np.all(nb >= 0) and np.all(nb <= slot)
    live = nb > 0                                     # a copy never leaves its trajectory's column or its slot
    assert np.all(src[live] >= idx[live] * stride + col_accu * T)
    assert np.all(src[live] + nb[live] <= idx[live] * stride + (col_accu + row) * T)
    assert np.all(dst[live] >= np.arange(n)[live] * slot) and np.all(dst[live] + nb[live] <= (np.arange(n)[live] + 1) * slot)
    table = rng.integers(0, 256, cap * stride, dtype=np.uint8)
    assert np.array_equal(O.fused_subcopy(table, idx, ts, ln, stride, col_accu, T, row, offset, length, pad_head),
                          O.np_gather(table, idx, ts, ln, stride, col_accu, T, row, offset, length, pad_head))


@settings(**SET)
@given(st.integers(1, 3 * 4096 + 50), st.floats(0.0, 0.9), st.integers(-20, 20), st.integers(0, 2**31 - 1))
def test_cumulative_table_properties(n, zero_frac, scale_exp, seed):
    rng = np.random.default_rng(seed)
    p = (rng.lognormal(0, 2, n) * 2.0 ** scale_exp).astype(np.float32)
    p[rng.random(n) < zero_frac] = 0.0
    cdf, l1, total, bad = O.scan(p)
    cdf2, l12, total2 = O.np_scan(p)[:3]
    assert np.array_equal(cdf, cdf2) and np.array_equal(l1, l12) and total == total2 and not bad
    # monotone inside every partition, level 1 monotone, total = last level-1 entry
    for lo in range(0, n, 4096):
        assert np.all(np.diff(cdf[lo:lo + 4096]) >= 0)
    assert np.all(np.diff(l1) >= 0) and l1[-1] == total
    if total > 0:
        u = rng.random(200)
        u[:2] = [0.0, np.nextafter(1.0, 0.0)]
        got = O.search(cdf, l1, u, scale=True)
        assert np.array_equal(got, O.np_search(cdf, l1, u, scale=True))
        assert np.all(p[got] > 0)                     # an entry without weight is never drawn
        # and the draw is within one index of an independent float64 running sum, where both have weight
        ref = O.search_f64(p, u * total)
        w = np.nonzero(p > 0)[0]
        rank_of = np.searchsorted(w, got) - np.searchsorted(w, np.minimum(ref, n - 1))
        assert np.all(np.abs(rank_of) <= 1)


@settings(**SET)
@given(st.sampled_from([1, 2, 3, 4, 8]), st.integers(1, 40), st.sampled_from(["contiguous", "scattered"]),
       st.integers(0, 2**31 - 1))
def test_sorted_routing_equals_request_by_request_routing(world, per_rank, layout, seed):
    rng = np.random.default_rng(seed)
    B = world * per_rank
    totals = rng.lognormal(0, 1, world)
    totals[rng.random(world) < 0.2] = 0.0
    if totals.sum() == 0:
        totals[0] = 1.0
    u = np.sort(rng.random(B))
    owner, residual, _ = sharded.route(totals, u, world)
    requester = sharded.requester_of(B, world, layout)
    assert np.all(np.diff(owner) >= 0)                # owners rise with the variate
    assert np.all(residual >= 0) and np.all(residual < np.maximum(totals[owner], np.finfo(np.float64).tiny) + 0)
    seen = np.zeros(B, int)
    for rank in range(world):
        want = sharded.exchange_plan(owner, requester, rank, world)
        plan, total, prefix, slot_map = sharded.plan_layout(totals, u, rank, world, layout)
        assert np.array_equal(np.asarray(plan.mine), want.mine)
        assert np.array_equal(plan.send_count, want.send_count) and np.array_equal(plan.recv_count, want.recv_count)
        assert np.array_equal(plan.send_first, want.send_first) and np.array_equal(plan.recv_first, want.recv_first)
        assert plan.send_count.sum() == len(want.mine) and plan.recv_count.sum() == per_rank
        seen[want.mine] += 1
    assert np.all(seen == 1)                          # every request has exactly one owner


@settings(**SET)
@given(st.sampled_from([2, 3, 4, 8]), st.integers(1, 30), st.integers(0, 2**31 - 1))
def test_scattered_slot_map_delivers_every_answer_to_its_place(world, per_rank, seed):
    """Simulate the all-to-all of the scattered layout with the slot maps alone: every owner writes
    its answers at base[q % world] + q // world, the regions travel as send_first/send_count say,
    and each requester must end up with its slice of the batch in order."""
    rng = np.random.default_rng(seed)
    B = world * per_rank
    totals = rng.lognormal(0, 1, world)
    totals[rng.random(world) < 0.25] = 0.0
    if totals.sum() == 0:
        totals[-1] = 2.0
    u = np.sort(rng.random(B))
    plans = [sharded.plan_layout(totals, u, r, world, "scattered") for r in range(world)]
    received = [np.full(per_rank, -1, np.int64) for _ in range(world)]
    for owner in range(world):
        plan, _, _, (mod, lo, base) = plans[owner]
        region = np.full(int(plan.send_count.sum()), -1, np.int64)      # the owner's send regions, by requester
        for q in plan.mine:                                              # what the owner's launch does per request
            slot = int(base[q % mod]) + q // mod
            assert region[slot] == -1
            region[slot] = q
        assert np.all(region >= 0)
        for req in range(world):                                         # what the exchange does per pair
            c, f = int(plan.send_count[req]), int(plan.send_first[req])
            rplan = plans[req][0]
            assert int(rplan.recv_count[owner]) == c
            dst = int(rplan.recv_first[owner])
            received[req][dst:dst + c] = region[f:f + c]
    for req in range(world):
        assert np.array_equal(received[req], np.arange(req, B, world))   # rank r's slice: positions r, r + world, ...


@settings(**SET)
@given(st.integers(1, 2 * 4096 + 9), st.integers(0, 2**31 - 1))
def test_any_variate_draws_an_entry_with_weight(n, seed):
    rng = np.random.default_rng(seed)
    p = rng.lognormal(0, 3, n).astype(np.float32)
    p[rng.random(n) < rng.random()] = 0.0
    if not p.any():
        p[int(rng.integers(0, n))] = 1.0
    cdf, l1, total, _ = O.scan(p)
    wild = np.array([0.0, -1.0, np.nan, np.inf, -np.inf, total, total * 2, np.nextafter(total, 0), 5e-324,
                     *(rng.random(50) * total), *l1, *np.nextafter(l1, 0), *np.nextafter(l1, np.inf)])
    got = O.search(cdf, l1, wild)
    assert np.all((got >= 0) & (got < n)) and np.all(p[got] > 0)
    assert np.array_equal(got, O.np_search(cdf, l1, wild))
    flat = O.uniform(rng.random(100), n)
    assert np.all((flat >= 0) & (flat < n))


@settings(deadline=None, max_examples=25, suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(1, 5), st.integers(1, 6),
       st.lists(st.tuples(st.integers(0, 9), st.integers(0, 4), st.booleans(), st.booleans(),
                          st.floats(0.1, 10.0, allow_nan=False)), min_size=1, max_size=150))
def test_index_protocol_equals_its_state_machine(m, cap, actions):
    """Any interleaving of simulator and trainer actions: the shared-memory index server and its
    clients report and hold what the plain state machine does."""
    import os
    from gear_b200 import _native as N
    from gear_b200._native import GearError
    from gear_b200.ingest import IndexClient, IndexServer
    key = 0x4B000000 + (os.getpid() % 50000) * 16 + 3
    srv = IndexServer(key, m, 7, cap)
    cls = [IndexClient(key, i, m) for i in range(m)]
    try:
        assert all(c.connect() == 0 for c in cls)
        model = O.IngestModel(m, 7, cap)
        pending = []
        for kind, who, term, alloc, w in actions:
            i = who % m
            if kind < 3:
                try:
                    got = cls[i].acquire(0)
                    assert model.acquire(i) and got == model.cl[i]["tindex"]
                except GearError as e:
                    assert e.code == N.ERR_TIMEOUT and not model.acquire(i)
            elif kind < 5:
                if model.cl[i]["fly"] and model.slots[i]["owner"] == 0:
                    assert cls[i].step_inc() == model.step(i)
            elif kind < 7:
                if model.cl[i]["fly"] and model.slots[i]["owner"] == 0:
                    assert cls[i].writeback(term, alloc, w) == model.writeback(i, term, alloc, w)
            elif kind < 9:
                ni, nu = srv.scan()
                infer, upd = model.scan()
                assert [(int(srv.infer_src[k]), int(srv.infer_idx[k]), int(srv.infer_ts[k])) for k in range(ni)] == infer
                assert [(int(srv.upd_idx[k]), int(srv.upd_ts[k]), np.float32(srv.upd_w[k])) for k in range(nu)] == upd
                srv.update(nu)
                model.update(upd)
                pending += [s for s, _, _ in infer]
            else:
                srv.callback(np.array(pending, np.int32))
                model.callback(pending)
                pending = []
            assert srv.free_count == len(model.free)
            np.testing.assert_array_equal(srv.weights, model.weights)
            np.testing.assert_array_equal(srv.timesteps, model.timesteps)
            # a trajectory is held by at most one simulator, and a held one is not in the free list
            held = [c_["tindex"] for c_, q in zip(model.cl, model.slots) if c_["fly"]]
            assert len(set(held)) == len(held) and not (set(held) & set(model.free))
    finally:
        for c in cls:
            c.close()
        srv.close()
