"""Scan / search / draw parity on the GPU: cumulative table, level-1 offsets and
sampled indices must equal the oracle's bit for bit on the same priorities and
the same variates."""
import numpy as np
import pytest
import torch

from gear_b200 import _native as N
from gear_b200 import core

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("n", [1, 2, 127, 128, 4095, 4096, 4097, 5 * 4096 + 123, 1 << 20])
def test_scan_bit_exact(O, n):
    p = O.synth_lognormal(21, n, n)
    cdf, l1, status = core.scan(dev(p))
    torch.cuda.synchronize()
    ocdf, ol1, total, bad = O.scan(p)
    assert np.array_equal(cdf.cpu().numpy(), ocdf)
    assert np.array_equal(l1.cpu().numpy(), ol1)
    assert status.cpu().tolist()[0] == 0


def test_scan_config2_and_search_bit_exact(O):
    # config 2: 1,048,576 LogNormal(0,1) priorities, 4096 variates U[0,total).
    n, b = 1 << 20, 4096
    p = O.synth_lognormal(0x6EA20102, 0, n)
    ocdf, ol1, total, _ = O.scan(p)
    u = O.synth_u01(0x6EA20202, 0, b) * total
    cdf, l1, status = core.scan(dev(p))
    got = core.search(cdf, l1, dev(u), status=status)
    torch.cuda.synchronize()
    want, near = O.search(ocdf, ol1, u, want_near=True)
    assert np.array_equal(got.cpu().numpy(), want)
    st = status.cpu().tolist()
    assert st[0] == 0 and st[1] == int(near.sum())
    # flips against an independent float64 running sum are neighbours and few
    ref = O.search_f64(p, u)
    flips = want != ref
    assert flips.sum() <= 32 and np.all(np.abs(want[flips] - ref[flips]) <= 1)


def test_search_edges_zero_priorities_and_scaling(O):
    n = 3 * 4096 + 77
    p = O.synth_lognormal(5, 1, n)
    p[::3] = 0.0
    p[4096:8192] = 0.0
    ocdf, ol1, total, _ = O.scan(p)
    cdf, l1, status = core.scan(dev(p))
    u = O.synth_u01(6, 1, 3000) * total
    u[:5] = [0.0, total, np.nextafter(total, 0), -1.0, np.nan]
    got = core.search(cdf, l1, dev(u)).cpu().numpy()
    assert np.array_equal(got, O.search(ocdf, ol1, u))
    assert np.all(p[got] > 0)
    u01 = O.synth_u01(6, 2, 777)
    got = core.search(cdf, l1, dev(u01), scale=True).cpu().numpy()
    assert np.array_equal(got, O.search(ocdf, ol1, u01, scale=True))


def test_all_zero_and_bad_priorities(O):
    p = np.zeros(5000, np.float32)
    cdf, l1, status = core.scan(dev(p))
    got = core.search(cdf, l1, dev(np.array([0.0, 0.7]))).cpu().numpy()
    assert list(got) == [4999, 4999]
    p = np.ones(9000, np.float32); p[8000] = -2.0
    _, _, status = core.scan(dev(p))
    assert status.cpu().tolist()[0] & N.ST_BAD_PRIORITY
    p[8000] = np.nan
    _, _, status = core.scan(dev(p))
    assert status.cpu().tolist()[0] & N.ST_BAD_PRIORITY


def test_inexact_level1_is_rebuilt_in_order(O):
    # Aggregates that differ by ~2^60 make float64 partial sums round; the kernel must
    # then fall back to the in-order sum, which is what the oracle computes.
    n = 64 * 4096
    p = np.full(n, 1.234e-3, np.float32)
    p[::8192] = 3e18            # every other partition sums to ~3e18, the rest to ~5
    p[4096 * 33 + 9] = 7.7e5
    ocdf, ol1, total, _ = O.scan(p)
    assert len(np.unique(np.diff(ol1))) > 2
    for _ in range(3):
        cdf, l1, status = core.scan(dev(p))
        assert np.array_equal(l1.cpu().numpy(), ol1)
        assert np.array_equal(cdf.cpu().numpy(), ocdf)
        assert status.cpu().tolist()[0] & N.ST_L1_RESUMMED


def test_sampler_object_repeated_scans(O):
    n = 37 * 4096 + 11
    s = core.PrioritySampler(n)
    for rep in range(4):
        p = O.synth_lognormal(100 + rep, 0, n)
        ocdf, ol1, total, _ = O.scan(p)
        s.scan(dev(p))
        u = O.synth_u01(200 + rep, 0, 1000)
        got = s.search(dev(u), scale=True)
        tot, st = s.result()
        assert tot == total and st[0] == 0
        assert np.array_equal(s.cdf.cpu().numpy(), ocdf)
        assert np.array_equal(s.l1.cpu().numpy(), ol1)
        assert np.array_equal(got.cpu().numpy(), O.search(ocdf, ol1, u, scale=True))


def test_uniform_draw_and_decode(O):
    u = O.synth_u01(1, 1, 5000)
    u[:3] = [0.0, 0.9999999999999999, 1.0]
    n = 4096 * 1000
    got = core.sample_uniform(n, dev(u))
    assert np.array_equal(got.cpu().numpy(), O.uniform(u, n))
    lengths = np.random.default_rng(0).integers(1, 1001, 4096).astype(np.int64)
    idx, ts, ln = core.decode(got, 1000, lengths=dev(lengths), index_offset=4096)
    oi, ot, ol = O.decode(got.cpu().numpy(), 1000, lengths=lengths, index_offset=4096)
    assert np.array_equal(idx.cpu().numpy(), oi) and np.array_equal(ts.cpu().numpy(), ot)
    assert np.array_equal(ln.cpu().numpy(), ol)
    idx, ts, ln = core.decode(got, 1000)
    assert torch.all(ln == 1000) and torch.all(idx * 1000 + ts == got)


def test_large_scan_properties_and_oracle(O):
    # 16M priorities (64 MB, beyond what fits a single wave): bit-exact against the
    # C oracle, which finishes this size in well under a second.
    n = 1 << 24
    p = torch.empty(n, dtype=torch.float32, device=DEV)
    core.fill(p, N.FILL_F32_LOGNORMAL, seed=31)
    cdf, l1, status = core.scan(p)
    hp = p.cpu().numpy()
    ocdf, ol1, total, _ = O.scan(hp)
    assert np.array_equal(l1.cpu().numpy(), ol1)
    assert np.array_equal(cdf.cpu().numpy(), ocdf)
    assert status.cpu().tolist()[0] == 0
    u = torch.empty(8192, dtype=torch.float64, device=DEV)
    core.fill(u, N.FILL_U01_F64, seed=32)
    got = core.search(cdf, l1, u, scale=True).cpu().numpy()
    assert np.array_equal(got, O.search(ocdf, ol1, u.cpu().numpy(), scale=True))


def test_fill_integer_kinds_match_oracle_philox(O):
    w = torch.empty(1001, dtype=torch.int32, device=DEV)
    core.fill(w, N.FILL_U32, seed=0xABCDEF0123, stream_id=5)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), O.philox_u32(0xABCDEF0123, 5, 0, 1001))
    core.fill(w, N.FILL_I32_RANGE, seed=9, stream_id=1, a=0, b=50257)
    assert np.array_equal(w.cpu().numpy(), O.synth_randint(9, 1, 1001, 0, 50257))
    b = torch.empty(1003, dtype=torch.uint8, device=DEV)
    core.fill(b[1:], N.FILL_U8, seed=4, count=1002)       # unaligned start
    assert np.array_equal(b[1:].cpu().numpy(), O.philox_u32(4, 0, 0, 251).view(np.uint8)[:1002])
    d = torch.empty(500, dtype=torch.float64, device=DEV)
    core.fill(d, N.FILL_U01_F64, seed=12, stream_id=3)
    assert np.array_equal(d.cpu().numpy(), O.philox_u01(12, 3, 0, 500))
    f = torch.empty(4000, dtype=torch.float32, device=DEV)
    core.fill(f, N.FILL_F32_UNIFORM, seed=13, a=-1.0, b=1.0)
    assert np.array_equal(f.cpu().numpy(), O.synth_uniform_pm1(13, 0, 4000))
    core.fill(f, N.FILL_F32_NORMAL, seed=14)
    np.testing.assert_allclose(f.cpu().numpy(), O.synth_normal(14, 0, 4000), rtol=1e-5, atol=1e-6)
    core.fill(f, N.FILL_F32_LOGNORMAL, seed=15)
    np.testing.assert_allclose(f.cpu().numpy(), O.synth_lognormal(15, 0, 4000), rtol=1e-5)


def test_scan_in_two_launches_equals_one_call(O):
    n = 9 * 4096 + 5
    p = O.synth_lognormal(91, 0, n)
    ocdf, ol1, ototal, _ = O.scan(p)
    s = core.PrioritySampler(n)
    for store in (True, False):
        s.scan_partitions(dev(p), store=store)
        s.scan_level1()
        tot, st = s.result()
        assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal and st[0] == 0
        if store:
            assert np.array_equal(s.cdf.cpu().numpy(), ocdf)


def test_totals_only_scan_gives_the_same_level1(O):
    for n in [1, 4095, 4097, 37 * 4096 + 11, 1 << 22]:
        p = O.synth_lognormal(77, n, n)
        s = core.PrioritySampler(n)
        s.scan(dev(p), store=False)
        tot, st = s.result()
        _, ol1, ototal, _ = O.scan(p)
        assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal and st[0] == 0


@pytest.mark.parametrize("n", [4096 * 3 + 17, 1 << 20])
def test_incremental_update_equals_full_scan(O, n):
    rng = np.random.default_rng(n)
    p = O.synth_lognormal(55, n, n)
    s = core.PrioritySampler(n)
    dp = dev(p)
    s.scan(dp)
    for rep in range(3):
        m = [1, 100, 3000][rep]
        idx = rng.integers(0, n, m).astype(np.int64)
        idx = np.unique(idx)                        # one writer per entry keeps the host copy well defined
        if rep == 1:
            idx[-1] = n - 1                         # the ragged last partition
        val = rng.lognormal(0, 1, len(idx)).astype(np.float32)
        val[::7] = 0.0
        p[idx] = val
        s.update(dp, dev(idx), dev(val))
        tot, st = s.result()
        ocdf, ol1, ototal, _ = O.scan(p)
        assert np.array_equal(dp.cpu().numpy(), p)
        assert np.array_equal(s.cdf.cpu().numpy(), ocdf)
        assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal and st[0] == 0
    # a full scan afterwards still works (scratch left consistent)
    s.scan(dp)
    assert np.array_equal(s.l1.cpu().numpy(), O.scan(p)[1])
    # the same updates on a table kept without its level-2 entries
    s.scan(dp, store=False)
    idx = np.unique(rng.integers(0, n, 500).astype(np.int64))
    val = rng.lognormal(0, 1, len(idx)).astype(np.float32)
    p[idx] = val
    s.update(dp, dev(idx), dev(val))
    tot, st = s.result()
    _, ol1, ototal, _ = O.scan(p)
    assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal and st[0] == 0


def test_incremental_update_inexact_level1_and_bad_index(O):
    n = 32 * 4096
    p = np.full(n, 1.234e-3, np.float32)
    s = core.PrioritySampler(n)
    dp = dev(p)
    s.scan(dp)
    idx = np.array([0, 8192, 5 * 4096 + 3], np.int64); val = np.array([3e18, 3e18, 7.7e5], np.float32)
    p[idx] = val
    s.update(dp, dev(idx), dev(val))
    tot, st = s.result()
    ocdf, ol1, _, _ = O.scan(p)
    assert np.array_equal(s.l1.cpu().numpy(), ol1) and np.array_equal(s.cdf.cpu().numpy(), ocdf)
    assert st[0] & N.ST_L1_RESUMMED
    s.update(dp, dev(np.array([n, -1], np.int64)), dev(np.array([1.0, 1.0], np.float32)))
    _, st = s.result()
    assert st[0] & N.ST_BAD_REQUEST
    assert np.array_equal(dp.cpu().numpy(), p)


def test_back_to_back_scans_of_one_sampler(O):
    # A totals-only scan may start while the launch before it in the stream is still finishing;
    # with nothing in between, that launch is the previous scan's level-1 launch.  Every scan must
    # still leave exactly its own table and no spurious status.
    n = 1500 * 4096 + 77                      # more than 1024 partitions: level 1 is its own launch
    ps = [O.synth_lognormal(10 + i, 0, n) for i in range(3)]
    ps[1][::3] *= 1e-3
    dps = [dev(p) for p in ps]
    want = O.scan(ps[2])
    s = core.PrioritySampler(n)
    for rep in range(5):
        for store in (False, True):
            for i in range(3):
                s.scan(dps[i], store=store)
            tot, st = s.result()
            assert np.array_equal(s.l1.cpu().numpy(), want[1]) and tot == want[2] and st[0] == 0
            if store:
                assert np.array_equal(s.cdf.cpu().numpy(), want[0])


def test_back_to_back_scans_of_a_small_table_without_host_sync(O):
    # Tables of at most 1024 partitions have their level 1 built by the scan's last CTA, so nothing
    # stands between two scans of one sampler in the stream.  They must still not run side by side
    # (they share the ticket and CTA counters): several scans queued without any host
    # synchronisation leave exactly the last one's table.
    n = 37 * 4096 + 11
    ps = [O.synth_lognormal(300 + i, 0, n) for i in range(4)]
    ps[2][::2] *= 1e-2
    dps = [dev(p) for p in ps]
    want = [O.scan(p) for p in ps]
    s = core.PrioritySampler(n)
    for rep in range(6):
        for store in (False, True):
            for i in range(4):
                s.scan(dps[i], store=store)
                s.scan(dps[(i + 1) % 4], store=store)
                s.scan(dps[i], store=store)
            tot, st = s.result()
            assert np.array_equal(s.l1.cpu().numpy(), want[3][1]) and tot == want[3][2] and st[0] == 0
            if store:
                assert np.array_equal(s.cdf.cpu().numpy(), want[3][0])


def test_small_table_scan_sample_scan_chain_without_host_sync(O):
    # scan_totals -> sample_gather -> scan_totals -> ... on a small table, and two small samplers
    # used in turn with the storing scan that may start early: every batch equals the oracle's.
    rows, T, cap, B, L = [36, 4, 1], 50, 400, 300, 5
    t = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
    t.connect()
    img = O.philox_u32(5, 3, 0, (t.nbytes + 3) // 4).view(np.uint8)[: t.nbytes].copy()
    t.write(0, img)
    h = core.StorageHandler(t)
    cols = [0, 1, 2]
    h.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * 3)
    n = cap * T
    ps = [O.synth_lognormal(310 + i, 0, n) for i in range(3)]
    dps = [dev(p) for p in ps]
    scans = [O.scan(p) for p in ps]
    us = [O.synth_u01(320 + i, 0, B) for i in range(6)]
    dus = [dev(u) for u in us]
    for mode in ("totals", "alternate"):
        sa, sb = core.PrioritySampler(n), core.PrioritySampler(n)
        flats = [torch.empty(B, dtype=torch.int64, device=DEV) for _ in range(6)]
        outs = [[torch.empty(B * L * r, dtype=torch.uint8, device=DEV) for r in rows] for _ in range(6)]
        for i in range(6):                                  # no host synchronisation inside this loop
            sm = sa if (mode == "totals" or i % 2 == 0) else sb
            if mode == "totals":
                sm.scan(dps[i % 3], store=False)
            else:
                sm.scan(dps[i % 3], store=True, alternate=True)
            sm.sample_gather(h, dus[i], cols, outs[i], scale=True, out_flat=flats[i])
        torch.cuda.synchronize()
        for i in range(6):
            ocdf, ol1, _, _ = scans[i % 3]
            want = O.search(ocdf, ol1, us[i], scale=True)
            assert np.array_equal(flats[i].cpu().numpy(), want), (mode, i)
            oi, ot, ol = O.decode(want, T)
            for c, r in enumerate(rows):
                w = O.fused_subcopy(img, oi, ot, ol, t.trajectory_stride, t.accu[c], T, r, 0, L, False)
                assert np.array_equal(outs[i][c].cpu().numpy(), w), (mode, i, c)
        assert sa.result()[1][0] == 0 and sb.result()[1][0] == 0


def test_lazy_level2_block_boundaries_and_block_totals(O):
    # A table kept without its level-2 entries is sampled through the block totals the scan leaves
    # (eight per partition): variates on, next to and far from every block boundary of a few
    # partitions must give the stored table's index; the block totals themselves must be the
    # tree's; an incremental update keeps them current.
    n = 6 * 4096 + 1000
    p = O.synth_lognormal(330, 0, n)
    p[4096 * 2: 4096 * 2 + 512] = 0.0          # a block without mass
    p[4096 * 3 + 100] = 5e4                    # a block dominated by one entry
    ocdf, ol1, total, _ = O.scan(p)
    rows, T = [8], 1
    cap = n
    t = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
    t.connect()
    h = core.StorageHandler(t)
    h.set([0], [core.SubscribePattern(0, 1, N.PAD_TAIL)])
    s = core.PrioritySampler(n)
    dp = dev(p)
    s.scan(dp, store=False)
    b0, b1, cur = s.block_totals()
    nparts = (n + 4095) // 4096
    blk = core.device_view((b0, b1)[cur], nparts * 8, torch.float32).cpu().numpy().reshape(nparts, 8)
    # block totals from the oracle's table: the aggregate is their in-order sum
    agg = np.zeros(nparts, np.float32)
    for q in range(nparts):
        x = np.float32(0)
        for w in range(8):
            x = np.float32(x + blk[q, w])
        agg[q] = x
    assert np.array_equal(np.diff(ol1).astype(np.float64), agg.astype(np.float64))
    # variates: every block boundary of every partition, a few ulps around it, plus random ones
    targets = []
    for q in range(nparts):
        x = np.float32(0)
        for w in range(8):
            x = np.float32(x + blk[q, w])
            for k in (-40, -3, -1, 0, 1, 3, 40):
                f = np.float32(x)
                for _ in range(abs(k)):
                    f = np.nextafter(f, np.float32(np.inf if k > 0 else -np.inf))
                targets.append(ol1[q] + float(f))
    u = np.array(targets + list(O.synth_u01(331, 0, 4000) * total), np.float64)
    u = u[(u >= 0) & (u < total)]
    du = dev(u)
    dst = [torch.empty(len(u) * 8, dtype=torch.uint8, device=DEV)]
    flat = torch.empty(len(u), dtype=torch.int64, device=DEV)
    s.sample_gather(h, du, [0], dst, scale=False, out_flat=flat)
    tot, st = s.result()
    want, near = O.search(ocdf, ol1, u, want_near=True)
    assert np.array_equal(flat.cpu().numpy(), want)
    assert st[0] == 0 and st[1] == int(near.sum())
    # update: new priorities in a few blocks; the block totals follow, the indices stay exact
    idx = np.array([5, 4096 * 3 + 100, 4096 * 5 + 600, n - 1], np.int64)
    val = np.array([9.0, 0.5, 77.0, 3.0], np.float32)
    p[idx] = val
    s.update(dp, dev(idx), dev(val))
    s.clear_status()
    ocdf, ol1, total, _ = O.scan(p)
    u2 = O.synth_u01(332, 0, 3000) * total
    flat2 = torch.empty(len(u2), dtype=torch.int64, device=DEV)
    dst2 = [torch.empty(len(u2) * 8, dtype=torch.uint8, device=DEV)]
    s.sample_gather(h, dev(u2), [0], dst2, scale=False, out_flat=flat2)
    want2, near2 = O.search(ocdf, ol1, u2, want_near=True)
    tot, st = s.result()
    assert tot == total and np.array_equal(flat2.cpu().numpy(), want2) and st[1] == int(near2.sum())


def test_draw_follows_the_priorities_in_distribution(O):
    # The reference's runnable weighted draw is torch.multinomial (gear/sampler/global_sampler.py:170):
    # P(i) = w_i / sum(w).  The bit-level definition of this library's draw is its own, so the law
    # is pinned statistically: 2,000,000 variates on 3,000 LogNormal weights with zeros, chi-square
    # against w / sum(w) (threshold: mean + 5 sigma of the chi-square distribution, i.e.
    # dof + 5 * sqrt(2 * dof); a wrong law -- e.g. uniform -- exceeds it by orders of magnitude),
    # zero-weight entries never drawn, and the same statistic for torch.multinomial's own counts
    # with replacement as a yardstick.
    k, draws = 3000, 2_000_000
    w = O.synth_lognormal(340, 0, k)
    w[::7] = 0.0
    dw = dev(w)
    cdf, l1, status = core.scan(dw)
    u = torch.empty(draws, dtype=torch.float64, device=DEV)
    core.fill(u, N.FILL_U01_F64, seed=341)
    got = core.search(cdf, l1, u, scale=True)
    counts = torch.bincount(got, minlength=k).cpu().numpy().astype(np.float64)
    pr = w.astype(np.float64) / w.astype(np.float64).sum()
    assert counts[w == 0].sum() == 0
    m = pr > 0
    dof = int(m.sum()) - 1
    limit = dof + 5.0 * np.sqrt(2.0 * dof)
    chi2 = float((((counts[m] - draws * pr[m]) ** 2) / (draws * pr[m])).sum())
    assert chi2 < limit, (chi2, limit)
    ref = torch.multinomial(dw.double(), draws, replacement=True)
    rc = torch.bincount(ref, minlength=k).cpu().numpy().astype(np.float64)
    chi2_ref = float((((rc[m] - draws * pr[m]) ** 2) / (draws * pr[m])).sum())
    assert chi2_ref < limit, (chi2_ref, limit)
    # and the two empirical laws agree with each other (two-sample chi-square, same threshold)
    two = float((((counts[m] - rc[m]) ** 2) / (counts[m] + rc[m]).clip(min=1)).sum())
    assert two < limit, (two, limit)
    uni = float((((np.full(int(m.sum()), draws / m.sum()) - draws * pr[m]) ** 2) / (draws * pr[m])).sum())
    assert uni > 100 * limit      # the statistic does tell a wrong law from the right one


def test_large_table_level1_falls_back_to_the_in_order_sum(O):
    # Above 1024 partitions level 1 is a launch of its own (a cluster of eight CTAs summing in
    # integer arithmetic).  Aggregates ~2^60 apart make float64 sums round: it must notice, redo
    # the sum strictly in order (the definition, which the oracle computes) and say so; a
    # well-behaved table right after it on the same sampler must come out exact again, no flag.
    n = 1300 * 4096 + 321
    p = np.full(n, 1.234e-3, np.float32)
    p[::8192] = 3e18
    p[4096 * 700 + 9] = 7.7e5
    ocdf, ol1, total, _ = O.scan(p)
    s = core.PrioritySampler(n)
    dp = dev(p)
    for store in (False, True, False):
        s.scan(dp, store=store)
        tot, st = s.result()
        assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == total
        assert st[0] & N.ST_L1_RESUMMED
        if store:
            assert np.array_equal(s.cdf.cpu().numpy(), ocdf)
    s.clear_status()
    q = O.synth_lognormal(350, 0, n)
    q[: 4096 * 130] = 0.0                       # a whole superblock (and a bit) without mass
    s.scan(dev(q), store=False)
    tot, st = s.result()
    _, ql1, qtotal, _ = O.scan(q)
    assert np.array_equal(s.l1.cpu().numpy(), ql1) and tot == qtotal and st[0] == 0
    # and through the entry point with caller-provided scratch, twice on one scratch block
    cdf, l1, status = core.scan(dev(q))
    assert np.array_equal(l1.cpu().numpy(), ql1) and status.cpu().tolist()[0] == 0


@pytest.mark.parametrize("n", [1, 4095, 3 * 4096 + 5, 1 << 20, 592 * 4096, 700 * 4096 + 9])
def test_scan_and_draw_in_one_call(O, n):
    # up to 592 partitions (4 CTAs of 63 registers x 256 threads per SM, 148 SMs) the call is one
    # cooperative launch; above that it is the two launches.  Either way: the bits of scan + search.
    s = core.PrioritySampler(n)
    two = core.PrioritySampler(n)
    rng = np.random.default_rng(n)
    for rep in range(3):                          # back to back: the launch leaves its counters at zero
        p = O.synth_lognormal(70 + rep, n, n)
        if rep == 1:
            p[:: 3] = 0.0
        b = [1, 4096, 777][rep]
        hu = rng.random(b)
        if b > 2:
            hu[0], hu[1] = 0.0, np.nextafter(1.0, 0.0)
        dp, du = dev(p), dev(hu)
        got = s.scan_search(dp, du, scale=True)
        tot, st = s.result()
        ocdf, ol1, ototal, _ = O.scan(p)
        want, near = O.search(ocdf, ol1, hu, scale=True, want_near=True)
        assert np.array_equal(got.cpu().numpy(), want)
        assert np.array_equal(s.cdf.cpu().numpy(), ocdf)
        assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal
        assert st[0] == 0 and st[1] == int(near.sum())
        two.scan(dp)
        assert np.array_equal(two.search(du, scale=True).cpu().numpy(), want)
        two.clear_status(); s.clear_status()
    # the tables it leaves serve the other consumers: a plain search and an incremental update
    assert np.array_equal(s.search(du, scale=True).cpu().numpy(), want)
    idx = np.unique(rng.integers(0, n, min(n, 50)).astype(np.int64))
    val = rng.random(len(idx)).astype(np.float32)
    p[idx] = val
    s.update(dp, dev(idx), dev(val))
    tot, _ = s.result()
    ocdf, ol1, ototal, _ = O.scan(p)
    assert np.array_equal(s.cdf.cpu().numpy(), ocdf) and np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal


def test_scan_and_draw_edge_tables(O):
    n = 5 * 4096
    s = core.PrioritySampler(n)
    z = torch.zeros(n, dtype=torch.float32, device=DEV)
    got = s.scan_search(z, dev(np.array([0.0, 0.5, 0.999])), scale=True)
    assert got.cpu().tolist() == [n - 1] * 3              # nothing selectable: defined as the last index
    p = np.zeros(n, np.float32); p[4096 * 2 + 17] = 2.0; p[n - 1] = 1.0
    got = s.scan_search(dev(p), dev(np.array([0.0, 1.999, 2.0, 2.999, 5.0, -1.0])), scale=False)
    assert got.cpu().tolist() == [4096 * 2 + 17] * 2 + [n - 1] * 3 + [4096 * 2 + 17]
    bad = p.copy(); bad[5] = -1.0
    s.scan_search(dev(bad), dev(np.array([0.5])), scale=True)
    _, st = s.result()
    assert st[0] & N.ST_BAD_PRIORITY
    s.clear_status()
    assert s.scan_search(dev(p), torch.empty(0, dtype=torch.float64, device=DEV)).numel() == 0
    # inexact level 1 (aggregates 2^70 apart): the in-order float64 sum, as in the separate launches
    q = np.full(n, 1e-3, np.float32); q[0] = 3e18; q[4096] = 3e18
    hu = np.random.default_rng(5).random(512)
    got = s.scan_search(dev(q), dev(hu), scale=True)
    ocdf, ol1, _, _ = O.scan(q)
    _, st = s.result()
    assert np.array_equal(got.cpu().numpy(), O.search(ocdf, ol1, hu, scale=True))
    assert np.array_equal(s.l1.cpu().numpy(), ol1) and st[0] & N.ST_L1_RESUMMED


def test_entries_of_weight_zero_are_never_drawn(O):
    # A chunk that begins with zeros would give them its offset, which can be an ulp above the
    # previous chunk's last value; the tree counts such entries as 0 in its running maximum, so
    # they repeat what came before bit for bit.  Variates aimed exactly at those places.
    n = 40 * 4096 + 1234
    rng = np.random.default_rng(11)
    p = rng.lognormal(0, 1, n).astype(np.float32)
    p[rng.random(n) < 0.7] = 0.0
    p[4096 * 3: 4096 * 5] = 0.0                      # whole partitions without weight
    dp = dev(p)
    s = core.PrioritySampler(n)
    s.scan(dp)
    cdf, l1 = s.cdf.cpu().numpy(), s.l1.cpu().numpy()
    ocdf, ol1, total, _ = O.scan(p)
    assert np.array_equal(cdf, ocdf) and np.array_equal(l1, ol1)
    prev = np.concatenate([[0], cdf[:-1]]); prev[::4096] = 0
    assert np.array_equal(cdf[p == 0], prev[p == 0])  # a zero priority repeats its predecessor's entry exactly
    # variates on, just below and just above every entry that precedes an entry of weight zero
    z = np.nonzero(p == 0)[0]
    part = z // 4096
    edge = prev[z].astype(np.float64) + l1[part]
    u = np.concatenate([edge, np.nextafter(edge, 0), np.nextafter(edge, np.inf), rng.random(500_000) * total])
    u = np.clip(u, 0, np.nextafter(total, 0))
    got = s.search(dev(u)).cpu().numpy()
    assert np.array_equal(got, O.search(ocdf, ol1, u))
    assert (p[got] > 0).all()
    # the same through the one-launch scan + draw (a small table) and the draw that rebuilds blocks
    m = 30 * 4096
    s2 = core.PrioritySampler(m)
    got2 = s2.scan_search(dev(p[:m]), dev(rng.random(100_000)), scale=True).cpu().numpy()
    assert (p[:m][got2] > 0).all()
