"""The one-launch prioritized sample + gather against the oracle and against the
three separate kernels (search, decode, gather), on the same table, priorities
and variates."""
import numpy as np
import pytest
import torch

from gear_b200 import _native as N
from gear_b200 import core

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def build(O, rows, T, cap, seed):
    t = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM)
    t.connect()
    img = O.philox_u32(seed, 3, 0, (t.nbytes + 3) // 4).view(np.uint8)[: t.nbytes].copy()
    t.write(0, img)
    return t, img


@pytest.mark.parametrize("rows,T,cap,B,L,pad,off", [
    ([156, 24, 4, 4, 1], 1000, 40, 1024, 64, N.PAD_TAIL, 0),    # config 3 rows, B and L
    ([68, 24, 4, 1], 1000, 16, 256, 20, N.PAD_TAIL, 0),         # config 1 rows, B and L
    ([4096, 4, 4], 100, 50, 64, 16, N.PAD_HEAD, -15),           # config 5 rows, head padding
    ([3, 7, 13], 37, 300, 333, 9, N.PAD_HEAD, -4),
])
@pytest.mark.parametrize("store", [True, False])      # False: level 2 rebuilt per request from the priorities
def test_fused_equals_oracle_and_separate_kernels(O, rows, T, cap, B, L, pad, off, store):
    t, img = build(O, rows, T, cap, seed=len(rows))
    h = core.StorageHandler(t)
    cols = list(range(len(rows)))
    pats = [core.SubscribePattern(off, L, pad)] * len(rows)
    h.set(cols, pats)
    n = cap * T
    prio = O.synth_lognormal(77, n, n)
    prio[::5] = 0.0
    lengths = np.random.default_rng(0).integers(1, T + 1, cap).astype(np.int64)
    u01 = O.synth_u01(78, n, B)

    s = core.PrioritySampler(n)
    dprio = dev(prio)
    s.scan(dprio, store=store)
    dl = dev(lengths)
    if not store:
        with pytest.raises(core.GearError):
            s.search(dev(u01), scale=True)
    dsts = [torch.full((B * L * r,), 0x5A, dtype=torch.uint8, device=DEV) for r in rows]
    outs = [torch.empty(B, dtype=torch.int64, device=DEV) for _ in range(4)]
    s.sample_gather(h, dev(u01), cols, dsts, scale=True, lengths=dl, index_offset=0,
                    out_flat=outs[0], out_idx=outs[1], out_ts=outs[2], out_len=outs[3])
    total, st = s.result()

    ocdf, ol1, ototal, _ = O.scan(prio)
    oflat, near = O.search(ocdf, ol1, u01, scale=True, want_near=True)
    oi, ot, ol = O.decode(oflat, T, lengths=lengths)
    assert total == ototal and st[0] == 0 and st[1] == int(near.sum())
    assert np.array_equal(outs[0].cpu().numpy(), oflat)
    assert np.array_equal(outs[1].cpu().numpy(), oi)
    assert np.array_equal(outs[2].cpu().numpy(), ot)
    assert np.array_equal(outs[3].cpu().numpy(), ol)
    for c, r in enumerate(rows):
        want = O.fused_subcopy(img, oi, ot, ol, t.trajectory_stride, t.accu[c], T, r, off, L, pad == N.PAD_HEAD)
        assert np.array_equal(dsts[c].cpu().numpy(), want), c

    # the three-kernel route gives the same bytes
    s.scan(dprio)
    flat = s.search(dev(u01), scale=True)
    idx, ts, ln = core.decode(flat, T, lengths=dl)
    dsts2 = [torch.full((B * L * r,), 0xA5, dtype=torch.uint8, device=DEV) for r in rows]
    h.gather(cols, idx, ts, ln, dsts2, zero_fill=True)
    for a, b in zip(dsts, dsts2):
        assert torch.equal(a, b)


def test_fused_subset_of_columns_and_offset(O):
    rows, T, cap, B, L = [20, 6, 2], 50, 30, 100, 7
    t, img = build(O, rows, T, cap, seed=9)
    h = core.StorageHandler(t)
    h.set([0, 2], [core.SubscribePattern(-2, L, N.PAD_TAIL), core.SubscribePattern(1, 3, N.PAD_HEAD)])
    n = cap * T
    prio = O.synth_lognormal(5, 5, n)
    u = O.synth_u01(6, 6, B)
    s = core.PrioritySampler(n)
    s.scan(dev(prio))
    d0 = torch.empty(B * L * 20, dtype=torch.uint8, device=DEV)
    d2 = torch.empty(B * 3 * 2, dtype=torch.uint8, device=DEV)
    oidx = torch.empty(B, dtype=torch.int64, device=DEV)
    s.sample_gather(h, dev(u), [0, 2], [d0, d2], scale=True, index_offset=1000, out_idx=oidx)
    ocdf, ol1, _, _ = O.scan(prio)
    oi, ot, ol = O.decode(O.search(ocdf, ol1, u, scale=True), T)
    assert np.array_equal(oidx.cpu().numpy(), oi + 1000)
    assert np.array_equal(d0.cpu().numpy(), O.fused_subcopy(img, oi, ot, ol, t.trajectory_stride, t.accu[0], T, 20, -2, L, False))
    assert np.array_equal(d2.cpu().numpy(), O.fused_subcopy(img, oi, ot, ol, t.trajectory_stride, t.accu[2], T, 2, 1, 3, True))
    with pytest.raises(core.GearError):      # more priorities than the table has steps
        core.PrioritySampler(n + 1).sample_gather(h, dev(u), [0], [d0])


@pytest.mark.parametrize("rows,T,cap,L,pad,off,ring", [
    ([4096, 4, 4], 100, 50, 16, N.PAD_TAIL, 0, False),       # config 5 rows: plain 16-byte loads
    ([4096, 4, 4], 100, 50, 16, N.PAD_HEAD, -15, True),      # the same through bulk-copy rings
    ([156, 24, 4, 4, 1], 200, 40, 64, N.PAD_TAIL, 0, False), # short requests: staged in shared memory
    ([3, 7, 13], 37, 300, 9, N.PAD_HEAD, -4, False),
])
@pytest.mark.parametrize("lazy", [False, True])   # True: no stored level-2 tables, blocks rebuilt from the owners' priorities
def test_pull_from_several_shards_on_one_device(O, rows, T, cap, L, pad, off, ring, lazy):
    # Three equal shards held by one process stand for three ranks: the kernel routes every
    # request by the shard totals and reads the owner's tables through the pointer arrays.  The
    # expected result is defined shard by shard: route() on the host, then the owner's search.
    from gear_b200.sharded import route
    W, B = 3, 255
    n = cap * T - 5                     # not a whole number of partitions, and fewer steps than the table
    shards = []
    dprios = []
    for j in range(W):
        t, img = build(O, rows, T, cap, seed=40 + j)
        prio = O.synth_lognormal(50 + j, 0, n)
        prio[j::4] = 0.0
        if j == 1:
            prio *= 3.0
        s = core.PrioritySampler(n)
        dprios.append(dev(prio))
        s.scan(dprios[j], store=not lazy)
        shards.append((t, img, prio, s, O.scan(prio)))
    cdfs = None if lazy else [sh[3].cdf_ptr for sh in shards]
    kw = dict(prios=[p.data_ptr() for p in dprios],
              blks=[sh[3].block_totals()[sh[3].block_totals()[2]] for sh in shards]) if lazy else {}
    h = core.StorageHandler(shards[0][0])
    cols = list(range(len(rows)))
    h.set(cols, [core.SubscribePattern(off, L, pad)] * len(rows))
    totals = np.array([sh[4][2] for sh in shards])
    for trial in range(3):
        u = np.sort(O.synth_u01(60 + trial, 0, B))
        if trial == 1:
            u[:4] = [0.0, 1e-300, 0.5, np.nextafter(1.0, 0.0)]
            u = np.sort(u)
        if trial == 2:
            totals_used = totals.copy(); totals_used[2] = 0.0   # a shard without mass owns nothing
        else:
            totals_used = totals
        dsts = [torch.empty(B * L * r, dtype=torch.uint8, device=DEV) for r in rows]
        oflat = torch.empty(B, dtype=torch.int64, device=DEV); oidx = torch.empty_like(oflat); ots = torch.empty_like(oflat)
        if trial == 0:
            # totals through a mailbox, as separate processes would exchange them: every shard's
            # sampler writes its own total and the epoch, the pull launch waits for all of them
            # (with `lazy`, every shard's level 1 travels into the mailbox too and is searched there)
            box = core.DeviceBuffer(core.mailbox_bytes(n if lazy else 0))
            for epoch in (1, 2, 3):                  # both slots, and a slot's second use
                for j, sh in enumerate(shards):
                    sh[3].publish(W, j, [box.ptr] * W, epoch, copy_l1=lazy)
                l1s = [box.ptr + core.mailbox_l1_offset(n, epoch, j) for j in range(W)] if lazy \
                    else [sh[3].l1_ptr for sh in shards]
                kw_box = dict(kw)
                if lazy:                              # ... and so do its block totals
                    kw_box["blks"] = [box.ptr + core.mailbox_blk_offset(n, epoch, j) for j in range(W)]
                shards[0][3].pull(h, None, cdfs, l1s,
                                  [sh[0].device_ptr for sh in shards], dev(u), cols, dsts, ring=ring,
                                  out_flat=oflat, out_idx=oidx, out_ts=ots, self_shard=(1 if ring else -1),
                                  mailbox=box.ptr, epoch=epoch, **kw_box)
            torch.cuda.synchronize()
            box.free()
        else:
            shards[0][3].pull(h, dev(totals_used), cdfs, [sh[3].l1_ptr for sh in shards],
                              [sh[0].device_ptr for sh in shards], dev(u), cols, dsts, ring=ring,
                              out_flat=oflat, out_idx=oidx, out_ts=ots, self_shard=(1 if ring else -1), **kw)
            torch.cuda.synchronize()
        owner, residual, _ = route(totals_used, np.resize(u, B + (-B) % W), W)   # padded to a multiple of W
        owner, residual = owner[:B], residual[:B]
        want_flat = np.empty(B, np.int64)
        for j in range(W):
            m = owner == j
            want_flat[m] = O.search(shards[j][4][0], shards[j][4][1], residual[m]) + j * n
        assert np.array_equal(oflat.cpu().numpy(), want_flat)
        loc = want_flat - owner * n
        assert np.array_equal(oidx.cpu().numpy(), loc // T + owner * cap)
        assert np.array_equal(ots.cpu().numpy(), loc % T)
        oi, ot, ol = O.decode(loc, T)
        for c, r in enumerate(rows):
            want = np.empty(B * L * r, np.uint8)
            for j in range(W):
                m = np.nonzero(owner == j)[0]
                t, img = shards[j][0], shards[j][1]
                part = O.fused_subcopy(img, oi[m], ot[m], ol[m], t.trajectory_stride, t.accu[c], T, r, off, L,
                                       pad == N.PAD_HEAD)
                want.reshape(B, L * r)[m] = part.reshape(len(m), L * r)
            assert np.array_equal(dsts[c].cpu().numpy(), want), (trial, c)
    assert shards[0][3].result()[1][0] == 0


@pytest.mark.parametrize("to_host", [True, False])       # False: the columns stay in device memory, only the ids travel
def test_host_batch_pipeline_delivers_the_same_batches(O, to_host):
    from gear_b200.pipeline import HostBatchPipeline
    rows, T, cap, B, L = [156, 24, 4, 4, 1], 200, 64, 96, 16
    t, img = build(O, rows, T, cap, seed=77)
    h = core.StorageHandler(t)
    cols = list(range(len(rows)))
    h.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * len(rows))
    n = cap * T
    prio = O.synth_lognormal(78, 0, n)
    dprio = dev(prio)
    s = core.PrioritySampler(n)
    ocdf, ol1, _, _ = O.scan(prio)
    pipe = HostBatchPipeline(s, h, cols, B, depth=2, batch_to_host=to_host)
    us = [torch.from_numpy(O.synth_u01(80 + i, 0, B)).pin_memory() for i in range(5)]
    got = []
    for i, u in enumerate(us):
        pipe.submit(dprio, u)
        if i >= 1:
            hc, hf = pipe.next()
            assert all(c.is_cuda != to_host for c in hc) and not hf.is_cuda
            got.append(([c.cpu().clone() for c in hc], hf.clone()))
    while len(got) < len(us):
        hc, hf = pipe.next()
        got.append(([c.cpu().clone() for c in hc], hf.clone()))
    with pytest.raises(core.GearError):
        pipe.next()
    for u, (hc, hf) in zip(us, got):
        want_flat = O.search(ocdf, ol1, u.numpy(), scale=True)
        assert np.array_equal(hf.numpy(), want_flat)
        oi, ot, ol = O.decode(want_flat, T)
        for c, r in enumerate(rows):
            want = O.fused_subcopy(img, oi, ot, ol, t.trajectory_stride, t.accu[c], T, r, 0, L, False)
            assert np.array_equal(hc[c].numpy(), want)


def test_pull_with_strided_variates_reads_every_kth(O):
    # A rank whose slice is every W-th request of the sorted batch passes the whole batch and a stride.
    rows, T, cap, L, W = [4096, 4], 60, 40, 8, 2
    n = cap * T
    shards = []
    for j in range(W):
        t, img = build(O, rows, T, cap, seed=70 + j)
        s = core.PrioritySampler(n)
        s.scan(dev(O.synth_lognormal(75 + j, 0, n)))
        shards.append((t, s))
    h = core.StorageHandler(shards[0][0])
    h.set([0, 1], [core.SubscribePattern(0, L, N.PAD_TAIL)] * 2)
    B, k = 90, 3
    u = dev(np.sort(O.synth_u01(79, 0, B)))
    totals = torch.stack([sh[1].l1[-1] for sh in shards])
    args = ([sh[1].cdf_ptr for sh in shards], [sh[1].l1_ptr for sh in shards], [sh[0].device_ptr for sh in shards])
    full = [torch.empty(B * L * r, dtype=torch.uint8, device=DEV) for r in rows]
    ffull = torch.empty(B, dtype=torch.int64, device=DEV)
    shards[0][1].pull(h, totals, *args, u, [0, 1], full, out_flat=ffull)
    for first in range(k):
        b = len(range(first, B, k))
        part = [torch.empty(b * L * r, dtype=torch.uint8, device=DEV) for r in rows]
        fpart = torch.empty(b, dtype=torch.int64, device=DEV)
        shards[0][1].pull(h, totals, *args, u[first:], [0, 1], part, out_flat=fpart, count=b, variate_stride=k)
        torch.cuda.synchronize()
        assert torch.equal(fpart, ffull[first::k])
        for c, r in enumerate(rows):
            assert torch.equal(part[c].view(b, L * r), full[c].view(B, L * r)[first::k])


def test_pull_gives_up_when_a_peer_never_publishes(O):
    # The wait on the peers' epoch words is bounded: with one shard's total missing the launch
    # comes back with GEARB_ST_SCAN_ABORTED, writes nothing, and the context stays usable.  The
    # batch is larger than the number of CTAs the GPU holds at once: the CTAs of the later waves
    # see that an earlier one ran out and leave at once, so giving up costs one wait, not several.
    import time
    rows, T, cap, L, W, B = [64, 4], 50, 40, 4, 3, 6000
    n = cap * T
    shards = []
    for j in range(W):
        t, img = build(O, rows, T, cap, seed=90 + j)
        s = core.PrioritySampler(n)
        s.scan(dev(O.synth_lognormal(95 + j, 0, n)))
        shards.append((t, s))
    h = core.StorageHandler(shards[0][0])
    cols = [0, 1]
    h.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * 2)
    u = dev(np.sort(O.synth_u01(99, 0, B)))
    dsts = [torch.full((B * L * r,), 0x77, dtype=torch.uint8, device=DEV) for r in rows]
    box = core.DeviceBuffer(N.MAILBOX_BYTES)
    args = ([sh[1].cdf_ptr for sh in shards], [sh[1].l1_ptr for sh in shards], [sh[0].device_ptr for sh in shards])
    for j in (0, 2):                                   # shard 1 stays silent
        shards[j][1].publish_total(W, j, [box.ptr] * W, 1)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    shards[0][1].pull(h, None, *args, u, cols, dsts, mailbox=box.ptr, epoch=1)
    _, st = shards[0][1].result()
    first_wait = time.perf_counter() - t0
    assert st[0] & N.ST_SCAN_ABORTED and st[2] == 1
    assert all(bool((d == 0x77).all()) for d in dsts)  # nothing was written
    assert N.lib.gearb_sampler_result(shards[0][1]._h, None, None, None) == N.ERR_TIMEOUT
    # a second launch at the same epoch finds the give-up mark and returns without waiting again
    t0 = time.perf_counter()
    shards[0][1].pull(h, None, *args, u, cols, dsts, mailbox=box.ptr, epoch=1)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5 * first_wait + 0.05
    assert first_wait < 20.0
    # the status words accumulate until cleared; a later scan of a small table (whose last CTA
    # builds level 1 itself) is not put off by the earlier time-out
    sm = shards[0][1]
    prio0 = O.synth_lognormal(98, 0, n)
    sm.scan(dev(prio0))
    assert np.array_equal(sm.l1.cpu().numpy(), O.scan(prio0)[1])
    assert sm.result()[1][0] & N.ST_SCAN_ABORTED        # still there: nothing cleared it
    sm.clear_status()
    assert sm.result()[1][:3] == [0, 0, 0]
    shards[1][1].publish_total(W, 1, [box.ptr] * W, 1)
    shards[0][1].pull(h, None, *args, u, cols, dsts, mailbox=box.ptr, epoch=1)
    torch.cuda.synchronize()
    assert not all(bool((d == 0x77).all()) for d in dsts)
    assert sm.result()[1][0] == 0
    box.free()


def _check_batch(O, s, h, t, img, rows, T, L, prio, u01, dsts, out_flat):
    ocdf, ol1, ototal, _ = O.scan(prio)
    oflat = O.search(ocdf, ol1, u01, scale=True)
    assert np.array_equal(out_flat.cpu().numpy(), oflat)
    oi, ot, ol = O.decode(oflat, T)
    for c, r in enumerate(rows):
        want = O.fused_subcopy(img, oi, ot, ol, t.trajectory_stride, t.accu[c], T, r, 0, L, False)
        assert np.array_equal(dsts[c].cpu().numpy(), want), c
    return ol1, ototal


def test_large_table_draws_before_its_level1_exists(O):
    # More than 1024 partitions and no stored level 2: the scan leaves level 1 owing, the sampling
    # launch finds partitions through the superblock sums, and the level-1 launch runs behind the
    # next scan.  Indices, bytes and (whenever it is asked for) level 1 are the oracle's.
    rows, T, cap, B, L = [8, 4], 1000, 6200, 1024, 16
    t, img = build(O, rows, T, cap, seed=9)
    h = core.StorageHandler(t)
    cols = [0, 1]
    h.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * 2)
    n = cap * T
    rng = np.random.default_rng(3)
    prios = [O.synth_lognormal(90 + k, n, n) for k in range(3)]
    prios[1][: 300 * 4096] = 0.0                         # whole superblocks without weight
    prios[2][::2] = 0.0
    dps = [dev(p) for p in prios]
    s = core.PrioritySampler(n)
    dsts = [torch.empty(B * L * r, dtype=torch.uint8, device=DEV) for r in rows]
    flat = torch.empty(B, dtype=torch.int64, device=DEV)
    for step in range(7):                                # scan, draw, scan, draw ...: level 1 always one step behind
        k = step % 3
        u01 = rng.random(B)
        u01[0], u01[1] = 0.0, np.nextafter(1.0, 0.0)
        s.scan(dps[k], store=False)
        s.sample_gather(h, dev(u01), cols, dsts, scale=True, out_flat=flat)
        if step in (2, 5):                               # without a host sync in between on the other steps
            ol1, ototal = _check_batch(O, s, h, t, img, rows, T, L, prios[k], u01, dsts, flat)
            if step == 5:                                # asking for the table has it built
                tot, st = s.result()
                assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal and st[0] == 0
    ol1, ototal = _check_batch(O, s, h, t, img, rows, T, L, prios[k], u01, dsts, flat)
    # two draws from one scan; then consumers that need the table itself
    u2 = rng.random(B)
    s.sample_gather(h, dev(u2), cols, dsts, scale=True, out_flat=flat)
    _check_batch(O, s, h, t, img, rows, T, L, prios[k], u2, dsts, flat)
    idx = np.unique(rng.integers(0, n, 400).astype(np.int64)); val = rng.random(len(idx)).astype(np.float32)
    prios[k][idx] = val
    s.update(dps[k], dev(idx), dev(val))
    s.sample_gather(h, dev(u2), cols, dsts, scale=True, out_flat=flat)
    ol1, ototal = _check_batch(O, s, h, t, img, rows, T, L, prios[k], u2, dsts, flat)
    tot, st = s.result()
    assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal and st[0] == 0
    # two scans in a row, a pinned slot, and the two-launch form of a scan
    s.scan(dps[0], store=False); s.scan(dps[1], store=False)
    s.sample_gather(h, dev(u2), cols, dsts, scale=True, out_flat=flat)
    _check_batch(O, s, h, t, img, rows, T, L, prios[1], u2, dsts, flat)
    for k in (2, 0, 2):
        s.select_slot(0)
        s.scan(dps[k], store=False)
        s.sample_gather(h, dev(u2), cols, dsts, scale=True, out_flat=flat)
    ol1, ototal = _check_batch(O, s, h, t, img, rows, T, L, prios[2], u2, dsts, flat)
    s.scan_partitions(dps[0], store=False); s.scan_level1()
    s.sample_gather(h, dev(u2), cols, dsts, scale=True, out_flat=flat)
    ol1, ototal = _check_batch(O, s, h, t, img, rows, T, L, prios[0], u2, dsts, flat)
    tot, st = s.result()
    assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal and st[0] == 0
    # a stored scan afterwards, and back
    s.scan(dps[1]); assert np.array_equal(s.search(dev(u2), scale=True).cpu().numpy(), O.search(*O.scan(prios[1])[:2], u2, scale=True))
    s.scan(dps[2], store=False)
    s.sample_gather(h, dev(u2), cols, dsts, scale=True, out_flat=flat)
    _check_batch(O, s, h, t, img, rows, T, L, prios[2], u2, dsts, flat)


def test_large_table_with_aggregates_too_far_apart_for_exact_sums(O):
    # Aggregates 2^30 apart: sums of subsets are no longer exact in float64 in every order, so the
    # sampling launch adds the aggregates in order itself; the answers stay the oracle's.
    rows, T, cap, B, L = [4], 1000, 5000, 256, 8
    t, img = build(O, rows, T, cap, seed=10)
    h = core.StorageHandler(t)
    h.set([0], [core.SubscribePattern(0, L, N.PAD_TAIL)])
    n = cap * T
    prio = O.synth_lognormal(95, n, n)
    prio[4096 * 7: 4096 * 9] *= np.float32(2.0 ** 30)
    prio[4096 * 900: 4096 * 901] *= np.float32(2.0 ** -12)
    s = core.PrioritySampler(n)
    dp = dev(prio)
    dsts = [torch.empty(B * L * 4, dtype=torch.uint8, device=DEV)]
    flat = torch.empty(B, dtype=torch.int64, device=DEV)
    rng = np.random.default_rng(4)
    for step in range(3):
        u01 = rng.random(B)
        u01[:64] *= 1e-9                                   # also draws outside the heavy partitions
        s.scan(dp, store=False)
        s.sample_gather(h, dev(u01), [0], dsts, scale=True, out_flat=flat)
        ol1, ototal = _check_batch(O, s, h, t, img, rows, T, L, prio, u01, dsts, flat)
    tot, st = s.result()
    assert np.array_equal(s.l1.cpu().numpy(), ol1) and tot == ototal


def test_large_stored_tables_draw_before_their_level1_exists(O):
    # The same for scans that store level 2: one sampler scanned and drawn from in a loop, and
    # two samplers used in turn (each one's scan may start under the other's sampling launch).
    rows, T, cap, B, L = [8, 4], 1000, 5000, 512, 16
    t, img = build(O, rows, T, cap, seed=11)
    h = core.StorageHandler(t)
    cols = [0, 1]
    h.set(cols, [core.SubscribePattern(0, L, N.PAD_TAIL)] * 2)
    n = cap * T
    rng = np.random.default_rng(6)
    prios = [O.synth_lognormal(96 + k, n, n) for k in range(2)]
    prios[1][1000 * 4096:] = 0.0
    dps = [dev(p) for p in prios]
    dsts = [torch.empty(B * L * r, dtype=torch.uint8, device=DEV) for r in rows]
    flat = torch.empty(B, dtype=torch.int64, device=DEV)
    a, b = core.PrioritySampler(n), core.PrioritySampler(n)
    for step in range(6):
        k = step % 2
        u01 = rng.random(B)
        a.scan(dps[k])
        a.sample_gather(h, dev(u01), cols, dsts, scale=True, out_flat=flat)
        if step >= 3:
            _check_batch(O, a, h, t, img, rows, T, L, prios[k], u01, dsts, flat)
    ocdf, ol1, ototal, _ = O.scan(prios[k])
    assert np.array_equal(a.search(dev(u01), scale=True).cpu().numpy(), O.search(ocdf, ol1, u01, scale=True))
    tot, st = a.result()
    assert np.array_equal(a.l1.cpu().numpy(), ol1) and np.array_equal(a.cdf.cpu().numpy(), ocdf) and tot == ototal
    for step in range(8):
        s, k = (a, b)[step % 2], (step // 2) % 2
        u01 = rng.random(B)
        s.scan(dps[k], alternate=True)
        s.sample_gather(h, dev(u01), cols, dsts, scale=True, out_flat=flat)
        if step >= 4:
            ol1, ototal = _check_batch(O, s, h, t, img, rows, T, L, prios[k], u01, dsts, flat)
    for s in (a, b):
        tot, st = s.result()
        assert st[0] == 0
    assert np.array_equal(b.l1.cpu().numpy(), ol1) and tot == ototal


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_call_sequences_keep_tables_and_draws_exact(O, seed):
    # Any order of the sampler's entry points on a table large enough to owe its level 1: every
    # draw, and the table whenever it is read, equals the oracle's for the priorities of the moment.
    rows, T, cap, B, L = [8], 500, 11000, 256, 4
    t, img = build(O, rows, T, cap, seed=20 + seed)
    h = core.StorageHandler(t)
    h.set([0], [core.SubscribePattern(0, L, N.PAD_TAIL)])
    n = cap * T                                           # 5,500,000 priorities: 1343 partitions
    rng = np.random.default_rng(seed)
    s = core.PrioritySampler(n)
    base = [O.synth_lognormal(30 + k, n, n) for k in range(2)]
    base[1][: n // 3] = 0.0
    cur = None            # host copy of the priorities the table was last built from
    dp = None
    stored = False
    dsts = [torch.empty(B * L * 8, dtype=torch.uint8, device=DEV)]
    flat = torch.empty(B, dtype=torch.int64, device=DEV)
    cache = {}

    def oracle():
        key = cur.tobytes()[:64] + cur[-8:].tobytes() + bytes([int(cur.sum() * 1000) % 251])
        if key not in cache:
            cache.clear()
            cache[key] = O.scan(cur)
        return cache[key]

    for op_i in range(45):
        op = rng.choice(["scan_lazy", "scan_store", "draw", "draw", "search", "update", "result", "pin", "two_launch", "scan_search"])
        if cur is None and op not in ("scan_lazy", "scan_store", "two_launch"):
            op = "scan_lazy"
        if op in ("scan_lazy", "scan_store", "two_launch", "pin"):
            k = int(rng.integers(0, 2))
            cur = base[k].copy()
            dp = dev(cur)
            stored = op == "scan_store" or (op in ("two_launch", "pin") and bool(rng.integers(0, 2)))
            if op == "pin":
                s.select_slot(int(rng.integers(0, 2)))
            if op == "two_launch":
                s.scan_partitions(dp, store=stored)
                s.scan_level1()
            else:
                s.scan(dp, store=stored)
        elif op == "draw":
            u01 = rng.random(B)
            s.sample_gather(h, dev(u01), [0], dsts, scale=True, out_flat=flat)
            ocdf, ol1, ototal, _ = oracle()
            want = O.search(ocdf, ol1, u01, scale=True)
            assert np.array_equal(flat.cpu().numpy(), want), (op_i, op)
            oi, ot, ol = O.decode(want, T)
            assert np.array_equal(dsts[0].cpu().numpy(),
                                  O.fused_subcopy(img, oi, ot, ol, t.trajectory_stride, t.accu[0], T, 8, 0, L, False))
        elif op == "search":
            u01 = rng.random(B)
            if stored:
                got = s.search(dev(u01), scale=True).cpu().numpy()
                ocdf, ol1, _, _ = oracle()
                assert np.array_equal(got, O.search(ocdf, ol1, u01, scale=True)), (op_i, op)
            else:
                with pytest.raises(core.GearError):
                    s.search(dev(u01), scale=True)
        elif op == "update":
            idx = np.unique(rng.integers(0, n, 300).astype(np.int64)); val = rng.random(len(idx)).astype(np.float32)
            cur[idx] = val
            s.update(dp, dev(idx), dev(val))
        elif op == "scan_search":
            k = int(rng.integers(0, 2))
            cur = base[k].copy()
            dp = dev(cur)
            stored = True
            u01 = rng.random(B)
            got = s.scan_search(dp, dev(u01), scale=True).cpu().numpy()
            ocdf, ol1, _, _ = oracle()
            assert np.array_equal(got, O.search(ocdf, ol1, u01, scale=True)), (op_i, op)
        else:
            tot, st = s.result()
            ocdf, ol1, ototal, _ = oracle()
            # (an update may leave aggregates so far apart that level 1 is summed in order: that is flagged)
            assert tot == ototal and st[0] & ~N.ST_L1_RESUMMED == 0, (op_i, op)
            assert np.array_equal(s.l1.cpu().numpy(), ol1)
            if stored:
                assert np.array_equal(s.cdf.cpu().numpy(), ocdf)
    tot, st = s.result()
    assert tot == oracle()[2] and st[0] & ~N.ST_L1_RESUMMED == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_tables_patterns_and_paths(O, seed):
    # Random row sets (which decide between the staged, the direct and -- for a host table -- the
    # ring path), offsets of either sign, both paddings, ragged lengths, stored and rebuilt level 2.
    rng = np.random.default_rng(100 + seed)
    for trial in range(7):
        ncols = int(rng.integers(1, 5))
        big = rng.random() < 0.35
        rows = [int(rng.integers(1, 700 if big else 90)) for _ in range(ncols)]
        T = int(rng.integers(8, 120))
        cap = int(rng.integers(3, 40))
        L = int(rng.integers(1, min(T, 48) + 1))
        host = rng.random() < 0.25
        t = core.TrajectoryTable(rows, T, cap, residency=N.RES_HOST if host else N.RES_HBM)
        t.connect()
        img = rng.integers(0, 256, t.nbytes, dtype=np.uint8)
        t.write(0, img)
        h = core.StorageHandler(t)
        cols = list(range(ncols))
        pats = [core.SubscribePattern(int(rng.integers(-L, L + 1)), L, int(rng.integers(1, 3))) for _ in cols]
        h.set(cols, pats)
        n = cap * T
        prio = rng.lognormal(0, 1.5, n).astype(np.float32)
        prio[rng.random(n) < 0.4] = 0.0
        if not prio.any():
            prio[0] = 1.0
        lengths = rng.integers(1, T + 1, cap).astype(np.int64)
        B = int(rng.integers(1, 200))
        u01 = rng.random(B)
        store = bool(rng.integers(0, 2))
        s = core.PrioritySampler(n)
        s.scan(dev(prio), store=store)
        dsts = [torch.full((B * L * r,), 0x3C, dtype=torch.uint8, device=DEV) for r in rows]
        flat = torch.empty(B, dtype=torch.int64, device=DEV)
        s.sample_gather(h, dev(u01), cols, dsts, scale=True, lengths=dev(lengths), out_flat=flat, zero_fill=True)
        _, st = s.result()
        ocdf, ol1, _, _ = O.scan(prio)
        want = O.search(ocdf, ol1, u01, scale=True)
        tag = (seed, trial, rows, T, cap, L, host, store, B)
        assert np.array_equal(flat.cpu().numpy(), want), tag
        assert st[0] & ~N.ST_L1_RESUMMED == 0, tag
        oi, ot, ol = O.decode(want, T, lengths=lengths)
        for c, r in enumerate(rows):
            exp = O.fused_subcopy(img, oi, ot, ol, t.trajectory_stride, t.accu[c], T, r, pats[c].offset, L,
                                  pats[c].pad == N.PAD_HEAD)
            assert np.array_equal(dsts[c].cpu().numpy(), exp), (tag, c)
        s.close(); h.close(); t.close()
