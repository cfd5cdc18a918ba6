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
def test_fused_equals_oracle_and_separate_kernels(O, rows, T, cap, B, L, pad, off):
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
    s.scan(dev(prio))
    dl = dev(lengths)
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
