"""Gather parity on the GPU: every byte the CUDA path writes is compared with the
oracle (itself pinned to the reference's compiled `sub`) on the same seeded table
and the same requests."""
import numpy as np
import pytest
import torch

from gear_b200 import _native as N
from gear_b200 import core

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def make_table(O, rows, T, cap, residency, seed=1):
    t = core.TrajectoryTable(rows, T, cap, residency=residency)
    t.connect()
    img = O.philox_u32(seed, 9, 0, (t.nbytes + 3) // 4).view(np.uint8)[: t.nbytes].copy()
    t.write(0, img)
    return t, img


def requests(rng, n, T, cap, ragged=True):
    idx = rng.integers(0, cap, n).astype(np.int64)
    ts = rng.integers(0, T, n).astype(np.int64)
    ln = rng.integers(0, T + 1, n).astype(np.int64) if ragged else np.full(n, T, np.int64)
    return idx, ts, ln


def oracle_column(O, img, t, col, pat, idx, ts, ln):
    return O.fused_subcopy(img, idx, ts, ln, t.trajectory_stride, t.accu[col], t.trajectory_length,
                           t.row_bytes[col], pat.offset, pat.length, pat.pad == N.PAD_HEAD)


def run_gather(h, cols, idx, ts, ln, zero_fill, fill_byte=0):
    t = h.table
    dev = [torch.from_numpy(a).to(DEV) for a in (idx, ts, ln)]
    dsts = [torch.full((len(idx) * h.patterns[c].length * t.row_bytes[c],), fill_byte, dtype=torch.uint8, device=DEV)
            for c in cols]
    h.gather(cols, *dev, dsts, zero_fill=zero_fill)
    torch.cuda.synchronize()
    return [d.cpu().numpy() for d in dsts]


@pytest.mark.parametrize("residency", [N.RES_HBM, N.RES_HOST, N.RES_HOST | N.RES_HBM])
def test_config1_shapes_all_columns(O, residency):
    # config 1 shapes (obs f32[17], act f32[6], rew f32, done u8), fewer trajectories.
    rows, T, cap = [68, 24, 4, 1], 1000, 64
    t, img = make_table(O, rows, T, cap, residency)
    h = core.StorageHandler(t)
    pats = [core.SubscribePattern(0, 20, N.PAD_TAIL)] * 4
    h.set([0, 1, 2, 3], pats)
    rng = np.random.default_rng(0)
    idx, ts, ln = requests(rng, 256, T, cap, ragged=False)
    got = run_gather(h, [0, 1, 2, 3], idx, ts, ln, zero_fill=True, fill_byte=0xCD)
    for c in range(4):
        assert np.array_equal(got[c], oracle_column(O, img, t, c, pats[c], idx, ts, ln)), c
    assert h.status() == 0


@pytest.mark.parametrize("rows,T,cap", [
    ([156, 24, 4, 4, 1], 1000, 48),      # config 3 rows
    ([28224, 4, 4, 1], 64, 6),            # config 4 rows (frame stacks)
    ([4096, 4, 4], 200, 12),              # config 5 rows
    ([3, 7, 13, 1, 2, 5], 37, 19),        # nothing aligned to anything
    ([2049, 2047, 16, 15, 17], 33, 7),    # around the 2 KiB piece size and the 16-byte vector
])
def test_random_patterns_all_alignments(O, rows, T, cap):
    t, img = make_table(O, rows, T, cap, N.RES_HBM, seed=len(rows))
    h = core.StorageHandler(t)
    rng = np.random.default_rng(sum(rows))
    for trial in range(4):
        cols = list(range(len(rows)))
        pats = [core.SubscribePattern(int(rng.integers(-T // 2, T // 2)), int(rng.integers(1, min(T, 70))),
                                      int(rng.integers(0, 3))) for _ in cols]
        h.set(cols, pats)
        idx, ts, ln = requests(rng, int(rng.integers(1, 300)), T, cap)
        for zero_fill in (True, False):
            got = run_gather(h, cols, idx, ts, ln, zero_fill=zero_fill, fill_byte=0xEE if zero_fill else 0)
            for c in cols:
                assert np.array_equal(got[c], oracle_column(O, img, t, c, pats[c], idx, ts, ln)), (trial, c, zero_fill)


def test_subcopy_leaves_padding_untouched(O):
    # Drop-in semantics of handler.subcopy: only the clipped segment is written
    # (the reference's loader relies on torch.zeros, offline_loader.py:181-189).
    rows, T, cap = [20, 6], 30, 5
    t, img = make_table(O, rows, T, cap, N.RES_HBM)
    h = core.StorageHandler(t)
    for pad in (N.PAD_HEAD, N.PAD_TAIL, N.PAD_INACTIVE):
        pat = core.SubscribePattern(-4, 12, pad)
        h.set([0], [pat])
        idx = np.array([0, 4, 2], np.int64); ts = np.array([0, 25, 10], np.int64); ln = np.array([30, 28, 0], np.int64)
        dst = torch.full((3 * 12 * 20,), 0x77, dtype=torch.uint8, device=DEV)
        h.subcopy(*[torch.from_numpy(a).to(DEV) for a in (idx, ts, ln)], 0, dst)
        torch.cuda.synchronize()
        want = O.fused_subcopy(img, idx, ts, ln, t.trajectory_stride, 0, T, 20, -4, 12, pad == N.PAD_HEAD,
                               dst=np.full(3 * 12 * 20, 0x77, np.uint8))
        assert np.array_equal(dst.cpu().numpy(), want)


def test_unaligned_destination_and_typed_tensors(O):
    rows, T, cap = [68, 1], 100, 9
    t, img = make_table(O, rows, T, cap, N.RES_HBM)
    h = core.StorageHandler(t)
    pat = core.SubscribePattern(0, 5, N.PAD_TAIL)
    h.set([0, 1], [pat, pat])
    rng = np.random.default_rng(5)
    idx, ts, ln = requests(rng, 33, T, cap)
    dev = [torch.from_numpy(a).to(DEV) for a in (idx, ts, ln)]
    obs = torch.zeros((33, 5, 17), dtype=torch.float32, device=DEV)
    backing = torch.zeros(33 * 5 + 3, dtype=torch.uint8, device=DEV)
    done = backing[3:]                      # destination that starts 3 bytes off alignment
    h.gather([0, 1], *dev, [obs, done], zero_fill=True)
    torch.cuda.synchronize()
    assert np.array_equal(obs.cpu().numpy().view(np.uint8).reshape(-1), oracle_column(O, img, t, 0, pat, idx, ts, ln))
    assert np.array_equal(done.cpu().numpy(), oracle_column(O, img, t, 1, pat, idx, ts, ln))
    assert backing[:3].sum().item() == 0


def test_bad_requests_are_skipped_and_flagged(O):
    rows, T, cap = [8], 10, 4
    t, img = make_table(O, rows, T, cap, N.RES_HBM)
    h = core.StorageHandler(t)
    h.set([0], [core.SubscribePattern(0, 4, N.PAD_TAIL)])
    idx = np.array([0, 4, -1, 3], np.int64); ts = np.array([1, 1, 1, 8], np.int64); ln = np.array([10, 10, 10, 99], np.int64)
    got = run_gather(h, [0], idx, ts, ln, zero_fill=True, fill_byte=0x55)[0]
    good = np.array([0, 0, 0, 3], np.int64)
    want = O.fused_subcopy(img, good, ts, np.array([10, 0, 0, 10], np.int64), t.trajectory_stride, 0, T, 8, 0, 4, False)
    assert np.array_equal(got, want)
    st = h.status()
    assert st & N.ST_BAD_REQUEST and st & N.ST_LEN_CLAMPED


def test_empty_batch_and_errors():
    t = core.TrajectoryTable([8], 10, 4, residency=N.RES_HBM); t.connect()
    h = core.StorageHandler(t)
    h.set([0], [core.SubscribePattern(0, 4, N.PAD_TAIL)])
    e = torch.empty(0, dtype=torch.int64, device=DEV)
    h.gather([0], e, e, e, [torch.empty(0, dtype=torch.uint8, device=DEV)])
    one = torch.zeros(1, dtype=torch.int64, device=DEV)
    with pytest.raises(core.GearError):   # destination too small
        h.gather([0], one, one, one, [torch.empty(8, dtype=torch.uint8, device=DEV)])
    with pytest.raises(core.GearError):   # pattern never set for column... there is only column 0
        h.gather([1], one, one, one, [torch.empty(64, dtype=torch.uint8, device=DEV)])
    with pytest.raises(core.GearError):   # host tensors are not accepted
        h.gather([0], one.cpu(), one, one, [torch.empty(64, dtype=torch.uint8, device=DEV)])


def test_vcopy_and_copy_match_reference_test_copy(O):
    # tests/test_copy.py of the reference: pinned host source, one 960-byte slice of ones.
    data = torch.ones((32, 100, 4, 3, 2), dtype=torch.float32).pin_memory()
    copied = torch.zeros((10, 4, 3, 2), dtype=torch.float32, device=DEV)
    z = torch.zeros(1, dtype=torch.long, device=DEV)
    stride = copied.numel() * copied.element_size() * torch.ones(1, dtype=torch.long, device=DEV)
    core.vcopy(data.data_ptr(), copied, z, z, stride, int(stride[0]))
    torch.cuda.synchronize()
    assert torch.all(copied == 1)
    # random offset lists, arbitrary alignment, against the oracle's vcopy
    rng = np.random.default_rng(9)
    src = rng.integers(0, 256, 1 << 16, dtype=np.uint8)
    n = 50
    lens = rng.integers(0, 700, n).astype(np.int64)
    so = rng.integers(0, (1 << 16) - 700, n).astype(np.int64)
    do = (np.arange(n) * 701).astype(np.int64)
    want = O.vcopy(src, np.zeros(n * 701, np.uint8), so, do, lens)
    dsrc = torch.from_numpy(src).to(DEV)
    dst = torch.zeros(n * 701, dtype=torch.uint8, device=DEV)
    core.vcopy(dsrc.data_ptr(), dst, *[torch.from_numpy(a).to(DEV) for a in (so, do, lens)], 700)
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy(), want)
    dst.zero_()
    core.copy(dsrc.data_ptr(), dst, torch.from_numpy(so).to(DEV), torch.from_numpy(do).to(DEV), 333)
    torch.cuda.synchronize()
    want = O.vcopy(src, np.zeros(n * 701, np.uint8), so, do, np.full(n, 333, np.int64))
    assert np.array_equal(dst.cpu().numpy(), want)


def test_large_table_roundtrip_property(O):
    # Size-independent property at a table larger than L2: what the gather returns
    # equals the same byte ranges read back from the device table by plain copies.
    rows, T, cap = [156, 24, 4, 4, 1], 1000, 2000        # 378 MB, device-filled
    t = core.TrajectoryTable(rows, T, cap, residency=N.RES_HBM); t.connect()
    core.fill_ptr(t.device_ptr, t.nbytes // 4, N.FILL_U32, seed=77)
    h = core.StorageHandler(t)
    pats = [core.SubscribePattern(0, 64, N.PAD_TAIL)] * 5
    h.set(range(5), pats)
    rng = np.random.default_rng(1)
    idx, ts, ln = requests(rng, 1024, T, cap, ragged=False)
    got = run_gather(h, list(range(5)), idx, ts, ln, zero_fill=True, fill_byte=0x11)
    for c in range(5):
        s, d, b, slot = h.sub(idx, ts, ln, c)
        want = np.zeros(1024 * slot, np.uint8)
        for i in range(0, 1024, 37):
            want_i = t.read(int(s[i]), int(b[i]))
            assert np.array_equal(got[c][d[i]:d[i] + b[i]], want_i)
            assert not got[c][i * slot + b[i]:(i + 1) * slot].any()
