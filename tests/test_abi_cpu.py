"""The C-ABI library without a GPU: it loads, exports every symbol that
include/gear_b200.h declares, and its host-side logic (layout, sub, argument
errors) agrees with the oracle and the reference-generated golden file."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import gear_b200
from gear_b200 import _native as N
from gear_b200 import core

GOLDEN = Path(__file__).resolve().parent / "golden" / "sub_golden.npz"


def test_library_exports_every_declared_symbol():
    names = N.declared_symbols()
    assert len(names) >= 35
    missing = [n for n in names if not hasattr(N.lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    assert N.lib.gearb_version() >= 100


def test_header_constants_match_python():
    text = (Path(N.PKG).parent / "include" / "gear_b200.h").read_text()
    import re
    defs = dict(re.findall(r"#define (GEARB_[A-Z0-9_]+) (0x[0-9a-fA-F]+|\d+)", text))
    assert int(defs["GEARB_PART"]) == N.PART
    assert int(defs["GEARB_MAX_COLUMNS"]) == N.MAX_COLUMNS
    assert int(defs["GEARB_PAD_HEAD"]) == N.PAD_HEAD and int(defs["GEARB_PAD_TAIL"]) == N.PAD_TAIL
    assert int(defs["GEARB_ST_BAD_REQUEST"], 16) == N.ST_BAD_REQUEST
    assert int(defs["GEARB_STATUS_WORDS"]) == N.STATUS_WORDS


def test_table_layout_matches_oracle(O):
    for rows, T, cap in [([68, 24, 4, 1], 1000, 4096), ([156, 24, 4, 4, 1], 1000, 100000),
                         ([28224, 4, 4, 1], 1000, 1000), ([4096, 4, 4], 1000, 32000)]:
        t = core.TrajectoryTable(rows, T, cap)
        accu, stride = O.table_layout(rows, T)
        assert t.trajectory_stride == stride and t.accu == list(accu)
        assert t.nbytes == stride * cap
    # config 5's shard is 131.3 GB: sizes must not wrap at 32 bits
    t = core.TrajectoryTable([4096, 4, 4], 1000, 32000)
    assert t.nbytes == 131_328_000_000


def test_handler_sub_matches_reference_golden():
    g = np.load(GOLDEN)
    for k in range(int(g["ncases"][0])):
        T, cap, col, off, length, pad, slot = [int(v) for v in g[f"case{k}_meta"]]
        rows = [int(r) for r in g[f"case{k}_rows"]]
        t = core.TrajectoryTable(rows, T, cap)
        h = core.StorageHandler(t)
        h.set([col], [core.SubscribePattern(off, length, pad)])
        idx, ts, ln = g[f"case{k}_req"]
        s, d, b, sl = h.sub(idx, ts, ln, col)
        assert sl == slot
        assert np.array_equal(np.stack([s, d, b]), g[f"case{k}_out"]), k


def test_errors_are_reported_not_fatal():
    t = core.TrajectoryTable([8, 4], 10, 3)
    h = core.StorageHandler(t)
    with pytest.raises(core.GearError, match="without setting its SubscribePattern"):
        h.sub([0], [0], [10], 1)          # same text as handler.cc:88-91
    with pytest.raises(core.GearError):
        h.set([5], [core.SubscribePattern(0, 1)])
    with pytest.raises(core.GearError):
        core.TrajectoryTable([], 10, 3)
    with pytest.raises(core.GearError):
        core.TrajectoryTable([4], 0, 3)
    with pytest.raises(core.GearError):
        core.TrajectoryTable([4] * 17, 10, 3)
    with pytest.raises(core.GearError):
        h.sub([0, 1], [0], [10], 0)


def test_host_table_write_view_read_roundtrip():
    t = core.TrajectoryTable([12, 3], 7, 5)
    assert t.connect() == t.nbytes
    h = core.StorageHandler(t)
    rng = np.random.default_rng(0)
    img = rng.integers(0, 256, t.nbytes, dtype=np.uint8)
    t.write(0, img)
    assert np.array_equal(t.host_view(), img)
    v = h.view(3, 1)
    lo = 3 * t.trajectory_stride + t.accu[1] * 7
    assert v.nbytes == 3 * 7 and np.array_equal(v, img[lo:lo + 21])
    assert np.array_equal(t.read(lo, 21), img[lo:lo + 21])
    with pytest.raises(core.GearError):
        t.write(t.nbytes - 1, np.zeros(2, np.uint8))


def test_sysv_shared_table_attach():
    key = 0x6EA20000 + (abs(hash(("gear_b200", id(object())))) % 0xFFFF)
    a = core.TrajectoryTable([16], 4, 2, key=key, create=True)
    a.connect()
    a.write(0, np.arange(a.nbytes, dtype=np.uint8))
    b = core.TrajectoryTable([16], 4, 2, key=key, create=False)
    b.connect()
    assert np.array_equal(b.host_view(), np.arange(a.nbytes, dtype=np.uint8))
    b.close(); a.close()
    c = core.TrajectoryTable([16], 4, 2, key=key, create=False)
    with pytest.raises(core.GearError):   # creator removed the segment (shared_memory.cc:65-82)
        c.connect()


def test_indexset_block_layout():
    s = core.Indexset(100, 10, 20)
    ts, w = s.timesteps_np, s.weights_np
    assert ts.dtype == np.int64 and w.dtype == np.float32 and len(ts) == len(w) == 10
    # weights follow the timesteps at a 128-byte aligned offset (include/index/set.h:49-69)
    assert w.ctypes.data - ts.ctypes.data == 128
    ts[:] = np.arange(10); w[:] = 0.5
    assert s.timesteps.tolist() == list(range(10)) and float(s.weights.sum()) == 5.0


def test_scratch_size_formula():
    up = lambda v: (v + 255) // 256 * 256
    for n in (1, 4096, 4097, 100_000_000):
        nparts = (n + 4095) // 4096
        assert N.lib.gearb_scan_scratch_bytes(n) == 256 + up(nparts * 4)   # header + one float per partition
    assert N.lib.gearb_scan_scratch_bytes(0) == 0
