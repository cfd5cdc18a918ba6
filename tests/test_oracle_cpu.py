"""The oracle against its pins: published Philox vectors, the reference's own
compiled `sub` (golden fixture), the reference's tests/test_copy.py case, and its
second (numpy) restatement."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden" / "sub_golden.npz"


def test_philox_known_answers(O):
    # Known-answer vectors published with the Random123 library for philox4x32-10.
    out = (C.c_uint32 * 4)()
    O.lib().gearo_philox4x32(C.c_uint64(0), C.c_uint64(0), C.c_uint64(0), out)
    assert [hex(x) for x in out] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    ones = 0xFFFFFFFFFFFFFFFF
    O.lib().gearo_philox4x32(C.c_uint64(ones), C.c_uint64(ones), C.c_uint64(ones), out)
    assert [hex(x) for x in out] == ["0x408f276d", "0x41c83b0e", "0xa20bc7c6", "0x6d5451fd"]
    # pi-digit vector: counter 243f6a88 85a308d3 13198a2e 03707344, key a4093822 299f31d0
    O.lib().gearo_philox4x32(C.c_uint64(0x299f31d0a4093822), C.c_uint64(0x0370734413198a2e),
                             C.c_uint64(0x85a308d3243f6a88), out)
    assert [hex(x) for x in out] == ["0xd16cfe09", "0x94fdcceb", "0x5001e420", "0x24126ea1"]


def test_philox_numpy_matches_c(O):
    ctr = np.arange(1000, dtype=np.uint64) * np.uint64(7919)
    a = O.np_philox4x32(0x1234567890ABCDEF, 42, ctr)
    out = (C.c_uint32 * 4)()
    for i in (0, 1, 17, 999):
        O.lib().gearo_philox4x32(C.c_uint64(0x1234567890ABCDEF), C.c_uint64(42), C.c_uint64(int(ctr[i])), out)
        assert list(out) == list(a[i])


def test_sub_matches_reference_golden(O):
    g = np.load(GOLDEN)
    n = int(g["ncases"][0])
    assert n >= 10
    for k in range(n):
        T, cap, col, off, length, pad, slot = [int(v) for v in g[f"case{k}_meta"]]
        rows = g[f"case{k}_rows"]
        idx, ts, ln = g[f"case{k}_req"]
        accu, stride = O.table_layout(rows, T)
        for fn in (O.sub, O.np_sub):
            s, d, b, sl = fn(idx, ts, ln, stride, int(accu[col]), T, int(rows[col]), off, length, pad == 1)
            assert sl == slot
            assert np.array_equal(np.stack([s, d, b]), g[f"case{k}_out"]), (k, fn.__name__)


def test_reference_test_copy_case(O):
    # tests/test_copy.py of the reference: one slice of 10*4*3*2 float32 ones, offsets 0.
    src = np.ones((32, 100, 4, 3, 2), np.float32).view(np.uint8).reshape(-1)
    dst = np.zeros(10 * 4 * 3 * 2 * 4, np.uint8)
    O.vcopy(src, dst, [0], [0], [dst.size])
    assert np.all(dst.view(np.float32) == 1.0)


@pytest.mark.parametrize("pad_head", [False, True])
def test_gather_c_vs_numpy(O, pad_head):
    rng = np.random.default_rng(3)
    rows = [68, 24, 4, 1]; T = 50; cap = 9
    accu, stride = O.table_layout(rows, T)
    table = rng.integers(0, 256, stride * cap, dtype=np.uint8)
    n = 40
    idx = rng.integers(0, cap, n); ts = rng.integers(0, T, n); ln = rng.integers(0, T + 1, n)
    for col in range(4):
        a = O.fused_subcopy(table, idx, ts, ln, stride, int(accu[col]), T, rows[col], -3, 11, pad_head)
        b = O.np_gather(table, idx, ts, ln, stride, int(accu[col]), T, rows[col], -3, 11, pad_head)
        assert np.array_equal(a, b)
        # zero_fill over a dirty destination gives the same bytes as a pre-zeroed one
        dirty = np.full(a.size, 0xAB, np.uint8)
        c = O.fused_subcopy(table, idx, ts, ln, stride, int(accu[col]), T, rows[col], -3, 11, pad_head,
                            dst=dirty, zero_fill=True)
        assert np.array_equal(a, c)


@pytest.mark.parametrize("n", [1, 3, 127, 128, 129, 4095, 4096, 4097, 3 * 4096 + 5, 50000])
def test_scan_c_vs_numpy(O, n):
    p = O.synth_lognormal(11, n, n)
    cdf, l1, total, bad = O.scan(p)
    cdf2, l12, total2 = O.np_scan(p)
    assert bad == 0
    assert np.array_equal(cdf, cdf2) and np.array_equal(l1, l12) and total == total2
    # monotone inside every partition, close to the float64 sum
    for s in range(0, n, O.PART):
        assert np.all(np.diff(cdf[s:s + O.PART]) >= 0)
    assert abs(total - p.astype(np.float64).sum()) <= 1e-5 * max(total, 1.0)


def test_scan_flags_bad_priority(O):
    p = np.ones(100, np.float32); p[7] = -1.0
    assert O.scan(p)[3] == 1
    p[7] = np.nan
    assert O.scan(p)[3] == 1


def test_search_c_vs_numpy_and_zero_priorities(O):
    n = 3 * 4096 + 77
    p = O.synth_lognormal(5, 1, n)
    p[::3] = 0.0                       # unselectable entries
    p[4096:8192] = 0.0                 # a whole partition without mass
    cdf, l1, total, _ = O.scan(p)
    u = O.synth_u01(6, 1, 4000) * total
    u[:4] = [0.0, total, np.nextafter(total, 0), -1.0]
    a = O.search(cdf, l1, u)
    b = O.np_search(cdf, l1, u)
    assert np.array_equal(a, b)
    assert np.all(p[a] > 0), "a zero priority was selected"
    assert np.all((a < 4096) | (a >= 8192))
    # scaled variates: same result as pre-multiplied ones
    u01 = O.synth_u01(6, 2, 500)
    assert np.array_equal(O.search(cdf, l1, u01, scale=True), O.search(cdf, l1, u01 * total))


def test_search_all_zero_is_defined(O):
    p = np.zeros(5000, np.float32)
    cdf, l1, total, _ = O.scan(p)
    assert total == 0.0
    assert np.array_equal(O.search(cdf, l1, np.array([0.0, 0.5])), [4999, 4999])


def test_flip_accounting_small(O):
    n = 1 << 16
    p = O.synth_lognormal(7, 1, n)
    cdf, l1, total, _ = O.scan(p)
    u = O.synth_u01(8, 1, 4096) * total
    a, near = O.search(cdf, l1, u, want_near=True)
    ref = O.search_f64(p, u)
    flips = a != ref
    # every disagreement with the float64 running sum is a neighbouring index
    assert np.all(np.abs(a[flips] - ref[flips]) <= 1)
    assert flips.sum() <= 64


def test_uniform_decode_owner_order(O):
    u = np.array([0.0, 0.5, 0.999999999, 1.0, -0.1])
    assert list(O.uniform(u, 10)) == [0, 5, 9, 9, 0]
    idx, ts, ln = O.decode([0, 999, 1000, 4095999], 1000)
    assert list(idx) == [0, 0, 1, 4095] and list(ts) == [0, 999, 0, 999] and list(ln) == [1000] * 4
    idx, ts, ln = O.decode([1500], 1000, lengths=[7, 9], index_offset=100)
    assert (int(idx[0]), int(ts[0]), int(ln[0])) == (101, 500, 9)
    o, l = O.owner([0, 31999, 32000, 95999], 32000)
    assert list(o) == [0, 0, 1, 2] and list(l) == [0, 31999, 0, 31999]
    assert list(O.comm_order(0, 4)) == [0, 1, 2, 3]
    assert list(O.comm_order(3, 4)) == [1, 2, 3, 0]


def test_threaded_drivers_equal_sequential(O):
    n = 9 * 4096 + 333
    p = O.synth_lognormal(3, 3, n)
    a = O.scan(p)
    for th in (1, 3, 8):
        b = O.scan_mt(p, th)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]) and a[2] == b[2]
    rows = [20, 3]; T = 40; cap = 11
    accu, stride = O.table_layout(rows, T)
    rng = np.random.default_rng(1)
    table = rng.integers(0, 256, stride * cap, dtype=np.uint8)
    m = 97
    idx = rng.integers(0, cap, m); ts = rng.integers(0, T, m); ln = rng.integers(0, T + 1, m)
    want = [O.fused_subcopy(table, idx, ts, ln, stride, int(accu[c]), T, rows[c], -2, 9, c == 1) for c in range(2)]
    dsts = [np.full(m * 9 * r, 0xEE, np.uint8) for r in rows]
    O.gather_mt(table, dsts, idx, ts, ln, stride, T, accu[:2], rows, [-2, -2], [9, 9], [0, 1], threads=4)
    assert all(np.array_equal(w, d) for w, d in zip(want, dsts))


def test_reference_library_when_present(O):
    if not O.Reference.available():
        pytest.skip("oracle/_ref/libgear_ref.so is not built on this machine")
    rows = [68, 24, 4, 1]; T = 1000; cap = 4096
    ref = O.Reference(rows, T, cap)
    accu, stride = O.table_layout(rows, T)
    rng = np.random.default_rng(2)
    idx = rng.integers(0, cap, 500); ts = rng.integers(0, T, 500); ln = rng.integers(0, T + 1, 500)
    for col, (off, L, pad) in enumerate([(0, 20, 2), (-7, 20, 1), (5, 3, 0), (-999, 1000, 1)]):
        ref.set(col, off, L, pad)
        s, d, b, slot = ref.sub(idx, ts, ln, col)
        s2, d2, b2, slot2 = O.sub(idx, ts, ln, stride, int(accu[col]), T, rows[col], off, L, pad == 1)
        assert slot == slot2 and np.array_equal(s, s2) and np.array_equal(d, d2) and np.array_equal(b, b2)
    ref.close()
