"""gearb_scan_static: the scan for callers that cannot allocate device memory.

Some users of this library are not in a position to call cudaMalloc when they need
a cumulative table: a sampler inside a training step must not stall the device the
way cudaMalloc does, and a process that gave all of its HBM to a framework's caching
allocator may find a late cudaMalloc refused.  For them the library carries its own
fixed scratch array; this test calls that entry point through the C ABI, twice in a
row on different priorities (the second call sees whatever the first left in the
shared array), and requires the same bits as gearb_scan with caller-provided scratch.

The file sorts last on purpose: with `-x` every other test has run before this one.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gear_b200 import _native as N

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _p(t):
    return C.c_void_p(t.data_ptr())


def _scan_both(prio_np):
    n = len(prio_np)
    nparts = (n + N.PART - 1) // N.PART
    prio = torch.from_numpy(prio_np).to(DEV)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    # existing entry point: caller-provided scratch
    cdf_a = torch.empty(n, dtype=torch.float32, device=DEV)
    l1_a = torch.empty(nparts + 1, dtype=torch.float64, device=DEV)
    st_a = torch.zeros(N.STATUS_WORDS, dtype=torch.int32, device=DEV)
    sb = N.lib.gearb_scan_scratch_bytes(n)
    scratch = torch.empty(sb, dtype=torch.uint8, device=DEV)
    N.check(N.lib.gearb_scan(_p(prio), n, _p(cdf_a), _p(l1_a), _p(scratch), sb, _p(st_a), stream))

    # the entry point under test: no scratch argument at all
    cdf_b = torch.full((n,), -1.0, dtype=torch.float32, device=DEV)
    l1_b = torch.full((nparts + 1,), -1.0, dtype=torch.float64, device=DEV)
    st_b = torch.zeros(N.STATUS_WORDS, dtype=torch.int32, device=DEV)
    N.check(N.lib.gearb_scan_static(_p(prio), n, _p(cdf_b), _p(l1_b), _p(st_b), stream))
    torch.cuda.synchronize()
    return (cdf_a.cpu().numpy(), l1_a.cpu().numpy(), st_a.cpu().tolist(),
            cdf_b.cpu().numpy(), l1_b.cpu().numpy(), st_b.cpu().tolist())


def test_static_scratch_scan_matches_scan_twice_in_a_row():
    rng = np.random.default_rng(20)
    # two calls back to back, different sizes and contents, the second smaller than the first
    for n in (5 * 4096 * 16 + 777, 3 * 4096 + 5):
        prio = rng.lognormal(0.0, 1.0, n).astype(np.float32)
        cdf_a, l1_a, st_a, cdf_b, l1_b, st_b = _scan_both(prio)
        assert np.array_equal(cdf_a, cdf_b)          # bit-exact: float32 table
        assert np.array_equal(l1_a, l1_b)            # bit-exact: float64 offsets
        assert st_a[0] == 0 and st_b[0] == 0
    # and once more with the first size, to see the array re-armed after a smaller call
    prio = rng.lognormal(0.0, 1.0, 5 * 4096 * 16 + 777).astype(np.float32)
    cdf_a, l1_a, _, cdf_b, l1_b, _ = _scan_both(prio)
    assert np.array_equal(cdf_a, cdf_b) and np.array_equal(l1_a, l1_b)


def test_static_scratch_scan_with_its_own_level1_launch_and_without_a_table():
    # Above 1024 partitions level 1 is a launch of its own that reads the exponent range of the
    # aggregates out of the built-in array's header; and the table argument may be NULL (offsets
    # and total only).  Both twice in a row, against the entry point with caller-provided scratch.
    rng = np.random.default_rng(21)
    for n in (5_000_000 + 3, 1200 * 4096, 5_000_000 + 3):
        prio = rng.lognormal(0.0, 1.0, n).astype(np.float32)
        cdf_a, l1_a, st_a, cdf_b, l1_b, st_b = _scan_both(prio)
        assert np.array_equal(cdf_a, cdf_b) and np.array_equal(l1_a, l1_b)
        assert st_a[0] == 0 and st_b[0] == 0
        # totals only: no table written, same offsets
        d = torch.from_numpy(prio).to(DEV)
        nparts = (n + N.PART - 1) // N.PART
        for _ in range(2):
            l1_c = torch.full((nparts + 1,), -1.0, dtype=torch.float64, device=DEV)
            st_c = torch.zeros(N.STATUS_WORDS, dtype=torch.int32, device=DEV)
            N.check(N.lib.gearb_scan_static(_p(d), n, None, _p(l1_c), _p(st_c),
                                            C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            N.check(N.lib.gearb_scan_static(_p(d), n, None, _p(l1_c), _p(st_c),
                                            C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            torch.cuda.synchronize()
            assert np.array_equal(l1_c.cpu().numpy(), l1_a) and st_c.cpu().tolist()[0] == 0


def test_static_scratch_scan_refuses_sizes_beyond_its_array():
    limit = N.lib.gearb_scan_static_max_n()
    assert limit == 1 << 28
    one = torch.zeros(4, dtype=torch.float32, device=DEV)   # never dereferenced: the size check comes first
    st = torch.zeros(N.STATUS_WORDS, dtype=torch.int32, device=DEV)
    rc = N.lib.gearb_scan_static(_p(one), limit + 1, _p(one), _p(one), _p(st), C.c_void_p(0))
    assert rc == N.ERR_UNSUPPORTED
    assert "exceed the built-in scratch" in N.last_error()
