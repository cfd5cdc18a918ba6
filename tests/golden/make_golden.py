"""Generate tests/golden/*.npz from the REFERENCE's own compiled code.

Run in a container that has the reference tree:
    make -C oracle ref && python tests/golden/make_golden.py

sub_golden.npz: outputs of CpuTrajectoryStorageHandler::sub
(src/storage/handler.cc:78-131 of bigrl-team/gear, compiled unchanged into
oracle/_ref/libgear_ref.so) for seeded random requests over several table
shapes and subscribe patterns, including clipping at both ends, empty
segments and every pad option.  The CPU oracle and the C ABI's host-side `sub`
are both checked against this file, so the check also runs where the reference
tree is absent.
"""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import torch  # noqa: F401  (libgear_ref.so resolves torch/pybind symbols from the process)

ROOT = Path(__file__).resolve().parents[2]
OUT = Path(__file__).resolve().parent / "sub_golden.npz"

CASES = [
    # (row_bytes, T, capacity, [(column, offset, length, pad)])
    ([68, 24, 4, 1], 1000, 4096, [(0, 0, 20, 2), (1, 0, 20, 2), (2, 0, 20, 2), (3, 0, 20, 2)]),
    ([156, 24, 4, 4, 1], 1000, 100000, [(0, 0, 64, 2), (1, -3, 64, 1), (4, 5, 64, 0)]),
    ([28224, 4, 4, 1], 1000, 1000, [(0, -31, 32, 1), (1, 0, 32, 2), (3, -1, 2, 1)]),
    ([4096, 4, 4], 1000, 32000, [(0, 0, 16, 2), (2, -15, 16, 1)]),
    ([96], 100, 32, [(0, -1, 100, 1)]),           # the shape of the reference's tests/test_sub.py
    ([3, 7, 13], 17, 11, [(0, -20, 5, 1), (1, 16, 9, 2), (2, 0, 0, 2), (2, -3, 40, 1)]),
]


def main():
    ref = C.CDLL(str(ROOT / "oracle" / "_ref" / "libgear_ref.so"))
    ref.gearref_create.restype = C.c_void_p
    ref.gearref_sub.restype = C.c_int64
    rng = np.random.default_rng(20240607)
    out = {}
    k = 0
    for row_bytes, T, cap, pats in CASES:
        rb = np.asarray(row_bytes, np.int64)
        h = C.c_void_p(ref.gearref_create(rb.ctypes.data_as(C.c_void_p), len(rb), C.c_int64(T), C.c_int64(cap)))
        for (col, off, length, pad) in pats:
            ref.gearref_set(h, col, off, C.c_int64(length), pad)
            n = 64
            idx = rng.integers(0, cap, n).astype(np.int64)
            ts = rng.integers(0, T, n).astype(np.int64)
            ln = rng.integers(0, T + 1, n).astype(np.int64)
            ts[:4] = [0, T - 1, 0, T - 1]
            ln[:4] = [T, T, 0, 1]
            s = np.zeros(n, np.int64); d = np.zeros(n, np.int64); b = np.zeros(n, np.int64)
            p = lambda a: a.ctypes.data_as(C.c_void_p)
            slot = ref.gearref_sub(h, p(idx), p(ts), p(ln), C.c_int64(n), col, p(s), p(d), p(b))
            out[f"case{k}_meta"] = np.asarray([T, cap, col, off, length, pad, slot], np.int64)
            out[f"case{k}_rows"] = rb
            out[f"case{k}_req"] = np.stack([idx, ts, ln])
            out[f"case{k}_out"] = np.stack([s, d, b])
            k += 1
        ref.gearref_destroy(h)
    out["ncases"] = np.asarray([k], np.int64)
    np.savez_compressed(OUT, **out)
    print(f"wrote {OUT} with {k} cases")


if __name__ == "__main__":
    sys.exit(main())
