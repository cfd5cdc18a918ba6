"""Drives the sanitizer build of the ingestion code (argv[1]) through the protocol, its error
paths and the state image.  Run by tests/test_ingest_cpu.py with libasan preloaded; any report
of the sanitizers ends the process with a non-zero code."""
import ctypes as C
import os
import sys

import numpy as np

lib = C.CDLL(sys.argv[1])
vp, i64 = C.c_void_p, C.c_int64
lib.gearb_ingest_server_create.argtypes = [C.c_int, C.c_int, i64, i64, C.POINTER(vp)]
lib.gearb_ingest_server_scan.argtypes = [vp, vp, vp, vp, i64, C.POINTER(i64), vp, vp, vp, i64, C.POINTER(i64)]
lib.gearb_ingest_server_update.argtypes = [vp, vp, vp, vp, i64]
lib.gearb_ingest_server_callback.argtypes = [vp, vp, i64]
lib.gearb_ingest_server_get_state.argtypes = [vp, vp, i64]
lib.gearb_ingest_server_get_state.restype = i64
lib.gearb_ingest_server_set_state.argtypes = [vp, vp, i64]
lib.gearb_ingest_server_free_count.argtypes = [vp]
lib.gearb_ingest_server_free_count.restype = i64
lib.gearb_ingest_server_destroy.argtypes = [vp]
lib.gearb_ingest_client_create.argtypes = [C.c_int, C.c_int, C.c_int, C.POINTER(vp)]
lib.gearb_ingest_client_acquire.argtypes = [vp, i64, C.POINTER(i64)]
lib.gearb_ingest_client_wait.argtypes = [vp, i64]
lib.gearb_ingest_client_step.argtypes = [vp]
lib.gearb_ingest_client_step.restype = i64
lib.gearb_ingest_client_writeback.argtypes = [vp, C.c_int, C.c_int, C.c_double]
lib.gearb_ingest_client_writeback.restype = i64
lib.gearb_ingest_client_status.argtypes = [vp, vp, C.POINTER(C.c_double)]
lib.gearb_ingest_client_destroy.argtypes = [vp]

key, m, cap = 0x4A000000 + os.getpid() % 100000, 3, 4
srv = vp(0)
assert lib.gearb_ingest_server_create(key, m, 10, cap, C.byref(srv)) == 0
assert lib.gearb_ingest_server_create(0, m, 10, cap, C.byref(vp(0))) != 0          # bad key
cls = []
for r in range(m):
    c = vp(0)
    assert lib.gearb_ingest_client_create(key, r, m, C.byref(c)) == 0
    cls.append(c)
assert lib.gearb_ingest_client_create(key, m, m, C.byref(vp(0))) != 0               # rank out of range
src, idx, ts = np.zeros(m, np.int32), np.zeros(m, np.int64), np.zeros(m, np.int64)
ui, ut, uw = np.zeros(2 * m, np.int64), np.zeros(2 * m, np.int64), np.zeros(2 * m, np.float32)
P = lambda a: a.ctypes.data_as(vp)
ni, nu = i64(0), i64(0)
rng = np.random.default_rng(0)
fly = [False] * m
for it in range(400):
    for r in range(m):
        t = i64(0)
        if not fly[r]:
            fly[r] = lib.gearb_ingest_client_acquire(cls[r], 0, C.byref(t)) == 0
            continue
        st = (i64 * 7)()
        lib.gearb_ingest_client_status(cls[r], st, None)
        if st[0] != 0:
            continue
        lib.gearb_ingest_client_step(cls[r])
        if rng.random() < 0.3:
            lib.gearb_ingest_client_writeback(cls[r], 1, int(rng.random() < 0.7), 1.5)
            fly[r] = False
        else:
            lib.gearb_ingest_client_writeback(cls[r], 0, 0, 0.0)
    assert lib.gearb_ingest_server_scan(srv, P(src), P(idx), P(ts), m, C.byref(ni), P(ui), P(ut), P(uw), 2 * m, C.byref(nu)) == 0
    assert lib.gearb_ingest_server_scan(srv, P(src), P(idx), P(ts), m - 1, C.byref(i64(0)), P(ui), P(ut), P(uw), 2 * m, C.byref(i64(0))) != 0
    assert lib.gearb_ingest_server_update(srv, P(ui), P(ut), P(uw), nu.value) == 0
    assert lib.gearb_ingest_server_callback(srv, P(src), ni.value) == 0
n = lib.gearb_ingest_server_get_state(srv, None, 0)
buf = C.create_string_buffer(n)
assert lib.gearb_ingest_server_get_state(srv, buf, n) == n
assert lib.gearb_ingest_server_get_state(srv, buf, n - 1) == -1
assert lib.gearb_ingest_server_set_state(srv, buf, n) == 0
assert lib.gearb_ingest_server_set_state(srv, buf, n - 8) != 0                       # truncated image
assert lib.gearb_ingest_client_wait(cls[0], 5) >= 0                                  # returns, with or without the slot
bad = np.array([10 + cap], np.int64)
assert lib.gearb_ingest_server_update(srv, P(bad), P(ut), P(uw), 1) != 0             # index outside the shard
for c in cls:
    lib.gearb_ingest_client_destroy(c)
lib.gearb_ingest_server_destroy(srv)
print("sanitized run ok")
