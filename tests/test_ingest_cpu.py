"""Online ingestion (host side): the shared-memory index server / client against the plain
state machine in the oracle, across processes, with waits that run out, and through the
libgear-named mirrors."""
import multiprocessing as mp
import os
import pickle
import time

import numpy as np
import pytest

from gear_b200 import _native as N
from gear_b200._native import GearError
from gear_b200.ingest import IndexClient, IndexServer
from oracle import oracle as O


def _key(salt: int) -> int:
    return 0x47000000 + (os.getpid() % 50000) * 16 + salt


def _slot_tuple(st):
    return (st["ownership"], st["terminated"], st["alloc"], st["valid"])


@pytest.mark.parametrize("m,cap,off,seed", [(3, 8, 0, 1), (5, 4, 100, 2), (8, 64, 7, 3), (2, 1, 0, 4)])
def test_protocol_matches_state_machine(m, cap, off, seed):
    """A seeded schedule of simulator and trainer actions, both sides in one process: after every
    action the server's report, its arrays and each slot equal the model's."""
    rng = np.random.default_rng(seed)
    srv = IndexServer(_key(1), m, off, cap)
    cls = [IndexClient(_key(1), i, m) for i in range(m)]
    assert all(c.connect() == 0 for c in cls)
    model = O.IngestModel(m, off, cap)
    pending = []                                     # inference requests not yet called back
    for it in range(600):
        a = rng.integers(0, 10)
        i = int(rng.integers(0, m))
        if a < 3:
            try:
                got = cls[i].acquire(0)
                assert model.acquire(i) and got == model.cl[i]["tindex"]
            except GearError as e:
                assert e.code == N.ERR_TIMEOUT and not model.acquire(i)
        elif a < 5:
            if model.cl[i]["fly"] and model.slots[i]["owner"] == 0:
                assert cls[i].step_inc() == model.step(i)
        elif a < 7:
            if model.cl[i]["fly"] and model.slots[i]["owner"] == 0:
                term, alloc, w = bool(rng.integers(0, 2)), bool(rng.integers(0, 2)), float(rng.random() + 0.1)
                assert cls[i].writeback(term, alloc, w) == model.writeback(i, term, alloc, w)
        elif a < 9:
            ni, nu = srv.scan()
            infer, upd = model.scan()
            assert [(int(srv.infer_src[k]), int(srv.infer_idx[k]), int(srv.infer_ts[k])) for k in range(ni)] == infer
            got = [(int(srv.upd_idx[k]), int(srv.upd_ts[k]), np.float32(srv.upd_w[k])) for k in range(nu)]
            assert got == upd
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
        for j in range(m):
            q = model.slots[j]
            assert _slot_tuple(cls[j].status()) == (q["owner"], q["terminated"], q["alloc"], q["valid"]), (it, j)
    for c in cls:
        c.close()
    srv.close()


def test_client_before_server_and_wait_runs_out():
    c = IndexClient(_key(2), 0, 2)
    assert c.connect() == -1                          # no segment yet: the caller retries
    srv = IndexServer(_key(2), 2, 0, 4)
    assert c.connect() == 0
    t0 = time.perf_counter()
    with pytest.raises(GearError) as e:               # nobody scans: the request for a trajectory stays unanswered
        c.acquire(50)
    assert e.value.code == N.ERR_TIMEOUT and 0.04 < time.perf_counter() - t0 < 2.0
    assert _slot_tuple(c.status()) == (1, 1, 1, 0)
    srv.scan()
    assert c.acquire(50) == 0                         # FIFO order: the first free index
    c.release()
    with pytest.raises(GearError):
        c.wait(20)
    c.close()
    srv.close()
    assert IndexClient(_key(2), 0, 2).connect() == -1  # the segment went with its creator


def test_bad_arguments():
    with pytest.raises(GearError):
        IndexServer(0, 1, 0, 4)
    with pytest.raises(GearError):
        IndexServer(_key(3), 0, 0, 4)
    srv = IndexServer(_key(3), 2, 10, 4)
    with pytest.raises(GearError):
        IndexClient(_key(3), 2, 2).connect()
    srv.upd_idx[0], srv.upd_ts[0], srv.upd_w[0] = 9, 1, 1.0
    with pytest.raises(GearError):
        srv.update(1)                                 # index below this shard's offset
    with pytest.raises(GearError):
        srv.callback(np.array([2], np.int32))
    with pytest.raises(GearError):
        srv.set_state(b"\0" * 48)
    srv.close()


def test_state_round_trip():
    srv = IndexServer(_key(4), 3, 5, 6)
    cls = [IndexClient(_key(4), i, 3) for i in range(3)]
    for c in cls:
        c.connect()
    for c in cls:
        with pytest.raises(GearError):
            c.acquire(0)
    srv.update(srv.scan()[1])
    assert [c.acquire(0) for c in cls] == [5, 6, 7]
    cls[1].step_inc(); cls[1].step_inc()
    cls[1].writeback(True, False, 2.5)
    srv.update(srv.scan()[1])
    state = srv.get_state()
    w, ts, free = srv.weights.copy(), srv.timesteps.copy(), srv.free_count
    assert w[1] == 2.5 and ts[1] == 2 and free == 4
    for c in cls:
        c.close()
    srv.close()
    again = IndexServer(_key(4), 3, 0, 6)             # the offset comes back with the state
    again.set_state(state)
    assert again.index_offset == 5
    np.testing.assert_array_equal(again.weights, w)
    np.testing.assert_array_equal(again.timesteps, ts)
    assert again.free_count == free
    c = IndexClient(_key(4), 1, 3)
    c.connect()
    with pytest.raises(GearError):
        c.acquire(0)
    again.scan()
    assert c.acquire(0) == 8                          # FIFO order survives: 8, 9, 10, then the recycled 6
    with pytest.raises(GearError):
        IndexServer(_key(5), 3, 5, 7).set_state(state)   # another shape is refused
    c.close()
    again.close()


def _simulator(key, rank, m, episodes, seed, q):
    rng = np.random.default_rng(seed)
    c = IndexClient(key, rank, m)
    deadline = time.time() + 20
    while c.connect() != 0:
        assert time.time() < deadline
        time.sleep(0.005)
    done = []
    for e in range(episodes):
        idx = c.acquire(20_000)
        steps = int(rng.integers(1, 12))
        for t in range(steps):
            assert c.step_inc() == t
            last = t == steps - 1
            if not last:
                c.writeback(False, False)             # an inference request; wait for the answer
                c.wait(20_000)
        w = float(np.float32(rng.random() + 0.5))
        assert c.writeback(True, e + 1 < episodes, w) == steps
        done.append((idx, steps, w))
    c.wait(20_000)                                    # the trainer has taken the last commit
    q.put((rank, done))
    c.close()


def test_simulators_in_other_processes():
    m, cap, episodes = 4, 6, 25
    key = _key(6)
    srv = IndexServer(key, m, 1000, cap)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_simulator, args=(key, r, m, episodes, 10 + r, q)) for r in range(m)]
    for p in procs:
        p.start()
    held, results, served = {}, {}, 0
    latest = {}                                       # index -> (steps, weight) of its latest commit, as the server saw it
    deadline = time.time() + 120
    while len(results) < m and time.time() < deadline:
        ni, nu = srv.scan()
        for k in range(nu):
            idx, ts, w = int(srv.upd_idx[k]), int(srv.upd_ts[k]), float(srv.upd_w[k])
            assert 1000 <= idx < 1000 + cap
            latest[idx] = (ts, w)
        srv.update(nu)
        srcs = srv.infer_src[:ni].copy()
        for k in range(ni):                           # no two simulators ever hold one trajectory
            held[int(srcs[k])] = int(srv.infer_idx[k])
        assert len(set(held.values())) == len(held)
        served += ni
        srv.callback(srcs)
        while not q.empty():
            r, done = q.get()
            results[r] = done
            held.pop(r, None)
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    assert len(results) == m
    total_steps = sum(s - 1 for d in results.values() for _, s, _ in d)
    assert served == total_steps                      # every non-final step was one inference request
    assert srv.free_count == cap                      # everything came back to the FIFO
    # the arrays hold, per index, the latest commit the server saw, and that commit is one a simulator made
    commits = {(i, s, np.float32(w)) for d in results.values() for i, s, w in d}
    for idx, (ts, w) in latest.items():
        assert srv.timesteps[idx - 1000] == ts and srv.weights[idx - 1000] == np.float32(w)
        assert (idx, ts, np.float32(w)) in commits
    srv.close()


def test_libgear_names():
    import gear_b200.dropin as dropin
    dropin.install()
    import libgear.core as glibc
    import torch

    srv = glibc.SharedMemoryIndexServer(_key(7), 2, 0, 4)
    cl = glibc.SharedMemoryIndexClient(_key(7), 1, 2)
    assert srv.connect() == 0 and cl.connect() == 0
    assert srv.get_capacity() == 4 and srv.get_num_clients() == 2 and cl.get_num_clients() == 2
    cl.timeout_ms = 0
    with pytest.raises(GearError):
        cl.acquire()
    cache = glibc.CachedRequest(4)
    srv.scan(cache)
    assert cache.warr.count == 1 and cache.iarr.count == 0
    srv.update(cache)
    cl.acquire()
    assert cl.get_index() == 0 and cl.get_timestep() == 0
    assert cl.step_inc() == 0
    cl.writeback(False, False)
    srv.scan(cache)
    assert cache.iarr.count == 1 and (cache.iarr.srcs[0], cache.iarr.idxs[0], cache.iarr.tss[0]) == (1, 0, 1)
    srv.callback(cache)
    cl.wait()
    assert cl.step_inc() == 1
    assert cl.writeback(True, False, 3.0) == 2
    srv.scan(cache)
    srv.update(cache)
    idxs, weights = torch.zeros(8, dtype=torch.int64), torch.zeros(4)
    assert cache.warr.continuous(idxs, weights) == 1   # index 0 once, with its latest values
    assert idxs[0] == 0 and idxs[4] == 2 and weights[0] == 3.0 and cache.warr.count == 0
    assert srv.get_weights()[0] == 3.0 and srv.get_timesteps()[0] == 2
    blob = pickle.dumps(srv)
    del srv
    back = pickle.loads(blob)
    assert back.get_weights()[0] == 3.0 and back.get_timesteps()[0] == 2


def test_ingestion_code_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """The host code of the ingestion path built on its own with -fsanitize=address,undefined and
    driven through the protocol, its error paths and the state image in a child process."""
    import shutil
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    gxx = shutil.which("g++")
    asan = subprocess.run([gxx, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    cuda_inc = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
    if not gxx or not Path(asan).is_file() or not (cuda_inc / "cuda_runtime.h").is_file():
        pytest.skip("g++ with libasan and the CUDA headers are needed")
    so = tmp_path / "libingest_san.so"
    build = subprocess.run(
        [gxx, "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
         "-fno-sanitize-recover=undefined", "-shared", "-fPIC", "-I", str(root / "include"), "-I", str(root / "gear_b200" / "csrc"),
         "-I", str(cuda_inc), str(root / "gear_b200" / "csrc" / "ingest.cc"), str(root / "tests" / "sanitize" / "host_stub.cc"),
         "-o", str(so), "-lpthread"], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-2000:]
    env = dict(os.environ, LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=23")
    run = subprocess.run([sys.executable, str(root / "tests" / "sanitize" / "drive_ingest.py"), str(so)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert run.returncode == 0 and "sanitized run ok" in run.stdout, (run.stdout[-500:], run.stderr[-3000:])
