"""CPU oracle for the sample + gather path -- TEST INFRASTRUCTURE ONLY.

Two independent restatements live here:

* ``C``: ctypes bindings to ``gear_oracle.c`` (plain C, sequential), used for
  everything up to full-size inputs;
* numpy functions (``np_*``) written separately from the C code, used on small
  inputs to cross-check the C restatement itself.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the shipped package never does.

Reference citations (paths inside bigrl-team/gear) are on each function of
``gear_oracle.c``; the numpy versions cite the same lines.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "libgear_oracle.so"

PART = 4096
TILE = 128
BLOCKS = 8


def build(force: bool = False) -> Path:
    """Compile gear_oracle.c (and the multi-threaded timing driver) with gcc."""
    srcs = [HERE / "gear_oracle.c", HERE / "cpu_baseline.c"]
    srcs = [s for s in srcs if s.exists()]
    if LIB_PATH.exists() and not force:
        if all(LIB_PATH.stat().st_mtime >= s.stat().st_mtime for s in srcs):
            return LIB_PATH
    LIB_PATH.parent.mkdir(exist_ok=True)
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared",
           "-pthread", "-o", str(LIB_PATH)] + [str(s) for s in srcs] + ["-lm"]
    subprocess.check_call(cmd)
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(LIB_PATH))
    return _lib


def _p(a: np.ndarray, ty=C.c_void_p):
    return a.ctypes.data_as(ty)


def _i64(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int64)


# --------------------------------------------------------------------------- #
# Philox4x32-10
# --------------------------------------------------------------------------- #
def philox_u32(seed: int, stream: int, first: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint32)
    lib().gearo_philox_u32(C.c_uint64(seed), C.c_uint64(stream), C.c_uint64(first),
                           C.c_int64(n), _p(out))
    return out


def philox_u01(seed: int, stream: int, first: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float64)
    lib().gearo_philox_u01(C.c_uint64(seed), C.c_uint64(stream), C.c_uint64(first),
                           C.c_int64(n), _p(out))
    return out


def np_philox4x32(seed: int, stream: int, counters: np.ndarray) -> np.ndarray:
    """Vectorised Philox4x32-10 in numpy; returns uint32[len(counters), 4]."""
    ctr = np.asarray(counters, dtype=np.uint64)
    c = [
        (ctr & np.uint64(0xFFFFFFFF)).astype(np.uint64),
        (ctr >> np.uint64(32)).astype(np.uint64),
        np.full(ctr.shape, stream & 0xFFFFFFFF, dtype=np.uint64),
        np.full(ctr.shape, (stream >> 32) & 0xFFFFFFFF, dtype=np.uint64),
    ]
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    m32 = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c[0]
        p1 = np.uint64(0xCD9E8D57) * c[2]
        n0 = ((p1 >> np.uint64(32)) ^ c[1] ^ np.uint64(k0)) & m32
        n1 = p1 & m32
        n2 = ((p0 >> np.uint64(32)) ^ c[3] ^ np.uint64(k1)) & m32
        n3 = p0 & m32
        c = [n0, n1, n2, n3]
        k0 = (k0 + 0x9E3779B9) & 0xFFFFFFFF
        k1 = (k1 + 0xBB67AE85) & 0xFFFFFFFF
    return np.stack(c, axis=-1).astype(np.uint32)


# --------------------------------------------------------------------------- #
# Synthetic data with the distributions of the benchmark configurations.
# Float values come from numpy's libm here; the device fill kernels use CUDA's,
# so host- and device-generated floats are NOT expected to match bit for bit --
# parity tests either upload host data or read the device table back.
# --------------------------------------------------------------------------- #
def synth_u01(seed, stream, n, first=0):
    return philox_u01(seed, stream, first, n)


def synth_normal(seed, stream, n):
    u = philox_u01(seed, stream, 0, 2 * n)
    u1 = 1.0 - u[0::2]  # (0,1]
    u2 = u[1::2]
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def synth_lognormal(seed, stream, n):
    return np.exp(synth_normal(seed, stream, n).astype(np.float64)).astype(np.float32)


def synth_uniform_pm1(seed, stream, n):
    return (philox_u01(seed, stream, 0, n) * 2.0 - 1.0).astype(np.float32)


def synth_randint(seed, stream, n, lo, hi, dtype=np.int32):
    w = philox_u32(seed, stream, 0, n).astype(np.uint64)
    return (lo + (w * np.uint64(hi - lo) >> np.uint64(32))).astype(dtype)


# --------------------------------------------------------------------------- #
# Table layout + gather addressing
# --------------------------------------------------------------------------- #
def table_layout(row_bytes, T):
    """(accu[ncols+1], trajectory_stride) -- src/storage/table.cc:8-25."""
    rb = _i64(row_bytes)
    accu = np.zeros(len(rb) + 1, dtype=np.int64)
    stride = lib().gearo_table_layout(_p(rb), C.c_int(len(rb)), C.c_int64(T), _p(accu))
    return accu, int(stride)


lib_restype_done = False


def _set_restypes():
    global lib_restype_done
    if not lib_restype_done:
        l = lib()
        l.gearo_table_layout.restype = C.c_int64
        l.gearo_sub.restype = C.c_int64
        l.gearo_scan.restype = C.c_int
        lib_restype_done = True


def sub(idx, ts, ln, traj_stride, col_accu, T, row, offset, length, pad_head):
    """(src_off, dst_off, copy_len, slot_bytes) -- src/storage/handler.cc:78-131."""
    _set_restypes()
    idx, ts, ln = _i64(idx), _i64(ts), _i64(ln)
    n = len(idx)
    s = np.zeros(n, np.int64); d = np.zeros(n, np.int64); b = np.zeros(n, np.int64)
    slot = lib().gearo_sub(_p(idx), _p(ts), _p(ln), C.c_int64(n), C.c_int64(traj_stride),
                           C.c_int64(col_accu), C.c_int64(T), C.c_int64(row),
                           C.c_int32(offset), C.c_int64(length), C.c_int(int(pad_head)),
                           _p(s), _p(d), _p(b))
    return s, d, b, int(slot)


def np_sub(idx, ts, ln, traj_stride, col_accu, T, row, offset, length, pad_head):
    """numpy restatement of the same addressing (handler.cc:78-131)."""
    idx, ts, ln = _i64(idx), _i64(ts), _i64(ln)
    start = np.maximum(ts + offset, 0)
    end = np.minimum(start + length, ln)
    nbytes = np.maximum(end * row - start * row, 0)
    slot = length * row
    src = idx * traj_stride + col_accu * T + start * row
    dst = np.arange(len(idx), dtype=np.int64) * slot + (slot - nbytes if pad_head else 0)
    return src, dst, nbytes, slot


def vcopy(src: np.ndarray, dst: np.ndarray, src_off, dst_off, copy_len):
    """Effect of vary_stride_copy_collect -- src/cuda/copy.cu:47-89."""
    assert src.dtype == np.uint8 and dst.dtype == np.uint8
    s, d, b = _i64(src_off), _i64(dst_off), _i64(copy_len)
    lib().gearo_vcopy(_p(src), _p(dst), C.c_int64(len(s)), _p(s), _p(d), _p(b))
    return dst


def fused_subcopy(table: np.ndarray, idx, ts, ln, traj_stride, col_accu, T, row,
                  offset, length, pad_head, dst: np.ndarray | None = None,
                  zero_fill: bool = False) -> np.ndarray:
    """Gather one column into [n, length*row] bytes -- src/cuda/copy.cu:91-134 +
    src/storage/handler.cc:133-154.  dst defaults to zeros (the loader's
    torch.zeros, gear/loader/offline_loader.py:181-189)."""
    assert table.dtype == np.uint8
    idx, ts, ln = _i64(idx), _i64(ts), _i64(ln)
    n = len(idx)
    if dst is None:
        dst = np.zeros(n * length * row, dtype=np.uint8)
    lib().gearo_fused_subcopy(_p(table), _p(dst), _p(idx), _p(ts), _p(ln), C.c_int64(n),
                              C.c_int64(traj_stride), C.c_int64(col_accu), C.c_int64(T),
                              C.c_int64(row), C.c_int32(offset), C.c_int64(length),
                              C.c_int(int(pad_head)), C.c_int(int(zero_fill)))
    return dst


def np_gather(table, idx, ts, ln, traj_stride, col_accu, T, row, offset, length, pad_head):
    """Pure numpy/Python gather (small inputs): sub + byte slices."""
    s, d, b, slot = np_sub(idx, ts, ln, traj_stride, col_accu, T, row, offset, length, pad_head)
    out = np.zeros(len(s) * slot, dtype=np.uint8)
    for i in range(len(s)):
        if b[i] > 0:
            out[d[i]:d[i] + b[i]] = table[s[i]:s[i] + b[i]]
    return out


# --------------------------------------------------------------------------- #
# Two-level cumulative priority table + search
# --------------------------------------------------------------------------- #
def scan(prio: np.ndarray):
    """(cdf float32[n], l1 float64[nparts+1], total, bad_flag)."""
    _set_restypes()
    prio = np.ascontiguousarray(prio, dtype=np.float32)
    n = len(prio)
    nparts = (n + PART - 1) // PART
    cdf = np.empty(n, np.float32)
    l1 = np.zeros(nparts + 1, np.float64)
    total = C.c_double(0.0)
    bad = lib().gearo_scan(_p(prio), C.c_int64(n), _p(cdf), _p(l1), C.byref(total))
    return cdf, l1, total.value, int(bad)


def _hs(v: np.ndarray, axis_len: int) -> np.ndarray:
    """Hillis-Steele inclusive float32 scan along the last axis."""
    d = 1
    while d < axis_len:
        nv = v.copy()
        nv[..., d:] = v[..., :-d] + v[..., d:]
        v = nv
        d <<= 1
    return v


def np_scan(prio: np.ndarray):
    """numpy restatement of the scan tree (one_dim_prefix_sum.cu:40-49,23-28,192-201):
    chunks of 4 in sequence, groups of 4 chunk totals in sequence, Hillis-Steele over the 32
    groups of a block, the 8 blocks of a partition in sequence, then a running maximum."""
    prio = np.asarray(prio, dtype=np.float32)
    n = len(prio)
    nparts = (n + PART - 1) // PART
    x = np.zeros(nparts * PART, np.float32)
    x[:n] = prio
    x = x.reshape(nparts, BLOCKS, 32, 4, 4)               # [P, block, group, chunk, value]
    s = np.empty_like(x)
    s[..., 0] = x[..., 0]
    for j in range(1, 4):
        s[..., j] = s[..., j - 1] + x[..., j]
    T = s[..., 3]                                          # [P,W,32,4] chunk totals
    g = np.empty_like(T)
    g[..., 0] = T[..., 0]
    for i in range(1, 4):
        g[..., i] = g[..., i - 1] + T[..., i]
    I = _hs(g[..., 3].copy(), 32)                          # [P,W,32]
    E = np.zeros_like(I)
    E[..., 1:] = I[..., :-1]
    X = np.zeros((nparts, BLOCKS), np.float32)             # block offsets, added in sequence
    for w in range(1, BLOCKS):
        X[:, w] = X[:, w - 1] + I[:, w - 1, 31]
    b = X[:, :, None] + E                                  # [P,W,32]
    off = np.empty_like(T)
    off[..., 0] = b
    for i in range(1, 4):
        off[..., i] = b + g[..., i - 1]
    o = off[..., None] + s                                 # [P,W,32,4,4]
    o = np.where(s == 0, np.float32(0), o)                 # a chunk's leading zeros take no part in the maximum
    o = o.reshape(nparts, PART).astype(np.float32)
    cdf = np.maximum.accumulate(o, axis=1)
    flat = cdf.reshape(-1)
    agg = X[:, BLOCKS - 1] + I[:, BLOCKS - 1, 31]          # block totals in sequence
    l1 = np.zeros(nparts + 1, np.float64)
    acc = 0.0
    for p in range(nparts):
        acc = acc + float(agg[p])
        l1[p + 1] = acc
    return flat[:n].copy(), l1, float(acc)


def search(cdf, l1, u, scale: bool = False, want_near: bool = False):
    cdf = np.ascontiguousarray(cdf, np.float32)
    l1 = np.ascontiguousarray(l1, np.float64)
    u = np.ascontiguousarray(u, np.float64)
    out = np.empty(len(u), np.int64)
    near = np.zeros(len(u), np.uint8) if want_near else None
    lib().gearo_search(_p(cdf), _p(l1), C.c_int64(len(cdf)), _p(u), C.c_int64(len(u)),
                       C.c_int(int(scale)), _p(out),
                       _p(near) if want_near else None)
    return (out, near) if want_near else out


def np_search(cdf, l1, u, scale=False):
    """searchsorted(right) at both levels -- numpy restatement."""
    cdf = np.asarray(cdf, np.float32); l1 = np.asarray(l1, np.float64)
    n = len(cdf); nparts = len(l1) - 1
    total = l1[nparts]
    v = np.asarray(u, np.float64).copy()
    if scale:
        v = v * total
    v = np.where(v >= 0.0, v, 0.0)
    v = np.where(v < total, v, np.nextafter(total, 0.0))
    p = np.searchsorted(l1[1:], v, side="right")
    p = np.minimum(p, nparts - 1)
    out = np.empty(len(v), np.int64)
    for i in range(len(v)):
        base = int(p[i]) * PART
        valid = min(PART, n - base)
        r = np.float32(v[i] - l1[p[i]])
        last = cdf[base + valid - 1]
        if not (r < last):
            r = np.nextafter(last, np.float32(0.0))
        j = int(np.searchsorted(cdf[base:base + valid], r, side="right"))
        out[i] = base + min(j, valid - 1)
    return out


def uniform(u01, n):
    u01 = np.ascontiguousarray(u01, np.float64)
    out = np.empty(len(u01), np.int64)
    lib().gearo_uniform(_p(u01), C.c_int64(len(u01)), C.c_int64(n), _p(out))
    return out


def decode(flat, T, lengths=None, index_offset=0):
    flat = _i64(flat)
    b = len(flat)
    idx = np.empty(b, np.int64); ts = np.empty(b, np.int64); ln = np.empty(b, np.int64)
    lp = _p(_i64(lengths)) if lengths is not None else None
    lib().gearo_decode(_p(flat), C.c_int64(b), C.c_int64(T), lp, C.c_int64(index_offset),
                       _p(idx), _p(ts), _p(ln))
    return idx, ts, ln


def search_f64(prio, u, scale_total: float = 0.0):
    """Flip-counting reference: float64 running sum + searchsorted(right)."""
    prio = np.ascontiguousarray(prio, np.float32)
    u = np.ascontiguousarray(u, np.float64)
    out = np.empty(len(u), np.int64)
    scratch = np.empty(len(prio), np.float64)
    lib().gearo_search_f64(_p(prio), C.c_int64(len(prio)), _p(u), C.c_int64(len(u)),
                           C.c_double(scale_total), _p(out), _p(scratch))
    return out


def owner(gidx, cap_per_rank):
    g = _i64(gidx)
    o = np.empty(len(g), np.int32); l = np.empty(len(g), np.int64)
    lib().gearo_owner(_p(g), C.c_int64(len(g)), C.c_int64(cap_per_rank), _p(o), _p(l))
    return o, l


def comm_order(rank, world):
    o = np.empty(world, np.int32)
    lib().gearo_comm_order(C.c_int(rank), C.c_int(world), _p(o))
    return o


# --------------------------------------------------------------------------- #
# Threaded drivers (timing of the CPU path) and the reference's compiled code
# --------------------------------------------------------------------------- #
def scan_mt(prio: np.ndarray, threads: int, cdf: np.ndarray | None = None):
    """gearo_scan with partitions striped over host threads; same result."""
    prio = np.ascontiguousarray(prio, dtype=np.float32)
    n = len(prio)
    nparts = (n + PART - 1) // PART
    if cdf is None:
        cdf = np.empty(n, np.float32)
    l1 = np.zeros(nparts + 1, np.float64)
    total = C.c_double(0.0)
    f = lib().gearo_scan_mt
    f.restype = C.c_int
    bad = f(_p(prio), C.c_int64(n), _p(cdf), _p(l1), C.byref(total), C.c_int(int(threads)))
    return cdf, l1, total.value, int(bad)


def gather_mt(table: np.ndarray, dsts, idx, ts, ln, traj_stride, T, col_accu, rows, offsets, lengths,
              pad_heads, threads: int):
    """All columns of a batch with zero-filled padding, requests striped over threads."""
    idx, ts, ln = _i64(idx), _i64(ts), _i64(ln)
    nc = len(rows)
    dptr = (C.c_void_p * nc)(*[d.ctypes.data for d in dsts])
    ca, rw, pl = _i64(col_accu), _i64(rows), _i64(lengths)
    po = np.ascontiguousarray(offsets, np.int32); ph = np.ascontiguousarray(pad_heads, np.int32)
    lib().gearo_gather_mt(_p(table), dptr, _p(idx), _p(ts), _p(ln), C.c_int64(len(idx)),
                          C.c_int64(traj_stride), C.c_int64(T), C.c_int(nc), _p(ca), _p(rw), _p(po), _p(pl),
                          _p(ph), C.c_int(int(threads)))


def plain_cumsum_search(prio: np.ndarray, u: np.ndarray, threads: int, scale: bool = True,
                        cum: np.ndarray | None = None):
    """The plain CPU draw, for timing: flat float64 running sum over host threads, then one
    upper_bound per variate.  Returns (indices, total)."""
    prio = np.ascontiguousarray(prio, dtype=np.float32)
    u = np.ascontiguousarray(u, dtype=np.float64)
    n = len(prio)
    if cum is None:
        cum = np.empty(n, np.float64)
    f = lib().gearo_plain_cumsum_mt
    f.restype = C.c_double
    total = f(_p(prio), C.c_int64(n), _p(cum), C.c_int(int(threads)))
    out = np.empty(len(u), np.int64)
    lib().gearo_plain_upper_bound(_p(cum), C.c_int64(n), _p(u), C.c_int64(len(u)), C.c_int(int(bool(scale))), _p(out))
    return out, float(total)


REF_LIB_PATH = HERE / "_ref" / "libgear_ref.so"


class IngestModel:
    """The online index protocol as a plain state machine, for small cases: the trainer's scan
    (src/index/server.cc:115-170), update (172-177, applied per index), callback (179-188) and
    the simulator's acquire / writeback (src/index/client.cc:30-91) over one status record per
    simulator (include/index/sim_status.h:7-17) and a FIFO of free indices
    (include/circular_buffer.h).  Single-threaded: a test drives both sides in a fixed order,
    so ownership is a plain field."""

    def __init__(self, num_clients: int, index_offset: int, capacity: int):
        self.m, self.off, self.cap = num_clients, index_offset, capacity
        self.slots = [dict(owner=0, terminated=0, alloc=0, valid=0, tindex=0, timestep=0, weight=0.0)
                      for _ in range(num_clients)]
        self.free = [index_offset + i for i in range(capacity)]
        self.weights = np.zeros(capacity, np.float32)
        self.timesteps = np.zeros(capacity, np.int64)
        self.cl = [dict(fly=False, tindex=0, timestep=0) for _ in range(num_clients)]

    # ---- trainer
    def scan(self):
        infer, upd = [], {}
        for i, q in enumerate(self.slots):
            if q["owner"] != 1:
                continue
            if not q["terminated"]:
                if q["valid"]:
                    infer.append((i, q["tindex"], q["timestep"]))
                continue
            if q["valid"]:
                self.free.append(q["tindex"])
                q["valid"] = 0
                upd[q["tindex"]] = (q["timestep"], np.float32(q["weight"]))
            if q["alloc"]:
                if self.free:
                    q["tindex"] = self.free.pop(0)
                    q.update(alloc=0, terminated=0, timestep=0, weight=0.0, valid=1, owner=0)
                    upd[q["tindex"]] = (0, np.float32(0.0))
            else:
                q["owner"] = 0
        return infer, [(k, v[0], v[1]) for k, v in upd.items()]      # dicts keep first-insertion order

    def update(self, upd):
        for idx, ts, w in upd:
            self.weights[idx - self.off] = w
            self.timesteps[idx - self.off] = ts

    def callback(self, srcs):
        for i in srcs:
            self.slots[i]["owner"] = 0

    # ---- simulator i; each returns False where the real client would have to wait
    def acquire(self, i):
        q, c = self.slots[i], self.cl[i]
        if q["owner"] != 0:
            return False
        if not q["valid"]:
            q.update(terminated=1, alloc=1, owner=1)
            return False
        c.update(fly=True, tindex=q["tindex"], timestep=0)
        return True

    def step(self, i):
        c = self.cl[i]
        c["timestep"] += 1
        return c["timestep"] - 1 if c["fly"] else 0

    def writeback(self, i, terminated, alloc_new, weight):
        q, c = self.slots[i], self.cl[i]
        if not c["fly"]:
            return 0
        q.update(terminated=int(terminated), timestep=c["timestep"], alloc=int(alloc_new), weight=float(weight), owner=1)
        c["fly"] = not terminated
        return c["timestep"]


class Reference:
    """The reference's own TableSpec / TrajectoryTable / CpuTrajectoryStorageHandler, compiled
    unchanged from the reference tree into oracle/_ref/libgear_ref.so (see oracle/Makefile)."""

    @staticmethod
    def available() -> bool:
        return REF_LIB_PATH.exists()

    def __init__(self, row_bytes, T, capacity):
        import torch  # noqa: F401  the library resolves torch / pybind11 symbols from the process
        self._lib = C.CDLL(str(REF_LIB_PATH))
        self._lib.gearref_create.restype = C.c_void_p
        self._lib.gearref_sub.restype = C.c_int64
        self._lib.gearref_time_gather.restype = C.c_double
        rb = _i64(row_bytes)
        self._h = C.c_void_p(self._lib.gearref_create(_p(rb), C.c_int(len(rb)), C.c_int64(T), C.c_int64(capacity)))

    def set(self, column, offset, length, pad):
        self._lib.gearref_set(self._h, C.c_int(column), C.c_int(offset), C.c_int64(length), C.c_int(pad))

    def sub(self, idx, ts, ln, column):
        idx, ts, ln = _i64(idx).copy(), _i64(ts).copy(), _i64(ln).copy()
        n = len(idx)
        s = np.zeros(n, np.int64); d = np.zeros(n, np.int64); b = np.zeros(n, np.int64)
        slot = self._lib.gearref_sub(self._h, _p(idx), _p(ts), _p(ln), C.c_int64(n), C.c_int(column),
                                     _p(s), _p(d), _p(b))
        return s, d, b, int(slot)

    def time_gather(self, table: np.ndarray, idx, ts, ln, columns, dsts, threads: int, iters: int) -> float:
        """Seconds for `iters` batches of reference sub() + one memcpy per request."""
        idx, ts, ln = _i64(idx).copy(), _i64(ts).copy(), _i64(ln).copy()
        cols = np.ascontiguousarray(columns, np.int32)
        dptr = (C.c_void_p * len(dsts))(*[d.ctypes.data for d in dsts])
        return float(self._lib.gearref_time_gather(self._h, _p(table), _p(idx), _p(ts), _p(ln),
                                                   C.c_int64(len(idx)), _p(cols), C.c_int(len(cols)), dptr,
                                                   C.c_int(int(threads)), C.c_int(int(iters))))

    def close(self):
        if self._h:
            self._lib.gearref_destroy(self._h)
            self._h = None
