"""Object layer over the C ABI: table, handler, index set, sampler.

torch tensors appear here only as owners of device memory and as the source of
the current CUDA stream; every operation is one call into libgear_b200.so.
Names follow the reference's host classes (TrajectoryTable, SubscribePattern,
CpuTrajectoryStorageHandler, Indexset; src/storage, include/index/set.h).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _native as N
from ._native import GearError, call, lib

__all__ = [
    "GearError", "SubscribePattern", "TrajectoryTable", "StorageHandler", "Indexset",
    "PrioritySampler", "scan", "search", "sample_uniform", "decode", "fill", "vcopy", "copy",
    "init", "device_count", "ipc_export", "ipc_open", "ipc_close", "DeviceBuffer",
]


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)
_HAVE_CUDA = None


def _stream(stream=None) -> C.c_void_p:
    """The cudaStream_t to launch on: the given torch stream (or raw handle), else torch's current
    stream.  On the path of every launch, so the raw accessors are used where torch has them."""
    global _HAVE_CUDA
    if stream is None:
        if _HAVE_CUDA is None:
            _HAVE_CUDA = bool(torch.cuda.is_available())
        if not _HAVE_CUDA:
            return C.c_void_p(0)
        if _RAW_STREAM is not None and _RAW_DEVICE is not None:
            return C.c_void_p(_RAW_STREAM(_RAW_DEVICE()))
        stream = torch.cuda.current_stream()
    return C.c_void_p(stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream))


def _dev_i64(t: torch.Tensor, what: str) -> C.c_void_p:
    if t.dtype != torch.int64 or not t.is_cuda or not t.is_contiguous():
        raise GearError(N.ERR_INVALID, f"{what} must be a contiguous int64 CUDA tensor")
    return C.c_void_p(t.data_ptr())


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


_TYPESTR = {torch.float32: "<f4", torch.float64: "<f8", torch.int32: "<i4", torch.int64: "<i8",
            torch.uint8: "|u1"}


class _DevArray:
    def __init__(self, ptr: int, n: int, dtype: torch.dtype):
        self.__cuda_array_interface__ = {"shape": (int(n),), "typestr": _TYPESTR[dtype],
                                         "data": (int(ptr), False), "version": 2}


def device_view(ptr: int, n: int, dtype: torch.dtype) -> torch.Tensor:
    """Zero-copy tensor over device memory owned by the native library."""
    return torch.as_tensor(_DevArray(ptr, n, dtype), device="cuda")


def init(device: int = 0) -> None:
    """gear::cuda::init (src/cuda/init.cu:6-13)."""
    call("gearb_init", int(device))


def device_count() -> int:
    n = C.c_int(0)
    call("gearb_device_count", C.byref(n))
    return n.value


@dataclass(frozen=True)
class SubscribePattern:
    """SubscribePattern (include/storage/handler.h:17-31): which timesteps of a
    column a request takes, relative to its timestep, and where padding goes."""
    offset: int = 0
    length: int = 1
    pad: int = N.PAD_TAIL


class TrajectoryTable:
    """TrajectoryTable (src/storage/table.cc): layout [trajectory][column][t][elem]."""

    def __init__(self, row_bytes: Sequence[int], trajectory_length: int, capacity: int,
                 residency: int = N.RES_HOST, key: int = 0, create: bool = True):
        self.row_bytes = [int(r) for r in row_bytes]
        self.trajectory_length = int(trajectory_length)
        self.capacity = int(capacity)
        self._h = C.c_void_p(0)
        rb = (C.c_int64 * len(self.row_bytes))(*self.row_bytes)
        call("gearb_table_create", rb, len(self.row_bytes), self.trajectory_length, self.capacity,
             int(residency), int(key), int(bool(create)), C.byref(self._h))
        stride, nbytes = C.c_int64(0), C.c_int64(0)
        accu = (C.c_int64 * (len(self.row_bytes) + 1))()
        call("gearb_table_layout", self._h, C.byref(stride), C.byref(nbytes), accu)
        self.trajectory_stride, self.nbytes, self.accu = stride.value, nbytes.value, list(accu)
        self.connected = False

    def connect(self) -> int:
        n = C.c_int64(0)
        call("gearb_table_connect", self._h, C.byref(n))
        self.connected = True
        return n.value

    @property
    def ncolumns(self) -> int:
        return len(self.row_bytes)

    @property
    def host_ptr(self) -> int:
        return lib.gearb_table_host_ptr(self._h) or 0

    @property
    def device_ptr(self) -> int:
        return lib.gearb_table_device_ptr(self._h) or 0

    def host_view(self) -> np.ndarray:
        """uint8 view of the host image (no copy)."""
        p = self.host_ptr
        if not p:
            raise GearError(N.ERR_STATE, "the table has no host copy")
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(self.nbytes,))

    def upload(self, stream=None) -> None:
        call("gearb_table_upload", self._h, _stream(stream))

    def upload_range(self, offset: int, nbytes: int, stream=None) -> None:
        """Bytes [offset, offset + nbytes) of the host copy into the device copy (after upload())."""
        call("gearb_table_upload_range", self._h, int(offset), int(nbytes), _stream(stream))

    def write(self, offset: int, data: np.ndarray, stream=None, sync: bool = True) -> None:
        """Bytes into every resident copy.  sync=False returns while the upload may still be
        reading `data` (page-locked memory the caller keeps alive and unchanged until it
        synchronises the stream)."""
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        call("gearb_table_write", self._h, int(offset), data.ctypes.data_as(C.c_void_p), data.nbytes,
             _stream(stream))
        if sync and torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()  # `data` may be freed by the caller

    def read_into(self, offset: int, out: np.ndarray) -> None:
        """Bytes [offset, offset + out.nbytes) of the table into `out` (contiguous uint8)."""
        call("gearb_table_read", self._h, int(offset), out.ctypes.data_as(C.c_void_p), int(out.nbytes))


    def read(self, offset: int, nbytes: int) -> np.ndarray:
        out = np.empty(int(nbytes), np.uint8)
        call("gearb_table_read", self._h, int(offset), out.ctypes.data_as(C.c_void_p), int(nbytes))
        return out

    def column_offset(self, column: int) -> int:
        return self.accu[column] * self.trajectory_length

    def close(self) -> None:
        if self._h:
            lib.gearb_table_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class StorageHandler:
    """CpuTrajectoryStorageHandler (src/storage/handler.cc) over either residency."""

    def __init__(self, table: TrajectoryTable, global_capacity: Optional[int] = None,
                 wregion=(0, 0), rregion: Optional[tuple] = None):
        self.table = table  # keeps the table alive: the native handler only borrows it
        gc = table.capacity if global_capacity is None else int(global_capacity)
        rregion = (0, table.capacity) if rregion is None else rregion
        self._h = C.c_void_p(0)
        call("gearb_handler_create", table._h, gc, int(wregion[0]), int(wregion[1]),
             int(rregion[0]), int(rregion[1]), C.byref(self._h))
        self.patterns: dict[int, SubscribePattern] = {}
        self._status: Optional[torch.Tensor] = None

    def set(self, cids: Sequence[int], patterns: Sequence[SubscribePattern]) -> None:
        n = len(cids)
        call("gearb_handler_set", self._h, (C.c_int64 * n)(*[int(c) for c in cids]), n,
             (C.c_int32 * n)(*[int(p.offset) for p in patterns]),
             (C.c_int64 * n)(*[int(p.length) for p in patterns]),
             (C.c_int32 * n)(*[int(p.pad) for p in patterns]))
        for c, p in zip(cids, patterns):
            self.patterns[int(c)] = p

    def sub(self, idx, ts, ln, column: int):
        """(src_off, dst_off, copy_len, slot_bytes) on the host (handler.cc:78-131)."""
        idx = np.ascontiguousarray(idx, np.int64); ts = np.ascontiguousarray(ts, np.int64)
        ln = np.ascontiguousarray(ln, np.int64)
        if not (len(idx) == len(ts) == len(ln)):
            raise GearError(N.ERR_INVALID, "Spans describing target properties have inconsistent size")
        n = len(idx)
        s = np.zeros(n, np.int64); d = np.zeros(n, np.int64); b = np.zeros(n, np.int64)
        slot = C.c_int64(0)
        vp = lambda a: a.ctypes.data_as(C.c_void_p)
        call("gearb_handler_sub", self._h, vp(idx), vp(ts), vp(ln), n, int(column), vp(s), vp(d), vp(b),
             C.byref(slot))
        return s, d, b, slot.value

    def status_tensor(self, device) -> torch.Tensor:
        if self._status is None or self._status.device != torch.device(device):
            self._status = torch.zeros(N.STATUS_WORDS, dtype=torch.int32, device=device)
        return self._status

    def subcopy(self, idx: torch.Tensor, ts: torch.Tensor, ln: torch.Tensor, column: int,
                dst: torch.Tensor, stream=None) -> None:
        """handler.subcopy (src/storage/pybind.cc:140-146)."""
        self.gather([column], idx, ts, ln, [dst], zero_fill=False, stream=stream)

    def gather(self, columns: Sequence[int], idx: torch.Tensor, ts: torch.Tensor, ln: torch.Tensor,
               dsts: Sequence[torch.Tensor], zero_fill: bool = True, stream=None) -> None:
        n = idx.numel()
        if not (ts.numel() == n and ln.numel() == n):
            raise GearError(N.ERR_INVALID, "idx, ts and len must have the same number of entries")
        if len(dsts) != len(columns):
            raise GearError(N.ERR_INVALID, "one destination per column is required")
        for c, d in zip(columns, dsts):
            p = self.patterns.get(int(c))
            if p is not None:
                need = n * p.length * self.table.row_bytes[int(c)]
                if not d.is_cuda or not d.is_contiguous() or d.numel() * d.element_size() < need:
                    raise GearError(N.ERR_INVALID,
                                    f"destination of column {c} must be a contiguous CUDA tensor of >= {need} bytes")
        if n == 0 or not columns:
            return
        nc = len(columns)
        st = self.status_tensor(idx.device)
        call("gearb_handler_gather", self._h, (C.c_int32 * nc)(*[int(c) for c in columns]), nc,
             _dev_i64(idx, "idx"), _dev_i64(ts, "ts"), _dev_i64(ln, "len"), n,
             (C.c_void_p * nc)(*[d.data_ptr() for d in dsts]), int(bool(zero_fill)), _ptr(st),
             _stream(stream))

    def view(self, index: int, column: int) -> np.ndarray:
        """Host bytes of one column of one trajectory (handler.cc:223-233)."""
        p, b = C.c_void_p(0), C.c_int64(0)
        call("gearb_handler_view", self._h, int(index), int(column), C.byref(p), C.byref(b))
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(b.value,))

    def status(self) -> int:
        return 0 if self._status is None else int(self._status[0].item())

    def close(self) -> None:
        if self._h:
            lib.gearb_handler_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Indexset:
    """Indexset (include/index/set.h:191-251): float32 weights + int64 timesteps."""

    def __init__(self, global_capacity: int, local_capacity: int, index_offset: int,
                 shared: bool = False, key: int = 0, create: bool = False):
        self.global_capacity, self.local_capacity = int(global_capacity), int(local_capacity)
        self.index_offset, self.is_sharing, self.shm_key = int(index_offset), bool(shared), int(key)
        self._h = C.c_void_p(0)
        call("gearb_indexset_create", self.global_capacity, self.local_capacity, self.index_offset,
             int(bool(shared)), int(key), int(bool(create)), C.byref(self._h))
        tp = lib.gearb_indexset_timesteps(self._h)
        wp = lib.gearb_indexset_weights(self._h)
        self.timesteps_np = np.ctypeslib.as_array(C.cast(tp, C.POINTER(C.c_int64)), shape=(self.local_capacity,))
        self.weights_np = np.ctypeslib.as_array(C.cast(wp, C.POINTER(C.c_float)), shape=(self.local_capacity,))

    @property
    def timesteps(self) -> torch.Tensor:
        return torch.from_numpy(self.timesteps_np)

    @property
    def weights(self) -> torch.Tensor:
        return torch.from_numpy(self.weights_np)

    def close(self) -> None:
        if self._h:
            self.timesteps_np = self.weights_np = None
            lib.gearb_indexset_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# --------------------------------------------------------------------------- #
# sampling
# --------------------------------------------------------------------------- #
def _nparts(n: int) -> int:
    return (n + N.PART - 1) // N.PART


def scan(priorities: torch.Tensor, stream=None):
    """Functional scan: returns (cdf f32[n], l1 f64[nparts+1], status i32[4])."""
    if priorities.dtype != torch.float32 or not priorities.is_cuda or not priorities.is_contiguous():
        raise GearError(N.ERR_INVALID, "priorities must be a contiguous float32 CUDA tensor")
    n = priorities.numel()
    dev = priorities.device
    cdf = torch.empty(n, dtype=torch.float32, device=dev)
    l1 = torch.empty(_nparts(max(n, 1)) + 1, dtype=torch.float64, device=dev)
    sb = lib.gearb_scan_scratch_bytes(max(n, 1))
    scratch = torch.empty(sb, dtype=torch.uint8, device=dev)
    status = torch.zeros(N.STATUS_WORDS, dtype=torch.int32, device=dev)
    call("gearb_scan", _ptr(priorities), n, _ptr(cdf), _ptr(l1), _ptr(scratch), sb, _ptr(status),
         _stream(stream))
    return cdf, l1, status


def search(cdf: torch.Tensor, l1: torch.Tensor, variates: torch.Tensor, scale: bool = False,
           status: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    if variates.dtype != torch.float64 or not variates.is_cuda or not variates.is_contiguous():
        raise GearError(N.ERR_INVALID, "variates must be a contiguous float64 CUDA tensor")
    out = torch.empty(variates.numel(), dtype=torch.int64, device=variates.device)
    call("gearb_search", _ptr(cdf), _ptr(l1), cdf.numel(), _ptr(variates), variates.numel(),
         N.SEARCH_SCALE if scale else 0, _ptr(out), _ptr(status), _stream(stream))
    return out


def sample_uniform(n: int, u01: torch.Tensor, stream=None) -> torch.Tensor:
    if u01.dtype != torch.float64 or not u01.is_cuda or not u01.is_contiguous():
        raise GearError(N.ERR_INVALID, "variates must be a contiguous float64 CUDA tensor")
    out = torch.empty(u01.numel(), dtype=torch.int64, device=u01.device)
    call("gearb_sample_uniform", int(n), _ptr(u01), u01.numel(), _ptr(out), _stream(stream))
    return out


def decode(flat: torch.Tensor, trajectory_length: int, lengths: Optional[torch.Tensor] = None,
           index_offset: int = 0, stream=None):
    b = flat.numel()
    idx = torch.empty(b, dtype=torch.int64, device=flat.device)
    ts = torch.empty_like(idx); ln = torch.empty_like(idx)
    call("gearb_decode", _dev_i64(flat, "flat"), b, int(trajectory_length), _ptr(lengths),
         int(index_offset), _ptr(idx), _ptr(ts), _ptr(ln), _stream(stream))
    return idx, ts, ln


class PrioritySampler:
    """Owns the cumulative table of n priorities on the current device."""

    def __init__(self, n: int):
        self.n = int(n)
        self._h = C.c_void_p(0)
        call("gearb_sampler_create", self.n, C.byref(self._h))
        c, l, s = C.c_void_p(0), C.c_void_p(0), C.c_void_p(0)
        call("gearb_sampler_buffers", self._h, C.byref(c), C.byref(l), C.byref(s))
        self.cdf_ptr, self.status_ptr = c.value, s.value

    @property
    def l1_ptr(self) -> int:
        """Address of the level-1 table of the LAST scan.  A sampler keeps two and a scan writes
        the one the previous scan did not (see select_slot), so ask again after every scan."""
        l = C.c_void_p(0)
        call("gearb_sampler_buffers", self._h, None, C.byref(l), None)
        return l.value

    def level1_buffers(self):
        """(address of level 1 in slot 0, in slot 1)."""
        a, b = C.c_void_p(0), C.c_void_p(0)
        call("gearb_sampler_level1_buffers", self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def scan(self, priorities: torch.Tensor, stream=None, store: bool = True, alternate: bool = False) -> None:
        """Build the two-level table.  store=False keeps only the partition offsets and the total
        (half the memory traffic); sample_gather then rebuilds the partition each request falls
        into from `priorities`, which must stay unchanged (and alive) until then.  search() and
        pull() need store=True.  alternate=True (with store): this is one of two samplers used in
        turn and the launch before this call in the stream reads only the other one's tables, so
        the scan may start while that launch is finishing."""
        if priorities.dtype != torch.float32 or not priorities.is_cuda or priorities.numel() != self.n:
            raise GearError(N.ERR_INVALID, f"priorities must be float32 CUDA with {self.n} entries")
        name = "gearb_sampler_scan_totals" if not store else ("gearb_sampler_scan_alternate" if alternate
                                                             else "gearb_sampler_scan")
        call(name, self._h, _ptr(priorities), _stream(stream))
        self._lazy_source = None if store else priorities      # keeps the array alive

    def scan_partitions(self, priorities: torch.Tensor, store: bool = True, stream=None) -> None:
        """First launch of a scan alone: one aggregate per partition (and, with store, the level-2
        table).  scan_level1() must follow before the table is used."""
        if priorities.dtype != torch.float32 or not priorities.is_cuda or priorities.numel() != self.n:
            raise GearError(N.ERR_INVALID, f"priorities must be float32 CUDA with {self.n} entries")
        call("gearb_sampler_scan_partitions", self._h, _ptr(priorities), int(bool(store)), _stream(stream))
        self._lazy_source = None if store else priorities

    def scan_level1(self, stream=None) -> None:
        """Second launch of a scan alone: the partition offsets from the aggregates."""
        call("gearb_sampler_scan_level1", self._h, _stream(stream))

    def update(self, priorities: torch.Tensor, idx: torch.Tensor, values: torch.Tensor, stream=None) -> None:
        """priorities[idx] = values, then rescan only the touched partitions (after a scan())."""
        if priorities.dtype != torch.float32 or not priorities.is_cuda or priorities.numel() != self.n:
            raise GearError(N.ERR_INVALID, f"priorities must be float32 CUDA with {self.n} entries")
        if values.dtype != torch.float32 or not values.is_cuda or values.numel() != idx.numel():
            raise GearError(N.ERR_INVALID, "values must be a float32 CUDA tensor, one per index")
        call("gearb_sampler_update", self._h, _ptr(priorities), _dev_i64(idx, "idx"), _ptr(values.contiguous()),
             idx.numel(), _stream(stream))

    def search(self, variates: torch.Tensor, scale: bool = False, out: Optional[torch.Tensor] = None,
               stream=None) -> torch.Tensor:
        if variates.dtype != torch.float64 or not variates.is_cuda:
            raise GearError(N.ERR_INVALID, "variates must be a float64 CUDA tensor")
        if out is None:
            out = torch.empty(variates.numel(), dtype=torch.int64, device=variates.device)
        call("gearb_sampler_search", self._h, _ptr(variates), variates.numel(),
             N.SEARCH_SCALE if scale else 0, _ptr(out), _stream(stream))
        return out

    def scan_search(self, priorities: torch.Tensor, variates: torch.Tensor, scale: bool = False,
                    out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """scan(priorities) followed by search(variates), as one launch where the table is small enough."""
        if priorities.dtype != torch.float32 or not priorities.is_cuda or priorities.numel() != self.n:
            raise GearError(N.ERR_INVALID, f"priorities must be float32 CUDA with {self.n} entries")
        if variates.dtype != torch.float64 or not variates.is_cuda or not variates.is_contiguous():
            raise GearError(N.ERR_INVALID, "variates must be a contiguous float64 CUDA tensor")
        if out is None:
            out = torch.empty(variates.numel(), dtype=torch.int64, device=variates.device)
        self._lazy_source = None
        call("gearb_sampler_scan_search", self._h, _ptr(priorities), _ptr(variates), variates.numel(),
             N.SEARCH_SCALE if scale else 0, _ptr(out), _stream(stream))
        return out

    def sample_gather(self, handler: "StorageHandler", variates: torch.Tensor, columns: Sequence[int],
                      dsts: Sequence[torch.Tensor], scale: bool = True,
                      lengths: Optional[torch.Tensor] = None, index_offset: int = 0,
                      zero_fill: bool = True, out_flat: Optional[torch.Tensor] = None,
                      out_idx: Optional[torch.Tensor] = None, out_ts: Optional[torch.Tensor] = None,
                      out_len: Optional[torch.Tensor] = None, stream=None,
                      affine: Optional[tuple] = None, flat_offset: int = 0,
                      slot_map: Optional[tuple] = None, dst_requests: Optional[int] = None) -> None:
        """Search every variate, decode it to (trajectory, timestep, length) and gather the
        listed columns of the handler's table, all in one launch.  affine=(mul, sub): the
        variates belong to a global draw over several shards and become u*mul - sub first;
        flat_offset is then added to out_flat, and slot_map=(mod, lo, base) says where the request
        at position q = lo + i of the global batch lands in the destinations: mod > 1: slot
        base[q % mod] + q // mod; mod == -1: slot q - base[0] for base[0] <= q < base[1], else
        base[2] + i (dst_requests: how many slots the destinations must hold, default one per variate)."""
        if variates.dtype != torch.float64 or not variates.is_cuda or not variates.is_contiguous():
            raise GearError(N.ERR_INVALID, "variates must be a contiguous float64 CUDA tensor")
        b = variates.numel()
        if len(dsts) != len(columns):
            raise GearError(N.ERR_INVALID, "one destination per column is required")
        for c, d in zip(columns, dsts):
            p = handler.patterns.get(int(c))
            if p is not None:
                need = (b if dst_requests is None else int(dst_requests)) * p.length * handler.table.row_bytes[int(c)]
                if not d.is_cuda or not d.is_contiguous() or d.numel() * d.element_size() < need:
                    raise GearError(N.ERR_INVALID,
                                    f"destination of column {c} must be a contiguous CUDA tensor of >= {need} bytes")
        for name, t in (("out_flat", out_flat), ("out_idx", out_idx), ("out_ts", out_ts), ("out_len", out_len)):
            if t is not None and (t.dtype != torch.int64 or not t.is_cuda
                                  or t.numel() < (b if dst_requests is None else int(dst_requests))):
                raise GearError(N.ERR_INVALID, f"{name} must be an int64 CUDA tensor with >= {b} entries")
        nc = len(columns)
        if affine is not None:
            mod, lo, base = (0, 0, None) if slot_map is None else slot_map
            base_arr = None if base is None else (C.c_int64 * len(base))(*[int(x) for x in base])
            call("gearb_sampler_sample_gather_affine", self._h, handler._h, _ptr(variates), b, float(affine[0]),
                 float(affine[1]), _ptr(lengths), int(index_offset), (C.c_int32 * nc)(*[int(c) for c in columns]), nc,
                 (C.c_void_p * nc)(*[d.data_ptr() for d in dsts]), int(bool(zero_fill)),
                 _ptr(out_flat), _ptr(out_idx), _ptr(out_ts), _ptr(out_len), int(flat_offset), int(mod), int(lo),
                 base_arr, _stream(stream))
            return
        call("gearb_sampler_sample_gather", self._h, handler._h, _ptr(variates), b,
             N.SEARCH_SCALE if scale else 0, _ptr(lengths), int(index_offset),
             (C.c_int32 * nc)(*[int(c) for c in columns]), nc,
             (C.c_void_p * nc)(*[d.data_ptr() for d in dsts]), int(bool(zero_fill)),
             _ptr(out_flat), _ptr(out_idx), _ptr(out_ts), _ptr(out_len), _stream(stream))

    def pull(self, handler: "StorageHandler", totals: Optional[torch.Tensor], cdfs: Optional[Sequence[int]],
             l1s: Sequence[int], tables: Sequence[int], variates: torch.Tensor, columns: Sequence[int],
             dsts: Sequence[torch.Tensor], zero_fill: bool = True, ring: bool = False,
             out_flat: Optional[torch.Tensor] = None, out_idx: Optional[torch.Tensor] = None,
             out_ts: Optional[torch.Tensor] = None, stream=None, self_shard: int = -1, mailbox: int = 0,
             epoch: int = 0, prios: Optional[Sequence[int]] = None, blks: Optional[Sequence[int]] = None,
             count: Optional[int] = None, variate_stride: int = 1) -> None:
        """This rank's slice of a global batch, read in place from `len(tables)` equal shards.

        totals: float64 CUDA tensor, one total priority per shard.  cdfs / l1s / tables: device
        addresses (ints) of every shard's tables, valid on the current device -- this process's
        own allocations or mappings from ipc_open().  variates are U[0,1) of the global draw.
        self_shard: the shard in this GPU's own memory (its large requests skip the ring).
        mailbox / epoch: instead of `totals`, take them from this rank's mailbox (device address) once
        every rank's publish() of this epoch has arrived there.
        cdfs=None with prios / blks: the shards keep no level-2 table (scan(store=False)); the launch
        rebuilds what each request needs from the owner's priorities and block totals.
        count / variate_stride: request g (of `count`) uses variates[g * variate_stride]."""
        a, _keep = self._marshal_pull(handler, totals, cdfs, l1s, tables, variates, columns, dsts, zero_fill, ring,
                                      out_flat, out_idx, out_ts, self_shard, mailbox, epoch, prios, blks, count,
                                      variate_stride)
        call("gearb_sampler_pull_ex", self._h, handler._h, C.byref(a), _stream(stream))

    def prepare_pull(self, handler: "StorageHandler", totals, cdfs, l1s, tables, variates, columns, dsts,
                     zero_fill: bool = True, ring: bool = False, out_flat=None, out_idx=None, out_ts=None,
                     self_shard: int = -1, mailbox: int = 0, prios=None, blks=None, count=None,
                     variate_stride: int = 1) -> "PreparedPull":
        """pull() with these arguments, checked and marshalled once: run(variates, epoch) of the returned
        object launches it for another batch of variates (same count, stride, tables and destinations).
        For loops in which the host's time per step matters (about 30 us per call otherwise)."""
        a, keep = self._marshal_pull(handler, totals, cdfs, l1s, tables, variates, columns, dsts, zero_fill, ring,
                                     out_flat, out_idx, out_ts, self_shard, mailbox, 0, prios, blks, count,
                                     variate_stride)
        return PreparedPull(self, handler, a, (keep, totals, dsts, out_flat, out_idx, out_ts), count, variate_stride)

    def _marshal_pull(self, handler, totals, cdfs, l1s, tables, variates, columns, dsts, zero_fill, ring, out_flat,
                      out_idx, out_ts, self_shard, mailbox, epoch, prios, blks, count, variate_stride):
        w = len(tables)
        lazy = cdfs is None
        if len(l1s) != w or (not lazy and len(cdfs) != w) or (lazy and (prios is None or len(prios) != w)):
            raise GearError(N.ERR_INVALID, "pull: one level-2 table (or priority array), l1 and table per shard")
        if not mailbox and (totals is None or totals.dtype != torch.float64 or not totals.is_cuda
                            or totals.numel() < w):
            raise GearError(N.ERR_INVALID, "pull: a float64 CUDA total per shard (or a mailbox) is required")
        if variates.dtype != torch.float64 or not variates.is_cuda or not variates.is_contiguous():
            raise GearError(N.ERR_INVALID, "variates must be a contiguous float64 CUDA tensor")
        stride = int(variate_stride)
        b = variates.numel() if count is None else int(count)
        if stride < 1 or (b > 0 and (b - 1) * stride >= variates.numel()):
            raise GearError(N.ERR_INVALID, "pull: count and variate_stride run past the variates")
        if len(dsts) != len(columns):
            raise GearError(N.ERR_INVALID, "one destination per column is required")
        for c, d in zip(columns, dsts):
            p = handler.patterns.get(int(c))
            if p is not None:
                need = b * p.length * handler.table.row_bytes[int(c)]
                if not d.is_cuda or not d.is_contiguous() or d.numel() * d.element_size() < need:
                    raise GearError(N.ERR_INVALID,
                                    f"destination of column {c} must be a contiguous CUDA tensor of >= {need} bytes")
        for name, t in (("out_flat", out_flat), ("out_idx", out_idx), ("out_ts", out_ts)):
            if t is not None and (t.dtype != torch.int64 or not t.is_cuda or t.numel() < b):
                raise GearError(N.ERR_INVALID, f"{name} must be an int64 CUDA tensor with >= {b} entries")
        nc = len(columns)
        arr = lambda v: None if v is None else (C.c_void_p * w)(*[int(x) for x in v])
        a = N.PullArgs()
        a.world, a.self = w, int(self_shard)
        a.totals = None if mailbox else totals.data_ptr()
        a.mailbox, a.epoch = (int(mailbox) or None), int(epoch)
        keep = [arr(cdfs), arr(prios if lazy else None), arr(blks if lazy else None), arr(l1s), arr(tables),
                (C.c_int32 * nc)(*[int(c) for c in columns]), (C.c_void_p * nc)(*[d.data_ptr() for d in dsts])]
        a.cdf = keep[0] if keep[0] is not None else C.POINTER(C.c_void_p)()
        a.prio = keep[1] if keep[1] is not None else C.POINTER(C.c_void_p)()
        a.blk = keep[2] if keep[2] is not None else C.POINTER(C.c_void_p)()
        a.l1, a.table = keep[3], keep[4]
        a.variates, a.b, a.variate_stride = variates.data_ptr(), b, stride
        a.columns, a.ncols, a.dst = keep[5], nc, keep[6]
        a.zero_fill, a.ring = int(bool(zero_fill)), int(bool(ring))
        a.out_flat = None if out_flat is None else out_flat.data_ptr()
        a.out_idx = None if out_idx is None else out_idx.data_ptr()
        a.out_ts = None if out_ts is None else out_ts.data_ptr()
        return a, keep

    def publish(self, world: int, rank: int, mailboxes: Sequence[int], epoch: int, copy_l1: bool = False,
                stream=None) -> None:
        """This shard's total, then `epoch`, into every rank's mailbox (device addresses valid on this
        device: the own one and the peers' as mapped by ipc_open); with copy_l1 the level-1 table goes
        into the other ranks' mailboxes first (they must then be mailbox_bytes(n) large)."""
        arr = (C.c_void_p * int(world))(*[int(x) for x in mailboxes])
        call("gearb_sampler_publish", self._h, int(world), int(rank), arr, C.c_uint64(int(epoch)),
             int(bool(copy_l1)), _stream(stream))

    def scan_publish(self, priorities: torch.Tensor, world: int, rank: int, mailboxes: Sequence[int], epoch: int,
                     stream=None) -> None:
        """scan(priorities, store=False) and publish(..., copy_l1=False) as one call: for tables of more
        than 1024 partitions the launch that builds level 1 also writes the mailboxes."""
        if priorities.dtype != torch.float32 or not priorities.is_cuda or priorities.numel() != self.n:
            raise GearError(N.ERR_INVALID, f"priorities must be float32 CUDA with {self.n} entries")
        key = (int(world), tuple(int(x) for x in mailboxes))
        cached = getattr(self, "_mailbox_arr", None)
        if cached is None or cached[0] != key:            # marshalled once: this call is made every step
            cached = (key, (C.c_void_p * int(world))(*key[1]))
            self._mailbox_arr = cached
        call("gearb_sampler_scan_totals_publish", self._h, _ptr(priorities), int(world), int(rank), cached[1],
             C.c_uint64(int(epoch)), _stream(stream))
        self._lazy_source = priorities

    def publish_total(self, world: int, rank: int, mailboxes: Sequence[int], epoch: int, stream=None) -> None:
        self.publish(world, rank, mailboxes, epoch, False, stream)

    def select_slot(self, slot: int) -> None:
        """Which of the two slots (level 1 and block totals) the NEXT scan writes; ranks of a pull
        agree on epoch & 1.  Pinning the same slot every time gives the tables a fixed address, at
        the price that a scan then never starts before the launch ahead of it has finished."""
        call("gearb_sampler_select_slot", self._h, int(slot))

    def block_totals(self):
        """(address of buffer 0, address of buffer 1, slot written by the last scan)."""
        a, b, cur = C.c_void_p(0), C.c_void_p(0), C.c_int(0)
        call("gearb_sampler_block_totals", self._h, C.byref(a), C.byref(b), C.byref(cur))
        return a.value, b.value, cur.value

    def clear_status(self, stream=None) -> None:
        """Zero the status words (they accumulate across launches)."""
        call("gearb_sampler_clear_status", self._h, _stream(stream))

    def result(self, stream=None):
        """(total, status words) after synchronising the stream.  ST_SCAN_ABORTED in status[0] means a
        bounded wait on the device ran out (the C call returns GEARB_ERR_TIMEOUT then)."""
        total = C.c_double(0.0)
        st = (C.c_int32 * N.STATUS_WORDS)()
        rc = lib.gearb_sampler_result(self._h, _stream(stream), C.byref(total), st)
        if rc not in (N.OK, N.ERR_TIMEOUT):     # a timed-out device wait is reported through the status words
            N.check(rc)
        return total.value, list(st)

    @property
    def cdf(self) -> torch.Tensor:
        """Level-2 table as a tensor view of the sampler's own memory."""
        return device_view(self.cdf_ptr, self.n, torch.float32)

    @property
    def l1(self) -> torch.Tensor:
        return device_view(self.l1_ptr, _nparts(self.n) + 1, torch.float64)

    @property
    def status(self) -> torch.Tensor:
        return device_view(self.status_ptr, N.STATUS_WORDS, torch.int32)

    def close(self) -> None:
        if self._h:
            lib.gearb_sampler_destroy(self._h)
            self._h = C.c_void_p(0)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def fill(dst: torch.Tensor, kind: int, seed: int, stream_id: int = 0, a: float = 0.0, b: float = 1.0,
         count: Optional[int] = None, stream=None) -> None:
    """Seeded synthetic data written on the device (benchmark tables)."""
    cnt = dst.numel() if count is None else int(count)
    call("gearb_fill", _ptr(dst), cnt, int(kind), C.c_uint64(seed), C.c_uint64(stream_id), float(a),
         float(b), _stream(stream))


def fill_ptr(ptr: int, count: int, kind: int, seed: int, stream_id: int = 0, a: float = 0.0,
             b: float = 1.0, stream=None) -> None:
    call("gearb_fill", C.c_void_p(ptr), int(count), int(kind), C.c_uint64(seed), C.c_uint64(stream_id),
         float(a), float(b), _stream(stream))


def vcopy(src_ptr: int, dst: torch.Tensor, src_off: torch.Tensor, dst_off: torch.Tensor,
          lengths: torch.Tensor, max_length: int, stream=None) -> None:
    """libgear.core.vcopy (src/cuda/copy.cu:175-215)."""
    n = min(src_off.numel(), dst_off.numel(), lengths.numel())
    call("gearb_vcopy", C.c_void_p(src_ptr), _ptr(dst), _dev_i64(src_off, "src_offsets"),
         _dev_i64(dst_off, "dst_offsets"), _dev_i64(lengths, "strides"), n, int(max_length),
         _stream(stream))


def copy(src_ptr: int, dst: torch.Tensor, src_off: torch.Tensor, dst_off: torch.Tensor, length: int,
         stream=None) -> None:
    """libgear.core.copy (src/cuda/copy.cu:138-173)."""
    n = min(src_off.numel(), dst_off.numel())
    call("gearb_copy", C.c_void_p(src_ptr), _ptr(dst), _dev_i64(src_off, "src_offsets"),
         _dev_i64(dst_off, "dst_offsets"), n, int(length), _stream(stream))


class PreparedPull:
    """A pull launch whose arguments were checked and marshalled once (PrioritySampler.prepare_pull)."""

    def __init__(self, sampler: "PrioritySampler", handler: "StorageHandler", args, keep, count, variate_stride):
        self._sampler, self._handler, self._a, self._keep = sampler, handler, args, keep
        self._count, self._stride = count, int(variate_stride)

    def run(self, variates: torch.Tensor, epoch: int = 0, stream=None) -> None:
        if variates.dtype != torch.float64 or not variates.is_cuda or not variates.is_contiguous():
            raise GearError(N.ERR_INVALID, "variates must be a contiguous float64 CUDA tensor")
        b = variates.numel() if self._count is None else int(self._count)
        if b != self._a.b or (b > 0 and (b - 1) * self._stride >= variates.numel()):
            raise GearError(N.ERR_INVALID, "prepared pull: another count of variates than it was prepared for")
        self._a.variates = variates.data_ptr()
        self._a.epoch = int(epoch)
        call("gearb_sampler_pull_ex", self._sampler._h, self._handler._h, C.byref(self._a), _stream(stream))

    def run_at(self, variates_ptr: int, epoch: int = 0, stream=None) -> None:
        """run() on variates given by their device address (float64, as many as the plan was prepared
        for, same stride): for callers that have checked the tensor once and only move inside it."""
        self._a.variates = int(variates_ptr)
        self._a.epoch = int(epoch)
        call("gearb_sampler_pull_ex", self._sampler._h, self._handler._h, C.byref(self._a), _stream(stream))


def mailbox_bytes(n: int = 0) -> int:
    """Size of a mailbox: the header alone (n = 0), or with room for the peers' level-1 copies."""
    return int(lib.gearb_mailbox_bytes(int(n)))


def mailbox_l1_offset(n: int, epoch: int, shard: int) -> int:
    """Byte offset, inside a mailbox_bytes(n) mailbox, of shard's level-1 copy for that epoch."""
    return int(lib.gearb_mailbox_l1_offset(int(n), C.c_uint64(int(epoch)), int(shard)))


def mailbox_blk_offset(n: int, epoch: int, shard: int) -> int:
    """Byte offset, inside a mailbox for shards of n priorities, of `shard`'s block-total copy for `epoch`."""
    return int(lib.gearb_mailbox_blk_offset(int(n), C.c_uint64(int(epoch)), int(shard)))


def ipc_export(device_ptr: int) -> bytes:
    """64-byte handle of a device allocation of this process, for the other ranks of the box."""
    buf = C.create_string_buffer(N.IPC_HANDLE_BYTES)
    call("gearb_ipc_export", C.c_void_p(int(device_ptr)), buf)
    return buf.raw


def ipc_open(handle: bytes) -> int:
    """Map another rank's allocation into this process; returns its address on the current device."""
    if len(handle) != N.IPC_HANDLE_BYTES:
        raise GearError(N.ERR_INVALID, f"an ipc handle has {N.IPC_HANDLE_BYTES} bytes")
    out = C.c_void_p(0)
    call("gearb_ipc_open", C.create_string_buffer(bytes(handle), N.IPC_HANDLE_BYTES), C.byref(out))
    return out.value


def ipc_close(device_ptr: int) -> None:
    call("gearb_ipc_close", C.c_void_p(int(device_ptr)))


class DeviceBuffer:
    """Zero-initialised device memory from the library's own allocator: unlike a tensor of a
    caching allocator it starts at the beginning of its allocation, so ipc_export() can hand it
    to other processes."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        p = C.c_void_p(0)
        call("gearb_device_alloc", self.nbytes, C.byref(p))
        self.ptr = p.value

    def view(self, dtype: torch.dtype) -> torch.Tensor:
        """The whole buffer as a tensor of `dtype` (the buffer must outlive the tensor)."""
        return device_view(self.ptr, self.nbytes // torch.empty(0, dtype=dtype).element_size(), dtype)

    def free(self) -> None:
        if self.ptr:
            call("gearb_device_free", C.c_void_p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
