"""`libgear.core`: the classes and functions GEAR's Python layer uses, same names and
argument meaning as the pybind registrations (file:line given per item), executed by
libgear_b200.so.  Host-side value types (specs, patterns, ranges, spans) are plain Python;
everything that touches table memory or the GPU goes through the C ABI.
"""
from __future__ import annotations

import builtins
import ctypes as C
import enum
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import _native as N
from .. import core as _c
from .._native import GearError

# --------------------------------------------------------------------------- #
# dtypes (src/common/pybind.cc:53-84, include/common/dtypes.h:18-76)
# --------------------------------------------------------------------------- #
class DataType(enum.IntEnum):
    """Same members and the same aliasing as the pybind enum: Python `int8` names kByte and
    `uint8` names kChar (pybind.cc:57-58); the span casts swap them back (span.h:100-102), so
    torch.uint8 columns round-trip as uint8."""
    bool = 0      # kBool
    int8 = 1      # kByte
    uint8 = 2     # kChar
    short = 3     # kShort
    int16 = 3
    int = 4       # kInt
    int32 = 4
    long = 5      # kLong
    int64 = 5
    half = 6      # kHalf
    float16 = 6
    float = 7     # kFloat
    float32 = 7
    double = 8    # kDouble
    float64 = 8


def __getattr__(name):
    """export_values(): `core.float32`, `core.int`, `core.bool` ... resolve to DataType members
    (looked up here rather than stored as globals, which would shadow the builtins)."""
    if name in DataType.__members__:
        return DataType[name]
    raise AttributeError(f"module 'libgear.core' has no attribute {name!r}")


_SIZEOF = {0: 1, 1: 1, 2: 1, 3: 2, 4: 4, 5: 8, 7: 4, 8: 8}           # no entry for half: sizeof_dtype throws
# tensor dtype a span of this DataType presents (span.h:100-107: kByte -> Char, kChar -> Byte swapped back)
_TORCH_OF = {0: torch.bool, 1: torch.int8, 2: torch.uint8, 3: torch.int16, 4: torch.int32, 5: torch.int64,
             7: torch.float32, 8: torch.float64}
_NUMPY_OF = {0: np.bool_, 1: np.int8, 2: np.uint8, 3: np.int16, 4: np.int32, 5: np.int64, 7: np.float32,
             8: np.float64}


def sizeof_dtype(dtype) -> int:
    try:
        return _SIZEOF[int(dtype)]
    except KeyError:
        raise RuntimeError("Unsupported type.")          # dtypes.h:71-73


def init(device_id: int) -> None:
    """core.init (src/cuda/init.cu:16-18)."""
    _c.init(device_id)


def print_environ() -> None:
    """core.print_environ (src/env.cc:55-58)."""
    print(f"<GEAR environ> visible CUDA devices: {_c.device_count()}")


def print_compile_options() -> None:
    print(f"<GEAR compile options> libgear_b200 version {N.lib.gearb_version()}, sm_100a, HAVE_CUDA")


# --------------------------------------------------------------------------- #
# value types
# --------------------------------------------------------------------------- #
class Range:
    """core.Range(lb, hb) (src/common/pybind.cc:86-91)."""

    def __init__(self, lb: int, hb: int):
        self.lb, self.hb = int(lb), int(hb)

    def __repr__(self):
        return f"Range({self.lb}, {self.hb})"


class MemoryPtr:
    """core.MemoryPtr(int) (src/memory/pybind.cc:13-17)."""

    def __init__(self, ptr: int):
        self.ptr = int(ptr)

    def get(self) -> int:
        return self.ptr

    def __repr__(self):
        return hex(self.ptr)


class ColumnSpec:
    """core.ColumnSpec(shape, dtype, name) (src/storage/pybind.cc:22-40; specs.cc:6-14)."""

    def __init__(self, shape: Sequence[int], dtype, name: str = ""):
        if not isinstance(dtype, DataType):
            raise TypeError("ColumnSpec: dtype must be a libgear DataType")
        self.shape = [int(s) for s in shape]
        self.dtype = dtype
        self.name = str(name)

    def size(self) -> int:
        n = sizeof_dtype(self.dtype)
        for s in self.shape:
            n *= s
        return n

    def __getstate__(self):
        return (self.shape, self.dtype, self.name)

    def __setstate__(self, t):
        if len(t) != 3:
            raise RuntimeError("Invalid state for ColumnSpec unpickling!")
        self.shape, self.dtype, self.name = list(t[0]), t[1], t[2]

    def __repr__(self):
        return f"<ColumnSpec {self.name!r} {self.shape} {self.dtype.name}>"


class TableSpec:
    """core.TableSpec(rank, worldsize, trajectory_length, capacity, num_columns, column_specs)
    (src/storage/pybind.cc:42-69; specs.cc:16-43)."""

    def __init__(self, rank, worldsize, trajectory_length, capacity, num_columns, column_specs):
        column_specs = list(column_specs)
        if len(column_specs) != int(num_columns):
            raise RuntimeError(f"column specs size mismatch with declared number of columns: spec num "
                               f"{len(column_specs)}, expected {num_columns}")
        self.rank, self.worldsize = int(rank), int(worldsize)
        self.trajectory_length, self.capacity = int(trajectory_length), int(capacity)
        self._num_columns, self._column_specs = int(num_columns), column_specs

    num_columns = property(lambda self: self._num_columns)
    column_specs = property(lambda self: self._column_specs)

    def index(self, name: str) -> int:
        for i, c in enumerate(self._column_specs):
            if c.name == name:
                return i
        return -1

    def size(self) -> int:
        return builtins.sum(c.size() for c in self._column_specs) * self.trajectory_length * self.capacity

    def __getstate__(self):
        return (self.rank, self.worldsize, self.trajectory_length, self.capacity, self._num_columns,
                self._column_specs)

    def __setstate__(self, t):
        if len(t) != 6:
            raise RuntimeError("Invalid state for TableSpec unpickling!")
        self.__init__(*t)


class SubscribePattern:
    """core.SubscribePattern(offset, length[, PadOption]) (src/storage/pybind.cc:73-105); the
    two-argument form pads at the tail (:78-81)."""

    class PadOption(enum.IntEnum):
        inactive = N.PAD_INACTIVE
        head = N.PAD_HEAD
        tail = N.PAD_TAIL

    def __init__(self, offset: int, length: int, pad_option: "SubscribePattern.PadOption" = None):
        self._offset, self._length = int(offset), int(length)
        self.pad_option = SubscribePattern.PadOption.tail if pad_option is None else SubscribePattern.PadOption(pad_option)

    offset = property(lambda self: self._offset)
    length = property(lambda self: self._length)

    def __repr__(self):
        names = {0: "PadOption::kInactive", 1: "PadOption::kHead", 2: "PadOption::kTail"}
        return f"<SubscribePattern: offset {self._offset}, length {self._length}, {names[int(self.pad_option)]}>"

    def __getstate__(self):
        return (self._offset, self._length, self.pad_option)

    def __setstate__(self, t):
        if len(t) != 3:
            raise RuntimeError("Invalid state for SubscribePattern unpickling")
        self._offset, self._length, self.pad_option = int(t[0]), int(t[1]), SubscribePattern.PadOption(t[2])

    def _native(self) -> _c.SubscribePattern:
        return _c.SubscribePattern(self._offset, self._length, int(self.pad_option))


inactive, head, tail = SubscribePattern.PadOption.inactive, SubscribePattern.PadOption.head, SubscribePattern.PadOption.tail


# --------------------------------------------------------------------------- #
# spans (include/common/span.h:51-107, src/common/pybind.cc:13-51)
# --------------------------------------------------------------------------- #
class _Span:
    """Borrowed view (pointer + element count) over host memory."""
    _np = np.uint8

    def __init__(self, array: np.ndarray, keep=None):
        self._a = array          # numpy view over the memory, dtype self._np
        self._keep = keep        # whatever owns the memory

    @property
    def ptr(self) -> int:
        return self._a.ctypes.data

    @property
    def size(self) -> int:
        return self._a.size

    @classmethod
    def from_tensor(cls, t: torch.Tensor):
        if t.is_cuda:
            raise RuntimeError("spans view host memory; pass device tensors to the GPU entry points directly")
        if not t.is_contiguous():
            # a span is a view (include/common/span.h:51-99): writes through it must reach the
            # tensor, which a copy made here would silently swallow
            raise RuntimeError("spans view memory in place; pass a contiguous tensor")
        a = t.detach().numpy()
        return cls(a.view(cls._np).reshape(-1), keep=t)

    @staticmethod
    def _as(arr, cls):
        return cls(arr.view(np.uint8).reshape(-1).view(cls._np), keep=arr)

    def as_bool(self): return _Span._as(self._a, BoolSpan)
    def as_int8(self): return _Span._as(self._a, Int8Span)
    def as_uint8(self): return _Span._as(self._a, Uint8Span)
    def as_int16(self): return _Span._as(self._a, Int16Span)
    def as_int32(self): return _Span._as(self._a, Int32Span)
    def as_int64(self): return _Span._as(self._a, Int64Span)
    def as_float32(self): return _Span._as(self._a, Float32Span)
    def as_float64(self): return _Span._as(self._a, Float64Span)

    def copy(self, t: torch.Tensor) -> None:
        """Span::copy (span.h:73-79): memcpy min(span bytes, tensor bytes) from the tensor."""
        src = t.detach().cpu().contiguous().view(-1).numpy().view(np.uint8).reshape(-1)
        dst = self._a.view(np.uint8).reshape(-1)
        n = min(dst.size, src.size)
        dst[:n] = src[:n]

    def tensor(self) -> torch.Tensor:
        return torch.from_numpy(self._a)

    def cast_tensor(self, dtype) -> torch.Tensor:
        """Span::cast_tensor (span.h:83-97): the same bytes as a tensor of `dtype`."""
        if int(dtype) not in _NUMPY_OF:
            raise RuntimeError("Unsupported type.")
        return torch.from_numpy(self._a.view(np.uint8).reshape(-1).view(_NUMPY_OF[int(dtype)]))

    @classmethod
    def Tensor(cls, span):  # noqa: N802  (static_as_tensor is bound as "Tensor")
        return span.tensor()

    def __len__(self):
        return self.size

    def __getitem__(self, i):
        return self._a[i]


class BoolSpan(_Span): _np = np.bool_
class Int8Span(_Span): _np = np.int8
class Uint8Span(_Span): _np = np.uint8
class Int16Span(_Span): _np = np.int16
class Int32Span(_Span): _np = np.int32
class Int64Span(_Span): _np = np.int64
class Float32Span(_Span): _np = np.float32
class Float64Span(_Span): _np = np.float64


def _i64_host(x) -> np.ndarray:
    """Tensor or Int64Span -> int64 numpy view (torch tensors convert implicitly, pybind.cc:28)."""
    if isinstance(x, _Span):
        return x._a.view(np.int64) if x._a.dtype != np.int64 else x._a
    if isinstance(x, torch.Tensor):
        if x.dtype != torch.int64:
            raise RuntimeError("expected an int64 tensor")
        return x.detach().cpu().contiguous().numpy() if x.is_cuda else x.detach().numpy()
    return np.ascontiguousarray(x, np.int64)


def _i64_out(x) -> np.ndarray:
    """An OUTPUT argument as a writable int64 view of the caller's own memory.  The reference's
    spans write through the tensor's data pointer (src/common/pybind.cc:28); a device tensor or a
    non-contiguous one would have to be copied first and the results would be lost, so both are
    refused."""
    if isinstance(x, _Span):
        return x._a.view(np.int64) if x._a.dtype != np.int64 else x._a
    if isinstance(x, torch.Tensor):
        if x.dtype != torch.int64 or x.is_cuda or not x.is_contiguous():
            raise RuntimeError("output offsets must be contiguous int64 host tensors (or Int64Span)")
        return x.detach().numpy()
    if isinstance(x, np.ndarray) and x.dtype == np.int64 and x.flags.c_contiguous and x.flags.writeable:
        return x
    raise RuntimeError("output offsets must be contiguous int64 host tensors (or Int64Span)")


# --------------------------------------------------------------------------- #
# table, handler, index set
# --------------------------------------------------------------------------- #
class TrajectoryTable:
    """core.TrajectoryTable(spec, key, create) (src/storage/pybind.cc:166-204; table.cc:8-43).
    `residency` is an extension: "host" (the reference's only mode), "hbm", or "host+hbm"."""

    def __init__(self, spec: TableSpec, key: int, create: bool, residency: str = "host"):
        self._spec, self._key, self._create = spec, int(key), bool(create)
        self._residency = residency
        res = {"host": N.RES_HOST, "hbm": N.RES_HBM, "host+hbm": N.RES_HOST | N.RES_HBM}[residency]
        self._t = _c.TrajectoryTable([c.size() for c in spec.column_specs], spec.trajectory_length,
                                     spec.capacity, residency=res, key=self._key, create=self._create)

    ncolumns = property(lambda self: self._spec.num_columns)

    def get_table_spec(self) -> TableSpec:
        return self._spec

    def get_column_spec(self, cid: int) -> ColumnSpec:
        return self._spec.column_specs[cid]

    def connect(self) -> int:
        """TrajectoryTable::connect (table.cc:27): size in bytes, or -1 while the segment is
        not there (callers retry: gear/dataset/shared_dataset.py:72-74)."""
        try:
            return self._t.connect()
        except GearError as e:
            if e.code == N.ERR_STATE:
                return -1
            raise

    def get_address(self) -> MemoryPtr:
        return MemoryPtr(self._t.host_ptr or self._t.device_ptr)

    def upload(self) -> None:
        """Copy the host image into HBM; later gathers read the HBM copy."""
        self._t.upload()
        self._residency = "host+hbm"

    def get_size(self) -> int:
        return self._t.nbytes

    def __getstate__(self):
        # the reference pickles (spec, key, size, create, raw bytes) (pybind.cc:178-186); a table that
        # lives in HBM only is read back for it (dump_stream below avoids the full host copy)
        img = np.array(self._t.host_view(), copy=True) if self._t.host_ptr else self._t.read(0, self._t.nbytes)
        return (self._spec, self._key, self._t.nbytes, self._create, img)

    # -- checkpoint at scale: the table's bytes as a stream of chunks --------------------------
    # The reference's pickle holds the whole table as ONE bytes object and casts its size to int
    # on load (src/storage/pybind.cc:178-204), which stops at 2 GiB and needs the table twice in
    # host memory.  The streamed form is a small pickled header followed by raw chunks, each
    # trailed by its CRC-32; a chunk goes through a pinned bounce buffer between the file and
    # whatever copies the table has (mapped host memory, HBM), so an HBM-only table of any size
    # is written and read back without a host image.
    STREAM_CHUNK = 64 << 20

    def dump_stream(self, f, chunk_bytes: int = 0) -> None:
        import pickle
        import zlib
        chunk = int(chunk_bytes) or self.STREAM_CHUNK
        n = self._t.nbytes
        pickle.dump(StreamedTableHeader(self._spec, self._key, n, self._create, chunk, self.residency_name()), f, protocol=4)
        bounce = _pinned(min(chunk, max(n, 1)))
        for off in range(0, n, chunk):
            m = min(chunk, n - off)
            view = bounce[:m]
            self._t.read_into(off, view)
            f.write(memoryview(view))
            f.write(int(zlib.crc32(memoryview(view))).to_bytes(4, "little"))

    @classmethod
    def load_stream(cls, header: "StreamedTableHeader", f, key=None, residency=None) -> "TrajectoryTable":
        import zlib
        t = cls(header.spec, header.key if key is None else key, True, residency=residency or header.residency)
        if t.connect() == -1:
            raise RuntimeError("TrajectoryTable: cannot allocate the table while loading")
        n, chunk = int(header.nbytes), int(header.chunk_bytes)
        if n != t._t.nbytes:
            raise RuntimeError(f"checkpoint holds {n} bytes, the spec describes {t._t.nbytes}")
        bounce = [_pinned(min(chunk, max(n, 1))) for _ in range(2)]     # one fills while the other uploads
        for i, off in enumerate(range(0, n, chunk)):
            m = min(chunk, n - off)
            view = bounce[i & 1][:m]
            if f.readinto(memoryview(view)) != m:
                raise RuntimeError("checkpoint truncated inside the table")
            crc = int.from_bytes(f.read(4), "little")
            if crc != zlib.crc32(memoryview(view)):
                raise RuntimeError(f"checkpoint corrupt: chunk at byte {off} fails its CRC-32")
            t._t.write(off, view, sync=i & 1 == 1)       # at most two uploads in flight
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()
        return t

    def residency_name(self) -> str:
        return self._residency

    def __setstate__(self, t):
        if len(t) != 5:
            raise RuntimeError("Invalid state!")
        self.__init__(t[0], t[1], t[3])
        if self.connect() == -1:
            raise RuntimeError("TrajectoryTable: cannot allocate the table while unpickling")
        self._t.write(0, np.asarray(t[4], np.uint8)[: int(t[2])])    # 64-bit size (the reference casts to int, :193)


class StreamedTableHeader:
    """What precedes a table's raw chunks in a streamed checkpoint (TrajectoryTable.dump_stream)."""

    def __init__(self, spec, key, nbytes, create, chunk_bytes, residency):
        self.spec, self.key, self.nbytes, self.create = spec, int(key), int(nbytes), bool(create)
        self.chunk_bytes, self.residency = int(chunk_bytes), str(residency)


def _pinned(nbytes: int) -> np.ndarray:
    """A page-locked uint8 buffer when CUDA is there (copies to and from it run at link speed and
    asynchronously), plain memory otherwise."""
    if torch.cuda.is_available():
        return torch.empty(int(nbytes), dtype=torch.uint8).pin_memory().numpy()
    return np.empty(int(nbytes), np.uint8)


class CpuTrajectoryStorageHandler:
    """CpuTrajectoryStorageHandler (src/storage/pybind.cc:108-155; handler.cc)."""

    def __init__(self, table: TrajectoryTable, global_capacity: int, wregion: Range, rregion: Range):
        self._table = table
        self._h = _c.StorageHandler(table._t, global_capacity, (wregion.lb, wregion.hb), (rregion.lb, rregion.hb))
        self._comm = None

    def set(self, cids: Sequence[int], patterns: Sequence[SubscribePattern]) -> None:
        self._h.set([int(c) for c in cids], [p._native() for p in patterns])

    def sub(self, indices, timesteps, lengths, column_id: int, src_offsets, dst_offsets, copy_lengths) -> int:
        """handler.sub (handler.cc:78-131): fills the three output spans, returns length*row."""
        try:
            s, d, b, slot = self._h.sub(_i64_host(indices), _i64_host(timesteps), _i64_host(lengths), int(column_id))
        except GearError as e:
            raise RuntimeError(str(e).split("] ", 1)[-1]) from None
        n = len(s)
        for out, val in ((src_offsets, s), (dst_offsets, d), (copy_lengths, b)):
            _i64_out(out)[:n] = val
        return slot

    sub_ = sub

    def subcopy(self, idxs: torch.Tensor, tss: torch.Tensor, lens: torch.Tensor, column: int, dst: torch.Tensor) -> None:
        """handler.subcopy (pybind.cc:140-146 -> handler.cc:133-154): int64 device tensors in,
        the clipped segments land in `dst`; padding is left as the caller prepared it."""
        try:
            self._h.subcopy(idxs, tss, lens, int(column), dst)
        except GearError as e:
            raise RuntimeError(str(e).split("] ", 1)[-1]) from None

    def gather(self, columns, idxs, tss, lens, dsts, zero_fill=True) -> None:
        """All listed columns in one launch (extension)."""
        self._h.gather(list(columns), idxs, tss, lens, list(dsts), zero_fill=zero_fill)

    def view(self, index: int, column_id: int) -> Uint8Span:
        return Uint8Span(self._h.view(int(index), int(column_id)), keep=self._table)

    def raw(self, offset: int, length: int) -> Uint8Span:
        v = self._table._t.host_view()
        return Uint8Span(v[int(offset):int(offset) + int(length)], keep=self._table)

    # -- cross-rank segment exchange (handler.cc:156-221) ------------------------------------
    def connect(self, rank: int, worldsize: int, id: bytes) -> None:  # noqa: A002
        from ..comm import Communicator
        self._comm = Communicator(rank, worldsize, bytes(id))

    def _segment_bytes(self, timesteps, lengths, column):
        p = self._h.patterns[int(column)]
        ts, ln = _i64_host(timesteps), _i64_host(lengths)
        start = np.maximum(ts + p.offset, 0)
        end = np.minimum(start + p.length, ln)
        return np.maximum(end - start, 0) * self._table._t.row_bytes[int(column)]

    def subsend(self, peer: int, indices, timesteps, lengths, column: int) -> None:
        """Owner side: the clipped segments of `column`, gathered in one launch into a staging
        buffer (slot-strided, like the requester's tensor) and sent with ONE message."""
        if self._comm is None:
            raise RuntimeError("call connect() first")
        idx, ts, ln = (torch.from_numpy(_i64_host(x).copy()).cuda() for x in (indices, timesteps, lengths))
        p = self._h.patterns[int(column)]
        slot = p.length * self._table._t.row_bytes[int(column)]
        buf = torch.empty(len(idx) * slot, dtype=torch.uint8, device="cuda")
        self._h.gather([int(column)], idx, ts, ln, [buf], zero_fill=True)
        self._comm.send(buf, int(peer))

    def subrecv(self, peer: int, dst: torch.Tensor, indices, timesteps, lengths, column: int) -> None:
        if self._comm is None:
            raise RuntimeError("call connect() first")
        p = self._h.patterns[int(column)]
        slot = p.length * self._table._t.row_bytes[int(column)]
        n = len(_i64_host(indices))
        self._comm.recv(dst.view(torch.uint8).view(-1)[: n * slot], int(peer))


def get_cpu_handler(table: TrajectoryTable, global_capacity: int, wregion: Range, rregion: Range):
    """core.get_cpu_handler (src/storage/pybind.cc:157-164)."""
    return CpuTrajectoryStorageHandler(table, global_capacity, wregion, rregion)


def get_cuda_handler(table: TrajectoryTable, global_capacity: int, wregion: Range, rregion: Range):
    """The HBM-resident handler the reference only declares (include/storage/handler.h:89-102):
    uploads the table's host image to HBM and gathers from there."""
    table.upload()
    return CpuTrajectoryStorageHandler(table, global_capacity, wregion, rregion)


class IndexsetState:
    """IndexsetState (include/index/set.h:146-182), pickled as (index_offset, local_capacity,
    global_capacity, bytes of timesteps followed by weights) (src/index/pybind.cc:15-50)."""

    def __init__(self, global_capacity, local_capacity, index_offset, timesteps: np.ndarray, weights: np.ndarray):
        self.global_capacity, self.local_capacity, self.index_offset = int(global_capacity), int(local_capacity), int(index_offset)
        self.timesteps = np.array(timesteps, np.int64, copy=True)
        self.weights = np.array(weights, np.float32, copy=True)

    def __getstate__(self):
        mem = np.concatenate([self.timesteps.view(np.uint8), self.weights.view(np.uint8)])
        return (self.index_offset, self.local_capacity, self.global_capacity, mem)

    def __setstate__(self, t):
        if len(t) != 4:
            raise RuntimeError("Invalid state for unpickling IndexsetState")
        off, loc, glob, mem = t
        mem = np.asarray(mem, np.uint8)
        self.__init__(glob, loc, off, mem[: loc * 8].view(np.int64), mem[loc * 8: loc * 12].view(np.float32))


class Indexset:
    """core.Indexset(global_capacity, local_capacity, index_offet, shared=False, key=0, create=False)
    (src/index/pybind.cc:293-356; include/index/set.h:191-251)."""

    def __init__(self, global_capacity, local_capacity, index_offet=0, shared=False, key=0, create=False,
                 index_offset=None):
        off = index_offet if index_offset is None else index_offset
        self._s = _c.Indexset(int(global_capacity), int(local_capacity), int(off), bool(shared), int(key), bool(create))

    timesteps = property(lambda self: self._s.timesteps)
    weights = property(lambda self: self._s.weights)
    global_capacity = property(lambda self: self._s.global_capacity)
    local_capacity = property(lambda self: self._s.local_capacity)
    capacity = property(lambda self: self._s.local_capacity)
    index_offset = property(lambda self: self._s.index_offset)
    is_sharing = property(lambda self: self._s.is_sharing)
    shm_key = property(lambda self: self._s.shm_key)

    def get_state(self) -> IndexsetState:
        return IndexsetState(self.global_capacity, self.local_capacity, self.index_offset,
                             self._s.timesteps_np, self._s.weights_np)

    @staticmethod
    def load_state(state: IndexsetState, shared=False, key=0, create=False) -> "Indexset":
        s = Indexset(state.global_capacity, state.local_capacity, state.index_offset, shared, key, create)
        s._s.timesteps_np[:] = state.timesteps
        s._s.weights_np[:] = state.weights
        return s

    def set_timestep(self, index: int, ts: int) -> None:
        self._s.timesteps_np[index] = ts

    def set_weight(self, index: int, w: float) -> None:
        self._s.weights_np[index] = w


# --------------------------------------------------------------------------- #
# kernels bound at module level (src/cuda/copy.cu:245-258, one_dim_*.cu)
# --------------------------------------------------------------------------- #
def vcopy(src: MemoryPtr, dst: torch.Tensor, src_offsets: torch.Tensor, dst_offsets: torch.Tensor,
          strides: torch.Tensor, max_stride: int) -> None:
    """core.vcopy (copy.cu:175-215).  A host MemoryPtr must be device-visible (mapped)."""
    _c.vcopy(_device_alias(src.get()), dst, src_offsets, dst_offsets, strides, int(max_stride))


def copy(src: MemoryPtr, dst: torch.Tensor, src_offsets: torch.Tensor, dst_offsets: torch.Tensor, stride: int) -> None:
    """core.copy (copy.cu:138-173)."""
    _c.copy(_device_alias(src.get()), dst, src_offsets, dst_offsets, int(stride))


def copy_debug(src: torch.Tensor, dst, src_offsets, dst_offsets, strides, max_stride) -> None:
    """core.copy_debug (copy.cu:248-257): vcopy with a tensor as the source."""
    _c.vcopy(src.data_ptr(), dst, src_offsets, dst_offsets, strides, int(max_stride))


def _device_alias(host_or_device_ptr: int) -> int:
    """Mapped pinned host memory is addressed by the same value on the device (unified
    addressing), so the pointer passes through."""
    return int(host_or_device_ptr)


def prefix_sum(input: torch.Tensor, output: torch.Tensor):  # noqa: A002
    """core.prefix_sum(in, out) (one_dim_prefix_sum.cu:246-276).  `output` receives the
    partition-local float32 cumulative table; the float64 partition offsets are returned
    (their last entry is the total)."""
    cdf, l1, _ = _c.scan(input)
    output.view(-1)[: cdf.numel()].copy_(cdf)
    return l1


def sum(val_tensor: torch.Tensor, sum_tensor: torch.Tensor, stride: int = 1) -> None:  # noqa: A001
    """core.sum(vals, out, stride) (one_dim_sum.cu:84-99): the total in a fixed order."""
    _, l1, _ = _c.scan(val_tensor)
    sum_tensor.view(-1)[:1].copy_(l1[-1:].to(sum_tensor.dtype))


# --------------------------------------------------------------------------- #
# online path: index server / client (src/index/pybind.cc:53-291)
# --------------------------------------------------------------------------- #
class _InferenceRequests:
    """InferenceRequestArray (include/index/request.h:19-35): count, srcs, idxs, tss."""

    def __init__(self, capacity: int):
        self.capacity, self.count = int(capacity), 0
        self.srcs = np.zeros(capacity, np.int32)
        self.idxs = np.zeros(capacity, np.int64)
        self.tss = np.zeros(capacity, np.int64)


class _WeightUpdates:
    """WeightUpdateRequestArray (include/index/request.h:37-55): the updates recorded since the
    last continuous() call, one per index."""

    def __init__(self, capacity: int):
        self.capacity, self.count = int(capacity), 0
        self.timesteps = np.zeros(capacity, np.int64)
        self.weights = np.zeros(capacity, np.float32)
        self._list = []

    def update(self, index: int, timestep: int, weight: float) -> None:
        if index not in self._list:
            self._list.append(int(index))
            self.count += 1
        self.timesteps[index] = timestep
        self.weights[index] = weight

    def continuous(self, idxs, weights) -> int:
        """request.cc:56-75: idxs[i] = index, idxs[capacity + i] = timestep, weights[i]; clears the list."""
        n = self.count
        idxs, weights = _i64_out(idxs), (weights._a if isinstance(weights, _Span) else weights.numpy())
        if len(idxs) < 2 * n or len(weights) < n:
            raise RuntimeError("Index output array for continuous weight update array has less space than required")
        for i, idx in enumerate(self._list):
            idxs[i] = idx
            idxs[self.capacity + i] = self.timesteps[idx]
            weights[i] = self.weights[idx]
        self._list, self.count = [], 0
        return n


class CachedRequest:
    """CachedRequest (include/index/request.h:57-63)."""

    def __init__(self, capacity: int):
        self.capacity = int(capacity)
        self.iarr = _InferenceRequests(capacity)
        self.warr = _WeightUpdates(capacity)


class SharedMemoryIndexServer:
    """core.SharedMemoryIndexServer(key, num_clients, index_offset, capacity) (src/index/server.cc)."""

    def __init__(self, key: int, num_clients: int, index_offset: int, capacity: int):
        from ..ingest import IndexServer
        self._s = IndexServer(key, num_clients, index_offset, capacity)

    def connect(self) -> int:
        return 0                                   # the segment is created with the object

    def get_capacity(self) -> int:
        return self._s.capacity

    def get_num_clients(self) -> int:
        return self._s.num_clients

    def scan(self, cache: CachedRequest) -> None:
        ni, nu = self._s.scan()
        cache.iarr.count = 0
        for k in range(ni):
            c = cache.iarr.count
            cache.iarr.srcs[c], cache.iarr.idxs[c], cache.iarr.tss[c] = self._s.infer_src[k], self._s.infer_idx[k], self._s.infer_ts[k]
            cache.iarr.count = c + 1
        off = self._s.index_offset
        for k in range(nu):
            cache.warr.update(int(self._s.upd_idx[k]) - off, int(self._s.upd_ts[k]), float(self._s.upd_w[k]))
        self._pending = nu

    def update(self, cache: CachedRequest) -> None:
        self._s.update(getattr(self, "_pending", 0))
        self._pending = 0

    def callback(self, cache: CachedRequest) -> None:
        self._s.callback(cache.iarr.srcs[: cache.iarr.count])
        cache.iarr.count = 0

    def get_weights(self) -> torch.Tensor:
        return torch.from_numpy(self._s.weights)

    def get_timesteps(self) -> torch.Tensor:
        return torch.from_numpy(self._s.timesteps)

    def __getstate__(self):
        return (self._s.key, self._s.num_clients, self._s.index_offset, self._s.capacity, self._s.get_state())

    def __setstate__(self, t):
        self.__init__(t[0], t[1], t[2], t[3])
        self._s.set_state(t[4])


class SharedMemoryIndexClient:
    """core.SharedMemoryIndexClient(key, client_rank, num_clients) (src/index/client.cc)."""

    def __init__(self, key: int, client_rank: int, num_clients: int):
        from ..ingest import IndexClient
        self._c = IndexClient(key, client_rank, num_clients)
        self.timeout_ms = 60_000

    def connect(self) -> int:
        return self._c.connect()

    def acquire(self) -> None:
        self._c.acquire(self.timeout_ms)

    def wait(self) -> None:
        self._c.wait(self.timeout_ms)

    def release(self) -> None:
        self._c.release()

    def writeback(self, terminated: bool, alloc_new: bool, weight: float = 0.0) -> int:
        return self._c.writeback(terminated, alloc_new, weight)

    def step_inc(self) -> int:
        return self._c.step_inc()

    def get_index(self) -> int:
        return self._c.get_index()

    def get_timestep(self) -> int:
        return self._c.get_timestep()

    def get_num_clients(self) -> int:
        return self._c.num_clients

    def get_status_unsafe(self):
        return self._c.status()
