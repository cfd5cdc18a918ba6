"""gear/dataset/shared_dataset.py: SharedDataset = TrajectoryTable + Indexset + handler.
Same methods and pickle layout (meta, table, index state) as the reference (:23-258)."""
import pathlib
import pickle
import random
from collections import namedtuple
from typing import Sequence, Union

import torch
from torch.utils.data.dataset import Dataset

from ...libgear import core as glibc
from ..config import KEY_T_RANGE
from ..utils import ensure_path, get_local_node_hashed_int32

SharedDatasetMeta = namedtuple("SharedDatasetMeta", ["storage", "index"])
IndexMeta = namedtuple("IndexMeta", ["global_capacity", "local_capacity", "index_offset", "shared", "key"])


def _keys(key):
    rng = random.Random(key)                       # shared_dataset.py:35-37
    return rng.randint(0, KEY_T_RANGE), rng.randint(0, KEY_T_RANGE)


class SharedDataset(Dataset):
    @staticmethod
    def create(spec=None, create: bool = True, shard_rank: int = 0, shard_world: int = 1, proc_rank: int = 0,
               key: Union[int, None] = None, residency: str = "host"):
        if key is None:
            key = get_local_node_hashed_int32()
        table_key, iset_key = _keys(key)
        if spec is None:
            raise RuntimeError("SharedDataset creator process should provide storage specs!")
        table = glibc.TrajectoryTable(spec, table_key, bool(create), residency=residency)
        iset = glibc.Indexset(int(spec.capacity * spec.worldsize), int(spec.capacity / shard_world),
                              int(spec.capacity * spec.rank + spec.capacity * shard_rank / shard_world),
                              shared=True, key=iset_key, create=bool(create))
        while table.connect() == -1:
            pass
        return SharedDataset(table, iset)

    def __init__(self, table=None, index_set=None) -> None:
        super().__init__()
        self._table, self._iset, self._handler = table, index_set, None
        if table and index_set:
            self._build()

    def _build(self):
        ncol = self._table.get_table_spec().num_columns
        self._entry_cls = namedtuple("SharedDatasetEntry", ["weight", "timestep"] + [f"column{i}" for i in range(ncol)])
        self._handler = glibc.get_cpu_handler(
            self._table, self._iset.global_capacity, glibc.Range(0, 0),
            glibc.Range(self._iset.index_offset, self._iset.index_offset + self._iset.local_capacity))

    weights = property(lambda self: self._iset.weights)
    timesteps = property(lambda self: self._iset.timesteps)
    num_col = property(lambda self: self._table.ncolumns)

    def to_hbm(self):
        """Upload the table to HBM; gathers then read device memory instead of mapped host memory."""
        self._table.upload()
        return self

    def __getitem__(self, index):
        return self._entry_cls(self.weights[index], self.timesteps[index], *self.get_tensor_view(index))

    def __len__(self):
        return self._iset.capacity

    def __setitem__(self, index, value):
        weight, timestep, columns = value
        self._iset.weights[index] = weight
        self._iset.timesteps[index] = timestep
        for cid in range(self.num_col):
            self._handler.view(index, cid).copy(columns[cid].view(-1))

    def get_column_spec(self, cid: int):
        return self._table.get_column_spec(cid)

    def get_column_dtype(self, cid: int):
        return self._table.get_column_spec(cid).dtype

    def get_column_shape(self, cid: int):
        return (self._table.get_table_spec().trajectory_length,) + tuple(self._table.get_column_spec(cid).shape)

    def get_raw_view(self, index: int, cids: Sequence[int] = None):
        cids = range(self.num_col) if cids is None else cids
        return tuple(self._handler.view(index, cid) for cid in cids)

    def get_tensor_view(self, index: int, cids: Sequence[int] = None):
        cids = list(range(self.num_col) if cids is None else cids)
        raw = self.get_raw_view(index, cids)
        return tuple(raw[i].cast_tensor(self.get_column_dtype(cid)).view(self.get_column_shape(cid))
                     for i, cid in enumerate(cids))

    STREAM_ABOVE = 1 << 30      # tables beyond this (or without a host image) are written as a stream of chunks

    def checkpoint(self, path, streamed: Union[bool, None] = None):
        """(meta, table, index state) like the reference (:179-199).  The table is either the
        reference's pickle (one bytes object) or, for large tables and tables that live in HBM
        only, a header followed by raw chunks (TrajectoryTable.dump_stream): no full host copy,
        64-bit sizes throughout.  load() reads both."""
        ensure_path(path)
        if streamed is None:
            streamed = self._table.get_size() > self.STREAM_ABOVE or self._table.residency_name() == "hbm"
        with open(path, "wb") as of:
            pickle.dump(SharedDatasetMeta(self._table.get_table_spec(),
                                          IndexMeta(self._iset.global_capacity, self._iset.local_capacity,
                                                    self._iset.index_offset, self._iset.is_sharing, self._iset.shm_key)),
                        of, protocol=4)                 # protocol 4: objects beyond 4 GiB
            if streamed:
                self._table.dump_stream(of)
            else:
                pickle.dump(self._table, of, protocol=4)
            pickle.dump(self._iset.get_state(), of, protocol=4)

    def load(self, path, key: Union[int, None] = None, create: bool = True, proc_rank: int = 0,
             residency: Union[str, None] = None):
        """residency (streamed checkpoints only): where the table goes, e.g. "hbm" to stream the
        file straight into device memory; default: where it was when it was written."""
        if key is None:
            key = get_local_node_hashed_int32()
        table_key, iset_key = _keys(key)
        with open(pathlib.Path(path), "rb") as f:
            meta = pickle.load(f)
            if create:
                obj = pickle.load(f)
                if isinstance(obj, glibc.StreamedTableHeader):
                    obj = glibc.TrajectoryTable.load_stream(obj, f, residency=residency)
                self._table = obj
                self._iset = glibc.Indexset.load_state(pickle.load(f), meta.index.shared, iset_key, True)
            else:
                self._table = glibc.TrajectoryTable(meta.storage, table_key, False)
                self._iset = glibc.Indexset(meta.index.global_capacity, meta.index.local_capacity,
                                            meta.index.index_offset, meta.index.shared, iset_key, False)
        while self._table.connect() == -1:
            pass
        self._build()
        return self
