"""gear/specs.py:8-46: ColumnSpec.create / TableSpec.create factories."""
from typing import Any, Dict, Sequence, Union

import torch

from ..libgear import core as glibc
from .dtypes import CVT_DTYPES_TORCH_TO_GEAR, DataType


class ColumnSpec:
    @staticmethod
    def create(shape: Sequence[int], dtype: torch.dtype = torch.float32, name: str = "", *args, **kwargs):
        if not isinstance(dtype, DataType):
            dtype = CVT_DTYPES_TORCH_TO_GEAR[dtype]
        return glibc.ColumnSpec(list(shape), dtype, name)


class TableSpec:
    @staticmethod
    def create(rank: int = 0, worldsize: int = 1, trajectory_length: int = 100, capacity: int = 32,
               column_specs: Union[Sequence[Dict[str, Any]], glibc.ColumnSpec] = None, *args, **kwargs):
        cspecs = []
        for column_spec in (column_specs or []):
            cspecs.append(column_spec if isinstance(column_spec, glibc.ColumnSpec) else ColumnSpec.create(**column_spec))
        return glibc.TableSpec(rank, worldsize, trajectory_length, capacity, len(cspecs), cspecs)
