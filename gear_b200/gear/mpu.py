"""Stand-in for gear/mpu.py:53-166.  The reference wraps DeepSpeed's PipelineParallelGrid only
to read the data-parallel rank, world size and group; this class answers the same three
questions from torch.distributed (or from its constructor arguments) and carries `device`."""
import os
from typing import Union

import torch
import torch.distributed as dist


class ModelParallelismUnit:
    def __init__(self, proc_coord=None, global_rank: Union[int, None] = None, local_rank: Union[int, None] = None,
                 device: Union[torch.device, None] = None, dp_rank: Union[int, None] = None,
                 dp_world_size: Union[int, None] = None, dp_group=None):
        inited = dist.is_available() and dist.is_initialized()
        self.global_rank = global_rank if global_rank is not None else (dist.get_rank() if inited else 0)
        self.local_rank = local_rank if local_rank is not None else int(os.environ.get("LOCAL_RANK", "0"))
        self._dp_rank = dp_rank if dp_rank is not None else (dist.get_rank(dp_group) if inited else 0)
        self._dp_world = dp_world_size if dp_world_size is not None else (dist.get_world_size(dp_group) if inited else 1)
        self._dp_group = dp_group
        self.device = device if device is not None else torch.device(f"cuda:{self.local_rank}")

    def get_global_rank(self):
        return self.global_rank

    def get_model_parallel_rank(self) -> int:
        return 0

    def get_model_parallel_world_size(self) -> int:
        return 1

    def get_data_parallel_rank(self):
        return self._dp_rank

    def get_data_parallel_world_size(self):
        return self._dp_world

    def get_data_parallel_group(self):
        return self._dp_group
