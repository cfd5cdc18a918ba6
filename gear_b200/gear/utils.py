"""gear/utils.py: path helper and the per-host shared-memory key."""
import os
import pathlib
import socket
import zlib
from typing import Union


def ensure_path(path: Union[str, pathlib.Path]) -> None:
    path = pathlib.Path(path)
    if not path.parent.exists():
        os.makedirs(path.parent)


def get_local_node_hashed_int32() -> int:
    """A key derived from the host name (gear/utils.py:19-23).  The reference uses Python's
    hash(), which is salted per process unless PYTHONHASHSEED is fixed, so two processes of one
    job could disagree on the key; a CRC of the name is the same in every process."""
    from .config import KEY_T_RANGE
    return zlib.crc32(socket.gethostname().encode()) % KEY_T_RANGE
