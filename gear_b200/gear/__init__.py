"""Mirror of GEAR's `gear` Python package (specs, dtypes, dataset, sampler, loader, mpu,
comm) on top of `gear_b200.libgear`.  Same public names and call signatures as the
reference's gear/__init__.py; `gear_b200.dropin.install()` registers it as `gear`.
"""
from ..libgear import core as glibc
from . import comm, dataset, dtypes, errors, loader, mpu, sampler, specs  # noqa: F401


def init(device_id: int = None):
    """gear.init (gear/__init__.py:8-24): pick the CUDA device from LOCAL_RANK unless given."""
    if device_id is None:
        import os
        try:
            device_id = int(os.environ["LOCAL_RANK"])
        except KeyError:
            device_id = 0
    glibc.init(device_id)


def check_visible_device():
    glibc.print_environ()


__all__ = ["init", "comm", "loader", "dataset", "sampler", "dtypes", "errors", "mpu", "specs"]
