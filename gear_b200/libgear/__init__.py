"""Mirror of GEAR's `libgear` pybind module (src/pybind.cc:75-109) on top of libgear_b200.so.

Submodules `core` and `comm` carry the names the in-scope Python of GEAR imports
(`import libgear.core as glibc`).  `gear_b200.dropin.install()` registers this package
under the name `libgear`.
"""
from . import comm, core  # noqa: F401

__all__ = ["core", "comm"]
