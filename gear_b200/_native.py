"""ctypes binding of libgear_b200.so (the C ABI declared in include/gear_b200.h).

The library is the product: if it is missing the import fails loudly -- there is
no Python or CPU fallback for any device operation.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = Path(os.environ.get("GEAR_B200_LIB", PKG / "lib" / "libgear_b200.so"))

OK = 0
ERR_INVALID, ERR_CUDA, ERR_NOMEM, ERR_STATE, ERR_TIMEOUT, ERR_NCCL, ERR_UNSUPPORTED = range(1, 8)

ST_L1_RESUMMED = 0x2
ST_BAD_PRIORITY = 0x4
ST_BAD_REQUEST = 0x8
ST_LEN_CLAMPED = 0x10
ST_SCAN_ABORTED = 0x20
STATUS_WORDS = 4

PART = 4096
RES_HOST, RES_HBM = 1, 2
PAD_INACTIVE, PAD_HEAD, PAD_TAIL = 0, 1, 2
MAX_COLUMNS = 16
MAX_SHARDS = 16
IPC_HANDLE_BYTES = 64
MAILBOX_BYTES = 2 * MAX_SHARDS * 16
SEARCH_SCALE = 1

DT_F32, DT_F64, DT_I64, DT_F16 = range(4)
FILL_U32, FILL_F32_NORMAL, FILL_F32_UNIFORM, FILL_F32_LOGNORMAL, FILL_I32_RANGE, FILL_U8, FILL_U01_F64 = range(7)


class GearError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference raises RuntimeError
    for argument/state errors, include/gear_errors.h:3-8)."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[gear_b200 status {code}] {msg}")
        self.code = code


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        if os.environ.get("GEAR_B200_AUTOBUILD", "1") != "0":
            from . import build as _b
            _b.build()
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m gear_b200.build` "
                "(gear_b200 has no fallback path)")
    return C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)


lib = _load()

vp, i32, i64, u64, f64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_double
pi64 = C.POINTER(C.c_int64)
pi32 = C.POINTER(C.c_int32)

_SIGS = {
    "gearb_last_error": (C.c_char_p, []),
    "gearb_version": (C.c_int, []),
    "gearb_init": (C.c_int, [C.c_int]),
    "gearb_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "gearb_table_create": (C.c_int, [pi64, C.c_int, i64, i64, C.c_int, C.c_int, C.c_int, C.POINTER(vp)]),
    "gearb_table_connect": (C.c_int, [vp, pi64]),
    "gearb_table_destroy": (C.c_int, [vp]),
    "gearb_table_layout": (C.c_int, [vp, pi64, pi64, pi64]),
    "gearb_table_host_ptr": (vp, [vp]),
    "gearb_table_device_ptr": (vp, [vp]),
    "gearb_table_upload": (C.c_int, [vp, vp]),
    "gearb_table_upload_range": (C.c_int, [vp, i64, i64, vp]),
    "gearb_table_write": (C.c_int, [vp, i64, vp, i64, vp]),
    "gearb_table_read": (C.c_int, [vp, i64, vp, i64]),
    "gearb_handler_create": (C.c_int, [vp, i64, i64, i64, i64, i64, C.POINTER(vp)]),
    "gearb_handler_destroy": (C.c_int, [vp]),
    "gearb_handler_set": (C.c_int, [vp, pi64, C.c_int, pi32, pi64, pi32]),
    "gearb_handler_sub": (C.c_int, [vp, vp, vp, vp, i64, C.c_int, vp, vp, vp, pi64]),
    "gearb_handler_subcopy": (C.c_int, [vp, vp, vp, vp, i64, C.c_int, vp, vp, vp]),
    "gearb_handler_gather": (C.c_int, [vp, pi32, C.c_int, vp, vp, vp, i64, C.POINTER(vp), C.c_int, vp, vp]),
    "gearb_handler_view": (C.c_int, [vp, i64, C.c_int, C.POINTER(vp), pi64]),
    "gearb_vcopy": (C.c_int, [vp, vp, vp, vp, vp, i64, i64, vp]),
    "gearb_copy": (C.c_int, [vp, vp, vp, vp, i64, i64, vp]),
    "gearb_indexset_create": (C.c_int, [i64, i64, i64, C.c_int, C.c_int, C.c_int, C.POINTER(vp)]),
    "gearb_indexset_destroy": (C.c_int, [vp]),
    "gearb_indexset_timesteps": (vp, [vp]),
    "gearb_indexset_weights": (vp, [vp]),
    "gearb_scan_scratch_bytes": (i64, [i64]),
    "gearb_scan": (C.c_int, [vp, i64, vp, vp, vp, i64, vp, vp]),
    "gearb_scan_static": (C.c_int, [vp, i64, vp, vp, vp, vp]),
    "gearb_scan_static_max_n": (i64, []),
    "gearb_search": (C.c_int, [vp, vp, i64, vp, i64, C.c_int, vp, vp, vp]),
    "gearb_sample_uniform": (C.c_int, [i64, vp, i64, vp, vp]),
    "gearb_decode": (C.c_int, [vp, i64, i64, vp, i64, vp, vp, vp, vp]),
    "gearb_sampler_create": (C.c_int, [i64, C.POINTER(vp)]),
    "gearb_sampler_destroy": (C.c_int, [vp]),
    "gearb_sampler_scan": (C.c_int, [vp, vp, vp]),
    "gearb_sampler_scan_totals": (C.c_int, [vp, vp, vp]),
    "gearb_sampler_scan_alternate": (C.c_int, [vp, vp, vp]),
    "gearb_sampler_scan_partitions": (C.c_int, [vp, vp, C.c_int, vp]),
    "gearb_sampler_scan_level1": (C.c_int, [vp, vp]),
    "gearb_sampler_update": (C.c_int, [vp, vp, vp, vp, i64, vp]),
    "gearb_sampler_search": (C.c_int, [vp, vp, i64, C.c_int, vp, vp]),
    "gearb_sampler_scan_search": (C.c_int, [vp, vp, vp, i64, C.c_int, vp, vp]),
    "gearb_sampler_sample_gather": (C.c_int, [vp, vp, vp, i64, C.c_int, vp, i64, pi32, C.c_int, C.POINTER(vp),
                                              C.c_int, vp, vp, vp, vp, vp]),
    "gearb_sampler_sample_gather_affine": (C.c_int, [vp, vp, vp, i64, f64, f64, vp, i64, pi32, C.c_int,
                                                     C.POINTER(vp), C.c_int, vp, vp, vp, vp, i64, C.c_int, i64,
                                                     pi64, vp]),
    "gearb_sampler_select_slot": (C.c_int, [vp, C.c_int]),
    "gearb_sampler_block_totals": (C.c_int, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(C.c_int)]),
    "gearb_sampler_level1_buffers": (C.c_int, [vp, C.POINTER(vp), C.POINTER(vp)]),
    "gearb_sampler_clear_status": (C.c_int, [vp, vp]),
    "gearb_mailbox_bytes": (i64, [i64]),
    "gearb_mailbox_l1_offset": (i64, [i64, u64, C.c_int]),
    "gearb_mailbox_blk_offset": (i64, [i64, u64, C.c_int]),
    "gearb_sampler_publish": (C.c_int, [vp, C.c_int, C.c_int, C.POINTER(vp), u64, C.c_int, vp]),
    "gearb_sampler_scan_totals_publish": (C.c_int, [vp, vp, C.c_int, C.c_int, C.POINTER(vp), u64, vp]),
    "gearb_sampler_pull_ex": (C.c_int, [vp, vp, vp, vp]),
    "gearb_ipc_export": (C.c_int, [vp, vp]),
    "gearb_ipc_open": (C.c_int, [vp, C.POINTER(vp)]),
    "gearb_ipc_close": (C.c_int, [vp]),
    "gearb_sampler_pull": (C.c_int, [vp, vp, C.c_int, C.c_int, vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), vp, i64,
                                     pi32, C.c_int, C.POINTER(vp), C.c_int, C.c_int, vp, vp, vp, vp]),
    "gearb_device_alloc": (C.c_int, [i64, C.POINTER(vp)]),
    "gearb_device_free": (C.c_int, [vp]),
    "gearb_sampler_publish_total": (C.c_int, [vp, C.c_int, C.c_int, C.POINTER(vp), u64, vp]),
    "gearb_sampler_pull_mailbox": (C.c_int, [vp, vp, C.c_int, C.c_int, vp, u64, C.POINTER(vp), C.POINTER(vp),
                                             C.POINTER(vp), vp, i64, pi32, C.c_int, C.POINTER(vp), C.c_int, C.c_int,
                                             vp, vp, vp, vp]),
    "gearb_sampler_buffers": (C.c_int, [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]),
    "gearb_sampler_result": (C.c_int, [vp, vp, C.POINTER(f64), pi32]),
    "gearb_comm_unique_id": (C.c_int, [C.c_char_p]),
    "gearb_comm_create": (C.c_int, [C.c_int, C.c_int, C.c_char_p, C.POINTER(vp)]),
    "gearb_comm_destroy": (C.c_int, [vp]),
    "gearb_comm_info": (C.c_int, [vp, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "gearb_comm_send": (C.c_int, [vp, vp, i64, C.c_int, vp]),
    "gearb_comm_recv": (C.c_int, [vp, vp, i64, C.c_int, vp]),
    "gearb_comm_allreduce_sum": (C.c_int, [vp, vp, i64, C.c_int, vp]),
    "gearb_comm_allgather": (C.c_int, [vp, vp, vp, i64, vp]),
    "gearb_comm_alltoallv": (C.c_int, [vp, C.c_int, C.POINTER(vp), pi64, pi64, C.POINTER(vp), pi64, pi64, vp]),
    "gearb_ingest_server_create": (C.c_int, [C.c_int, C.c_int, i64, i64, C.POINTER(vp)]),
    "gearb_ingest_server_destroy": (C.c_int, [vp]),
    "gearb_ingest_server_scan": (C.c_int, [vp, vp, vp, vp, i64, pi64, vp, vp, vp, i64, pi64]),
    "gearb_ingest_server_update": (C.c_int, [vp, vp, vp, vp, i64]),
    "gearb_ingest_server_callback": (C.c_int, [vp, vp, i64]),
    "gearb_ingest_server_weights": (vp, [vp]),
    "gearb_ingest_server_timesteps": (vp, [vp]),
    "gearb_ingest_server_free_count": (i64, [vp]),
    "gearb_ingest_server_get_state": (i64, [vp, vp, i64]),
    "gearb_ingest_server_set_state": (C.c_int, [vp, vp, i64]),
    "gearb_ingest_client_create": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(vp)]),
    "gearb_ingest_client_destroy": (C.c_int, [vp]),
    "gearb_ingest_client_acquire": (C.c_int, [vp, i64, pi64]),
    "gearb_ingest_client_wait": (C.c_int, [vp, i64]),
    "gearb_ingest_client_release": (C.c_int, [vp]),
    "gearb_ingest_client_step": (i64, [vp]),
    "gearb_ingest_client_writeback": (i64, [vp, C.c_int, C.c_int, f64]),
    "gearb_ingest_client_status": (C.c_int, [vp, pi64, C.POINTER(f64)]),
    "gearb_fill": (C.c_int, [vp, i64, C.c_int, u64, u64, f64, f64, vp]),
}

# Entry points added after the first slice are optional at bind time so that the
# symbol test can report exactly which declared names are missing.
for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.gearb_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != OK:
        raise GearError(code, last_error())


def call(name: str, *args):
    check(getattr(lib, name)(*args))


class PullArgs(C.Structure):
    """gearb_pull_args of include/gear_b200.h."""
    _fields_ = [("world", C.c_int), ("self", C.c_int), ("totals", vp), ("mailbox", vp), ("epoch", u64),
                ("cdf", C.POINTER(vp)), ("prio", C.POINTER(vp)), ("blk", C.POINTER(vp)), ("l1", C.POINTER(vp)),
                ("table", C.POINTER(vp)), ("variates", vp), ("b", i64), ("variate_stride", i64),
                ("columns", pi32), ("ncols", C.c_int), ("dst", C.POINTER(vp)), ("zero_fill", C.c_int),
                ("ring", C.c_int), ("out_flat", vp), ("out_idx", vp), ("out_ts", vp)]


def declared_symbols() -> list[str]:
    """Names declared in include/gear_b200.h (parsed from the header text)."""
    import re
    text = (PKG.parent / "include" / "gear_b200.h").read_text()
    return sorted(set(re.findall(r"\b(gearb_[a-z0-9_]+)\s*\(", text)))
