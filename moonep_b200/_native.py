"""ctypes binding of ``libmoonep_b200.so`` (plain ``extern "C"`` ABI).

The structs mirror ``csrc/mep_types.h`` and the per-kernel argument structs field by
field.  Every native function returns 0 on success; on failure ``check`` raises
``MoonEPNativeError`` with the library's thread-local message.

Takes the place of the reference's pybind11 module ``moonep._C`` (csrc/bindings.cu:13-53), which
exposes only the symmetric-memory calls; here the same library also carries every kernel
launcher, and it loads without a CUDA driver (the driver API is resolved at first use).
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch  # noqa: F401  (loads the CUDA runtime the library links against)

MAX_RANKS = 128
MAX_VRANKS = 8
BAR_ROWS = 4

_LIB = None


class MoonEPNativeError(RuntimeError):
    pass


class MepStatus(C.Structure):
    _fields_ = [("code", C.c_int32), ("kernel", C.c_int32), ("site", C.c_int32), ("rank", C.c_int32),
                ("peer", C.c_int32), ("observed", C.c_uint32), ("expected", C.c_uint32), ("reserved", C.c_int32)]


class MepRankCtx(C.Structure):
    _fields_ = (
        [(n, C.c_int32) for n in ("rank", "R", "S", "H", "K", "E", "epn", "N", "NvS", "token_padding",
                                  "vblock_entries", "num_vblocks", "num_sms", "checked")]
        + [("heap_base", C.c_void_p), ("chunk_stride", C.c_int64)]
        + [(n, C.c_int64) for n in ("off_hidden", "off_weights", "off_tpe", "off_bar", "off_dupcnt",
                                    "off_dupgroups", "off_duploffs", "off_ready",
                                    "dup_group_cap", "dup_loff_cap")]
        + [(n, C.c_void_p) for n in ("grid_bar", "epoch", "hist", "count", "tpe_prefix", "remaining", "alloc",
                                     "alloc_cumsum", "expert_off", "etc_all", "stats_all", "send_cnt", "status")]
        + [("wait_budget_ns", C.c_uint64), ("trace", C.c_void_p), ("trace_cap", C.c_int64), ("mc_base", C.c_void_p), ("vb_flags", C.c_void_p)]
        + [("status_host", C.c_void_p), ("off_rowsrc", C.c_int64), ("tile_done", C.c_void_p), ("flag_epoch", C.c_void_p),
           ("ntiles", C.c_int32), ("reserved1", C.c_int32), ("counters", C.c_void_p),
           ("off_slotflag", C.c_int64), ("slot_done", C.c_void_p), ("pf_epoch", C.c_void_p)]
    )

COUNTER_SLOTS = 64
COUNTER_NAMES = {0: "dispatches", 1: "rows_sent", 2: "rows_sent_remote", 3: "padding_rows_cleared", 4: "barrier_wait_ns",
                 5: "barriers", 6: "combines", 7: "rows_pulled", 8: "duplicate_rows_expanded"}
COUNTER_PEER_BASE = 16


class PlanArgs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("topk", "tpe", "dst", "cu_seqlens", "experts_to_copy",
                                          "zero_fill", "remote_stats")] + [("epoch", C.c_uint32), ("pad", C.c_int32)]


class DispatchArgs(C.Structure):
    _fields_ = [("hidden", C.c_void_p), ("weights", C.c_void_p), ("dst", C.c_void_p), ("zero_fill", C.c_void_p),
                ("fresh", C.c_int32), ("entry_barrier", C.c_int32), ("srcinfo_off", C.c_int64),
                ("send_list", C.c_void_p), ("send_meta", C.c_void_p)]


class SendOrderArgs(C.Structure):
    _fields_ = [("dst", C.c_void_p), ("cu_seqlens", C.c_void_p), ("send_list", C.c_void_p), ("send_meta", C.c_void_p),
                ("hist", C.c_void_p), ("bucket", C.c_void_p)]


class PushReduceArgs(C.Structure):
    _fields_ = [("out", C.c_void_p), ("out_weights", C.c_void_p), ("push_off", C.c_int64), ("pushw_off", C.c_int64)]


class DupFinalizeArgs(C.Structure):
    _fields_ = [("dup_groups", C.c_void_p), ("dup_loffs", C.c_void_p), ("dup_counts", C.c_void_p)]


class DupArgs(C.Structure):
    _fields_ = [("buf", C.c_void_p), ("dup_groups", C.c_void_p), ("dup_loffs", C.c_void_p), ("dup_counts", C.c_void_p)]


class CombineArgs(C.Structure):
    _fields_ = [("dst", C.c_void_p), ("out", C.c_void_p), ("out_weights", C.c_void_p), ("entry_barrier", C.c_int32)]


class CopyTensor(C.Structure):
    _fields_ = [("local", C.c_void_p), ("pool", C.c_void_p), ("expert_bytes", C.c_int64), ("rank_stride", C.c_int64)]


class PrefetchArgs(C.Structure):
    _fields_ = [("etc", C.c_void_p), ("ntensors", C.c_int32), ("pad", C.c_int32), ("t", CopyTensor * 6)]


class ReduceTensor(C.Structure):
    _fields_ = [("local", C.c_void_p), ("pool", C.c_void_p), ("expert_elems", C.c_int64), ("rank_stride", C.c_int64)]


class GradReduceArgs(C.Structure):
    _fields_ = [("etc", C.c_void_p), ("ntensors", C.c_int32), ("flags", C.c_int32), ("t", ReduceTensor * 3)]


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "_lib" / "libmoonep_b200.so"


def load(build_if_missing: bool = True):
    """Load (building first if the library is missing or older than its sources and nvcc exists)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    from . import _build
    p = lib_path()
    if build_if_missing and _build.nvcc_path() is not None and os.environ.get("MOONEP_NO_AUTOBUILD") != "1":
        if _build.is_stale():
            _build.build()
    if not p.exists():
        raise MoonEPNativeError(
            f"{p} is missing: build it with `python -m moonep_b200._build` (needs nvcc); "
            "the CUDA kernels are the only implementation of the device ops")
    lib = C.CDLL(str(p), mode=C.RTLD_GLOBAL)
    lib.mep_last_error.restype = C.c_char_p
    lib.mep_launch_count.restype = C.c_longlong
    # size_t / pointer arguments must not be squeezed through the default C int conversion
    vp, sz, i32 = C.c_void_p, C.c_size_t, C.c_int
    lib.mep_vmm_granularity.argtypes = [i32, i32, C.POINTER(sz)]
    lib.mep_multicast_granularity.argtypes = [i32, i32, i32, sz, C.POINTER(sz)]
    lib.mep_chunk_create.argtypes = [i32, sz, i32, C.POINTER(vp), C.POINTER(C.c_ubyte)]
    lib.mep_chunk_release.argtypes = [vp]
    lib.mep_map_all.argtypes = [i32, i32, i32, vp, C.POINTER(C.c_ubyte), C.POINTER(vp), C.POINTER(C.c_ulonglong)]
    lib.mep_unmap_all.argtypes = [vp]
    lib.mep_map_remote_one.argtypes = [i32, i32, sz, C.POINTER(C.c_ubyte), C.POINTER(vp), C.POINTER(C.c_ulonglong)]
    lib.mep_alias_map.argtypes = [i32, sz, vp, C.POINTER(vp), C.POINTER(C.c_ulonglong)]
    lib.mep_alias_unmap.argtypes = [vp]
    lib.mep_mc_create.argtypes = [i32, i32, sz, i32, C.POINTER(vp), C.POINTER(C.c_ubyte)]
    lib.mep_mc_import.argtypes = [i32, sz, i32, C.POINTER(C.c_ubyte), C.POINTER(vp)]
    lib.mep_mc_add_device.argtypes = [vp]
    lib.mep_mc_bind_map.argtypes = [vp, vp, C.POINTER(C.c_ulonglong)]
    lib.mep_mc_destroy.argtypes = [vp]
    _LIB = lib
    return lib


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = load().mep_last_error().decode(errors="replace")
        raise MoonEPNativeError(f"{what}: {msg}" if what else msg)


def ptr(t) -> int | None:
    """Device pointer of a tensor (None stays None)."""
    return None if t is None else t.data_ptr()


def ctx_array(ctx_ptrs):
    arr = (C.c_void_p * len(ctx_ptrs))(*ctx_ptrs)
    return arr


def cur_stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)
