"""ctypes binding of ``libcoresets_b200.so`` (declared in ``include/coresets_b200.h``).

This module replaces the reference's JIT loader (src/coresets/cuda/extension.py:15-85).  The
library is built in-tree with nvcc (``python -m coresets_b200.build``); when it is missing and
nvcc is on the machine it is compiled on first use, like the reference does, and when it can
be neither found nor built every entry point raises ``RuntimeError`` -- there is no CPU or
PyTorch fallback behind this boundary.
"""
from __future__ import annotations

import ctypes
from typing import Optional

from . import build as _build

CS_ABI_VERSION = 9
SELECT_SCRATCH_BYTES = 8192
F_ELEMENT_ORDER = 1
F_PDL = 2
F_X_HALF = 4
F_TEST_STALL_PIPE = 0x100
CS_CTL_BYTES = 256
CELL_TILE = 256
CELLS_META_BYTES = 128

MODE_PRUNE = 0
MODE_DENSE = 1
MODE_DENSE_LDG = 3
MODE_PRUNE_INLINE = 2
RULE_NONE = 0
RULE_SIM_SINGLE = 1
RULE_SIM_SHARDED = 2
RULE_STOP_NONPOS = 3
XCHG_GATHER = 0
XCHG_PEER = 1
MAX_PEERS = 8

EXPORTS = (
    "cs_version", "cs_error_string", "cs_last_cuda_error", "cs_device_check", "cs_init_state",
    "cs_reset_ctl", "cs_force_pick", "cs_commit_bound", "cs_fps_step", "cs_sim_begin",
    "cs_sim_final_check", "cs_xchg_window_words", "cs_xchg_wait", "cs_scan_argmax", "cs_fps_step_lanes", "cs_fps_step_noalloc",
    "cs_select_kth_largest", "cs_pool_argmax", "cs_cells_build", "cs_cells_select", "cs_fps_step_cells", "cs_force_pick_list", "cs_pool_pick",
)


class CsState(ctypes.Structure):
    """``cs_state`` of include/coresets_b200.h."""
    _fields_ = [
        ("X", ctypes.c_void_p),
        ("norms", ctypes.c_void_p),
        ("h", ctypes.c_void_p),
        ("voronoi", ctypes.c_void_p),
        ("N_local", ctypes.c_int64),
        ("shard_offset", ctypes.c_int64),
        ("D", ctypes.c_int32),
        ("world_size", ctypes.c_int32),
        ("X_sel", ctypes.c_void_p),
        ("norms_sel", ctypes.c_void_p),
        ("dSL_quarter", ctypes.c_void_p),
        ("cap", ctypes.c_int64),
        ("selected", ctypes.c_void_p),
        ("eps", ctypes.c_void_p),
        ("ctl", ctypes.c_void_p),
        ("pack_local", ctypes.c_void_p),
        ("pack_all", ctypes.c_void_p),
        ("rank", ctypes.c_int32),
        ("xchg", ctypes.c_int32),
        ("peer_win", ctypes.c_void_p * MAX_PEERS),
        ("xchg_timeout_ms", ctypes.c_int32),
        ("flags", ctypes.c_int32),
    ]


class CsCells(ctypes.Structure):
    """``cs_cells`` of include/coresets_b200.h."""
    _fields_ = [
        ("perm", ctypes.c_void_p),
        ("hp", ctypes.c_void_p),
        ("vp", ctypes.c_void_p),
        ("cell0", ctypes.c_void_p),
        ("slots", ctypes.c_int64),
        ("seg_start", ctypes.c_void_p),
        ("seg_count", ctypes.c_void_p),
        ("seg_key", ctypes.c_void_p),
        ("seg_h0", ctypes.c_void_p),
        ("cursor", ctypes.c_void_p),
        ("work_cell", ctypes.c_void_p),
        ("work_cum", ctypes.c_void_p),
        ("meta", ctypes.c_void_p),
        ("queue", ctypes.c_void_p),
        ("row_norm_max", ctypes.c_float),
        ("q_cap", ctypes.c_int32),
    ]


class CellsMetaView(ctypes.Structure):
    """``cs_cells_meta_view`` of include/coresets_b200.h."""
    _fields_ = [
        ("n_cells", ctypes.c_int32),
        ("n_work", ctypes.c_int32),
        ("n_chunks", ctypes.c_int32),
        ("total_slots", ctypes.c_int32),
        ("visited_slots", ctypes.c_uint64),
        ("picks", ctypes.c_uint64),
        ("q_count", ctypes.c_uint32),
        ("q_inline", ctypes.c_uint32),
        ("reserved", ctypes.c_uint8 * (CELLS_META_BYTES - 40)),
    ]


assert ctypes.sizeof(CellsMetaView) == CELLS_META_BYTES


def decode_key(key: int):
    """``(value, global index)`` of a 64-bit arg-max key (include/coresets_b200.h, cs_pool_argmax);
    ``(-inf, -1)`` for key 0."""
    import struct
    key &= 0xFFFFFFFFFFFFFFFF
    if key == 0:
        return float("-inf"), -1
    o = key >> 32
    b = (o & 0x7FFFFFFF) if o & 0x80000000 else (~o) & 0xFFFFFFFF
    return struct.unpack("<f", struct.pack("<I", b))[0], 0xFFFFFFFF - (key & 0xFFFFFFFF)


class SelectResult(ctypes.Structure):
    """``cs_select_result`` of include/coresets_b200.h."""
    _fields_ = [("value", ctypes.c_float), ("valid", ctypes.c_int32), ("n_alive", ctypes.c_int64)]


class CtlView(ctypes.Structure):
    """``cs_ctl_view`` of include/coresets_b200.h."""
    _fields_ = [
        ("key", ctypes.c_uint64 * 2),
        ("n_sel", ctypes.c_int32),
        ("ticket", ctypes.c_uint32),
        ("status", ctypes.c_int32),
        ("viable", ctypes.c_int32),
        ("sep", ctypes.c_float),
        ("steps", ctypes.c_int32),
        ("live_rows", ctypes.c_uint64),
        ("last_val", ctypes.c_float),
        ("last_idx", ctypes.c_int32),
        ("xseq", ctypes.c_uint32),
        ("halt", ctypes.c_int32),
        ("reserved", ctypes.c_uint8 * (CS_CTL_BYTES - 64)),
    ]


assert ctypes.sizeof(CtlView) == CS_CTL_BYTES


class NativeError(RuntimeError):
    pass


class Native:
    """Thin, typed wrapper over the C entry points.  Methods take a ``CsState`` (or an array of
    them) and a raw ``cudaStream_t`` value; a non-zero return code raises ``NativeError``."""

    def __init__(self, path: Optional[str] = None):
        lib_path = path or str(_build.LIB)
        try:
            self.lib = ctypes.CDLL(lib_path)
        except OSError as e:
            raise NativeError(
                f"cannot load {lib_path}: {e}. Build it with `python -m coresets_b200.build`."
            ) from e
        L = self.lib
        missing = [n for n in EXPORTS if not hasattr(L, n)]
        if missing:
            raise NativeError(f"{lib_path} lacks symbols {missing}; rebuild it")
        L.cs_version.restype = ctypes.c_int
        L.cs_error_string.restype = ctypes.c_char_p
        L.cs_error_string.argtypes = [ctypes.c_int]
        L.cs_last_cuda_error.restype = ctypes.c_char_p
        L.cs_device_check.restype = ctypes.c_int
        sp = ctypes.POINTER(CsState)
        vp = ctypes.c_void_p
        for name, args in (
            ("cs_init_state", [sp, vp]),
            ("cs_reset_ctl", [sp, ctypes.c_int32, vp]),
            ("cs_force_pick", [sp, ctypes.c_int64, ctypes.c_float, vp]),
            ("cs_force_pick_list", [sp, vp, vp, ctypes.c_float, vp]),
            ("cs_pool_pick", [sp, vp, vp, vp]),
            ("cs_commit_bound", [sp, ctypes.c_uint32, vp]),
            ("cs_fps_step", [sp, ctypes.c_uint32, vp]),
            ("cs_sim_begin", [sp, ctypes.c_float, vp]),
            ("cs_sim_final_check", [sp, vp]),
            ("cs_scan_argmax", [sp, vp]),
            ("cs_select_kth_largest", [vp, ctypes.c_int64, ctypes.c_int64, vp, vp]),
            ("cs_pool_argmax", [vp, vp, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, vp, vp]),
            ("cs_xchg_wait", [sp, vp]),
            ("cs_fps_step_lanes", [sp, ctypes.c_int32, ctypes.c_uint32, vp]),
            ("cs_cells_build", [sp, ctypes.POINTER(CsCells), vp]),
            ("cs_cells_select", [sp, ctypes.POINTER(CsCells), vp]),
            ("cs_fps_step_cells", [sp, ctypes.POINTER(CsCells), vp]),
        ):
            fn = getattr(L, name)
            fn.restype = ctypes.c_int
            fn.argtypes = args
        L.cs_xchg_window_words.restype = ctypes.c_int64
        L.cs_xchg_window_words.argtypes = [ctypes.c_int32, ctypes.c_int32]
        L.cs_fps_step_noalloc.restype = ctypes.c_int
        L.cs_fps_step_noalloc.argtypes = [vp, vp, vp, vp, ctypes.c_int64, ctypes.c_int32, ctypes.c_int64, vp,
                                          ctypes.c_float, vp, ctypes.c_int32, ctypes.c_uint32, vp, vp, vp]
        if L.cs_version() != CS_ABI_VERSION:
            raise NativeError(f"{lib_path}: ABI {L.cs_version()} != expected {CS_ABI_VERSION}; rebuild it")

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            msg = self.lib.cs_error_string(rc).decode()
            if rc == -4:
                msg += ": " + self.lib.cs_last_cuda_error().decode()
            raise NativeError(f"{what} failed ({rc}): {msg}")

    def device_check(self) -> int:
        sms = self.lib.cs_device_check()
        if sms < 0:
            self._check(sms, "cs_device_check")
        return sms

    def init_state(self, s: CsState, stream: int) -> None:
        self._check(self.lib.cs_init_state(ctypes.byref(s), stream), "cs_init_state")

    def reset_ctl(self, s: CsState, n_sel: int, stream: int) -> None:
        self._check(self.lib.cs_reset_ctl(ctypes.byref(s), n_sel, stream), "cs_reset_ctl")

    def force_pick(self, s: CsState, global_idx: int, val: float, stream: int) -> None:
        self._check(self.lib.cs_force_pick(ctypes.byref(s), global_idx, val, stream), "cs_force_pick")

    def force_pick_list(self, s: CsState, list_ptr: int, vals_ptr, val: float, stream: int) -> None:
        self._check(self.lib.cs_force_pick_list(ctypes.byref(s), list_ptr, vals_ptr, val, stream), "cs_force_pick_list")

    def pool_pick(self, s: CsState, pool_ptr: int, n_pool_ptr: int, stream: int) -> None:
        self._check(self.lib.cs_pool_pick(ctypes.byref(s), pool_ptr, n_pool_ptr, stream), "cs_pool_pick")

    def commit_bound(self, s: CsState, rules: int, stream: int) -> None:
        self._check(self.lib.cs_commit_bound(ctypes.byref(s), rules, stream), "cs_commit_bound")

    def fps_step(self, s: CsState, mode: int, stream: int) -> None:
        self._check(self.lib.cs_fps_step(ctypes.byref(s), mode, stream), "cs_fps_step")

    def sim_begin(self, s: CsState, sep: float, stream: int) -> None:
        self._check(self.lib.cs_sim_begin(ctypes.byref(s), sep, stream), "cs_sim_begin")

    def sim_final_check(self, s: CsState, stream: int) -> None:
        self._check(self.lib.cs_sim_final_check(ctypes.byref(s), stream), "cs_sim_final_check")

    def xchg_window_words(self, world_size: int, D: int) -> int:
        n = int(self.lib.cs_xchg_window_words(world_size, D))
        if n < 0:
            self._check(n, "cs_xchg_window_words")
        return n

    def xchg_wait(self, s: CsState, stream: int) -> None:
        self._check(self.lib.cs_xchg_wait(ctypes.byref(s), stream), "cs_xchg_wait")

    def pool_argmax(self, h: int, pool: int, n_pool: int, shard_offset: int, n_local: int, out_key: int,
                    stream: int) -> None:
        self._check(self.lib.cs_pool_argmax(h, pool, n_pool, shard_offset, n_local, out_key, stream), "cs_pool_argmax")

    def select_kth_largest(self, h: int, n: int, k: int, scratch: int, stream: int) -> None:
        self._check(self.lib.cs_select_kth_largest(h, n, k, scratch, stream), "cs_select_kth_largest")

    def scan_argmax(self, s: CsState, stream: int) -> None:
        self._check(self.lib.cs_scan_argmax(ctypes.byref(s), stream), "cs_scan_argmax")

    def fps_step_noalloc(self, X: int, norms: int, h: int, voronoi: int, N_local: int, D: int,
                         shard_offset: int, centre: int, norm_new: float, dSL: Optional[int], sel_pos: int,
                         mode: int, out_key: int, out_live_rows: Optional[int], stream: int) -> None:
        """``cs_fps_step_noalloc``: the fused step for hosts that may not allocate device memory;
        every pointer argument is a raw device address.  Raises on a non-zero return code."""
        self._check(self.lib.cs_fps_step_noalloc(X, norms, h, voronoi, N_local, D, shard_offset, centre,
                                                 norm_new, dSL, sel_pos, mode, out_key, out_live_rows, stream),
                    "cs_fps_step_noalloc")

    def cells_build(self, s: CsState, c: CsCells, stream: int) -> None:
        self._check(self.lib.cs_cells_build(ctypes.byref(s), ctypes.byref(c), stream), "cs_cells_build")

    def cells_select(self, s: CsState, c: CsCells, stream: int) -> None:
        self._check(self.lib.cs_cells_select(ctypes.byref(s), ctypes.byref(c), stream), "cs_cells_select")

    def fps_step_cells(self, s: CsState, c: CsCells, stream: int) -> None:
        self._check(self.lib.cs_fps_step_cells(ctypes.byref(s), ctypes.byref(c), stream), "cs_fps_step_cells")

    def fps_step_lanes(self, lanes, n_lanes: int, mode: int, stream: int) -> None:
        self._check(self.lib.cs_fps_step_lanes(lanes, n_lanes, mode, stream), "cs_fps_step_lanes")


_native: Optional[Native] = None


def ensure_compiled() -> None:
    """Load the native library, compiling it first if it is absent and nvcc is available.
    Mirrors ``ensure_compiled`` of the reference (src/coresets/cuda/extension.py:15-74)."""
    global _native
    if _native is not None:
        return
    if not _build.LIB.is_file():
        try:
            print("Compiling coresets_b200 CUDA kernels for sm_100a (first use)...")
            _build.build()
        except Exception as e:  # no nvcc, or the compile failed: fail loudly
            raise NativeError(
                f"{_build.LIB} is missing and could not be built ({e}). "
                "Run `python -m coresets_b200.build` on a machine with nvcc (CUDA >= 12.8)."
            ) from e
    _native = Native()


def get_native() -> Native:
    ensure_compiled()
    assert _native is not None
    return _native


def set_native_for_tests(obj) -> None:
    """Install a stand-in for the native library.  Only the CPU test-suite calls this (with an
    implementation backed by the oracle); it exists because multi-rank host logic has to be
    testable on machines without a GPU."""
    global _native
    _native = obj
