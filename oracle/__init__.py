"""ctypes front end of the CPU restatement in ``fps_oracle.c``.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline leg of ``bench.py``; the shipped package never imports it.  Arrays are numpy,
C-contiguous; ``voronoi`` is int64 as in the reference (src/coresets/cuda/fps.py:43).
"""
from __future__ import annotations

import contextlib
import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libfps_oracle.so"
_lib = None

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
_i64 = ctypes.c_int64
_int = ctypes.c_int


def build(force: bool = False) -> Path:
    """Compile ``fps_oracle.c`` with the Makefile next to it (gcc)."""
    src = _HERE / "fps_oracle.c"
    if force or not _LIB_PATH.is_file() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "libfps_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        L.oracle_warp_dot.restype = ctypes.c_float
        L.oracle_warp_dot.argtypes = [_f32p, _f32p, _int]
        L.oracle_fps_update.restype = None
        L.oracle_fps_update.argtypes = [_f32p, _f32p, _f32p, ctypes.c_float, _f32p, _i64p, _i64, _i64, _int]
        L.oracle_voronoi_update.restype = _i64
        L.oracle_voronoi_update.argtypes = [_f32p, _f32p, _f32p, ctypes.c_float, _f32p, _f32p, _i64p,
                                            _i64, _i64, _int]
        L.oracle_argmax.restype = None
        L.oracle_argmax.argtypes = [_f32p, _i64, ctypes.POINTER(ctypes.c_float),
                                    ctypes.POINTER(ctypes.c_int32)]
        L.oracle_dsl_quarter.restype = None
        L.oracle_dsl_quarter.argtypes = [_f32p, _f32p, _f32p, _i64, _int]
        L.oracle_fps_cuda.restype = _int
        L.oracle_fps_cuda.argtypes = [_f32p, _f32p, _i64, _int, _i64, _i64p, _i64, _i64p, _f32p, _f32p, _i64p]
        L.oracle_fps_sharded.restype = _int
        L.oracle_fps_sharded.argtypes = [_f32p, _f32p, _int, _i64, _int, _i64p, _i64, _i64p, _f32p, _f32p, _i64p]
        L.oracle_simulate.restype = _int
        L.oracle_simulate.argtypes = [_f32p, _f32p, _i64, _int, _f32p, _i64p, _f32p, _f32p, _i64,
                                      ctypes.c_double, _i64, ctypes.POINTER(_i64),
                                      ctypes.POINTER(ctypes.c_float)]
        L.oracle_simulate_sharded.restype = _int
        L.oracle_simulate_sharded.argtypes = [_f32p, _f32p, _int, _int, _i64p, _f32p, _i64p, _f32p, _f32p,
                                              _i64, ctypes.c_double, _i64, ctypes.POINTER(_i64),
                                              ctypes.POINTER(ctypes.c_float)]
        L.oracle_set_element_order.restype = None
        L.oracle_set_element_order.argtypes = [_int]
        _lib = L
    return _lib


@contextlib.contextmanager
def element_order(on: bool = True):
    """Within the block every dot is summed element-wise (the reference's order for float16 /
    float64 inputs, _shared.cuh:55-58); the caller passes the rows converted to float32."""
    lib().oracle_set_element_order(1 if on else 0)
    try:
        yield
    finally:
        lib().oracle_set_element_order(0)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def row_norms_f32(X: np.ndarray) -> np.ndarray:
    """A float32 row-norm vector for CPU-only cases.  The reference computes norms with
    torch on the GPU (src/coresets/cuda/fps.py:34); every kernel and every oracle function
    takes norms as an INPUT, so any float32 vector works for kernel-vs-oracle parity."""
    X = _c(X, np.float32)
    return (X * X).sum(axis=1, dtype=np.float32).astype(np.float32)


def warp_dot(row, c) -> float:
    row = _c(row, np.float32); c = _c(c, np.float32)
    return float(lib().oracle_warp_dot(row, c, int(row.shape[0])))


def fps_update(X, norms, x_new, norm_new, h, v, sel_idx):
    X = _c(X, np.float32)
    lib().oracle_fps_update(X, _c(norms, np.float32), _c(x_new, np.float32), float(norm_new), h, v,
                            int(sel_idx), int(X.shape[0]), int(X.shape[1]))


def voronoi_update(X, norms, x_new, norm_new, dSL, h, v, sel_idx) -> int:
    X = _c(X, np.float32)
    return int(lib().oracle_voronoi_update(X, _c(norms, np.float32), _c(x_new, np.float32),
                                           float(norm_new), _c(dSL, np.float32), h, v, int(sel_idx),
                                           int(X.shape[0]), int(X.shape[1])))


def argmax(h):
    val = ctypes.c_float(); idx = ctypes.c_int32()
    h = _c(h, np.float32)
    lib().oracle_argmax(h, int(h.shape[0]), ctypes.byref(val), ctypes.byref(idx))
    return np.float32(val.value), int(idx.value)


def dsl_quarter(X_sel, norms_sel, n_sel):
    X_sel = _c(X_sel, np.float32)
    out = np.zeros(max(int(n_sel), 1), dtype=np.float32)
    lib().oracle_dsl_quarter(X_sel, _c(norms_sel, np.float32), out, int(n_sel), int(X_sel.shape[1]))
    return out[: int(n_sel)]


def fps_cuda(X, norms, k, seed=None):
    """Reference ``fps_cuda`` (src/coresets/cuda/fps.py:13-130).  Returns
    (selected int64[k], eps float32[k], h float32[N], voronoi int64[N])."""
    X = _c(X, np.float32); norms = _c(norms, np.float32)
    N, D = X.shape
    seed = np.array([0], dtype=np.int64) if seed is None else _c(seed, np.int64)
    sel = np.empty(k, dtype=np.int64); eps = np.empty(k, dtype=np.float32)
    h = np.empty(N, dtype=np.float32); v = np.empty(N, dtype=np.int64)
    rc = lib().oracle_fps_cuda(X, norms, N, D, int(k), seed, int(seed.shape[0]), sel, eps, h, v)
    if rc != 0:
        raise ValueError("oracle_fps_cuda: bad arguments")
    return sel, eps, h, v


def fps_sharded(X, norms, k, sizes, first=0):
    """Reference ``fps_sharded`` over W emulated ranks (src/coresets/cuda/multi/fps_sharded.py).
    ``X``/``norms`` are the concatenated global arrays; ``sizes`` the shard sizes."""
    X = _c(X, np.float32); norms = _c(norms, np.float32)
    N, D = X.shape
    sizes = _c(sizes, np.int64)
    assert int(sizes.sum()) == N
    sel = np.empty(k, dtype=np.int64); eps = np.empty(k, dtype=np.float32)
    h = np.empty(N, dtype=np.float32); v = np.empty(N, dtype=np.int64)
    rc = lib().oracle_fps_sharded(X, norms, D, int(k), int(sizes.shape[0]), sizes, int(first), sel,
                                  eps, h, v)
    if rc != 0:
        raise ValueError("oracle_fps_sharded: bad arguments")
    return sel, eps, h, v


def simulate(X, norms, h, v, X_sel_init, norms_sel_init, sep, points_left):
    """Reference ``simulate_fps_voronoi`` (kernels/simulate.cu:10-90); h, v updated in place.
    Returns (viable bool, steps_used, final sep)."""
    X = _c(X, np.float32)
    N, D = X.shape
    Xi = _c(X_sel_init, np.float32).reshape(-1, D)
    ni = _c(norms_sel_init, np.float32)
    if Xi.shape[0] == 0:
        Xi = np.zeros((1, D), np.float32); ni = np.zeros(1, np.float32); n_init = 0
    else:
        n_init = Xi.shape[0]
    steps = _i64(); sep_out = ctypes.c_float()
    rc = lib().oracle_simulate(X, _c(norms, np.float32), N, D, h, v, Xi, ni, n_init, float(sep),
                               int(points_left), ctypes.byref(steps), ctypes.byref(sep_out))
    if rc < 0:
        raise RuntimeError("oracle_simulate failed")
    return bool(rc), int(steps.value), np.float32(sep_out.value)


def simulate_sharded(X, norms, sizes, h, v, X_sel_init, norms_sel_init, sep, points_left):
    """Reference ``simulate_fps_voronoi_multi_sharded`` (kernels/multi.cu:428-528)."""
    X = _c(X, np.float32)
    N, D = X.shape
    sizes = _c(sizes, np.int64)
    Xi = _c(X_sel_init, np.float32).reshape(-1, D)
    ni = _c(norms_sel_init, np.float32)
    if Xi.shape[0] == 0:
        Xi = np.zeros((1, D), np.float32); ni = np.zeros(1, np.float32); n_init = 0
    else:
        n_init = Xi.shape[0]
    steps = _i64(); sep_out = ctypes.c_float()
    rc = lib().oracle_simulate_sharded(X, _c(norms, np.float32), D, int(sizes.shape[0]), sizes, h, v,
                                       Xi, ni, n_init, float(sep), int(points_left),
                                       ctypes.byref(steps), ctypes.byref(sep_out))
    if rc < 0:
        raise RuntimeError("oracle_simulate_sharded failed")
    return bool(rc), int(steps.value), np.float32(sep_out.value)
