"""A CPU stand-in for ``libcoresets_b200.so`` used ONLY by the CPU test-suite.

It implements the C entry points of include/coresets_b200.h on host memory, with every piece of
arithmetic delegated to the oracle, so that the host-side drivers (pick sequencing, all-gather
exchange over gloo, checkpoints, accretion control flow) can run on a machine without a GPU.
It validates host logic; kernel parity is the job of the ``-m gpu`` tests.
"""
from __future__ import annotations

import ctypes
import struct

import numpy as np

import oracle
from coresets_b200._native import CsState, CtlView, MODE_DENSE, RULE_SIM_SHARDED, RULE_SIM_SINGLE


def _view(ptr, n, dtype):
    if not ptr or n == 0:
        return np.zeros(0, dtype=dtype)
    nbytes = int(n) * np.dtype(dtype).itemsize
    buf = (ctypes.c_uint8 * nbytes).from_address(ptr)
    return np.frombuffer(buf, dtype=dtype)


def f2ord(h) -> int:
    h = np.float32(h)
    if np.isnan(h):
        return 1
    b = struct.unpack("<I", struct.pack("<f", 0.0 if h == 0 else float(h)))[0]
    return (~b) & 0xFFFFFFFF if b & 0x80000000 else b | 0x80000000


def ord2f(o: int) -> np.float32:
    b = (o & 0x7FFFFFFF) if o & 0x80000000 else (~o) & 0xFFFFFFFF
    return np.float32(struct.unpack("<f", struct.pack("<I", b))[0])


def make_key(h, gidx: int) -> int:
    return (f2ord(h) << 32) | (0xFFFFFFFF - int(gidx))


def key_val(k: int) -> np.float32:
    return ord2f(k >> 32) if k else np.float32(-np.inf)


def key_idx(k: int) -> int:
    return (0xFFFFFFFF - (k & 0xFFFFFFFF)) if k else -1


class FakeNative:
    def _ctl(self, s: CsState) -> CtlView:
        return CtlView.from_address(s.ctl)

    def _arrays(self, s: CsState):
        N, D = s.N_local, s.D
        return dict(
            X=_view(s.X, N * D, np.float32).reshape(N, D), norms=_view(s.norms, N, np.float32),
            h=_view(s.h, N, np.float32), v=_view(s.voronoi, N, np.int32),
            X_sel=_view(s.X_sel, s.cap * D, np.float32).reshape(s.cap, D),
            norms_sel=_view(s.norms_sel, s.cap, np.float32), dSL=_view(s.dSL_quarter, s.cap, np.float32),
            selected=_view(s.selected, s.cap, np.int64), eps=_view(s.eps, s.cap, np.float32),
            pack_local=_view(s.pack_local, 4 + D, np.uint32) if s.world_size > 1 else None,
            pack_all=_view(s.pack_all, s.world_size * (4 + D), np.uint32).reshape(s.world_size, 4 + D)
            if s.world_size > 1 else None,
        )

    def device_check(self) -> int:
        return 148

    def init_state(self, s, stream):
        a = self._arrays(s)
        a["h"][:] = np.inf
        a["v"][:] = 0
        ctypes.memset(s.ctl, 0, 256)

    def reset_ctl(self, s, n_sel, stream):
        ctypes.memset(s.ctl, 0, 256)
        self._ctl(s).n_sel = n_sel

    def _publish(self, s, a, k: int):
        if s.world_size <= 1:
            return
        p = a["pack_local"]
        p[:] = 0
        p[0] = k & 0xFFFFFFFF
        p[1] = k >> 32
        if k:
            l = key_idx(k) - s.shard_offset
            p[2] = a["norms"][l : l + 1].view(np.uint32)[0]
            p[4:] = a["X"][l].view(np.uint32)

    def force_pick(self, s, gidx, val, stream):
        a = self._arrays(s)
        ctl = self._ctl(s)
        l = gidx - s.shard_offset
        owner = 0 <= l < s.N_local
        k = make_key(val, gidx) if owner else 0
        ctl.key[ctl.n_sel & 1] = k
        if s.world_size <= 1 and not owner:
            ctl.status = 2
        self._publish(s, a, k)

    def _winner(self, s, a, ctl, i):
        if s.world_size <= 1:
            k = int(ctl.key[i & 1])
            if not k:
                return 0, None, np.float32(0)
            l = key_idx(k) - s.shard_offset
            return k, a["X"][l].copy(), a["norms"][l]
        best, br = 0, -1
        for r in range(s.world_size):
            p = a["pack_all"][r]
            k = int(p[0]) | (int(p[1]) << 32)
            if k > best:
                best, br = k, r
        if br < 0:
            return 0, None, np.float32(0)
        p = a["pack_all"][br]
        return best, p[4:].view(np.float32).copy(), p[2:3].view(np.float32)[0]

    def commit_bound(self, s, rules, stream):
        a = self._arrays(s)
        ctl = self._ctl(s)
        i = ctl.n_sel
        if i >= s.cap:
            ctl.status = 1
            return
        k, row, norm = self._winner(s, a, ctl, i)
        val, gidx = key_val(k), key_idx(k)
        if s.selected:
            a["selected"][i] = gidx
        if s.eps:
            a["eps"][i] = val
        ctl.last_val = float(val) if np.isfinite(val) else (float("inf") if val > 0 else float("-inf"))
        ctl.last_idx = gidx
        ctl.key[(i + 1) & 1] = 0
        ctl.live_rows = 0
        sep = np.float32(ctl.sep)
        if rules == RULE_SIM_SINGLE:
            if sep > val:
                ctl.viable = 1
            if val < sep:
                ctl.sep = float(val)
            ctl.steps += 1
        elif rules == RULE_SIM_SHARDED:
            if sep > val or val <= 0 or gidx < 0:
                ctl.viable = 1
            if val > 0 and val < sep:
                ctl.sep = float(val)
            ctl.steps += 1
        if gidx < 0:
            return
        a["norms_sel"][i] = norm
        l = gidx - s.shard_offset
        if 0 <= l < s.N_local:
            a["h"][l] = -1.0
            a["v"][l] = i
        a["X_sel"][i] = row
        if i > 0:
            with oracle.element_order(bool(s.flags & 1)):
                a["dSL"][:i] = oracle.dsl_quarter(a["X_sel"][: i + 1], a["norms_sel"][: i + 1], i)

    def fps_step(self, s, mode, stream):
        a = self._arrays(s)
        ctl = self._ctl(s)
        i = ctl.n_sel
        if i >= s.cap:
            ctl.status = 1
            return
        N = s.N_local
        if N > 0:
            v64 = a["v"].astype(np.int64)
            with oracle.element_order(bool(s.flags & 1)):
                if i == 0:
                    oracle.fps_update(a["X"], a["norms"], a["X_sel"][0], a["norms_sel"][0], a["h"], v64, 0)
                    live = int((a["h"] >= 0).sum())
                else:
                    live = oracle.voronoi_update(a["X"], a["norms"], a["X_sel"][i], a["norms_sel"][i],
                                                 a["dSL"][:i], a["h"], v64, i)
                    if mode & MODE_DENSE:
                        live = int((~(a["h"] < 0)).sum())
            a["v"][:] = v64.astype(np.int32)
            ctl.live_rows = live
            val, li = oracle.argmax(a["h"])
            k = make_key(val, li + s.shard_offset) if li >= 0 else 0
        else:
            k = 0
        ctl.key[(i + 1) & 1] = k
        self._publish(s, a, k)
        ctl.n_sel = i + 1

    def pool_argmax(self, h_ptr, pool_ptr, n_pool, shard_offset, n_local, out_ptr, stream):
        h = _view(h_ptr, n_local, np.float32)
        pool = _view(pool_ptr, n_pool, np.int64)
        best = 0
        for p in pool[(pool >= shard_offset) & (pool < shard_offset + n_local)]:
            best = max(best, make_key(h[p - shard_offset], int(p)))
        ctypes.c_uint64.from_address(out_ptr).value = best

    def select_kth_largest(self, h_ptr, n, k, scratch_ptr, stream):
        from coresets_b200._native import SelectResult
        h = _view(h_ptr, n, np.float32)
        alive = np.sort(h[h >= 0])
        res = SelectResult.from_address(scratch_ptr)
        res.n_alive = int(alive.size)
        res.valid = 1 if 1 <= k <= alive.size else 0
        res.value = float(alive[alive.size - k]) if res.valid else 0.0

    def scan_argmax(self, s, stream):
        a = self._arrays(s)
        ctl = self._ctl(s)
        if s.N_local > 0:
            val, li = oracle.argmax(a["h"])
            k = make_key(val, li + s.shard_offset) if li >= 0 else 0
        else:
            k = 0
        ctl.key[ctl.n_sel & 1] = k
        self._publish(s, a, k)

    def sim_begin(self, s, sep, stream):
        ctl = self._ctl(s)
        ctl.viable = 0
        ctl.steps = 0
        ctl.sep = sep

    def sim_final_check(self, s, stream):
        a = self._arrays(s)
        ctl = self._ctl(s)
        k, _, _ = self._winner(s, a, ctl, ctl.n_sel)
        if np.float32(ctl.sep) > key_val(k):
            ctl.viable = 1

    def fps_step_lanes(self, lanes, n_lanes, mode, stream):
        for l in range(n_lanes):
            self.fps_step(lanes[l], mode, stream)
