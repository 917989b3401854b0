"""Host-side engine: owns one rank's device buffers and drives the per-pick launch sequence.

One pick on every rank is
    [all-gather of the candidate packs]  ->  cs_commit_bound  ->  cs_fps_step
with the pick counter, the arg-max key and the winning row all staying on the device, so a
run of picks needs no host synchronisation and is replayed from a CUDA graph.  This replaces
the reference's per-pick Python loops, which read the winner back to the host every pick
(src/coresets/cuda/fps.py:105-128, src/coresets/cuda/multi/fps_sharded.py:385-402).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from . import _native
from ._native import (CsCells, CsState, CtlView, MODE_DENSE, MODE_PRUNE, RULE_NONE, RULE_STOP_NONPOS, XCHG_GATHER,
                      XCHG_PEER)

_NORM_CHUNK_ELEMS = 1 << 28  # elements of the X*X temporary per chunk (1 GiB of fp32)


def row_norms(X: torch.Tensor) -> torch.Tensor:
    """Squared row norms with the reference's own expression, ``(X * X).sum(dim=1)``
    (src/coresets/cuda/fps.py:34, src/coresets/cuda/multi/fps_sharded.py:90), evaluated in row
    chunks so that no N x D temporary is ever allocated.  Every chunk has the same number of
    rows (the last one overlaps its predecessor) so each call reduces with the same launch
    shape as one big call would; the values are bit-identical to the unchunked expression."""
    N, D = X.shape
    chunk = max(1, _NORM_CHUNK_ELEMS // max(D, 1))
    if N <= chunk:
        return (X * X).sum(dim=1).to(torch.float32)
    out = torch.empty(N, dtype=torch.float32, device=X.device)
    a = 0
    while a < N:
        b = min(a + chunk, N)
        if b - a < chunk:
            a = N - chunk
        out[a:b] = (X[a:b] * X[a:b]).sum(dim=1).to(torch.float32)
        a = b
    return out


_CONVERT_CHUNK_ELEMS = 1 << 28


def engine_matrix(X: torch.Tensor):
    """Return ``(X_kernels, element_order)``: the row-major matrix the kernels read and whether
    its dots must be summed element-wise.

    The reference dispatches float32, float64 and float16 (``AT_DISPATCH_FLOATING_TYPES_AND_HALF``,
    src/coresets/cuda/kernels/warp.cu:167) and for the last two converts every element to float
    before an element-wise fma chain (``_shared.cuh:55-58``).  Converting the matrix once gives
    the same float values (float16 -> float32 is exact, float64 -> float32 rounds to nearest as
    the kernel's cast does), so those inputs run the float32 kernels with the element-wise order.
    float16 rows on the device are read where they lie (``CS_F_X_HALF``: every element widened at the
    load, 2 bytes of HBM per element and no float32 copy); ``CORESETS_B200_NATIVE_HALF=0`` converts."""
    if X.dtype == torch.float32:
        return X.contiguous(), False
    if X.dtype == torch.float16 and X.is_cuda and _knob("NATIVE_HALF", 1):
        return X.contiguous(), True
    if X.dtype not in (torch.float16, torch.float64):
        raise ValueError(f"X must be float32, float64 or float16 (the reference's dispatch), got {X.dtype}")
    N, D = X.shape
    out = torch.empty((N, D), dtype=torch.float32, device=X.device)
    chunk = max(1, _CONVERT_CHUNK_ELEMS // max(D, 1))
    for a in range(0, N, chunk):
        out[a : a + chunk].copy_(X[a : a + chunk])
    return out, True


def default_mode() -> int:
    m = os.environ.get("CORESETS_B200_MODE", "prune").strip().lower()
    if m not in ("prune", "dense"):
        raise ValueError(f"CORESETS_B200_MODE must be 'prune' or 'dense', got {m!r}")
    return MODE_DENSE if m == "dense" else MODE_PRUNE


def exchange_mode() -> str:
    """How candidates travel between ranks: ``nccl`` = one all-gather per pick, ``p2p`` = the step
    kernel stores its candidate into every peer's symmetric-memory window over NVLink and the next
    commit kernel waits on flags (no collective launch at all)."""
    m = os.environ.get("CORESETS_B200_EXCHANGE", "nccl").strip().lower()
    if m not in ("nccl", "p2p"):
        raise ValueError(f"CORESETS_B200_EXCHANGE must be 'nccl' or 'p2p', got {m!r}")
    return m


def _cells_env() -> bool:
    """``CORESETS_B200_CELLS=0`` keeps every pick on the full scan of h / voronoi."""
    return bool(int(os.environ.get("CORESETS_B200_CELLS", "1")))


# Cell index (see cs_cells in include/coresets_b200.h): the first picks run on the scan kernels,
# the index is built when this many centres exist and rebuilt every time their number has doubled.
# Each constant can be overridden through the environment (tests build tiny indexes often).
def _knob(name: str, default, kind=int):
    return kind(os.environ.get("CORESETS_B200_" + name, default))


_CELLS_FIRST_BUILD = 64          # CELLS_FIRST_BUILD
_CELLS_GROWTH = 2.0              # CELLS_GROWTH
_CELLS_MIN_ROWS = 1 << 18        # CELLS_MIN_ROWS: below this a full scan costs less than the launches of an indexed pick
_CELLS_PROBE_PICKS = 32          # CELLS_PROBE_PICKS: picks after a build before the visited share is read back
_CELLS_GIVE_UP_SHARE = 0.2       # CELLS_GIVE_UP_SHARE: above this share of the slots per pick the scan kernel wins
_CELLS_LIVE_GATE = 0.1           # CELLS_LIVE_GATE: no index while a pick still evaluates this share of the rows
_HALF_RING_SHARE = 0.3          # HALF_RING_SHARE: float16 rows stay on the bulk-copy ring (2 bytes per element, every row)
                                 # while a pick still evaluates this share of them; 0 = never
_EARLY_DENSE_PICKS = 24          # EARLY_DENSE_PICKS: nearly every row passes the triangle test this early, so
                                 # X is streamed with the bulk-copy ring


def _graph_picks() -> int:
    return max(1, int(os.environ.get("CORESETS_B200_GRAPH_PICKS", "32")))


def _graphs_enabled() -> bool:
    return bool(int(os.environ.get("CORESETS_B200_GRAPH", "1")))


class ShardEngine:
    """State of one rank: ``X_local`` (borrowed), norms, ``h``, ``voronoi`` (int32), the
    replicated centre table and the control block.  ``world_size > 1`` adds the candidate packs
    and the all-gather on ``group``."""

    def __init__(self, X_local: torch.Tensor, norms: torch.Tensor, cap: int, *, shard_offset: int = 0,
                 world_size: int = 1, group=None, mode: Optional[int] = None,
                 h: Optional[torch.Tensor] = None, voronoi: Optional[torch.Tensor] = None,
                 record: bool = True, element_order: bool = False, cells: bool = False,
                 cells_any_rules: bool = False):
        if X_local.dim() != 2:
            raise ValueError(f"X_local must be 2-D, got shape {tuple(X_local.shape)}")
        self.half_rows = X_local.dtype == torch.float16
        if X_local.dtype != torch.float32 and not (self.half_rows and element_order and X_local.is_cuda):
            raise ValueError("the engine reads float32 rows, or float16 rows on the device with the element-wise "
                             f"order (see engine_matrix), got {X_local.dtype}")
        if not X_local.is_contiguous():
            raise ValueError("X_local must be contiguous (row-major)")
        self.native = _native.get_native()
        self.X = X_local
        self.norms = norms
        self.device = X_local.device
        self.on_cuda = X_local.is_cuda
        self.N_local, self.D = int(X_local.shape[0]), int(X_local.shape[1])
        self.cap = int(cap)
        self.shard_offset = int(shard_offset)
        self.world_size = int(world_size)
        self.group = group
        self.mode = default_mode() if mode is None else int(mode)
        self.element_order = bool(element_order)
        self._extra_flags = 0            # test hooks of the C ABI (CS_F_TEST_*)
        dev = self.device
        f32, i32, i64 = torch.float32, torch.int32, torch.int64
        n_alloc = max(self.N_local, 1)
        self.h = h if h is not None else torch.empty(n_alloc, dtype=f32, device=dev)
        self.voronoi = voronoi if voronoi is not None else torch.empty(n_alloc, dtype=i32, device=dev)
        self.X_sel = torch.empty((self.cap, self.D), dtype=f32, device=dev)
        self.norms_sel = torch.empty(self.cap, dtype=f32, device=dev)
        self.dSL = torch.empty(self.cap, dtype=f32, device=dev)
        self.selected = torch.empty(self.cap, dtype=i64, device=dev) if record else None
        self.eps = torch.empty(self.cap, dtype=f32, device=dev) if record else None
        self.ctl = torch.zeros(_native.CS_CTL_BYTES // 8, dtype=i64, device=dev)
        self.pack_local = self.pack_all = self.window = None
        self.peer_ptrs = []
        self.rank = 0
        self.xchg = XCHG_GATHER
        self._unconsumed = False       # a candidate was published and no commit has consumed it yet
        if self.world_size > 1:
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
            if self.on_cuda and exchange_mode() == "p2p":
                self._open_peer_windows()
            else:
                self.pack_local = torch.zeros(4 + self.D, dtype=i32, device=dev)
                self.pack_all = torch.zeros((self.world_size, 4 + self.D), dtype=i32, device=dev)
        self._ctl_host = torch.empty(_native.CS_CTL_BYTES // 8, dtype=i64,
                                     pin_memory=self.on_cuda)
        self._graphs = {}
        self.state = self._make_state()
        # cell index: only for plain farthest-point runs on the device (the caller asks for it)
        self.n_host: Optional[int] = None      # picks committed so far, when the host can tell
        self._first_build = max(1, _knob("CELLS_FIRST_BUILD", _CELLS_FIRST_BUILD))
        self._growth = max(1.05, _knob("CELLS_GROWTH", _CELLS_GROWTH, float))
        self._probe_picks = max(1, _knob("CELLS_PROBE_PICKS", _CELLS_PROBE_PICKS))
        self._give_up_share = _knob("CELLS_GIVE_UP_SHARE", _CELLS_GIVE_UP_SHARE, float)
        self._early_dense = max(0, _knob("EARLY_DENSE_PICKS", _EARLY_DENSE_PICKS))
        self._live_gate = _knob("CELLS_LIVE_GATE", _CELLS_LIVE_GATE, float)
        # float16 rows in whole 16-byte units: dense picks stream them through the bulk-copy ring at
        # HBM speed, pruned picks gather them with 2-byte loads
        self._ring_share = _knob("HALF_RING_SHARE", _HALF_RING_SHARE, float)
        self.half_ring = bool(self.half_rows and self.on_cuda and self.mode == MODE_PRUNE and self._ring_share > 0
                              and self.D % 8 == 0 and self.D <= 1024
                              and self.N_local >= _knob("CELLS_MIN_ROWS", _CELLS_MIN_ROWS))
        self._ring_until = 0                   # picks below this count take the ring
        self._ring_off = False                 # the evaluated share fell below the threshold
        self.cells_enabled = bool(
            cells and self.on_cuda and _cells_env() and self.mode == MODE_PRUNE and not self.element_order
            and self.D % 4 == 0 and self.D <= 1024 and self.cap <= 65536
            and self.N_local >= _knob("CELLS_MIN_ROWS", _CELLS_MIN_ROWS)
            and self.N_local + self.cap * _native.CELL_TILE < 2 ** 31)
        self.cells_any_rules = bool(cells_any_rules)   # also for picks with simulation rules (accretion probes)
        self.cells_hold = False                # the caller's veto for the run in hand (e.g. a short probe)
        self._cells: Optional[CsCells] = None
        self._cells_ok = False                 # the index mirrors h / voronoi
        self._cells_next_build = 0
        self._cells_scan_until = 0             # an epoch the index lost: scan kernels up to this pick count
        self.cells_log = []                    # (built at, visited share of the probe) per build

    # -- plumbing ------------------------------------------------------------------------------
    def _open_peer_windows(self) -> None:
        """Allocate this rank's exchange window in symmetric memory and map every peer's window
        (a collective: all ranks construct their engines in the same order)."""
        import torch.distributed._symmetric_memory as symm_mem
        if self.world_size > _native.MAX_PEERS:
            raise ValueError(f"p2p exchange addresses at most {_native.MAX_PEERS} ranks")
        words = self.native.xchg_window_words(self.world_size, self.D)
        self.window = symm_mem.empty(words, dtype=torch.int32, device=self.device)
        self.window.zero_()
        handle = symm_mem.rendezvous(self.window, self.group if self.group is not None else dist.group.WORLD)
        self.peer_ptrs = [int(p) for p in handle.buffer_ptrs]
        self._symm_handle = handle
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)      # every window is zeroed before any peer may store into it
        self.xchg = XCHG_PEER

    def _make_state(self) -> CsState:
        s = CsState()
        s.X = self.X.data_ptr() if self.N_local > 0 else None
        s.norms = self.norms.data_ptr() if self.N_local > 0 else None
        s.h = self.h.data_ptr()
        s.voronoi = self.voronoi.data_ptr()
        s.N_local = self.N_local
        s.shard_offset = self.shard_offset
        s.D = self.D
        s.world_size = self.world_size
        s.X_sel = self.X_sel.data_ptr()
        s.norms_sel = self.norms_sel.data_ptr()
        s.dSL_quarter = self.dSL.data_ptr()
        s.cap = self.cap
        s.selected = self.selected.data_ptr() if self.selected is not None else None
        s.eps = self.eps.data_ptr() if self.eps is not None else None
        s.ctl = self.ctl.data_ptr()
        s.pack_local = self.pack_local.data_ptr() if self.pack_local is not None else None
        s.pack_all = self.pack_all.data_ptr() if self.pack_all is not None else None
        s.rank = self.rank
        s.xchg = self.xchg
        for r, ptr in enumerate(self.peer_ptrs):
            s.peer_win[r] = ptr
        s.xchg_timeout_ms = int(os.environ.get("CORESETS_B200_XCHG_TIMEOUT_MS", "10000"))
        s.flags = ((_native.F_ELEMENT_ORDER if self.element_order else 0) | self._extra_flags
                   | (_native.F_X_HALF if self.half_rows else 0)
                   | (_native.F_PDL if self.on_cuda and _knob("PDL", 1) else 0))
        return s

    def rebind(self, *, h: Optional[torch.Tensor] = None, voronoi: Optional[torch.Tensor] = None) -> None:
        """Point the engine at other ``h`` / ``voronoi`` buffers (snapshots, probe scratch).
        Captured graphs hold the old pointers, so they are dropped."""
        if h is not None:
            self.h = h
        if voronoi is not None:
            self.voronoi = voronoi
        self.state = self._make_state()
        self._graphs.clear()
        self._cells_ok = False

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream if self.on_cuda else 0

    # -- single launches -------------------------------------------------------------------------
    def init_state(self) -> None:
        self.native.init_state(self.state, self._stream())
        self.n_host = 0
        self._cells_ok = False
        self._ring_until, self._ring_off = 0, False

    def reset_ctl(self, n_sel: int) -> None:
        self.native.reset_ctl(self.state, int(n_sel), self._stream())
        self.n_host = int(n_sel)
        self._cells_ok = False
        self._cells_scan_until = 0
        self._ring_until, self._ring_off = 0, False

    def _before_publish(self) -> None:
        # peer exchange: sequence s+1 may only be published once every peer's s has been seen
        if self.xchg == XCHG_PEER and self._unconsumed:
            self.native.xchg_wait(self.state, self._stream())
        self._unconsumed = True

    def force_pick(self, global_idx: int, val: float = float("inf")) -> None:
        self._before_publish()
        self.native.force_pick(self.state, int(global_idx), float(val), self._stream())

    def exchange(self) -> None:
        if self.world_size > 1 and self.xchg == XCHG_GATHER:
            dist.all_gather_into_tensor(self.pack_all.view(-1), self.pack_local, group=self.group)

    def scan(self) -> None:
        """Recompute the next pick's key (and candidate) from the current ``h``."""
        self._before_publish()
        self.native.scan_argmax(self.state, self._stream())

    def sim_begin(self, sep: float) -> None:
        self.native.sim_begin(self.state, float(sep), self._stream())

    def sim_final_check(self) -> None:
        self.native.sim_final_check(self.state, self._stream())
        self._unconsumed = False

    def commit(self, rules: int = RULE_NONE) -> None:
        self.native.commit_bound(self.state, int(rules), self._stream())
        self._unconsumed = False

    def step(self, mode: Optional[int] = None) -> None:
        self.native.fps_step(self.state, self.mode if mode is None else int(mode), self._stream())
        self._unconsumed = True
        self._cells_ok = False             # h changed behind the index
        if self.n_host is not None:
            self.n_host += 1

    # -- picks -------------------------------------------------------------------------------------
    def _pick_body(self, rules: int, how=None) -> None:
        """One pick.  ``how``: None = the engine's mode, an int = that step mode, "cells" = through
        the cell index."""
        if how == "forced":
            if self.world_size > 1 and self.xchg == XCHG_PEER:
                self.native.xchg_wait(self.state, self._stream())     # see _before_publish
            self.native.force_pick_list(self.state, self._forced_list.data_ptr(), self._forced_vals.data_ptr(),
                                        float("inf"), self._stream())
            how = None
        elif how == "pool":
            if self.world_size > 1 and self.xchg == XCHG_PEER:
                self.native.xchg_wait(self.state, self._stream())     # see _before_publish
            self.native.pool_pick(self.state, self._pool_buf.data_ptr(), self._pool_n.data_ptr(), self._stream())
            how = None
        self.exchange()
        self.commit(rules)
        if how == "cells":
            st = self._stream()
            self.native.cells_select(self.state, self._cells, st)
            self.native.fps_step_cells(self.state, self._cells, st)
            self._unconsumed = True
            if self.n_host is not None:
                self.n_host += 1
        else:
            self.step(how)

    def pick_forced(self, global_idx: int, val: float = float("inf"), rules: int = RULE_NONE) -> None:
        """Commit a prescribed row as the next centre and run its update."""
        self.force_pick(global_idx, val)
        self._pick_body(rules)

    def run_forced(self, indices, rules: int = RULE_NONE, values=None) -> None:
        """Commit the prescribed global rows ``indices`` one after the other as the next centres, each
        with its update -- ``pick_forced`` for a whole list.  On the device the rows are read from a
        list indexed by the pick counter, so the run replays from CUDA graphs like free picks
        (a resumed checkpoint of 16 384 picks is 512 graph replays instead of 65 536 host calls)."""
        idx = [int(v) for v in (indices.tolist() if hasattr(indices, "tolist") else indices)]
        if not idx:
            return
        vals = [float("inf")] * len(idx) if values is None else [float(v) for v in values]
        if not (self.on_cuda and _graphs_enabled() and self.n_host is not None) or len(idx) < 4:
            for g, v in zip(idx, vals):
                self.pick_forced(g, v, rules=rules)
            return
        if self.n_host + len(idx) > self.cap:
            raise ValueError(f"{len(idx)} forced picks after {self.n_host} exceed the capacity {self.cap}")
        if not hasattr(self, "_forced_list"):
            self._forced_list = torch.zeros(self.cap, dtype=torch.int64, device=self.device)
            self._forced_vals = torch.zeros(self.cap, dtype=torch.float32, device=self.device)
        lo, hi = self.n_host, self.n_host + len(idx)
        self._forced_list[lo:hi] = torch.tensor(idx, dtype=torch.int64).to(self.device)
        self._forced_vals[lo:hi] = torch.tensor(vals, dtype=torch.float32).to(self.device)
        self._replay(len(idx), rules, "forced")

    def run_restricted(self, pool: torch.Tensor, n: int):
        """Up to ``n`` greedy picks restricted to the global rows in ``pool`` (int64, on the device):
        each takes the largest ``h`` among the pool's rows (ties to the smaller index), commits it
        and runs its update -- the forward walk of accretion (block_forward.py:38-53,
        sharded.py:174-215) without a host round trip per pick.  The run stops by itself when the
        best value is not positive.  Returns ``(picks made, ran dry)``; one read-back."""
        if not (self.on_cuda and self.n_host is not None):
            raise RuntimeError("run_restricted needs a CUDA engine whose pick count the host knows")
        n = int(n)
        if n <= 0:
            return 0, False
        if not hasattr(self, "_pool_buf"):
            self._pool_buf = torch.zeros(max(self.cap, 1), dtype=torch.int64, device=self.device)
            self._pool_n = torch.zeros(1, dtype=torch.int64, device=self.device)
        if pool.numel() > self._pool_buf.numel():
            self._pool_buf = torch.zeros(int(pool.numel()), dtype=torch.int64, device=self.device)
            self._graphs = {k: g for k, g in self._graphs.items() if k[2] != "pool"}
        self._pool_buf[: pool.numel()].copy_(pool)
        self._pool_n.fill_(int(pool.numel()))
        before = self.n_host
        n = min(n, self.cap - before)
        self._replay(n, RULE_STOP_NONPOS, "pool")
        ctl = self.read_ctl()
        made = int(ctl.n_sel) - before
        self.n_host = int(ctl.n_sel)
        dry = bool(ctl.halt)
        if dry:
            # the halt word silences every later launch: clear it (and with it the key slots, so the
            # caller recomputes the key before the next free pick)
            self.reset_ctl(self.n_host)
            self._unconsumed = False
        return made, dry

    def _graph(self, n: int, rules: int, how=None):
        key = (n, rules, self.mode if how is None else how)
        g = self._graphs.get(key)
        if g is None:
            n_before, ok_before = self.n_host, self._cells_ok
            # Nothing may be in flight while the stream captures: with collectives in the body the
            # process group's watchdog thread polls the events of earlier eager collectives, and
            # an event query from another thread invalidates a capture in the default "global"
            # error mode.  Drain the device first and confine capture errors to this thread.
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                for _ in range(n):
                    self._pick_body(rules, how)
            self._graphs[key] = g
            self.n_host, self._cells_ok = n_before, ok_before      # capturing ran nothing
        return g

    _UNITS = (32, 16, 8, 4, 2, 1)

    def _units(self, n: int):
        """Binary decomposition of ``n`` picks into the graph sizes (largest first)."""
        top = min(_graph_picks(), self._UNITS[0])
        for unit in self._UNITS:
            if unit <= top:
                while n >= unit:
                    yield unit
                    n -= unit

    def prepare(self, n: int, rules: int = RULE_NONE) -> None:
        """Capture (without running) the graphs ``run_picks(n)`` will replay."""
        if not (self.on_cuda and _graphs_enabled()):
            return
        kinds = [None]
        if self._uses_cells(rules):
            self._alloc_cells()
            kinds.append("cells")
            if self.n_host < self._early_dense:
                kinds.append(MODE_DENSE)
        for how in kinds:
            for unit in set(self._units(n)):
                self._graph(unit, rules, how)

    def _replay(self, n: int, rules: int, how) -> None:
        """Enqueue ``n`` picks of one kind: graph replays, or single launches when graphs are off."""
        if self.on_cuda and _graphs_enabled():
            for unit in self._units(n):
                self._graph(unit, rules, how).replay()
                self._unconsumed = True
                if self.n_host is not None:
                    self.n_host += unit
                if how != "cells":
                    self._cells_ok = False
            return
        for _ in range(n):
            self._pick_body(rules, how)

    def _uses_cells(self, rules: int) -> bool:
        return (self.cells_enabled and not self.cells_hold and self.n_host is not None
                and (rules == RULE_NONE or self.cells_any_rules))

    def run_picks(self, n: int, rules: int = RULE_NONE) -> None:
        """Enqueue ``n`` farthest-point picks, replayed from CUDA graphs of 32, 16, ... 1 picks
        (binary decomposition of ``n``).  Without the cell index nothing here synchronises with the
        host.  With it (plain farthest-point runs) the picks are cut at the points where the
        index is built (64 centres, then every doubling), and once per build the host reads back
        how much of the index the first picks visited, to fall back to the scan kernels on data
        the index does not help."""
        n = int(n)
        if n <= 0:
            return
        if self.half_ring and rules == RULE_NONE and self.n_host is not None and not self._ring_off:
            # float16 rows: the ring while many rows are still evaluated (one read-back per stretch
            # of picks: 24, then every 25 % more), the pruned scan for the rest of the run
            while n > 0 and not self._ring_off:
                cur = self.n_host
                if cur >= max(self._ring_until, self._early_dense):
                    if cur > 0 and self.read_ctl().live_rows <= self._ring_share * self.N_local:
                        self._ring_off = True
                        break
                    self._ring_until = max(cur + 16, int(cur * 1.25))
                m = min(n, max(self._ring_until, self._early_dense) - cur)
                self._replay(m, rules, MODE_DENSE)
                n -= m
            if n <= 0:
                return
        if not self._uses_cells(rules):
            self._replay(n, rules, None)
            return
        while n > 0:
            cur = self.n_host
            if cur < self._early_dense:
                m = min(n, self._early_dense - cur)
                self._replay(m, rules, MODE_DENSE)
            elif cur < max(self._first_build, self._cells_scan_until):
                m = min(n, max(self._first_build, self._cells_scan_until) - cur)
                self._replay(m, rules, None)
            else:
                if not self._cells_ok or cur >= self._cells_next_build:
                    # an index pays once a pick leaves most rows alone; while the last pick still
                    # evaluated a large share of them the scan kernels stay (one read-back)
                    if self.read_ctl().live_rows > self._live_gate * self.N_local:
                        self._cells_scan_until = max(cur + 16, int(cur * 1.25))
                        continue
                    self._build_cells()
                m = min(n, self._cells_next_build - cur)
                if self._cells_probe_left > 0:
                    m = min(m, self._cells_probe_left)
                    self._replay(m, rules, "cells")
                    self._cells_probe_left -= m
                    if self._cells_probe_left == 0:
                        self._assess_cells()
                else:
                    self._replay(m, rules, "cells")
            n -= m

    # -- cell index ----------------------------------------------------------------------------------
    def _alloc_cells(self) -> None:
        if self._cells is not None:
            return
        dev, i32 = self.device, torch.int32
        slots = (self.N_local + self.cap * _native.CELL_TILE + 3) & ~3
        bufs = dict(
            perm=torch.empty(slots, dtype=i32, device=dev), hp=torch.empty(slots, dtype=torch.float32, device=dev),
            vp=torch.empty(slots, dtype=i32, device=dev), cell0=torch.empty(self.N_local, dtype=i32, device=dev),
            seg_start=torch.zeros(self.cap + 1, dtype=i32, device=dev), seg_count=torch.zeros(self.cap, dtype=i32, device=dev),
            seg_key=torch.zeros(self.cap, dtype=torch.int64, device=dev), seg_h0=torch.zeros(self.cap, dtype=torch.float32, device=dev),
            cursor=torch.zeros(self.cap, dtype=i32, device=dev), work_cell=torch.zeros(self.cap, dtype=i32, device=dev),
            work_cum=torch.zeros(self.cap, dtype=i32, device=dev),
            meta=torch.zeros(_native.CELLS_META_BYTES // 8, dtype=torch.int64, device=dev))
        # rows of one pick that wait for a distance: a quarter of the shard is far more than a pick
        # needs once the index is in use (the kernels stay correct when it overflows, only slower)
        q_cap = max(_native.CELL_TILE, _knob("CELLS_QUEUE", max(1 << 16, self.N_local // 4)))
        bufs["queue"] = torch.empty((q_cap, 2), dtype=i32, device=dev)
        c = CsCells()
        for name, t in bufs.items():
            setattr(c, name, t.data_ptr())
        c.slots = slots
        c.q_cap = q_cap
        c.row_norm_max = float(self.norms.max().item())           # one read-back, at the first build
        self._cells_bufs = bufs
        self._cells_meta_host = torch.empty(_native.CELLS_META_BYTES // 8, dtype=torch.int64, pin_memory=True)
        self._cells = c

    def _build_cells(self) -> None:
        self._alloc_cells()
        cur = self.n_host
        self.native.cells_build(self.state, self._cells, self._stream())
        self._cells_ok = True
        self._cells_built_at = cur
        self._cells_next_build = max(cur + min(self._first_build, 64), int(cur * self._growth))
        self._cells_probe_left = self._probe_picks

    def read_cells_meta(self) -> "_native.CellsMetaView":
        """Copy the index's statistics block to the host (synchronises the current stream)."""
        self._cells_meta_host.copy_(self._cells_bufs["meta"], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        view = _native.CellsMetaView()
        ctypes.memmove(ctypes.addressof(view), self._cells_meta_host.data_ptr(), _native.CELLS_META_BYTES)
        return view

    def _assess_cells(self) -> None:
        """After the first picks on a fresh index: if they visited most of it, the data does not
        separate into cells (or not yet) and the scan kernels take the rest of this epoch."""
        mv = self.read_cells_meta()
        share = mv.visited_slots / max(1, mv.picks) / max(1, mv.total_slots)
        self.cells_log.append((self._cells_built_at, round(share, 4)))
        if share > self._give_up_share:
            self._cells_scan_until = self._cells_next_build

    # -- several states in one pass over X ("lanes") --------------------------------------------------
    @staticmethod
    def step_lanes(engines, mode: Optional[int] = None) -> None:
        """One fused step for several engines that share ``X`` (bisect probes): ``X`` is streamed
        once, every engine ends exactly as after its own ``step()``."""
        e0 = engines[0]
        m = e0.mode if mode is None else int(mode)
        arr = (CsState * len(engines))(*[e.state for e in engines])
        e0.native.fps_step_lanes(arr, len(engines), m, e0._stream())
        for e in engines:
            e._unconsumed = True
            e._cells_ok = False
            e.n_host = None

    @staticmethod
    def run_lane_picks(engines, n: int, rules: int) -> None:
        """``n`` lock-step picks on every engine of ``engines`` (graph-replayed on the GPU)."""
        e0 = engines[0]
        if e0.mode == MODE_PRUNE and any(e._uses_cells(rules) for e in engines):
            # prune mode steps the lanes one by one anyway (cs_fps_step_lanes); with a cell index each
            # lane runs its own picks, through its own index
            for e in engines:
                e.run_picks(n, rules)
            return

        def body():
            for e in engines:
                e.exchange()
                e.commit(rules)
            ShardEngine.step_lanes(engines)

        if not (e0.on_cuda and _graphs_enabled()):
            for _ in range(n):
                body()
            return
        key = ("lanes", tuple(id(e) for e in engines), n, rules, e0.mode)
        g = e0._graphs.get(key)
        if g is None:
            torch.cuda.synchronize(e0.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                for _ in range(n):
                    body()
            e0._graphs[key] = g
        g.replay()
        for e in engines:
            e._unconsumed = True
            e._cells_ok = False
            e.n_host = None

    def kth_largest_live(self, k: int):
        """``(value, n_alive)``: the exact ``k``-th largest entry of this engine's ``h`` among the
        rows that are not selected (``h >= 0``) and how many such rows there are; ``value`` is
        ``None`` when ``k`` is outside ``[1, n_alive]``.  Equals
        ``torch.kthvalue(h[h >= 0], n_alive - k + 1)`` (cuda/_internal/bisect.py:64-71): a selection
        returns one of its inputs.  One 16-byte read-back."""
        if not hasattr(self, "_select_scratch"):
            self._select_scratch = torch.zeros(_native.SELECT_SCRATCH_BYTES // 8, dtype=torch.int64, device=self.device)
            self._select_host = torch.empty(2, dtype=torch.int64, pin_memory=self.on_cuda)
        self.native.select_kth_largest(self.h.data_ptr(), self.N_local, int(k), self._select_scratch.data_ptr(),
                                       self._stream())
        if self.on_cuda:
            self._select_host.copy_(self._select_scratch[:2], non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            src = self._select_host
        else:
            src = self._select_scratch
        res = _native.SelectResult()
        ctypes.memmove(ctypes.addressof(res), src.data_ptr(), ctypes.sizeof(res))
        return (float(res.value) if res.valid else None), int(res.n_alive)

    # -- read-back -----------------------------------------------------------------------------------
    def read_ctl(self) -> CtlView:
        """Copy the control block to the host (synchronises the current stream)."""
        if self.on_cuda:
            self._ctl_host.copy_(self.ctl, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            src = self._ctl_host
        else:
            src = self.ctl
        view = CtlView()
        ctypes.memmove(ctypes.addressof(view), src.data_ptr(), _native.CS_CTL_BYTES)
        return view

    def check_status(self) -> CtlView:
        view = self.read_ctl()
        if view.status != 0:
            what = {1: "more picks were launched than the centre table can hold",
                    2: "a forced pick named a row this rank does not own",
                    3: "timed out waiting for a peer's candidate (peer exchange)",
                    4: "timed out waiting for a bulk copy (dense-mode pipe)"}.get(view.status, "unknown")
            raise RuntimeError(f"coresets_b200 device status {view.status}: {what}")
        return view
