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
from ._native import CsState, CtlView, MODE_DENSE, MODE_PRUNE, RULE_NONE, XCHG_GATHER, XCHG_PEER

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
    """Return ``(X32, element_order)``: the float32 row-major matrix the kernels read and whether
    its dots must be summed element-wise.

    The reference dispatches float32, float64 and float16 (``AT_DISPATCH_FLOATING_TYPES_AND_HALF``,
    src/coresets/cuda/kernels/warp.cu:167) and for the last two converts every element to float
    before an element-wise fma chain (``_shared.cuh:55-58``).  Converting the matrix once gives
    the same float values (float16 -> float32 is exact, float64 -> float32 rounds to nearest as
    the kernel's cast does), so those inputs run the float32 kernels with the element-wise order."""
    if X.dtype == torch.float32:
        return X.contiguous(), False
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
                 record: bool = True, element_order: bool = False):
        if X_local.dim() != 2:
            raise ValueError(f"X_local must be 2-D, got shape {tuple(X_local.shape)}")
        if X_local.dtype != torch.float32:
            raise ValueError(f"the engine reads float32 rows (see engine_matrix), got {X_local.dtype}")
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
        s.flags = (_native.F_ELEMENT_ORDER if self.element_order else 0) | self._extra_flags
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

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream if self.on_cuda else 0

    # -- single launches -------------------------------------------------------------------------
    def init_state(self) -> None:
        self.native.init_state(self.state, self._stream())

    def reset_ctl(self, n_sel: int) -> None:
        self.native.reset_ctl(self.state, int(n_sel), self._stream())

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

    # -- picks -------------------------------------------------------------------------------------
    def _pick_body(self, rules: int) -> None:
        self.exchange()
        self.commit(rules)
        self.step()

    def pick_forced(self, global_idx: int, val: float = float("inf"), rules: int = RULE_NONE) -> None:
        """Commit a prescribed row as the next centre and run its update."""
        self.force_pick(global_idx, val)
        self._pick_body(rules)

    def _graph(self, n: int, rules: int):
        key = (n, rules, self.mode)
        g = self._graphs.get(key)
        if g is None:
            # Nothing may be in flight while the stream captures: with collectives in the body the
            # process group's watchdog thread polls the events of earlier eager collectives, and
            # an event query from another thread invalidates a capture in the default "global"
            # error mode.  Drain the device first and confine capture errors to this thread.
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                for _ in range(n):
                    self._pick_body(rules)
            self._graphs[key] = g
        return g

    _UNITS = (32, 16, 8, 4, 2, 1)

    def prepare(self, n: int, rules: int = RULE_NONE) -> None:
        """Capture (without running) the graphs ``run_picks(n)`` will replay."""
        if not (self.on_cuda and _graphs_enabled()):
            return
        top = min(_graph_picks(), self._UNITS[0])
        for unit in self._UNITS:
            if unit <= top and n >= unit:
                self._graph(unit, rules)
                n %= unit

    def run_picks(self, n: int, rules: int = RULE_NONE) -> None:
        """Enqueue ``n`` farthest-point picks.  No host synchronisation happens here: the picks
        are replayed from CUDA graphs of 32, 16, ... 1 picks (binary decomposition of ``n``)."""
        n = int(n)
        if n <= 0:
            return
        if self.on_cuda and _graphs_enabled():
            top = min(_graph_picks(), self._UNITS[0])
            for unit in self._UNITS:
                if unit > top:
                    continue
                while n >= unit:
                    self._graph(unit, rules).replay()
                    self._unconsumed = True
                    n -= unit
        for _ in range(n):
            self._pick_body(rules)

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

    @staticmethod
    def run_lane_picks(engines, n: int, rules: int) -> None:
        """``n`` lock-step picks on every engine of ``engines`` (graph-replayed on the GPU)."""
        e0 = engines[0]

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
