"""Accretion (merging new candidates into an anchor's FPS ordering) on the B200 engine.

One driver class serves both public entry points:

* ``flavour="single"``  -- ``accrete`` (reference: src/coresets/cuda/accrete.py:26-272 with
  cuda/_internal/{bisect,block_forward,reconstruct}.py): one GPU, no process group, the
  single-GPU simulation rules and the k-th-value early exit of its bisect;
* ``flavour="sharded"`` -- ``accrete_sharded`` (reference: src/coresets/cuda/multi/_base.py:37-873
  and multi/sharded.py:18-775): rows sharded over ranks, the sharded simulation rules, seeded
  search, lazy forward, batched fill, checkpoints.

The three hot loops -- restricted forward, bisect simulations, unconstrained fill -- run on
``ShardEngine``: forced picks for the forward / replay, graph-replayed picks for the fill, and
16-pick graph chunks with a 256-byte control-block read-back for the simulations.  The host logic
around them (nested anchor blocks, snapshots, reconstruction with the reference's torch
expressions, the searches) keeps the reference's decisions so that the result is the same list.
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Set, Tuple

import numpy as np
import torch
import torch.distributed as dist
from torch import Tensor

from .. import engine as _engine
from .._native import RULE_NONE, RULE_SIM_SHARDED, RULE_SIM_SINGLE, decode_key
from . import search
from .diag import PhaseTimer, Tracer, fmt_gap, invariant_numbers, level_counts
from .multi.layout import ShardLayout

_SIM_POLL = 16          # the host looks at the viability flag every 16 simulated picks
_GROSS_REL = 1e-3       # tolerated relative shortfall of sep^2 against cov^2 (float32 noise)


@dataclass
class _Snapshot:
    sep: float
    n_selected: int
    selected: List[int]


def _env_int(name: str, default: int) -> int:
    return int(os.environ.get(name, str(default)))


class AccreteDriver:
    def __init__(self, X_local: Tensor, norms_local: Tensor, layout: ShardLayout, anchor_order: List[int],
                 n_anchor: int, n_global: int, max_k: int, max_sel: int, *, flavour: str, verbose: bool,
                 profile: bool, trace_path: Optional[str], checkpoint_path: Optional[str] = None,
                 resume_from: Optional[str] = None, checkpoint_every: int = 0,
                 X_src: Optional[Tensor] = None):
        """``X_local`` is the float32 matrix the kernels read.  ``X_src`` is the caller's matrix when
        it was float16 / float64: the kernels then sum element-wise (``engine.engine_matrix``) and the
        reconstruct step multiplies in the caller's dtype, as the reference does."""
        assert flavour in ("single", "sharded")
        self.flavour = flavour
        self.multi = flavour == "sharded"
        self.name = "accrete_voronoi_multi_sharded" if self.multi else "accrete"
        self.layout = layout
        self.device = X_local.device
        self.dim = int(X_local.shape[1])
        self.max_k, self.max_sel = int(max_k), int(max_sel)
        self.n_anchor, self.n_global = int(n_anchor), int(n_global)
        self.verbose, self.profile = verbose, profile
        self.chatty = verbose and layout.rank == 0
        self.checkpoint_path, self.resume_from = checkpoint_path, resume_from
        self.checkpoint_every = int(checkpoint_every)
        self._last_ckpt_n = 0
        self.rules = RULE_SIM_SHARDED if self.multi else RULE_SIM_SINGLE

        world = layout.world_size if self.multi else 1
        self.X_src = X_src
        kw = dict(shard_offset=layout.shard_offset, world_size=world, element_order=X_src is not None)
        self.E = _engine.ShardEngine(X_local, norms_local, self.max_sel, **kw)
        # Probes can run through the cell index (built per probe from the reconstructed state) on shards
        # of at least CORESETS_B200_CELLS_SIM_MIN_ROWS rows.  Off unless that knob is set: at 25 M rows
        # per GPU it shortens the probes' steps by a quarter but a run by 6 % only, because three quarters
        # of a large run go into the reconstruct step, whose arithmetic is the reference's.
        self._sim_cells = (X_local.is_cuda and int(X_local.shape[0]) >= _env_int("CORESETS_B200_CELLS_SIM_MIN_ROWS", 1 << 40))
        self._sim_cells_min_steps = _env_int("CORESETS_B200_CELLS_SIM_MIN_STEPS", 256)
        self.S = _engine.ShardEngine(X_local, norms_local, self.max_sel, record=False, cells=self._sim_cells,
                                     cells_any_rules=True, **kw)
        self.E.init_state()
        n_alloc = self.E.h.shape[0]
        mk = lambda dt: torch.empty(n_alloc, dtype=dt, device=self.device)  # noqa: E731
        self.h_snap, self.h_final = mk(torch.float32), mk(torch.float32)
        self.v_snap, self.v_final = mk(torch.int32), mk(torch.int32)

        self.anchor_indices = list(anchor_order)
        self.nested_blocks: List[Set[int]] = [
            set(self.anchor_indices[: min(2 ** i, self.n_anchor)]) for i in range(1, self.max_k + 1)
        ]
        self.selected: List[int] = []
        self.selected_set: Set[int] = set()
        self.sep = float("inf")
        self._key_valid = False        # does the control block hold the arg-max of the current h?

        # knobs of the sharded driver (read once; _base.py:107-137, sharded.py:70)
        seeded = _env_int("CORESETS_BISECT_SEED", 0) if self.multi else 0
        self.bisect_seeded = seeded
        self.cov_relax = float(os.environ.get("CORESETS_ANCHOR_COV_RELAX", "1.0")) if self.multi else 1.0
        self.lazy_forward = bool(seeded) and bool(_env_int("CORESETS_LAZY_FORWARD", 1))
        self.bisect_lanes = max(0, min(8, _env_int("CORESETS_BISECT_LANES", 4))) if seeded else 0
        self.lanes_min_steps = _env_int("CORESETS_LANES_MIN_STEPS", 768)
        self.gallop_deep = bool(seeded) and bool(_env_int("CORESETS_BISECT_GALLOP_DEEP", 0))
        self.fill_chunk = _env_int("CORESETS_FILL_CHUNK", 0) if self.multi else 0
        self._seed_by_pos: Dict[int, int] = {}
        self._seed_prev_by_pos: Dict[int, int] = {}
        self._bisect_seed = 0
        self._has_seed = False
        if self.multi and dist.is_initialized():
            flags = torch.tensor([seeded, int(self.lazy_forward), self.bisect_lanes, int(self.gallop_deep)],
                                 dtype=torch.long, device=self.device)
            lo, hi = flags.clone(), flags.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            if not torch.equal(lo, hi):
                raise RuntimeError(
                    f"{self.name}: CORESETS_BISECT_SEED/CORESETS_LAZY_FORWARD/CORESETS_BISECT_LANES differ "
                    "across ranks - set them identically on every rank (they steer collective control flow)."
                )
        self.timer = PhaseTimer(profile, X_local.is_cuda)
        self.trace = Tracer(trace_path if layout.rank == 0 else None)
        self._k = 0
        self._pos = 0
        self._n_probe = 0

    # ------------------------------------------------------------------ primitives
    def _record(self, idx: int) -> int:
        pos = len(self.selected)
        self.selected.append(idx)
        self.selected_set.add(idx)
        return pos

    def _commit_known(self, idx: int, val: float) -> None:
        """Commit global row ``idx`` as the next centre and run its update (3 launches)."""
        with self.timer("voronoi_step_s"):
            self.E.pick_forced(idx, val)
        self._key_valid = True

    def _restricted_argmax(self, pool: Tensor) -> Tuple[float, int]:
        """Largest ``h`` over the global indices in ``pool``, ties to the smallest index
        (block_forward.py:38-53, sharded.py:174-210): one kernel reduces this shard's part to a
        64-bit key (value, then smaller index), the ranks' keys are gathered, one read-back.
        Rows of the pool that are already selected carry ``h = -1`` and can only win when nothing
        else is left, which the caller reads as "dry" exactly like an empty pool."""
        E = self.E
        if not hasattr(self, "_pool_key"):
            world = self.layout.world_size if self.multi else 1
            self._pool_key = torch.zeros(1, dtype=torch.int64, device=self.device)
            self._pool_keys = torch.zeros(world, dtype=torch.int64, device=self.device)
            self._pool_host = torch.empty(world, dtype=torch.int64, pin_memory=E.on_cuda)
        E.native.pool_argmax(E.h.data_ptr(), pool.data_ptr(), int(pool.numel()), self.layout.shard_offset,
                             self.layout.N_shard, self._pool_key.data_ptr(), E._stream())
        src = self._pool_key
        if self.multi:
            dist.all_gather_into_tensor(self._pool_keys, self._pool_key)
            src = self._pool_keys
        if E.on_cuda:
            self._pool_host[: src.numel()].copy_(src, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            keys = self._pool_host[: src.numel()].tolist()
        else:
            keys = src.tolist()
        val, idx = decode_key(max(k & 0xFFFFFFFFFFFFFFFF for k in keys))
        return float(val), int(idx)

    def _global_max(self, h: Tensor) -> float:
        n = self.layout.N_shard
        t = h[:n].max().reshape(1) if n > 0 else torch.full((1,), float("-inf"), device=self.device)
        if self.multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def _take_snapshot(self) -> _Snapshot:
        self.h_snap.copy_(self.E.h)
        self.v_snap.copy_(self.E.voronoi)
        return _Snapshot(self.sep, len(self.selected), list(self.selected))

    def _rollback(self, snap: _Snapshot) -> None:
        self.E.h.copy_(self.h_snap)
        self.E.voronoi.copy_(self.v_snap)
        self.E.reset_ctl(snap.n_selected)
        self._key_valid = False
        self.selected = list(snap.selected)
        self.selected_set = set(snap.selected)
        self.sep = snap.sep

    def _reconstruct(self, snap: _Snapshot, added_t: Tensor, sel_start_t: Tensor, m: int, target=None) -> None:
        """State after keeping only the first ``m`` forward picks, written into the simulation
        engine's ``h`` / ``voronoi``.  Rows whose final centre lies in the dropped tail are
        recomputed against the kept picks with the reference's expression
        ``n_a + n_b - 2 * (X_a @ X_b.T)`` in the same column chunks (reconstruct.py:75-157,
        _shared.py:67-152), so the values are the ones the reference feeds its simulations."""
        n_snap = snap.n_selected
        n = self.layout.N_shard
        target = self.S if target is None else target
        h_mid, v_mid = target.h, target.voronoi
        h_mid.copy_(self.h_final)
        v_mid.copy_(self.v_final)
        if n > 0:
            affected = torch.where(self.v_final[:n] >= (n_snap + m))[0]
            if affected.numel() > 0:
                if m == 0:
                    h_mid[affected] = self.h_snap[affected]
                    v_mid[affected] = self.v_snap[affected]
                else:
                    X_added = self.E.X_sel[n_snap : n_snap + m]
                    n_added = self.E.norms_sel[n_snap : n_snap + m]
                    if self.X_src is None:
                        X_aff = self.E.X[affected]
                    else:
                        # float16 / float64 input: the product runs in the caller's dtype.  The
                        # single-GPU reference gathers the added rows from X (reconstruct.py:102),
                        # the sharded one keeps them in an X_sel of X's dtype that was filled from
                        # the float32 exchange pack (sharded.py:52, multi.cu:245)
                        X_aff = self.X_src[affected]
                        X_added = X_added.to(self.X_src.dtype) if self.multi else self.X_src[added_t[:m]]
                    n_aff = self.E.norms[affected]
                    cnt = affected.numel()
                    best = torch.full((cnt,), float("inf"), dtype=torch.float32, device=self.device)
                    arg = torch.zeros(cnt, dtype=torch.long, device=self.device)
                    chunk = max(1, 10_000_000 // max(cnt, 1))
                    for a in range(0, m, chunk):
                        b = min(a + chunk, m)
                        d = n_aff.unsqueeze(1) + n_added[a:b].unsqueeze(0) - 2.0 * (X_aff @ X_added[a:b].T)
                        vals, rel = d.min(dim=1)
                        better = vals < best
                        best = torch.where(better, vals, best)
                        arg = torch.where(better, rel + a, arg)
                    snap_vals = self.h_snap[affected]
                    keep_snap = snap_vals <= best
                    h_mid[affected] = torch.where(keep_snap, snap_vals, best)
                    v_mid[affected] = torch.where(keep_snap, self.v_snap[affected], (n_snap + arg).to(torch.int32))
        pre = sel_start_t if m == 0 else torch.cat((sel_start_t, added_t[:m]))
        if pre.numel() > 0 and n > 0:
            lo = self.layout.shard_offset
            mine = pre[(pre >= lo) & (pre < lo + n)] - lo
            if mine.numel() > 0:
                h_mid[mine] = -1.0

    def _sim_start(self, S, sep_mid: float, n_init: int, points_left: int = 0) -> None:
        S.cells_hold = points_left < self._sim_cells_min_steps      # an index does not pay for a short probe
        if n_init > 0:
            S.X_sel[:n_init].copy_(self.E.X_sel[:n_init])
            S.norms_sel[:n_init].copy_(self.E.norms_sel[:n_init])
        S.reset_ctl(n_init)
        S.sim_begin(sep_mid)
        S.scan()

    def _sim_finish(self, S, done: int, points_left: int) -> Tuple[bool, int]:
        """Run a started probe from ``done`` (a multiple of 16) picks to its verdict."""
        while done < points_left:
            n = min(_SIM_POLL, points_left - done)
            S.run_picks(n, self.rules)
            done += n
            if n == _SIM_POLL and S.read_ctl().viable:
                return True, done
        S.exchange()
        S.sim_final_check()
        return bool(S.check_status().viable), points_left

    def _simulate(self, sep_mid: float, points_left: int, n_init: int) -> Tuple[bool, int]:
        """One bisect probe on the simulation engine's state: up to ``points_left`` unrestricted
        picks, viable as soon as the running separation beats the coverage
        (simulate.cu:10-90, multi.cu:428-528)."""
        self._sim_start(self.S, sep_mid, n_init, points_left)
        return self._sim_finish(self.S, 0, points_left)

    def _lane_engines(self, n: int):
        """Simulation engines for fused probes; lane 0 is the sequential one.  The count is capped
        by CORESETS_LANES_MEM_GB (default 8) like the reference's lane scratch (sharded.py:78-97)."""
        if not hasattr(self, "_lanes"):
            self._lanes = [self.S]
        budget = float(os.environ.get("CORESETS_LANES_MEM_GB", "8")) * (1 << 30)
        per_lane = max(self.layout.sizes) * (26 if self._sim_cells else 8) + self.max_sel * (self.dim * 4 + 12)
        n = max(1, min(n, 1 + int(budget // max(per_lane, 1))))
        world = self.layout.world_size if self.multi else 1
        while len(self._lanes) < n:
            self._lanes.append(_engine.ShardEngine(self.E.X, self.E.norms, self.max_sel, record=False,
                                                   shard_offset=self.layout.shard_offset, world_size=world,
                                                   element_order=self.E.element_order, cells=self._sim_cells,
                                                   cells_any_rules=True))
        return self._lanes[:n]

    def _simulate_lanes(self, engines, probes) -> List[bool]:
        """Several probes as lanes of one loop: one pass over X per step serves them all
        (multi.cu:800-1019).  Every lane polls its flag after each 16 picks like a lone probe, so
        each verdict is the lone probe's verdict."""
        W = len(probes)
        for S, p in zip(engines, probes):
            self._sim_start(S, float(p["sep"]), p["n_init"], p["points_left"])
        left = [p["points_left"] for p in probes]
        verdict: List[Optional[bool]] = [None] * W
        active = list(range(W))
        done = 0
        while len(active) >= 2 and min(left[w] for w in active) - done >= _SIM_POLL:
            _engine.ShardEngine.run_lane_picks([engines[w] for w in active], _SIM_POLL, self.rules)
            done += _SIM_POLL
            for w in list(active):
                if engines[w].read_ctl().viable:
                    verdict[w] = True
                    active.remove(w)
        for w in active:                      # tails (and a lone survivor) finish on their own
            verdict[w], _ = self._sim_finish(engines[w], done, left[w])
        return [bool(v) for v in verdict]

    def _fill(self, budget: int, k: int) -> int:
        """Unrestricted FPS for ``budget`` picks (hot loop C).  Same picks in the same order as the
        reference's per-pick loop; the host synchronises once per chunk."""
        if budget <= 0:
            return budget
        if not self._key_valid:
            self.E.scan()
            self._key_valid = True
        # Safe points (where a mid-layer checkpoint may be written) follow the reference: after every
        # chunk of CORESETS_FILL_CHUNK picks when that knob is set (sharded.py:219-295), after every
        # pick otherwise (_base.py:528-540) -- there the picks still run in chunks, cut so that the
        # checkpoint cadence falls on a chunk end.
        if self.trace.active:
            chunk = 1
        elif self.fill_chunk > 0 and len(self.selected) > 0:
            chunk = self.fill_chunk
        else:
            chunk = 256
            if self.checkpoint_every:
                chunk = max(1, min(chunk, self.checkpoint_every))
        while budget > 0:
            m = min(chunk, budget)
            n0 = len(self.selected)
            self.E.run_picks(m)
            idx = self.E.selected[n0 : n0 + m].tolist()
            val = self.E.eps[n0 : n0 + m].tolist()
            if min(idx) < 0 or min(val) < -0.5:
                # a selected row was picked again: the pool ran dry (sharded.py:274-283)
                raise RuntimeError(
                    f"{self.name}: fill committed an invalid pick (min idx={min(idx)}, "
                    f"min val={min(val):.3e}) - candidate pool exhausted. This cannot happen for "
                    "n_target <= N_global."
                )
            self._absorb(idx, val)
            budget -= m
            self._maybe_midlayer_ckpt(k)
        return budget

    def _absorb(self, idx: List[int], val: List[float]) -> None:
        for g, v in zip(idx, val):
            self.sep = min(self.sep, v)
            pos = self._record(int(g))
            self.trace("fill", pos, int(g), v, self.sep)

    # ------------------------------------------------------------------ one nested block
    def _do_block(self, desired: List[int], budget: int, pos: int) -> int:
        """snapshot -> restricted greedy forward -> largest viable prefix -> roll back -> replay
        (_base.py:375-509, accrete.py:122-222).  Returns the budget left."""
        self._pos, self._n_probe = pos, 0
        if self.chatty and self.multi:
            print(f"  [block] k={self._k} pos={pos}: bisect start (desired={len(desired):,}, budget={budget:,})",
                  flush=True)
        with self.timer("snapshot_s"):
            snap = self._take_snapshot()

        if self.bisect_seeded:                       # seed of the walk (_base.py:386-403)
            prev, prev2 = self._seed_by_pos.get(pos), self._seed_prev_by_pos.get(pos)
            self._has_seed = prev is not None
            if self.gallop_deep and prev is not None and prev2 is not None and prev2 > 0:
                est = round(prev * prev / prev2)
                self._bisect_seed = max(prev // 2, min(2 * prev, est))
            elif prev is None:
                self._bisect_seed = search.GALLOP_MAX_SEED + 1
            else:
                self._bisect_seed = 2 * prev if pos == 0 else prev

        added: List[int] = []
        step_seps: List[float] = [snap.sep]
        max_add = min(budget, len(desired))
        state = {"pool": torch.tensor(desired, dtype=torch.long, device=self.device), "dry": False}

        device_walk = self.E.on_cuda and self.E.n_host is not None and _env_int("CORESETS_B200_DEVICE_FORWARD", 1) == 1

        def forward_to(n_picks: int) -> int:
            with self.timer("select_block_s"):
                want = min(n_picks, max_add) - len(added)
                if device_walk and want > 0 and not state["dry"]:
                    # the whole walk on the device (the pool keeps its selected rows: they carry h = -1 and
                    # can only win when nothing positive is left, which ends the walk)
                    n0 = len(self.selected)
                    made, dry = self.E.run_restricted(state["pool"], want)
                    idxs = self.E.selected[n0 : n0 + made].tolist()
                    vals = self.E.eps[n0 : n0 + made].tolist()
                    for idx, val in zip(idxs, vals):
                        self.sep = min(self.sep, val)
                        step_seps.append(self.sep)
                        added.append(int(idx))
                        self.trace("forward", self._record(int(idx)), int(idx), val, self.sep)
                    state["dry"] = dry or made < want
                    self._key_valid = made > 0 and not dry
                    return len(added)
                while len(added) < min(n_picks, max_add) and not state["dry"]:
                    val, idx = self._restricted_argmax(state["pool"])
                    if val <= 0.0 or idx < 0:        # every remaining pool row is already selected
                        state["dry"] = True
                        break
                    self.sep = min(self.sep, val)
                    step_seps.append(self.sep)
                    added.append(idx)
                    sel_pos = self._record(idx)
                    self.trace("forward", sel_pos, idx, val, self.sep)
                    self._commit_known(idx, val)
                    state["pool"] = state["pool"][state["pool"] != idx]
            return len(added)

        deep_walk = self.gallop_deep and self._has_seed and pos >= 1
        lazy = self.lazy_forward and (self._bisect_seed <= search.GALLOP_MAX_SEED or deep_walk)
        forward_to(self._bisect_seed + 1 if lazy else max_add)
        if not added:
            return budget

        def freeze_final() -> None:
            self.h_final.copy_(self.E.h)
            self.v_final.copy_(self.E.voronoi)

        freeze_final()
        sel_start_t = torch.tensor(snap.selected, dtype=torch.long, device=self.device)
        extend_to = None
        if lazy:
            def extend_to(m: int) -> int:
                before = len(added)
                now = forward_to(m)
                if now > before:
                    freeze_final()
                return now

        t0 = time.perf_counter()
        with self.timer("bisect_s"):
            if self.multi:
                best_m = self._bisect_sharded(snap, added, sel_start_t, step_seps, budget, max_add, extend_to)
            else:
                best_m = self._bisect_single(snap, added, sel_start_t, step_seps, budget)
        if self.chatty and self.multi:
            print(f"  [block] k={self._k} pos={pos}: best_m={best_m:,}  (bisect {time.perf_counter() - t0:.1f}s, "
                  f"{self._n_probe} sim-probes) -> replay + fill", flush=True)
        if self.bisect_seeded:
            if pos in self._seed_by_pos:
                self._seed_prev_by_pos[pos] = self._seed_by_pos[pos]
            self._seed_by_pos[pos] = best_m

        self._rollback(snap)
        with self.timer("replay_s"):
            for j in range(best_m):
                idx = added[j]
                sel_pos = self._record(idx)
                self.sep = step_seps[j + 1]
                self.trace("replay", sel_pos, idx, self.sep, self.sep)
            # the kept picks go back in as one run of prescribed picks (replayed from CUDA graphs on
            # the device) instead of one forced pick at a time
            if best_m > 0:
                self.E.run_forced(added[:best_m], values=step_seps[1 : best_m + 1])
                self._key_valid = True
        return budget - best_m

    # ------------------------------------------------------------------ bisect, single-GPU flavour
    def _bisect_single(self, snap: _Snapshot, added: List[int], sel_start_t: Tensor, step_seps: List[float],
                       total_budget: int) -> int:
        """Plain binary search with the reference's shortcuts (cuda/_internal/bisect.py:15-129)."""
        added_t = torch.tensor(added, dtype=torch.long, device=self.device)
        n_start = snap.n_selected
        N = self.n_global

        def viable(mid: int) -> bool:
            sep_mid = step_seps[mid]
            points_left = total_budget - mid
            if n_start + mid + points_left >= N:
                return True
            self._reconstruct(snap, added_t, sel_start_t, mid)
            # after a fill of points_left picks the coverage is at most the (points_left + 1)-th
            # largest live h: the reference's kthvalue early exit (bisect.py:64-71) as one exact
            # device-side selection (count and value in a single read-back)
            cov_upper, n_pos = self.S.kth_largest_live(points_left + 1)
            if 0 < points_left < n_pos:
                if sep_mid > cov_upper:
                    return True
            elif points_left >= n_pos:
                return True
            if points_left == 0:
                return sep_mid > cov_upper           # k = 1: the maximum of the live rows (bisect.py:78-80)
            ok, _ = self._simulate(float(sep_mid), points_left, n_start + mid)
            self._n_probe += 1
            return ok

        return search.binary_search(viable, len(added))

    # ------------------------------------------------------------------ bisect, sharded flavour
    def _bisect_sharded(self, snap: _Snapshot, added: List[int], sel_start_t: Tensor, step_seps: List[float],
                        total_budget: int, max_add: int, extend_to: Optional[Callable[[int], int]]) -> int:
        """Largest viable prefix with the sharded driver's shortcuts, memo, seeded walk and lazy
        forward (_base.py:556-732)."""
        ctx = {"n_added": len(added), "added_t": torch.tensor(added, dtype=torch.long, device=self.device)}

        def refresh() -> None:
            ctx["n_added"] = len(added)
            ctx["added_t"] = torch.tensor(added, dtype=torch.long, device=self.device)

        memo: Dict[int, bool] = {}

        def classify(mid: int, target=None):
            if mid > ctx["n_added"]:
                if extend_to is not None and extend_to(mid) > ctx["n_added"]:
                    refresh()
                if mid > ctx["n_added"]:
                    return False                      # past the natural end of the forward pass
            sep_mid = step_seps[mid] / self.cov_relax
            points_left = total_budget - mid
            if snap.n_selected + mid + points_left >= self.n_global:
                return True
            # rows outside the prefix (selected rows are distinct, so the all-reduced count of
            # _base.py:574-597 is N_global minus the prefix length)
            if points_left >= self.n_global - (snap.n_selected + mid):
                return True
            self._reconstruct(snap, ctx["added_t"], sel_start_t, mid, target)
            if points_left == 0:
                return sep_mid > self._global_max((target or self.S).h)
            return {"sep": sep_mid, "points_left": points_left, "n_init": snap.n_selected + mid}

        def viable(mid: int) -> bool:
            if mid in memo:
                return memo[mid]
            probe = classify(mid)
            if isinstance(probe, bool):
                memo[mid] = probe
                return probe
            t0 = time.perf_counter()
            ok, _ = self._simulate(float(probe["sep"]), probe["points_left"], probe["n_init"])
            memo[mid] = ok
            self._n_probe += 1
            if self.chatty:
                print(f"    [bisect] k={self._k} pos={self._pos} probe#{self._n_probe} mid={mid:,} "
                      f"sim_fill={probe['points_left']:,} -> viable={ok} ({time.perf_counter() - t0:.1f}s)",
                      flush=True)
            return ok

        deep_walk = self.gallop_deep and self._has_seed and self._pos >= 1
        if self.bisect_seeded and (self._bisect_seed <= search.GALLOP_MAX_SEED or deep_walk):
            high = max_add if extend_to is not None else ctx["n_added"]
            seed = max(0, min(int(self._bisect_seed), high))
            first_probe = seed if seed > 0 else 1            # the walk never probes m = 0
            # the walk's first probes as fused lanes; the walk then reads the memo (_base.py:702-726)
            if self.bisect_lanes >= 2 and total_budget - seed >= self.lanes_min_steps:
                engines = self._lane_engines(self.bisect_lanes)
                probes, mids = [], []
                for mid in range(first_probe, min(first_probe + len(engines), high + 1)):
                    if mid in memo:
                        continue
                    probe = classify(mid, engines[len(probes)])
                    if isinstance(probe, bool):
                        memo[mid] = probe
                    else:
                        probes.append(probe)
                        mids.append(mid)
                if len(probes) >= 2:
                    t0 = time.perf_counter()
                    for mid, ok in zip(mids, self._simulate_lanes(engines[: len(probes)], probes)):
                        memo[mid] = ok
                        self._n_probe += 1
                    if self.chatty:
                        print(f"    [bisect] k={self._k} pos={self._pos} lanes mids={mids} -> "
                              f"{[memo[m_] for m_ in mids]} ({time.perf_counter() - t0:.1f}s)", flush=True)
            return search.largest_true(viable, high, self._bisect_seed)
        return search.binary_search(viable, ctx["n_added"])

    # ------------------------------------------------------------------ layers
    def _check_invariant(self, k: int, target_size: int):
        """sep^2 must not fall grossly below cov^2 (diag.py:88-109, _shared.py:339-372)."""
        sep_sq = self.sep
        relax = self.cov_relax if self.multi else 1.0
        if self.multi and math.isfinite(sep_sq):
            sep_sq = max(0.0, sep_sq)
        cov_sq = max(0.0, self._global_max(self.E.h))
        sep_val, cov_val, rel_gap = invariant_numbers(cov_sq, sep_sq)
        if math.isfinite(sep_sq) and sep_sq < cov_sq * relax * relax * (1.0 - _GROSS_REL):
            where = f"k={k}" if self.multi else f"level k={k}"        # the two flavours' wording (_shared.py:365, diag.py:103)
            raise RuntimeError(
                f"{self.name}: sep > cov violated at {where} (size={target_size}): sep={sep_val:.8e}, "
                f"cov={cov_val:.8e}, rel_gap={rel_gap:.3e}. Gross violation, not float noise."
            )
        return sep_val, cov_val, rel_gap

    def _do_layer(self, k: int) -> None:
        target = min(2 ** k, self.max_sel)
        budget = target - len(self.selected)
        if budget <= 0:
            return
        self._k = k
        if self.E.on_cuda and not self.multi:
            torch.cuda.synchronize()
        t_layer = time.perf_counter()
        if self.chatty and self.multi:
            print(f"  [layer] k={k} start: budget={budget:,}  n_selected={len(self.selected):,}", flush=True)
        for pos, block in enumerate(self.nested_blocks[k - 1 :]):
            if budget <= 0:
                break
            desired = sorted(block - self.selected_set)
            if not desired:
                continue
            budget = self._do_block(desired, budget, pos)
            self._maybe_midlayer_ckpt(k)
        t_fill = time.perf_counter()
        with self.timer("fill_s"):
            budget = self._fill(budget, k)
        if self.E.on_cuda and not self.multi:
            torch.cuda.synchronize()
        t_end = time.perf_counter()
        sep_val, cov_val, rel_gap = self._check_invariant(k, target)
        if self.chatty:
            in_bk, from_a = level_counts(self.selected, target, self.nested_blocks[k - 1], self.n_anchor)
            if self.multi:
                print(f"{k:<4} | {target:<6} | {in_bk:>6} | {from_a:>7} | {target - from_a:>7} | "
                      f"{sep_val:>9.5f} | {cov_val:>9.5f} | {fmt_gap(rel_gap)} | {time.perf_counter() - t_layer:>8.2f}",
                      flush=True)
                print(f"  [time] k={k} block_bisect={t_fill - t_layer:8.1f}s  fill={t_end - t_fill:8.1f}s", flush=True)
            else:
                print(f"{k:<4} | {target:<10} | {in_bk:>10} | {from_a:>10} | {target - from_a:>10} | "
                      f"{t_end - t_layer:>9.2f} | {sep_val:>9.5f} | {cov_val:>9.5f} | {fmt_gap(rel_gap)}", flush=True)
        if self.multi:
            if self.checkpoint_path is not None and self.layout.rank == 0:
                self._write_layer_checkpoint(k, target)
                self._dump_seeds()
            self._last_ckpt_n = len(self.selected)

    def run(self) -> Tensor:
        if self.chatty:
            if self.multi:
                print(f"{self.name}: N={self.n_global}, D={self.dim}, max_k={self.max_k}, "
                      f"world_size={self.layout.world_size}")
                print(f"  shard sizes = {self.layout.sizes}")
                print(f"{'k':<4} | {'size':<6} | {'in_Bk':>6} | {'from_A':>7} | {'from_C':>7} | "
                      f"{'sep':>9} | {'cov':>9} | {'rel_gap':>11} | {'dt_s':>8}")
                print("-" * 90)
            else:
                print(f"{'k':<4} | {'size':<10} | {'in_Bk':>10} | {'from_A':>10} | {'from_C':>10} "
                      f"| {'time_s':>9} | {'sep':>9} | {'cov':>9} | {'rel_gap':>11}")
                print("-" * 104)
        if self.resume_from is not None:
            start_k = self._resume(self.resume_from)
        else:
            first = self.anchor_indices[0]
            self._record(first)
            self._commit_known(first, float("inf"))
            start_k = 1
        for k in range(start_k, self.max_k + 1):
            self._do_layer(k)
        self.E.check_status()
        if self.profile and self.layout.rank == 0:
            self.timer.report(f"{self.name} phases")
        self.trace.close()
        return torch.tensor(self.selected, dtype=torch.long, device=self.device)

    # ------------------------------------------------------------------ checkpoints (sharded flavour)
    @staticmethod
    def _save(path: str, arr: np.ndarray) -> None:
        with open(path + ".tmp", "wb") as f:
            np.save(f, arr, allow_pickle=False)
        os.replace(path + ".tmp", path)

    @staticmethod
    def _save_text(path: str, text: str) -> None:
        with open(path + ".tmp", "w") as f:
            f.write(text)
        os.replace(path + ".tmp", path)

    def _write_layer_checkpoint(self, k: int, target_size: int) -> None:
        """`<prefix>_kKK.npy`, `<prefix>_kKK_sep.npy`, then `<prefix>_latest.txt` = "k"
        (sharded.py:754-775)."""
        p = self.checkpoint_path
        self.E.check_status()     # a device-side time-out leaves garbage picks: raise, do not publish them
        ids = np.asarray(self.selected[:target_size], dtype=np.int64)
        self._save(f"{p}_k{k:02d}.npy", ids)
        self._save(f"{p}_k{k:02d}_sep.npy", np.asarray([self.sep], dtype=np.float64))
        self._save_text(f"{p}_latest.txt", f"{k}\n")
        if self.verbose:
            print(f"  [checkpoint] k={k} => {p}_k{k:02d}.npy ({len(ids):,} points)")

    def _dump_seeds(self) -> None:
        """Seeds side-car int64[n, 3] = (position, best_m, best_m two layers ago or -1)
        (sharded.py:498-519)."""
        if self.checkpoint_path is None or self.layout.rank != 0 or not self._seed_by_pos:
            return
        rows = [[p, m, self._seed_prev_by_pos.get(p, -1)] for p, m in self._seed_by_pos.items()]
        self._save(f"{self.checkpoint_path}_seeds.npy", np.asarray(rows, dtype=np.int64))

    def _maybe_midlayer_ckpt(self, k: int) -> None:
        """Rolling mid-layer dump every ``checkpoint_every`` picks at safe points; latest.txt then
        holds "k n" (_base.py:812-821, sharded.py:521-549)."""
        if not (self.multi and self.checkpoint_every):
            return
        n = len(self.selected)
        if n >= min(2 ** k, self.max_sel) or n - self._last_ckpt_n < self.checkpoint_every:
            return
        self._last_ckpt_n = n
        if self.checkpoint_path is None or self.layout.rank != 0:
            return
        p = self.checkpoint_path
        self.E.check_status()
        self._save(f"{p}_mid.npy", np.asarray(self.selected, dtype=np.int64))
        self._save(f"{p}_mid_sep.npy", np.asarray([self.sep], dtype=np.float64))
        self._save_text(f"{p}_latest.txt", f"{k} {n}\n")
        self._dump_seeds()
        if self.verbose:
            print(f"  [checkpoint] mid-layer k={k} n={n:,} => {p}_mid.npy", flush=True)

    def _resume(self, prefix: str) -> int:
        """Restore from the last layer or mid-layer checkpoint (_base.py:212-299).  The state is
        rebuilt by replaying the stored picks through the same kernels, so the continued run is
        bit-identical to an uninterrupted one."""
        latest = f"{prefix}_latest.txt"
        if not os.path.exists(latest):
            raise FileNotFoundError(f"resume requires {latest}; not found.")
        toks = open(latest).read().split()
        k0 = int(toks[0])
        if k0 > self.max_k:
            raise ValueError(f"resume checkpoint is at layer k0={k0} but max_k={self.max_k}; "
                             "the checkpoint already exceeds the requested target. Increase max_k to extend.")
        if len(toks) >= 2:
            n0 = int(toks[1])
            ids = np.load(f"{prefix}_mid.npy").astype(np.int64, copy=False)
            if ids.shape[0] != n0:
                raise ValueError(f"resume {prefix}_mid.npy has {ids.shape[0]} ids, latest says {n0}")
            lo, hi = 2 ** (k0 - 1), min(2 ** k0, self.max_sel)
            if not lo <= n0 <= hi:
                raise ValueError(f"mid-layer resume n={n0} outside layer k={k0} range [{lo},{hi}]")
            sep_file = f"{prefix}_mid_sep.npy"
            start_k = k0 if n0 < hi else k0 + 1
        else:
            ids = np.load(f"{prefix}_k{k0:02d}.npy").astype(np.int64, copy=False)
            expected = min(2 ** k0, self.max_sel)
            if ids.shape[0] != expected:
                raise ValueError(f"resume {prefix} k={k0}: {ids.shape[0]} ids, expected {expected}")
            sep_file = f"{prefix}_k{k0:02d}_sep.npy"
            start_k = k0 + 1
        if os.path.exists(sep_file):
            sep_prev = float(np.load(sep_file)[0])
        else:
            sep_prev = float("inf")
            if self.layout.rank == 0:
                print(f"  [resume] WARNING: {sep_file} missing - sep restored as inf, so the sep>cov layer "
                      "check is vacuous until new picks re-establish it.", flush=True)
        for g in ids.tolist():
            self._record(int(g))
            self._commit_known(int(g), float("inf"))
        self.sep = sep_prev
        self._last_ckpt_n = len(self.selected)
        seeds_file = f"{prefix}_seeds.npy"
        if os.path.exists(seeds_file):
            try:
                arr = np.load(seeds_file)
                self._seed_by_pos = {int(r[0]): int(r[1]) for r in arr}
                if arr.shape[1] >= 3:
                    self._seed_prev_by_pos = {int(r[0]): int(r[2]) for r in arr if int(r[2]) >= 0}
            except Exception as e:  # unreadable side-car: cold start of the search
                if self.chatty:
                    print(f"  [resume] seeds sidecar unreadable ({e}); cold-start binary search", flush=True)
        if self.chatty:
            print(f"  [resume] restored {len(self.selected):,} centers (k={k0}, sep={sep_prev:.6g}); "
                  f"continuing from layer {start_k} to {self.max_k}", flush=True)
        return start_k


def resolve_max_k(max_k: Optional[int], n_total: int, dim: int, elem_bytes: int, device: torch.device,
                  *, strict: bool, collective: bool) -> Tuple[int, int]:
    """``max_k`` from free device memory when the caller did not pin it: 30 % of the free bytes
    for two copies of the centre rows plus five scalars per centre, capped by ``log2 N``.
    ``strict`` (single-GPU entry, scratch.py:62-90) also rejects a pinned value that does not fit;
    ``collective`` (sharded entry, _shared.py:316-336) takes the minimum over ranks."""
    per_row = 2 * dim * elem_bytes + 5 * 4
    if device.type == "cuda":
        free_bytes, _ = torch.cuda.mem_get_info(device)
    else:
        free_bytes = 1 << 40
    budget = int(free_bytes * 0.30)
    fit_k = max(1, int(math.log2(max(1, budget // per_row))))
    if max_k is None:
        max_k = min(int(math.log2(n_total)), fit_k)
        if collective:
            t = torch.tensor([max_k], dtype=torch.long, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            max_k = int(t.item())
    max_sel = 2 ** max_k
    if strict:
        need = 2 * max_sel * dim * elem_bytes + 5 * max_sel * 4
        if need > budget:
            raise ValueError(
                f"Coreset buffers need {need / 1e9:.1f} GB (2^max_k={max_sel}, D={dim}) but budget is "
                f"{budget / 1e9:.1f} GB (30% of {free_bytes / 1e9:.1f} GB free). Safe max_k for this GPU: {fit_k}"
            )
    return max_k, max_sel
