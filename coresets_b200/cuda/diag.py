"""Tracing, phase timing and the per-level report of the accretion drivers.

Same observable behaviour as the reference's helpers (src/coresets/cuda/_internal/diag.py:11-141,
src/coresets/cuda/multi/_shared.py:339-414): the trace is an append-only TSV with hex floats so a
test can recover every bit; phase totals are wall-clock seconds with a device synchronise on
both sides of a scope when profiling is on.
"""
from __future__ import annotations

import math
import time
from contextlib import contextmanager
from typing import Dict, Iterable, Optional, Set

import torch

PHASES = ("snapshot_s", "select_block_s", "bisect_s", "replay_s", "fill_s", "voronoi_step_s")


class Tracer:
    """``phase<TAB>sel_pos<TAB>idx<TAB>val.hex()<TAB>sep.hex()`` per commit; no-op without a path."""

    def __init__(self, path: Optional[str]):
        self._f = open(path, "w") if path else None

    @property
    def active(self) -> bool:
        return self._f is not None

    def __call__(self, phase: str, sel_pos: int, idx: int, val: float, sep: float) -> None:
        if self._f is not None:
            self._f.write(f"{phase}\t{sel_pos}\t{idx}\t{float(val).hex()}\t{float(sep).hex()}\n")

    def close(self) -> None:
        if self._f is not None:
            self._f.close()
            self._f = None


class PhaseTimer:
    def __init__(self, enabled: bool, on_cuda: bool):
        self.enabled = enabled
        self.on_cuda = on_cuda
        self.totals: Dict[str, float] = {}

    @contextmanager
    def __call__(self, phase: str):
        if not self.enabled:
            yield
            return
        if self.on_cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if self.on_cuda:
                torch.cuda.synchronize()
            self.totals[phase] = self.totals.get(phase, 0.0) + time.perf_counter() - t0

    def report(self, header: str) -> None:
        total = sum(self.totals.values())
        print(f"\n[Profile: {header}]")
        for key in PHASES:
            val = self.totals.get(key, 0.0)
            pct = 100.0 * val / total if total > 0 else 0.0
            print(f"  {key:<14} {val:8.3f}s  ({pct:5.1f}%)")


def invariant_numbers(cov_sq: float, sep_sq: float):
    """(sep, cov, relative gap) as the level report shows them."""
    sep_val = math.sqrt(max(sep_sq, 0.0)) if math.isfinite(sep_sq) else float("inf")
    cov_val = math.sqrt(cov_sq)
    rel_gap = (sep_sq / cov_sq - 1.0) if (cov_sq > 0 and math.isfinite(sep_sq)) else float("inf")
    return sep_val, cov_val, rel_gap


def level_counts(selected: Iterable[int], target_size: int, block_k: Set[int], n_anchor: int):
    sel_set = set(list(selected)[:target_size])
    return len(sel_set & block_k), sum(1 for s in sel_set if s < n_anchor)


def fmt_gap(rel_gap: float) -> str:
    return f"{rel_gap:>11.3e}" if math.isfinite(rel_gap) else f"{'inf':>11}"
