"""Searches for the largest viable prefix length of a bisect block.

``viable(m)`` is monotone (true up to some boundary, false after), and every evaluation may cost
a whole simulated FPS fill, so the number and the kind of probes matter: a false probe runs its
full budget.  Two strategies, both returning the same boundary for every monotone predicate:

* ``binary_search``  -- the plain exact search of the reference
  (src/coresets/cuda/multi/_base.py:735-747);
* ``largest_true``   -- start at a seed (the previous layer's answer), walk in the direction the
  seed's verdict points to, stride 1 for the first ``linear`` successes and doubling afterwards,
  then bisect the bracket (the reference's seeded walk, _base.py:751-809).  A walk that starts at
  seed 0 never spends a probe on m = 0, which cannot move the floor.
"""
from __future__ import annotations

from typing import Callable

GALLOP_MAX_SEED = 32   # seeds above this fall back to binary search (_base.py:41-42)
GALLOP_LINEAR = 4      # stride-1 probes before the stride doubles (_base.py:44-45)


def binary_search(viable: Callable[[int], bool], n: int) -> int:
    """Largest m in [0, n] with viable(m); 0 when nothing is viable."""
    lo, hi, best = 0, n, 0
    while lo <= hi:
        mid = (lo + hi) // 2
        if viable(mid):
            best, lo = mid, mid + 1
        else:
            hi = mid - 1
    return best


def _bracket(viable, start: int, limit: int, direction: int, linear: int):
    """Walk from ``start`` in ``direction`` (+1 / -1) while the verdict stays what it was at
    ``start``; returns (last position with the old verdict, first position with the new one or
    None when the range ended)."""
    stride, moves = 1, 0
    here = start
    probe = here + direction
    while (probe <= limit) if direction > 0 else (probe >= limit):
        flipped = (not viable(probe)) if direction > 0 else viable(probe)
        if flipped:
            return here, probe
        here = probe
        moves += 1
        if moves >= linear:
            stride *= 2
        probe = here + direction * stride
    return here, None


def largest_true(viable: Callable[[int], bool], n: int, seed: int, linear: int = GALLOP_LINEAR) -> int:
    """Largest m in [0, n] with viable(m) for a monotone predicate, searched outward from
    ``seed`` (clamped into [0, n]); 0 when nothing is viable."""
    seed = min(max(int(seed), 0), n)
    if seed == 0 or viable(seed):
        lo, hi = _bracket(viable, seed, n, +1, linear)      # lo viable (or the unprobed 0)
        if hi is None:
            hi = n + 1                                       # virtual "false" past the range
    else:
        hi, lo = _bracket(viable, seed, 0, -1, linear)      # hi not viable
        if lo is None:
            lo = -1                                          # virtual "true" below the range
    while hi - lo > 1:
        mid = (lo + hi) // 2
        if viable(mid):
            lo = mid
        else:
            hi = mid
    return max(lo, 0)
