"""``accrete`` in plain torch: the reference's Python backend of the accretion algorithm
(src/coresets/pytorch/accrete.py:12-247, src/coresets/pytorch/_internal/phases.py:11-225).  Runs on
whatever device the matrices live on; the CUDA drivers (``coresets_b200.accrete``,
``accrete_sharded``) never come through here.

Algorithm.  The global matrix is ``cat(X_anchor, X_candidates)``; layer ``k`` brings the selection to
``2**k`` rows.  For every nested anchor block (the first ``2**i`` entries of ``anchor_order``, i >= k)
while budget is left: snapshot the state, run a greedy farthest-point walk restricted to the block's
unselected rows, find by binary search the largest prefix ``m`` of that walk after which an
unrestricted fill of the remaining budget still ends with separation > coverage, roll back and
replay ``m`` picks.  What is left of the layer's budget is filled by unrestricted picks.  A layer
whose separation falls more than 1e-3 (relative, squared) below its coverage aborts.

Every pick is one step with the triangle bound (``_State.commit``): rows of cell ``j`` whose ``h`` is
not above a quarter of the squared distance between centre ``j`` and the new centre cannot move and
are left out; above half of the rows the dense product is used instead.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
from torch import Tensor


class _State:
    """``h`` (squared distance to the nearest pick, -1 on picks), the cell of every row and the table
    of picked rows, advanced one pick at a time."""

    def __init__(self, X: Tensor):
        n, dim = X.shape
        self.n_rows, self.dim, self.device = n, dim, X.device
        self.opts = dict(dtype=X.dtype, device=X.device)
        self.X = X
        self.norms = (X * X).sum(dim=1)
        self.h = torch.full((n,), float("inf"), **self.opts)
        self.cell = torch.zeros(n, dtype=torch.long, device=X.device)
        self.scratch = torch.empty(n, **self.opts)
        self.dense_above = int(0.5 * n)

    def reserve(self, capacity: int) -> None:
        self.centres = torch.empty((capacity, self.dim), **self.opts)
        self.centre_norms = torch.empty(capacity, **self.opts)

    def dense(self, h: Tensor, cell: Tensor, row: int, pos: int) -> None:
        """Dense update of (h, cell) for the pick ``row`` at position ``pos`` (fps.py:8-28)."""
        d = self.scratch
        d.copy_(self.norms).add_(self.norms[row])
        torch.addmv(d, self.X, self.X[row], beta=1, alpha=-2, out=d)
        cell.masked_fill_(d < h, pos)
        torch.minimum(h, d, out=h)
        h[row] = -1.0

    def commit(self, row: int, pos: int) -> None:
        """One pick with the triangle bound (phases.py:11-70)."""
        X, norms, h, cell = self.X, self.norms, self.h, self.cell
        self.centres[pos] = X[row]
        self.centre_norms[pos] = norms[row]
        c, c_norm = self.centres[pos], self.centre_norms[pos]
        if pos == 0:
            self.dense(h, cell, row, pos)
            return
        quarter = (self.centre_norms[:pos] + c_norm - 2.0 * (self.centres[:pos] @ c)) * 0.25
        active = quarter[cell] < h
        if bool(active.any()):
            if int(active.sum().item()) <= self.dense_above:
                rows = torch.where(active)[0]
                d_rows = norms[rows] + c_norm - 2.0 * (X[rows] @ c)
                closer = d_rows < h[rows]
                moved = rows[closer]
                h[moved] = d_rows[closer]
                cell[moved] = pos
            else:
                d = self.scratch
                d.copy_(norms).add_(c_norm)
                torch.addmv(d, X, c, beta=1, alpha=-2, out=d)
                cell.masked_fill_(d < h, pos)
                torch.minimum(h, d, out=h)
        h[row] = -1.0
        cell[row] = pos

    def h_after_prefix(self, h_snap: Tensor, h_final: Tensor, cell_final: Tensor, before: List[int], added: List[int],
                       m: int) -> Tensor:
        """``h`` as it was after only the first ``m`` walk picks: rows whose final cell lies in the
        dropped tail are recomputed against the snapshot and the kept picks (phases.py:74-138)."""
        X, norms = self.X, self.norms
        out = h_final.clone()
        stale = cell_final >= (len(before) + m)
        if m != len(added) and bool(stale.any()):
            rows = torch.where(stale)[0]
            if m == 0:
                out[rows] = h_snap[rows]
            else:
                kept = torch.tensor(added[:m], dtype=torch.long, device=X.device)
                X_kept, n_kept = X[kept], norms[kept]
                X_rows, n_rows = X[rows], norms[rows]
                nearest = torch.full((len(rows),), float("inf"), dtype=X.dtype, device=X.device)
                step = max(1, 10_000_000 // max(len(rows), 1))
                for lo in range(0, m, step):
                    hi = min(lo + step, m)
                    tile = n_rows.unsqueeze(1) + n_kept[lo:hi].unsqueeze(0) - 2.0 * (X_rows @ X_kept[lo:hi].T)
                    torch.minimum(nearest, tile.min(dim=1).values, out=nearest)
                out[rows] = torch.minimum(h_snap[rows], nearest)
        out[torch.tensor(before + added[:m], dtype=torch.long, device=X.device)] = -1.0
        return out

    def largest_viable_prefix(self, h_snap: Tensor, h_final: Tensor, cell_final: Tensor, before: List[int],
                              added: List[int], seps: List[float], budget: int) -> int:
        """Binary search over the walk's prefixes (phases.py:142-225); a prefix ``m`` is viable when a fill
        of ``budget - m`` unrestricted picks ends with separation above coverage."""
        n = self.n_rows
        cell_unused = torch.zeros(n, dtype=torch.long, device=self.device)
        lo, hi, best = 0, len(added), 0
        while lo <= hi:
            m = (lo + hi) // 2
            left = budget - m
            ok = False
            if len(before) + m + left >= n:
                ok = True
            else:
                h = self.h_after_prefix(h_snap, h_final, cell_final, before, added, m)
                live = int((h >= 0).sum().item())
                if left >= live:
                    ok = True
                elif 0 < left and seps[m] > float(torch.kthvalue(h[h >= 0], live - left).values.item()):
                    ok = True                      # the coverage after the fill is at most that value
                else:
                    sep, pos = seps[m], len(before) + m
                    for _ in range(left):
                        far = int(torch.argmax(h).item())
                        sep = min(sep, float(h[far].item()))
                        self.dense(h, cell_unused, far, pos)
                        pos += 1
                        if sep > float(torch.max(h).item()):
                            ok = True
                            break
                    if not ok:
                        ok = sep > float(torch.max(h).item())
            if ok:
                best, lo = m, m + 1
            else:
                hi = m - 1
        return best


def _run(st: "_State", order, n_anchor: int, max_k: Optional[int], talk: bool, label: str) -> Tensor:
    """The accretion loop over a state (local or sharded); ``order`` lists the anchors' global rows."""
    n = st.n_rows
    if max_k is None:
        max_k = int(math.log2(n))
    blocks = [set(order[: min(2 ** i, n_anchor)]) for i in range(1, max_k + 1)]
    st.reserve(2 ** max_k)
    picked: List[int] = [order[0]]
    picked_set = {order[0]}
    sep = float("inf")
    st.commit(order[0], 0)

    def take(row: int) -> None:
        picked.append(row)
        picked_set.add(row)
        st.commit(row, len(picked) - 1)

    if talk:
        print(f"{'k':<4} | {'size':<6} | {'in_Bk':>6} | {'from_A':>7} | {'from_C':>7} | "
              f"{'sep':>9} | {'cov':>9} | {'rel_gap':>11}")
        print("-" * 79)

    for k in range(1, max_k + 1):
        size = 2 ** k
        budget = size - len(picked)
        if budget <= 0:
            continue
        for block in blocks[k - 1:]:
            if budget <= 0:
                break
            pool = sorted(block - picked_set)
            if not pool:
                continue
            h_snap, cell_snap, sep_snap, before = st.h.clone(), st.cell.clone(), sep, list(picked)
            added: List[int] = []
            seps: List[float] = [sep_snap]
            for _ in range(min(budget, len(pool))):              # greedy walk restricted to the pool
                at = int(torch.argmax(st.h[torch.tensor(pool, dtype=torch.long, device=st.device)]).item())
                row = pool[at]
                val = float(st.h[row].item())
                if val <= 0:
                    break
                sep = min(sep, val)
                seps.append(sep)
                added.append(row)
                take(row)
                pool[at] = pool[-1]
                pool.pop()
            if not added:
                continue
            keep = st.largest_viable_prefix(h_snap, st.h.clone(), st.cell.clone(), before, added, seps, budget)
            st.h.copy_(h_snap)                                   # roll back, then replay the kept prefix
            st.cell.copy_(cell_snap)
            picked = list(before)
            picked_set = set(before)
            for j in range(keep):
                take(added[j])
            sep = seps[keep]
            budget -= keep
        while budget > 0:                                        # unrestricted fill
            row = int(torch.argmax(st.h).item())
            sep = min(sep, float(st.h[row].item()))
            take(row)
            budget -= 1

        cov_sq = max(0.0, float(st.h.max().item()))
        sep_val = math.sqrt(max(sep, 0.0)) if math.isfinite(sep) else float("inf")
        cov_val = math.sqrt(cov_sq)
        rel_gap = (sep / cov_sq - 1.0) if (cov_sq > 0 and math.isfinite(sep)) else float("inf")
        if math.isfinite(sep) and sep < cov_sq * (1.0 - 1e-3):
            raise RuntimeError(
                f"{label}: sep > cov violated at k={k} (size={size}): "
                f"sep={sep_val:.8e}, cov={cov_val:.8e}, rel_gap={rel_gap:.3e}. "
                "Gross violation, not float noise."
            )
        if talk:
            layer = set(picked[:size])
            from_a = sum(1 for s in layer if s < n_anchor)
            gap = f"{rel_gap:>11.3e}" if math.isfinite(rel_gap) else f"{'inf':>11}"
            print(f"{k:<4} | {size:<6} | {len(layer & blocks[k - 1]):>6} | {from_a:>7} | {size - from_a:>7} | "
                  f"{sep_val:>9.5f} | {cov_val:>9.5f} | {gap}")
    return torch.tensor(picked, dtype=torch.long, device=st.device)


def accrete(X_anchor: Tensor, X_candidates: Tensor, anchor_order: Tensor, candidate_order: Tensor,
            max_k: Optional[int] = None, verbose: bool = True) -> Tensor:
    """int64 indices over ``cat(X_anchor, X_candidates)`` in selection order (indices below
    ``len(X_anchor)`` are anchors).  ``candidate_order`` is unused, kept for the reference's signature."""
    st = _State(torch.cat([X_anchor, X_candidates], dim=0))
    return _run(st, anchor_order.tolist(), int(X_anchor.shape[0]), max_k, verbose, "accrete")
