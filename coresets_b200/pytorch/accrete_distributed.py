"""``accrete`` in plain torch over ``torch.distributed`` ranks: the reference's distributed Python
backend (src/coresets/pytorch/accrete_distributed.py:12-237, _internal/distributed_state.py:10-120,
_internal/phases_distributed.py:13-260).  The rows are sharded (the local slices in rank order form
the global matrix); ``h``, the cells and the table of picked rows are replicated, so every decision
is taken identically on every rank.  Communication per pick: one broadcast of the new centre's row
from its owner and one all-gather of the ranks' distance slices; a reconstruct step all-reduces (min)
the distances of the affected rows, each computed by the rank that owns the row.

The loop itself is the one of ``coresets_b200.pytorch.accrete``; only the state differs.
"""
from __future__ import annotations

import bisect
from typing import List, Optional

import torch
import torch.distributed as dist
from torch import Tensor

from .accrete import _State, _run


class _ShardedState(_State):
    """Rows on their owners, everything else replicated."""

    def __init__(self, X_local: Tensor, rank: int, world_size: int):
        self.rank, self.world = rank, world_size
        self.device = X_local.device
        self.opts = dict(dtype=X_local.dtype, device=X_local.device)
        self.dim = int(X_local.shape[1])
        mine = torch.tensor([X_local.shape[0]], dtype=torch.int64, device=self.device)
        sizes = [torch.zeros(1, dtype=torch.int64, device=self.device) for _ in range(world_size)]
        dist.all_gather(sizes, mine)
        self.sizes = [int(t.item()) for t in sizes]
        self.n_rows = sum(self.sizes)
        self.bounds = [0]
        for n in self.sizes:
            self.bounds.append(self.bounds[-1] + n)
        self.lo = self.bounds[rank]
        self.X = X_local
        self.norms = (X_local * X_local).sum(dim=1)
        self.h = torch.full((self.n_rows,), float("inf"), **self.opts)
        self.cell = torch.zeros(self.n_rows, dtype=torch.long, device=self.device)
        self.dense_above = int(0.5 * self.n_rows)
        self._d_local = torch.empty(self.sizes[rank], **self.opts)
        self._d_parts = [torch.empty(n, **self.opts) for n in self.sizes]
        self._d_full = torch.empty(self.n_rows, **self.opts)
        self._row = torch.empty(self.dim, **self.opts)

    # -- communication primitives (distributed_state.py:50-106) ------------------------------------
    def _centre(self, row: int) -> Tensor:
        """The row of global index ``row``, broadcast from its owner into a shared buffer."""
        owner = bisect.bisect_right(self.bounds, row) - 1
        if owner == self.rank:
            self._row.copy_(self.X[row - self.bounds[owner]])
        dist.broadcast(self._row, src=owner)
        return self._row

    def _gathered(self) -> Tensor:
        dist.all_gather(self._d_parts, self._d_local)
        at = 0
        for part in self._d_parts:
            self._d_full[at : at + part.shape[0]].copy_(part)
            at += part.shape[0]
        return self._d_full

    def _all_distances(self, c: Tensor) -> Tensor:
        c_norm = (c * c).sum()
        self._d_local.copy_(self.norms).add_(c_norm)
        torch.addmv(self._d_local, self.X, c, beta=1, alpha=-2, out=self._d_local)
        return self._gathered()

    def _active_distances(self, c: Tensor, active: Tensor) -> Tensor:
        """Distances of the active rows only (inf elsewhere); each rank computes its own rows."""
        c_norm = (c * c).sum()
        mine = active[self.lo : self.lo + self.sizes[self.rank]]
        self._d_local.fill_(float("inf"))
        if bool(mine.any()):
            rows = torch.where(mine)[0]
            self._d_local[rows] = self.norms[rows] + c_norm - 2.0 * (self.X[rows] @ c)
        return self._gathered()

    # -- the state's steps ---------------------------------------------------------------------------
    def dense(self, h: Tensor, cell: Tensor, row: int, pos: int) -> None:
        d = self._all_distances(self._centre(row))
        cell.masked_fill_(d < h, pos)
        torch.minimum(h, d, out=h)
        h[row] = -1.0

    def commit(self, row: int, pos: int) -> None:
        """One pick with the triangle bound on the replicated state (phases_distributed.py:13-72)."""
        h, cell = self.h, self.cell
        c = self._centre(row)
        c_norm = (c * c).sum()
        self.centres[pos] = c
        self.centre_norms[pos] = c_norm
        if pos == 0:
            d = self._all_distances(c)
            cell.masked_fill_(d < h, pos)
            torch.minimum(h, d, out=h)
            h[row] = -1.0
            return
        quarter = (self.centre_norms[:pos] + c_norm - 2.0 * (self.centres[:pos] @ c)) * 0.25
        active = quarter[torch.clamp(cell, max=pos - 1)] < h
        if bool(active.any()):
            if int(active.sum().item()) <= self.dense_above:
                d = self._active_distances(c, active)
                closer = (d < h) & active
                h[closer] = d[closer]
                cell.masked_fill_(closer, pos)
            else:
                d = self._all_distances(c)
                cell.masked_fill_(d < h, pos)
                torch.minimum(h, d, out=h)
        h[row] = -1.0
        cell[row] = pos

    def h_after_prefix(self, h_snap: Tensor, h_final: Tensor, cell_final: Tensor, before: List[int], added: List[int],
                       m: int) -> Tensor:
        """As the local version, with the affected rows split over their owners and an all-reduce (min)
        of the result (phases_distributed.py:76-164); the kept picks come from the replicated table."""
        n_before = len(before)
        out = h_final.clone()
        stale = cell_final >= (n_before + m)
        if m != len(added) and bool(stale.any()):
            rows = torch.where(stale)[0]
            if m == 0:
                out[rows] = h_snap[rows]
            else:
                X_kept = self.centres[n_before : n_before + m]
                n_kept = self.centre_norms[n_before : n_before + m]
                nearest = torch.full((len(rows),), float("inf"), **self.opts)
                own = (rows >= self.lo) & (rows < self.lo + self.sizes[self.rank])
                if bool(own.any()):
                    local = rows[own] - self.lo
                    X_rows, n_rows = self.X[local], self.norms[local]
                    best = torch.full((int(own.sum().item()),), float("inf"), **self.opts)
                    step = max(1, 10_000_000 // max(best.shape[0], 1))
                    for lo in range(0, m, step):
                        hi = min(lo + step, m)
                        tile = n_rows.unsqueeze(1) + n_kept[lo:hi].unsqueeze(0) - 2.0 * (X_rows @ X_kept[lo:hi].T)
                        torch.minimum(best, tile.min(dim=1).values, out=best)
                    nearest[torch.where(own)[0]] = best
                dist.all_reduce(nearest, op=dist.ReduceOp.MIN)
                out[rows] = torch.minimum(h_snap[rows], nearest)
        out[torch.tensor(before + added[:m], dtype=torch.long, device=self.device)] = -1.0
        return out


def accrete(X_local: Tensor, anchor_order: Tensor, n_anchor: int, rank: int, world_size: int,
            max_k: Optional[int] = None, verbose: bool = True) -> Tensor:
    """int64 global indices in selection order, identical on every rank.  ``X_local`` is this rank's
    slice of ``cat(anchors, candidates)``; the first ``n_anchor`` global rows are the anchors."""
    st = _ShardedState(X_local, rank, world_size)
    return _run(st, anchor_order.tolist(), int(n_anchor), max_k, verbose and rank == 0, "accrete (distributed)")
