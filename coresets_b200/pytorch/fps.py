"""``fps``: farthest point sampling in plain torch, the reference's Python backend
(src/coresets/pytorch/fps.py:32-73).  Works on any device and float dtype torch supports.

Every pick is one dense pass: ``d = norms + norms[c] - 2 * X @ X[c]`` for the new centre ``c``
(:19-20), rows with ``d < h`` move to the new cell and take ``h = d`` (:23-27), the centre is marked
``h = -1``; the next pick is the first maximum of ``h`` (:66).  Summation order is torch's, not the
CUDA kernels': the two backends agree on radii to rounding, not bit for bit.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor


def fps(X: Tensor, n_to_select: int, selected_idx: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """Return ``(selected, epsilons, hausdorff, voronoi)``.

    ``selected`` int64 ``[n_to_select]`` starts with ``selected_idx`` (default: row 0);
    ``epsilons[i]`` is ``max h`` before pick ``i`` (0.0 for a seeded pick made while nothing is
    selected, :59-62); ``hausdorff`` is the final squared distance of every row to its nearest
    pick (-1 on picks) and ``voronoi`` the position of that pick in ``selected``.
    """
    n_rows = X.shape[0]
    opts = dict(dtype=X.dtype, device=X.device)
    norms = (X * X).sum(dim=1)
    h = torch.full((n_rows,), float("inf"), **opts)
    cell = torch.zeros(n_rows, dtype=torch.long, device=X.device)
    picks = torch.empty(n_to_select, dtype=torch.long, device=X.device)
    radii = torch.zeros(n_to_select, **opts)
    dist = torch.empty(n_rows, **opts)
    given = [0] if selected_idx is None else [int(v) for v in selected_idx.tolist()]
    picks[: len(given)] = torch.as_tensor(given, dtype=torch.long, device=X.device)

    for pos in range(n_to_select):
        if pos < len(given):
            centre = given[pos]
            before = float(h[centre])
            radii[pos] = 0.0 if before == float("inf") else before
        else:
            centre = int(torch.argmax(h))
            radii[pos] = h[centre]
            picks[pos] = centre
        dist.copy_(norms).add_(norms[centre])
        torch.addmv(dist, X, X[centre], beta=1, alpha=-2, out=dist)
        cell.masked_fill_(dist < h, pos)
        torch.minimum(h, dist, out=h)
        h[centre] = -1.0
    return picks, radii, h, cell


def fps_update(X: Tensor, norms: Tensor, d: Tensor, hausdorff: Tensor, voronoi: Tensor, new_idx: int, sel_idx: int) -> None:
    """One dense update in place for the new centre ``X[new_idx]`` committed at position ``sel_idx``
    (src/coresets/pytorch/fps.py:8-28); ``d`` is scratch of the rows' shape."""
    d.copy_(norms).add_(norms[new_idx])
    torch.addmv(d, X, X[new_idx], beta=1, alpha=-2, out=d)
    voronoi.masked_fill_(d < hausdorff, sel_idx)
    torch.minimum(hausdorff, d, out=hausdorff)
    hausdorff[new_idx] = -1.0


def voronoi_fps(X: Tensor, n_to_select: int, selected_idx: Optional[Tensor] = None,
                full_fraction: float = 0.5) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """``fps`` with the triangle bound (src/coresets/pytorch/fps.py:77-176): a row of cell ``j`` can
    only move to the new centre when a quarter of the squared distance between the two centres is
    below its ``h``; rows that cannot are left out of the distance pass, and when more than
    ``full_fraction`` of the rows remain the dense update is used instead.  Same return value as ``fps``."""
    n_rows, dim = X.shape
    opts = dict(dtype=X.dtype, device=X.device)
    norms = (X * X).sum(dim=1)
    h = torch.full((n_rows,), float("inf"), **opts)
    cell = torch.zeros(n_rows, dtype=torch.long, device=X.device)
    picks = torch.empty(n_to_select, dtype=torch.long, device=X.device)
    radii = torch.zeros(n_to_select, **opts)
    dist = torch.empty(n_rows, **opts)
    centres = torch.empty((n_to_select, dim), **opts)
    centre_norms = torch.empty(n_to_select, **opts)
    given = [0] if selected_idx is None else [int(v) for v in selected_idx.tolist()]
    picks[: len(given)] = torch.as_tensor(given, dtype=torch.long, device=X.device)
    for pos, c in enumerate(given):                       # seeds: dense updates, radii stay 0 (:111-118)
        centres[pos], centre_norms[pos] = X[c], norms[c]
        fps_update(X, norms, dist, h, cell, c, pos)
    dense_above = int(full_fraction * n_rows)
    for pos in range(len(given), n_to_select):
        c = int(torch.argmax(h))
        picks[pos], radii[pos] = c, h[c]
        centres[pos], centre_norms[pos] = X[c], norms[c]
        quarter = (centre_norms[:pos] + norms[c] - 2.0 * (centres[:pos] @ X[c])) * 0.25
        active = quarter[cell] < h
        n_active = int(active.sum())
        if n_active == 0:
            pass
        elif n_active <= dense_above:
            rows = torch.where(active)[0]
            d_rows = norms[rows] + norms[c] - 2.0 * (X[rows] @ X[c])
            closer = d_rows < h[rows]
            h[rows[closer]] = d_rows[closer]
            cell[rows[closer]] = pos
        else:
            dist.copy_(norms).add_(norms[c])
            torch.addmv(dist, X, X[c], beta=1, alpha=-2, out=dist)
            cell.masked_fill_(dist < h, pos)
            torch.minimum(h, dist, out=h)
        h[c] = -1.0
        cell[c] = pos
    return picks, radii, h, cell
