"""Single-GPU accretion: drop-in for the reference's ``accrete``
(src/coresets/cuda/accrete.py:26-272)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .. import engine as _engine
from .accrete_core import AccreteDriver, resolve_max_k
from .multi.layout import ShardLayout

# the CPU test-suite clears this to drive the host logic with a stand-in native library
_REQUIRE_CUDA = True


def accrete(
    X_anchor: Tensor,
    X_candidates: Tensor,
    anchor_order: Tensor,
    max_k: Optional[int] = None,
    *,
    verbose: bool = True,
    profile: bool = False,
    trace_path: Optional[str] = None,
) -> Tensor:
    """Merge ``X_candidates`` into the FPS ordering ``anchor_order`` of ``X_anchor``.

    Returns ``2 ** max_k`` int64 indices into ``cat(X_anchor, X_candidates)`` (entries below
    ``len(X_anchor)`` come from the anchor) such that every prefix of length ``2 ** k`` is a valid
    coreset that keeps as much of the anchor hierarchy as the new data allows.  ``max_k`` is
    derived from free device memory when ``None``.  Validation and errors follow the reference
    (accrete.py:39-48)."""
    n_anchor, n_cand = X_anchor.shape[0], X_candidates.shape[0]
    if n_anchor == 0:
        raise ValueError("X_anchor is empty - need at least one anchor point.")
    if n_cand > 0 and X_anchor.shape[1] != X_candidates.shape[1]:
        raise ValueError(
            f"feature-dim mismatch: X_anchor={X_anchor.shape[1]}, X_candidates={X_candidates.shape[1]}"
        )
    if _REQUIRE_CUDA and not X_anchor.is_cuda:
        raise ValueError(f"X_anchor must be on a CUDA device, got {X_anchor.device}")
    if X_anchor.dtype not in (torch.float32, torch.float16):
        # float64 is not offered: the reference's reconstruct step cannot finish with it either (it
        # assigns a float64 result into the float32 h, which torch's index_put rejects)
        raise ValueError(f"X_anchor must be float32 or float16, got {X_anchor.dtype}")
    n_total, dim = n_anchor + n_cand, int(X_anchor.shape[1])
    X = (torch.cat([X_anchor, X_candidates], dim=0) if n_cand > 0 else X_anchor).contiguous()
    norms = _engine.row_norms(X)
    max_k, max_sel = resolve_max_k(max_k, n_total, dim, X.element_size(), X.device, strict=True, collective=False)
    layout = ShardLayout(rank=0, world_size=1, sizes=[n_total], offsets=[0])
    X32, element_order = _engine.engine_matrix(X)
    driver = AccreteDriver(X32, norms, layout, anchor_order.tolist(), n_anchor, n_total, max_k, max_sel,
                           flavour="single", verbose=verbose, profile=profile, trace_path=trace_path,
                           X_src=X if element_order else None)
    return driver.run()
