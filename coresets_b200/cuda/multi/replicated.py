"""Accretion with the whole matrix on every rank: drop-in for the reference's
``accrete_voronoi_multi`` (src/coresets/cuda/multi/replicated.py:252-308).

The reference keeps a second driver for this case because its sharded driver has to gather the
rows of new centres from their owners; here the candidate row travels with the arg-max key on
every pick anyway (one exchange per pick, resolved on the device), so a replicated matrix needs no
driver of its own: every rank takes the rows ``compute_shard_layout`` gives it and runs the
sharded driver on that slice.  The picks depend only on the rows and their global order, not on
who holds them -- which is also what the reference's determinism test demands of its three
drivers (tests/test_determinism.py: single, replicated and sharded give one list).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
from torch import Tensor

from .layout import compute_shard_layout
from .sharded import accrete_voronoi_multi_sharded


def accrete_voronoi_multi(
    X_A: Tensor,
    X_C: Tensor,
    idx_A: Tensor,
    rank: int,
    world_size: int,
    max_k: Optional[int] = None,
    verbose: bool = True,
    profile: bool = False,
    trace_path: Optional[str] = None,
) -> Tensor:
    """Global coreset indices over ``cat(X_A, X_C)``, identical on every rank.  ``X_A`` (anchors) and
    ``X_C`` (candidates) are the FULL matrices on every rank; ``idx_A`` orders the anchors."""
    if not dist.is_initialized():
        raise RuntimeError(
            "torch.distributed is not initialised. "
            "Call dist.init_process_group(backend='nccl') first."
        )
    n_anchor, n_cand = int(X_A.shape[0]), int(X_C.shape[0])
    if n_anchor == 0:
        raise ValueError("X_A is empty — need at least one anchor point.")
    dim = int(X_A.shape[1])
    if n_cand > 0 and X_C.shape[1] != dim:
        raise ValueError(f"feature-dim mismatch: X_A={dim}, X_C={X_C.shape[1]}")
    n_global = n_anchor + n_cand
    sizes, offsets = compute_shard_layout(n_global, world_size)
    lo, hi = offsets[rank], offsets[rank] + sizes[rank]
    # this rank's rows of cat(X_A, X_C), taken from the two parts without building the whole matrix
    parts = []
    if lo < n_anchor:
        parts.append(X_A[lo : min(hi, n_anchor)])
    if hi > n_anchor and n_cand > 0:
        parts.append(X_C[max(lo, n_anchor) - n_anchor : hi - n_anchor])
    X_local = (torch.cat(parts, dim=0) if len(parts) > 1 else parts[0]).contiguous() if parts \
        else X_A.new_empty((0, dim))
    return accrete_voronoi_multi_sharded(
        X_local, rank=rank, world_size=world_size, N_A_global=n_anchor, N_global=n_global, shard_sizes=sizes,
        idx_A=idx_A, max_k=max_k, verbose=verbose, profile=profile, trace_path=trace_path,
    )
