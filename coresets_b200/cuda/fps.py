"""Single-GPU farthest point sampling: drop-in for the reference's ``fps_cuda``
(src/coresets/cuda/fps.py:13-130)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .. import engine as _engine

# the CPU test-suite clears this to drive the host logic with a stand-in native library
_REQUIRE_CUDA = True


def fps(
    X: Tensor,
    n_to_select: int,
    *,
    seed: Optional[Tensor] = None,
    return_epsilons: bool = False,
):
    """Return int64 row indices of ``X`` in selection order (a device tensor).

    ``seed`` holds the first picks (1-D integer tensor, length in ``[1, n_to_select]``) and
    defaults to row 0.  Same validation and errors as the reference (fps.py:22-31, 57-66).
    ``return_epsilons=True`` (an addition) also returns the float32 device tensor of ``max h``
    before each pick (``+inf`` for seed picks).

    The whole loop runs on the device: per pick one bound kernel and one fused
    distance / min-update / arg-max kernel, replayed from a CUDA graph, no host read-back.
    """
    if _REQUIRE_CUDA and not X.is_cuda:
        raise ValueError(f"X must be on a CUDA device, got {X.device}")
    if X.dim() != 2:
        raise ValueError(f"X must be 2-D (N, D), got shape {tuple(X.shape)}")
    n_total, dim = X.shape
    if not 1 <= n_to_select <= n_total:
        raise ValueError(f"n_to_select={n_to_select} must be in [1, N={n_total}]")
    if X.dtype not in (torch.float32, torch.float64, torch.float16):
        raise ValueError(f"X must be float32, float64 or float16, got X.dtype={X.dtype}")

    if seed is not None:
        if seed.dim() != 1:
            raise ValueError(f"seed must be 1-D int64, got shape {tuple(seed.shape)}")
        seed_list = [int(v) for v in seed.to(dtype=torch.long).cpu().tolist()]
        n_seed = len(seed_list)
        if n_seed == 0 or n_seed > n_to_select:
            raise ValueError(f"seed length {n_seed} must be in [1, n_to_select={n_to_select}]")
        for v in seed_list:
            if not 0 <= v < n_total:
                raise ValueError(f"seed index {v} must be in [0, N={n_total})")
    else:
        seed_list = [0]

    X = X.contiguous()
    norms = _engine.row_norms(X)                       # in X's own dtype, as fps.py:34 does
    X32, element_order = _engine.engine_matrix(X)
    eng = _engine.ShardEngine(X32, norms, n_to_select, element_order=element_order, cells=True)
    eng.init_state()
    for idx in seed_list:
        eng.pick_forced(idx)
    eng.run_picks(n_to_select - len(seed_list))
    eng.check_status()
    if return_epsilons:
        return eng.selected, eng.eps
    return eng.selected
