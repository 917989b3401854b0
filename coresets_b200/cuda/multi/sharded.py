"""Multi-GPU accretion over row shards: drop-ins for the reference's ``accrete_sharded`` and
``accrete_voronoi_multi_sharded`` (src/coresets/cuda/multi/sharded.py:553-751)."""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
from torch import Tensor

from ... import engine as _engine
from ..accrete_core import AccreteDriver, resolve_max_k
from .layout import ShardLayout

# the CPU test-suite clears this to drive the host logic with gloo and a stand-in native library
_REQUIRE_CUDA = True


def accrete_voronoi_multi_sharded(
    X_local: Tensor,
    rank: int,
    world_size: int,
    N_A_global: int,
    N_global: int,
    shard_sizes: List[int],
    idx_A: Tensor,
    *,
    max_k: Optional[int] = None,
    n_target: Optional[int] = None,
    verbose: bool = True,
    profile: bool = False,
    trace_path: Optional[str] = None,
    checkpoint_path: Optional[str] = None,
    resume_from: Optional[str] = None,
    checkpoint_every: int = 0,
) -> Tensor:
    """Global coreset indices, identical on every rank.  Concatenating ``X_local`` over ranks in
    rank order must give ``cat(X_anchor, X_candidates)``; the first ``N_A_global`` rows are anchors."""
    if not dist.is_initialized():
        raise RuntimeError(
            "torch.distributed is not initialised. Call dist.init_process_group(backend='nccl') first."
        )
    # validation in the reference's order (sharded.py:692-726)
    if N_global >= 2 ** 31:
        raise ValueError(
            f"N_global={N_global} exceeds int32 range (2^31 - 1). The arg-max key carries the global "
            "row index in 32 bits."
        )
    if len(shard_sizes) != world_size:
        raise ValueError(f"shard_sizes has {len(shard_sizes)} entries; world_size={world_size}")
    if sum(shard_sizes) != N_global:
        raise ValueError(f"shard_sizes sums to {sum(shard_sizes)}, expected {N_global}")
    if any(s < 0 for s in shard_sizes):
        raise ValueError(f"shard_sizes has negatives: {shard_sizes}")
    if X_local.shape[0] != shard_sizes[rank]:
        raise ValueError(
            f"rank {rank}: X_local has {X_local.shape[0]} rows, expected shard_sizes[{rank}]={shard_sizes[rank]}"
        )
    if X_local.dim() != 2:
        raise ValueError(f"X_local must be 2-D, got shape {tuple(X_local.shape)}")
    if idx_A.numel() == 0:
        raise ValueError("idx_A is empty - need at least one anchor point.")
    if not 0 <= N_A_global <= N_global:
        raise ValueError(f"N_A_global={N_A_global} must be in [0, N_global={N_global}]")
    if _REQUIRE_CUDA and not X_local.is_cuda:
        raise ValueError(f"X_local must be on a CUDA device, got {X_local.device}")
    if X_local.dtype not in (torch.float32, torch.float16):
        # float64 is not offered: the reference's reconstruct step cannot finish with it either (it
        # assigns a float64 result into the float32 h, which torch's index_put rejects)
        raise ValueError(f"X_local must be float32 or float16, got {X_local.dtype}")

    X_local = X_local.contiguous()
    sizes = [int(s) for s in shard_sizes]
    offsets = [sum(sizes[:i]) for i in range(world_size)]
    layout = ShardLayout(rank=rank, world_size=world_size, sizes=sizes, offsets=offsets)
    device, dim = X_local.device, int(X_local.shape[1])

    d_pair = torch.tensor([dim, -dim], dtype=torch.long, device=device)
    dist.all_reduce(d_pair, op=dist.ReduceOp.MAX)
    d_max, d_min = int(d_pair[0].item()), -int(d_pair[1].item())
    if d_max != dim or d_min != dim:
        raise ValueError(
            f"D={dim} disagrees with peers (cluster min={d_min}, max={d_max}). "
            "Every rank must hold the same feature dim."
        )
    a_min, a_max = int(idx_A.min().item()), int(idx_A.max().item())
    if a_min < 0 or a_max >= N_global:
        raise ValueError(f"idx_A out of range: min={a_min}, max={a_max}; expected [0, {N_global})")

    norms_local = _engine.row_norms(X_local)
    max_k, max_sel = resolve_max_k(max_k, N_global, dim, X_local.element_size(), device,
                                   strict=False, collective=True)
    if n_target is not None:
        if not (2 ** (max_k - 1) < n_target <= 2 ** max_k):
            raise ValueError(
                f"n_target={n_target} must satisfy 2**(max_k-1) < n_target <= 2**max_k "
                f"({2 ** (max_k - 1)} < n_target <= {2 ** max_k} for max_k={max_k})"
            )
        if n_target > N_global:
            raise ValueError(f"n_target={n_target} exceeds the pool size N_global={N_global}")
        max_sel = n_target

    X32, element_order = _engine.engine_matrix(X_local)
    driver = AccreteDriver(X32, norms_local, layout, idx_A.tolist(), N_A_global, N_global, max_k, max_sel,
                           flavour="sharded", verbose=verbose, profile=profile, trace_path=trace_path,
                           checkpoint_path=checkpoint_path, resume_from=resume_from,
                           checkpoint_every=checkpoint_every, X_src=X_local if element_order else None)
    return driver.run()


def accrete_sharded(
    X_local: Tensor,
    anchor_order: Tensor,
    n_anchor: int,
    *,
    max_k: Optional[int] = None,
    n_target: Optional[int] = None,
    checkpoint_path: Optional[str] = None,
    resume_from: Optional[str] = None,
    checkpoint_every: int = 0,
    trace_path: Optional[str] = None,
    verbose: bool = True,
    profile: bool = False,
) -> Tensor:
    """Recommended entry: rank and shard layout are discovered from ``torch.distributed``; the
    first ``n_anchor`` rows of the global matrix are anchors, the rest candidates."""
    if not dist.is_initialized():
        raise RuntimeError(
            "torch.distributed must be initialised before accrete_sharded(). "
            "Call dist.init_process_group(backend='nccl', ...) first. "
            "For single-GPU runs, use coresets_b200.accrete instead."
        )
    if _REQUIRE_CUDA and not X_local.is_cuda:
        raise ValueError(
            f"X_local must be on a CUDA device, got {X_local.device}. "
            "Place each rank's shard on its local GPU before calling."
        )
    rank, world_size = dist.get_rank(), dist.get_world_size()
    sizes_t = torch.zeros(world_size, dtype=torch.long, device=X_local.device)
    sizes_t[rank] = X_local.shape[0]
    dist.all_reduce(sizes_t, op=dist.ReduceOp.SUM)
    shard_sizes = [int(v) for v in sizes_t.cpu().tolist()]
    return accrete_voronoi_multi_sharded(
        X_local, rank=rank, world_size=world_size, N_A_global=n_anchor, N_global=int(sum(shard_sizes)),
        shard_sizes=shard_sizes, idx_A=anchor_order, max_k=max_k, n_target=n_target, verbose=verbose,
        profile=profile, trace_path=trace_path, checkpoint_path=checkpoint_path, resume_from=resume_from,
        checkpoint_every=checkpoint_every,
    )
