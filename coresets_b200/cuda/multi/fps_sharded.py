"""Multi-GPU farthest point sampling over row shards: drop-in for the reference's
``fps_sharded`` (src/coresets/cuda/multi/fps_sharded.py:21-418).

Each rank holds a contiguous row range of X.  Per pick every rank runs the fused step kernel on
its rows; the rank's candidate -- a 64-bit (value, ~global index) key, the row's norm and the
row itself -- is published by the last block of that kernel and exchanged with ONE all-gather
over NCCL/NVLink; every rank then resolves the same winner on the device.  The pick counter,
the winner and its row never visit the host, so the loop is replayed from CUDA graphs and the
host synchronises only at log / checkpoint points.
"""
from __future__ import annotations

import math
import os
import socket
import time
from typing import Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist
from torch import Tensor

from ... import engine as _engine
from .layout import ShardLayout

# the CPU test-suite clears this to drive the host logic with gloo and a stand-in native library
_REQUIRE_CUDA = True


def fps_sharded(
    X_local: Tensor,
    n_to_select: int,
    *,
    seed: Optional[int] = None,
    checkpoint_path: Optional[str] = None,
    checkpoint_every: int = 0,
    resume_from: Optional[str] = None,
    log_every: Optional[int] = None,
    verbose: bool = True,
) -> Tuple[Tensor, Tensor]:
    """Return ``(selected, epsilons)``: global int64 picks in selection order on the device and
    the float32 CPU tensor of squared coverage radii before each pick (``epsilons[0] = inf``).

    Arguments, validation order, exceptions, checkpoint file names and cadence follow the
    reference.  ``resume_from`` replays the checkpointed picks through the same kernels, so a
    resumed run is bit-identical to an uninterrupted one (the reference rebuilds ``h`` with a
    GEMM instead, src/coresets/cuda/multi/_shared.py:243-312, which is not).
    """
    if not dist.is_initialized():
        raise RuntimeError(
            "torch.distributed must be initialised before fps_sharded(). "
            "Call dist.init_process_group(backend='nccl', ...) first. "
            "For single-GPU runs, use coresets_b200.fps_cuda instead."
        )
    if _REQUIRE_CUDA and not X_local.is_cuda:
        raise ValueError(
            f"X_local must be on a CUDA device, got {X_local.device}. "
            "Place each rank's shard on its local GPU before calling."
        )
    if X_local.dim() != 2:
        raise ValueError(f"X_local must be 2-D (N_shard, D), got shape {tuple(X_local.shape)}")

    rank = dist.get_rank()
    world_size = dist.get_world_size()
    device = X_local.device

    # shard layout from every rank's row count (fps_sharded.py:56-63)
    sizes_t = torch.zeros(world_size, dtype=torch.long, device=device)
    sizes_t[rank] = X_local.shape[0]
    dist.all_reduce(sizes_t, op=dist.ReduceOp.SUM)
    sizes = [int(v) for v in sizes_t.cpu().tolist()]
    offsets = [sum(sizes[:i]) for i in range(world_size)]
    layout = ShardLayout(rank=rank, world_size=world_size, sizes=sizes, offsets=offsets)
    n_global = sum(sizes)

    if not 1 <= n_to_select <= n_global:
        raise ValueError(f"n_to_select={n_to_select} must be in [1, N_global={n_global}]")
    if n_global >= 2**31:
        raise ValueError(
            f"N_global={n_global} exceeds int32 range (2^31 - 1). The arg-max key carries the "
            "global row index in 32 bits."
        )

    dim = int(X_local.shape[1])
    d_pair = torch.tensor([dim, -dim], dtype=torch.long, device=device)
    dist.all_reduce(d_pair, op=dist.ReduceOp.MAX)
    d_max, d_min = int(d_pair[0].item()), -int(d_pair[1].item())
    if d_max != dim or d_min != dim:
        raise ValueError(
            f"D={dim} disagrees with peers (cluster min={d_min}, max={d_max}). "
            "Every rank must hold the same feature dim."
        )
    if X_local.dtype not in (torch.float32, torch.float64, torch.float16):
        raise ValueError(f"X_local must be float32, float64 or float16, got X_local.dtype={X_local.dtype}")

    X_local = X_local.contiguous()
    norms_local = _engine.row_norms(X_local)           # in X's own dtype, as fps_sharded.py:90 does
    X32, element_order = _engine.engine_matrix(X_local)
    eng = _engine.ShardEngine(
        X32, norms_local, n_to_select, shard_offset=layout.shard_offset,
        world_size=world_size, group=None, element_order=element_order, cells=True,
    )
    eng.init_state()

    # checkpoint cadence (fps_sharded.py:269-281): every `checkpoint_every` picks or at powers
    # of two, plus the last pick
    if checkpoint_path is not None:
        if checkpoint_every > 0:
            ckpt_steps = set(range(checkpoint_every, n_to_select, checkpoint_every))
        else:
            max_pow = int(math.log2(n_to_select)) if n_to_select > 1 else 0
            ckpt_steps = {1 << p for p in range(1, max_pow + 1)}
        ckpt_steps.add(n_to_select - 1)
        ckpt_steps = {s for s in ckpt_steps if s < n_to_select}
    else:
        ckpt_steps = set()
    if log_every is None:
        log_every = max(1, n_to_select // 100)
    chatty = verbose and rank == 0

    eps_prev: Optional[np.ndarray] = None
    if resume_from is not None:
        k0_done, selected_prev = _load_resume(resume_from)
        k_prev = k0_done + 1
        if k_prev > n_to_select:
            raise ValueError(
                f"resume checkpoint has K_prev={k_prev} picks but n_to_select={n_to_select}. "
                "Increase n_to_select to extend beyond the checkpoint."
            )
        eps_file = f"{resume_from}_k{k0_done:010d}_eps.npy"
        if os.path.exists(eps_file):
            eps_prev = np.load(eps_file).astype(np.float32, copy=False)
        if chatty:
            print(
                f"fps_sharded: resume from {resume_from}  K_prev={k_prev:,}  "
                f"new target K={n_to_select:,}  N_global={n_global:,}  D={dim}  "
                f"world_size={world_size}  host={socket.gethostname()}"
            )
        t_resume = time.time()
        bad = selected_prev[(selected_prev < 0) | (selected_prev >= n_global)]
        if bad.size:
            raise ValueError(f"resume checkpoint holds row {int(bad[0])}, outside [0, N_global={n_global})")
        eng.run_forced(selected_prev)
        if chatty:
            eng.read_ctl()
            print(f"  resume state rebuilt in {time.time() - t_resume:.1f}s (replayed {k_prev:,} picks)")
        start_i = k_prev
    else:
        first = 0 if seed is None else int(seed)
        if not 0 <= first < n_global:
            raise ValueError(f"seed={first} must be in [0, N_global={n_global})")
        eng.pick_forced(first)
        if chatty:
            print(
                f"fps_sharded: N_global={n_global:,}  D={dim}  K={n_to_select:,}  "
                f"world_size={world_size}  host={socket.gethostname()}"
            )
            print(f"  shard sizes = {sizes}")
            print(f"  seed = global row {first} (owner rank {layout.owner_of(first)})")
        start_i = 1

    def host_eps(upto: int) -> np.ndarray:
        e = eng.eps[:upto].cpu().numpy().astype(np.float32, copy=True)
        if eps_prev is not None:
            n = min(eps_prev.shape[0], upto)
            e[:n] = eps_prev[:n]
        return e

    # host events: progress lines (rank 0, verbose) and checkpoints (rank 0)
    events = set()
    if chatty:
        events.update(i for i in range(start_i, n_to_select) if i % log_every == 0 or i == n_to_select - 1)
    if rank == 0 and checkpoint_path is not None:
        events.update(s for s in ckpt_steps if s >= start_i)

    t0 = time.time()
    pos = start_i
    for ev in sorted(events):
        eng.run_picks(ev - pos + 1)
        pos = ev + 1
        best_val = float(eng.eps[ev].item())          # synchronises this rank's stream
        if chatty and (ev % log_every == 0 or ev == n_to_select - 1):
            elapsed = time.time() - t0
            done = ev - start_i + 1
            rate = done / elapsed if elapsed > 0 else 0.0
            print(
                f"  {ev:>10,}/{n_to_select:,}  "
                f"({rate:>7.1f} pick/s, eps={math.sqrt(max(best_val, 0.0)):.4e}, cum {elapsed:.1f}s)"
            )
        if ev in ckpt_steps and rank == 0 and checkpoint_path is not None:
            eng.check_status()        # a device-side time-out leaves garbage picks: raise, do not publish them
            _write_checkpoint(checkpoint_path, ev, eng.selected, host_eps(ev + 1))
    eng.run_picks(n_to_select - pos)
    eng.check_status()

    epsilons_np = host_eps(n_to_select)
    if chatty:
        elapsed = time.time() - t0
        new = n_to_select - start_i
        rate = new / elapsed if elapsed > 0 else 0.0
        eps_final_sq = float(epsilons_np[-1])
        print(
            f"fps_sharded: done. K={n_to_select:,} (+{new:,} new) in {elapsed:.1f}s "
            f"({rate:.1f} pick/s)  eps_final={math.sqrt(max(eps_final_sq, 0.0)):.6e}  "
            f"eps_final_sq={eps_final_sq:.6e}"
        )
    return eng.selected, torch.from_numpy(epsilons_np)


def _write_checkpoint(path_prefix: str, k: int, selected: Tensor, epsilons_np: np.ndarray) -> None:
    """Rank-0 dump of the first ``k + 1`` ids and radii; ``<prefix>_latest.txt`` is written last
    and every file goes through ``.tmp`` + rename (same names as fps_sharded.py:422-446)."""
    arrays = {
        f"{path_prefix}_k{k:010d}_ids.npy": selected[: k + 1].cpu().numpy().astype(np.int64, copy=False),
        f"{path_prefix}_k{k:010d}_eps.npy": epsilons_np[: k + 1].astype(np.float32, copy=False),
    }
    for name, arr in arrays.items():
        with open(name + ".tmp", "wb") as f:
            np.save(f, arr, allow_pickle=False)
        os.replace(name + ".tmp", name)
    latest = f"{path_prefix}_latest.txt"
    with open(latest + ".tmp", "w") as f:
        f.write(f"{k}\n")
    os.replace(latest + ".tmp", latest)


def _load_resume(path_prefix: str) -> Tuple[int, np.ndarray]:
    """Last completed step and the ids up to it (fps_sharded.py:450-475)."""
    latest_path = f"{path_prefix}_latest.txt"
    if not os.path.exists(latest_path):
        raise FileNotFoundError(
            f"resume requires {latest_path}; not found. "
            f"Either disable resume or point at a different prefix."
        )
    with open(latest_path) as f:
        k_last = int(f.read().strip())
    ids_path = f"{path_prefix}_k{k_last:010d}_ids.npy"
    if not os.path.exists(ids_path):
        raise FileNotFoundError(f"resume ids file missing: {ids_path}")
    ids = np.load(ids_path).astype(np.int64, copy=False)
    if ids.shape[0] != k_last + 1:
        raise ValueError(f"resume {ids_path} has {ids.shape[0]} entries, expected k_last+1 = {k_last + 1}")
    return k_last, ids
