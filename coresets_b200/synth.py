"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

They stand in for the real embedding / feature matrices the reference is run on (none of which
ship with it).  Rows are generated block-wise from (seed, block index), so any rank of any world
size materialises exactly the same bytes for a given global row range, on the device, without
ever holding the whole matrix on the host.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

import numpy as np
import torch

BLOCK_ROWS = 1 << 18  # rows per generation block; a block's bytes depend only on (seed, block)


@dataclass(frozen=True)
class Workload:
    name: str
    n_rows: int
    dim: int
    n_comp: int
    seed: int
    k: int
    mean_scale: float = 4.0
    sigma: float = 1.0
    dirichlet: bool = False      # component weights ~ Dirichlet(1) instead of equal
    unit_sphere: bool = False    # unit-norm means, rows L2-normalised after the noise
    describe: str = ""
    extra_comp: int = 0          # further components drawn after the first n_comp ...
    extra_scale: float = 0.0     # ... with means ~N(0, extra_scale^2 I) ...
    extra_share: float = 0.0     # ... that together own this share of the rows
    stream: int = 0              # separates the row noise of workloads that share a seed


WORKLOADS = {
    # CPU-runnable reference case
    "c1": Workload("c1", 20_000, 64, 16, 0, 512,
                   describe="20k x 64, 16 isotropic Gaussians, means ~N(0,16 I), sigma 1"),
    # single-GPU case
    "c2": Workload("c2", 20_000_000, 256, 64, 1, 10_000,
                   describe="20M x 256, 64 isotropic Gaussians, means ~N(0,16 I), sigma 1"),
    # headline scaling case
    "c3": Workload("c3", 300_000_000, 128, 256, 2, 16_384, dirichlet=True,
                   describe="300M x 128, 256 Gaussians, Dirichlet(1) weights, means ~N(0,16 I), sigma 1"),
    # wide embeddings
    "c4": Workload("c4", 40_000_000, 1024, 128, 3, 8_192, sigma=0.3, unit_sphere=True,
                   describe="40M x 1024 unit vectors, 128 vMF-like components, sigma 0.3"),
    # accretion case: the anchors, and candidates of which half come from 64 components the
    # anchors do not have (the two share seed 4, hence the first 128 component means)
    "c5a": Workload("c5a", 50_000_000, 256, 128, 4, 1 << 14,
                    describe="50M x 256 anchors, 128 isotropic Gaussians, means ~N(0,16 I), sigma 1"),
    "c5c": Workload("c5c", 50_000_000, 256, 128, 4, 1 << 14, extra_comp=64, extra_scale=6.0, extra_share=0.5, stream=1,
                    describe="50M x 256 candidates, half from the anchors' 128 components, half from 64 new "
                             "ones with means ~N(0,36 I)"),
}


def scaled(w: Workload, n_rows: int, k: Optional[int] = None) -> Workload:
    """Same law, fewer rows (tests, CPU samples)."""
    return replace(w, n_rows=int(n_rows), k=int(k if k is not None else min(w.k, n_rows)))


class MixtureSource:
    """Row-addressable generator of one workload."""

    def __init__(self, w: Workload):
        self.w = w
        rng = np.random.default_rng(1_000_003 * (w.seed + 1))
        means = rng.standard_normal((w.n_comp, w.dim)).astype(np.float32)
        if w.unit_sphere:
            means /= np.linalg.norm(means, axis=1, keepdims=True)
        else:
            means *= np.float32(w.mean_scale)
        if w.dirichlet:
            weights = rng.dirichlet(np.ones(w.n_comp))
        else:
            weights = np.full(w.n_comp, 1.0 / w.n_comp)
        if w.extra_comp:
            extra = rng.standard_normal((w.extra_comp, w.dim)).astype(np.float32) * np.float32(w.extra_scale)
            means = np.concatenate([means, extra])
            weights = np.concatenate([weights * (1.0 - w.extra_share),
                                      np.full(w.extra_comp, w.extra_share / w.extra_comp)])
        self.means = torch.from_numpy(means)
        self.weights = torch.from_numpy(weights.astype(np.float64))
        self._means_dev = {}

    def _block(self, b: int, device: torch.device) -> torch.Tensor:
        w = self.w
        lo = b * BLOCK_ROWS
        n = min(BLOCK_ROWS, w.n_rows - lo)
        g = torch.Generator(device=device)
        g.manual_seed(7_919 * (w.seed + 1) + 104_729 * b + 15_485_863 * w.stream)
        key = str(device)
        if key not in self._means_dev:
            self._means_dev[key] = (self.means.to(device), self.weights.to(device))
        means, weights = self._means_dev[key]
        # always draw a full block so that a partial tail does not change the stream
        comp = torch.multinomial(weights, BLOCK_ROWS, replacement=True, generator=g)
        x = torch.randn((BLOCK_ROWS, w.dim), dtype=torch.float32, device=device, generator=g)
        x.mul_(w.sigma).add_(means[comp])
        if w.unit_sphere:
            x.div_(x.norm(dim=1, keepdim=True))
        return x[:n]

    def fill(self, out: torch.Tensor, start: int) -> torch.Tensor:
        """Write global rows ``[start, start + out.shape[0])`` into ``out`` (on out's device)."""
        count = int(out.shape[0])
        if start < 0 or start + count > self.w.n_rows or out.shape[1] != self.w.dim:
            raise ValueError("row range or width outside the workload")
        pos = start
        end = start + count
        while pos < end:
            b = pos // BLOCK_ROWS
            blk = self._block(b, out.device)
            lo = pos - b * BLOCK_ROWS
            n = min(blk.shape[0] - lo, end - pos)
            out[pos - start : pos - start + n].copy_(blk[lo : lo + n])
            pos += n
        return out

    def rows(self, start: int, count: int, device) -> torch.Tensor:
        out = torch.empty((count, self.w.dim), dtype=torch.float32, device=device)
        return self.fill(out, start)


class StackedSource:
    """Several sources one after the other in the global row order (accretion: the anchors, then the
    candidates, src/coresets/cuda/multi/sharded.py:633-634), row-addressable like its parts."""

    def __init__(self, parts):
        self.parts = list(parts)
        self.dim = self.parts[0].w.dim
        self.n_rows = sum(p.w.n_rows for p in self.parts)

    def fill(self, out: torch.Tensor, start: int) -> torch.Tensor:
        count = int(out.shape[0])
        if start < 0 or start + count > self.n_rows or out.shape[1] != self.dim:
            raise ValueError("row range or width outside the stacked workload")
        base = 0
        for p in self.parts:
            lo, hi = max(start, base), min(start + count, base + p.w.n_rows)
            if lo < hi:
                p.fill(out[lo - start : hi - start], lo - base)
            base += p.w.n_rows
        return out

    def rows(self, start: int, count: int, device) -> torch.Tensor:
        out = torch.empty((count, self.dim), dtype=torch.float32, device=device)
        return self.fill(out, start)


def accretion_sources(n_anchor: int = 0, n_cand: int = 0):
    """``(anchors, candidates, stacked)`` of the accretion benchmark case; row counts may be scaled down."""
    a = MixtureSource(scaled(WORKLOADS["c5a"], n_anchor or WORKLOADS["c5a"].n_rows))
    c = MixtureSource(scaled(WORKLOADS["c5c"], n_cand or WORKLOADS["c5c"].n_rows))
    return a, c, StackedSource([a, c])
