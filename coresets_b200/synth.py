"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

They stand in for the real embedding / feature matrices the reference is run on (none of which
ship with it).  Rows are generated block-wise from (seed, block index), so any rank of any world
size materialises exactly the same bytes for a given global row range, on the device, without
ever holding the whole matrix on the host.
"""
from __future__ import annotations

from dataclasses import dataclass
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
}


def scaled(w: Workload, n_rows: int, k: Optional[int] = None) -> Workload:
    """Same law, fewer rows (tests, CPU samples)."""
    return Workload(w.name, int(n_rows), w.dim, w.n_comp, w.seed, int(k if k is not None else min(w.k, n_rows)),
                    w.mean_scale, w.sigma, w.dirichlet, w.unit_sphere, w.describe)


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
        self.means = torch.from_numpy(means)
        if w.dirichlet:
            weights = rng.dirichlet(np.ones(w.n_comp))
        else:
            weights = np.full(w.n_comp, 1.0 / w.n_comp)
        self.weights = torch.from_numpy(weights.astype(np.float64))
        self._means_dev = {}

    def _block(self, b: int, device: torch.device) -> torch.Tensor:
        w = self.w
        lo = b * BLOCK_ROWS
        n = min(BLOCK_ROWS, w.n_rows - lo)
        g = torch.Generator(device=device)
        g.manual_seed(7_919 * (w.seed + 1) + 104_729 * b)
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
