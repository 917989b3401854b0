"""Coverage / separation invariants of the accretion output, by brute force on the CPU.

For every layer k the first 2**k picks S_k must satisfy, in float64,
  cov_k = max_x min_{s in S_k} |x - s|  is non-increasing in k, and
  sep_k = min_{s != s'} |s - s'| >= cov_k,
within 1e-4 relative (float32 kernels against float64 arithmetic).  The reference states the same
two properties in tests/test_invariants.py (one anchor row, mildly clustered rows).  The CPU
version drives the package's `accrete` through the oracle-backed stand-in native library; the
GPU version runs the real kernels on the reference's sizes."""
import importlib

import numpy as np
import pytest
import torch

from coresets_b200 import _native

acc_mod = importlib.import_module("coresets_b200.cuda.accrete")


def clustered(N, D, n_clusters, seed):
    rng = np.random.default_rng(seed)
    centres = rng.standard_normal((n_clusters, D)).astype(np.float32)
    ids = rng.integers(0, n_clusters, size=N)
    return centres[ids] + 0.1 * rng.standard_normal((N, D)).astype(np.float32)


def check_layers(X_np, sel, max_k, eps_rel=1e-4):
    X = torch.from_numpy(X_np).double()
    prev = float("inf")
    for k in range(1, max_k + 1):
        S = X[sel[: 2 ** k]]
        cov = float(torch.cdist(X, S).min(dim=1).values.max())
        dS = torch.cdist(S, S)
        dS.fill_diagonal_(float("inf"))
        sep = float(dS.min())
        tol = eps_rel * max(cov, 1e-9)
        assert cov <= prev + tol, f"layer {k}: coverage grew from {prev} to {cov}"
        assert sep >= cov - tol, f"layer {k}: separation {sep} below coverage {cov}"
        prev = cov


def test_layers_keep_separation_above_coverage_cpu(monkeypatch):
    from tests.fake_native import FakeNative
    monkeypatch.setattr(_native, "_native", FakeNative())
    monkeypatch.setattr(acc_mod, "_REQUIRE_CUDA", False)
    for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
        monkeypatch.delenv(k, raising=False)
    N, D, max_k = 768, 8, 6
    X_np = clustered(N, D, 12, seed=0)
    X = torch.from_numpy(X_np)
    sel = acc_mod.accrete(X[:1], X[1:], torch.tensor([0]), max_k=max_k, verbose=False).numpy()
    assert len(sel) == 2 ** max_k and len(set(sel.tolist())) == len(sel)
    check_layers(X_np, sel, max_k)


@pytest.mark.gpu
@pytest.mark.parametrize("knobs", [{}, {"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"}])
def test_layers_keep_separation_above_coverage_gpu(monkeypatch, knobs):
    import coresets_b200
    for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
        monkeypatch.delenv(k, raising=False)
    for k, v in knobs.items():
        monkeypatch.setenv(k, v)
    N, D, K = 4096, 16, 1024                       # the reference's sizes
    max_k = int(np.log2(K))
    X_np = clustered(N, D, 32, seed=0)
    X = torch.from_numpy(X_np).cuda()
    coresets_b200.warmup_fast_fps()
    sel = coresets_b200.accrete(X[:1], X[1:], torch.tensor([0], device="cuda"), max_k=max_k, verbose=False).cpu().numpy()
    assert len(sel) == 2 ** max_k and len(set(sel.tolist())) == len(sel)
    check_layers(X_np, sel, max_k)
