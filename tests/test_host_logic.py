"""Host-side drivers on CPU: the pick sequencing of fps_cuda / fps_sharded is driven with the
oracle-backed stand-in native library and compared with the oracle's own whole-run functions."""
import numpy as np
import pytest
import torch

import oracle
from coresets_b200 import _native
import importlib

fps_mod = importlib.import_module("coresets_b200.cuda.fps")
from tests.data import clustered_jitter, gaussian_mixture, with_duplicates
from tests.fake_native import FakeNative


@pytest.fixture()
def fake_native(monkeypatch):
    monkeypatch.setattr(_native, "_native", FakeNative())
    monkeypatch.setattr(fps_mod, "_REQUIRE_CUDA", False)
    yield


def _norms_t(X):
    return (X * X).sum(dim=1).to(torch.float32).numpy()


@pytest.mark.parametrize("N,D,k", [(1, 4, 1), (33, 8, 33), (500, 32, 64), (777, 6, 50), (2048, 64, 128)])
def test_fps_cuda_driver_matches_oracle(fake_native, N, D, k):
    X = torch.from_numpy(gaussian_mixture(N, D, 8, seed=N))
    sel, eps = fps_mod.fps(X, k, return_epsilons=True)
    o_sel, o_eps, _, _ = oracle.fps_cuda(X.numpy(), _norms_t(X), k)
    assert sel.dtype == torch.int64
    np.testing.assert_array_equal(sel.numpy(), o_sel)
    np.testing.assert_array_equal(eps.numpy().view(np.int32), o_eps.view(np.int32))


def test_fps_cuda_seed_tensor(fake_native):
    X = torch.from_numpy(with_duplicates(clustered_jitter(600, 16), 40, seed=1))
    seed = torch.tensor([5, 17, 301])
    sel = fps_mod.fps(X, 40, seed=seed)
    o_sel, _, _, _ = oracle.fps_cuda(X.numpy(), _norms_t(X), 40, seed=seed.numpy())
    np.testing.assert_array_equal(sel.numpy(), o_sel)
    assert sel[:3].tolist() == [5, 17, 301]


def test_fps_cuda_validation(fake_native):
    X = torch.zeros(10, 4)
    with pytest.raises(ValueError):
        fps_mod.fps(torch.zeros(10), 2)
    with pytest.raises(ValueError):
        fps_mod.fps(X, 0)
    with pytest.raises(ValueError):
        fps_mod.fps(X, 11)
    with pytest.raises(ValueError):
        fps_mod.fps(X, 2, seed=torch.zeros((2, 2), dtype=torch.long))
    with pytest.raises(ValueError):
        fps_mod.fps(X, 2, seed=torch.tensor([1, 2, 3]))
    with pytest.raises(ValueError):
        fps_mod.fps(X, 2, seed=torch.tensor([], dtype=torch.long))
    with pytest.raises(ValueError):
        fps_mod.fps(X.to(torch.bfloat16), 2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float64])
@pytest.mark.parametrize("N,D,k", [(400, 64, 40), (333, 10, 30)])
def test_fps_cuda_float16_and_float64(fake_native, dtype, N, D, k):
    """Norms in the input's own dtype (fps.py:34), rows cast to float, dots summed element-wise
    (_shared.cuh:55-58)."""
    X = torch.from_numpy(gaussian_mixture(N, D, 8, seed=N)).to(dtype)
    if dtype == torch.float64:
        X = X * 1.000000123
    sel, eps = fps_mod.fps(X, k, return_epsilons=True)
    with oracle.element_order():
        o_sel, o_eps, _, _ = oracle.fps_cuda(X.float().numpy(), _norms_t(X), k)
    np.testing.assert_array_equal(sel.numpy(), o_sel)
    np.testing.assert_array_equal(eps.numpy().view(np.int32), o_eps.view(np.int32))


def test_fps_cuda_requires_cuda_tensor():
    with pytest.raises(ValueError, match="CUDA"):
        fps_mod.fps(torch.zeros(10, 4), 2)


def test_resolve_max_k_budget_rule(monkeypatch):
    """30 % of the free device bytes for two copies of the centre rows plus five scalars per
    centre, capped by log2 N (src/coresets/cuda/multi/_shared.py:316-336, _internal/scratch.py:62-90)."""
    from coresets_b200.cuda.accrete_core import resolve_max_k
    dev = torch.device("cuda", 0)
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (10 * 10**9, 180 * 10**9))
    # budget 3e9 / (2*256*4 + 20) = 1 450 676 rows -> 2^20 fits, N = 1e6 caps at 19
    assert resolve_max_k(None, 1_000_000, 256, 4, dev, strict=False, collective=False) == (19, 2 ** 19)
    assert resolve_max_k(None, 10**9, 256, 4, dev, strict=False, collective=False) == (20, 2 ** 20)
    assert resolve_max_k(7, 10**9, 256, 4, dev, strict=False, collective=False) == (7, 128)   # a pinned value is kept
    assert resolve_max_k(20, 10**9, 256, 4, dev, strict=True, collective=False) == (20, 2 ** 20)
    with pytest.raises(ValueError, match="Safe max_k for this GPU: 20"):
        resolve_max_k(21, 10**9, 256, 4, dev, strict=True, collective=False)
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (1000, 1000))
    assert resolve_max_k(None, 10**6, 256, 4, dev, strict=False, collective=False) == (1, 2)  # never below one level


def test_torch_backend_fps_reproduces_the_reference_python_fps():
    """``coresets_b200.fps`` (plain torch) against the outputs of the reference's own ``coresets.fps``
    (tests/golden/cpu_fps_c1.npz, written by tests/golden/make_golden_cpu.py)."""
    from pathlib import Path
    import numpy as np
    import torch
    import coresets_b200
    from tests.data import gaussian_mixture
    z = np.load(Path(__file__).resolve().parent / "golden" / "cpu_fps_c1.npz")
    X = torch.from_numpy(gaussian_mixture(20000, 64, 16, seed=0))
    torch.set_num_threads(1)
    sel, eps, h, v = coresets_b200.fps(X, 512)
    np.testing.assert_array_equal(sel.numpy(), z["selected"])
    np.testing.assert_allclose(eps.numpy(), z["eps"], rtol=1e-6)
    np.testing.assert_array_equal(v.numpy().astype(np.int16), z["voronoi"])
    assert eps[0] == 0.0 and "fps" in coresets_b200.__all__
    seeded = coresets_b200.fps(X[:500], 5, torch.tensor([7, 3]))
    assert seeded[0][:2].tolist() == [7, 3] and float(seeded[1][0]) == 0.0 and float(seeded[1][1]) > 0.0


def test_torch_backend_voronoi_fps_equals_fps():
    """The triangle-bound variant picks what the dense one picks (the reference's own claim for its
    two torch functions), sparse and dense branches both taken."""
    import torch
    from coresets_b200.pytorch import fps, voronoi_fps
    from tests.data import gaussian_mixture
    X = torch.from_numpy(gaussian_mixture(4000, 16, 8, seed=5))
    a = fps(X, 200)
    for frac in (0.5, 0.0):
        b = voronoi_fps(X, 200, full_fraction=frac)
        assert torch.equal(a[0], b[0]) and torch.equal(a[3], b[3])
        assert torch.allclose(a[1], b[1], rtol=1e-5, atol=1e-5) and torch.allclose(a[2], b[2], rtol=1e-4, atol=1e-4)
    s = voronoi_fps(X, 50, torch.tensor([9, 4]))
    assert s[0][:2].tolist() == [9, 4] and torch.equal(s[0], fps(X, 50, torch.tensor([9, 4]))[0])


def test_torch_backend_accrete_reproduces_the_reference():
    """``coresets_b200.pytorch.accrete`` against the lists (and the printed table) the reference's own
    plain-torch ``accrete`` produced (tests/golden/torch_accrete.npz, make_golden_torch_accrete.py)."""
    import contextlib
    import io
    from pathlib import Path
    import numpy as np
    import torch
    from coresets_b200.pytorch import accrete
    from tests.golden.make_golden_torch_accrete import CASES, case_inputs
    z = np.load(Path(__file__).resolve().parent / "golden" / "torch_accrete.npz")
    torch.set_num_threads(1)
    for name, c in CASES.items():
        Xa, Xc, order = case_inputs(c)
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            out = accrete(Xa, Xc, order, torch.arange(Xc.shape[0]), max_k=c["max_k"], verbose=True)
        np.testing.assert_array_equal(out.numpy(), z[name])
        assert buf.getvalue() == str(z[name + "_table"])
