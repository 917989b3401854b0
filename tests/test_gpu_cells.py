"""The cell index (cs_cells_build / cs_cells_select / cs_fps_step_cells) against the oracle, the
reference's golden vectors and the scan kernels, through the C ABI.

Bar: bit-exact -- the index only decides which rows are LOOKED AT; every row that could change is
still tested with the reference's predicate and evaluated with the reference's arithmetic.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

from coresets_b200 import engine
from coresets_b200._native import MODE_PRUNE
from tests.data import clustered_jitter, gaussian_mixture, with_duplicates
from tests.test_gpu_parity import assert_matches_oracle, bits

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"

# tiny indexes, rebuilt often, never abandoned: every kernel of the index runs many times per case
EAGER = {"CORESETS_B200_CELLS_MIN_ROWS": "1", "CORESETS_B200_CELLS_FIRST_BUILD": "3", "CORESETS_B200_CELLS_GROWTH": "1.4",
         "CORESETS_B200_EARLY_DENSE_PICKS": "2", "CORESETS_B200_CELLS_GIVE_UP_SHARE": "2.0",
         "CORESETS_B200_CELLS_PROBE_PICKS": "5", "CORESETS_B200_CELLS_LIVE_GATE": "2.0"}


def cells_engine(X_np_or_dev, k, monkeypatch, env=EAGER, seed=(0,), graph=True):
    for key, val in env.items():
        monkeypatch.setenv(key, val)
    monkeypatch.setenv("CORESETS_B200_GRAPH", "1" if graph else "0")
    X = X_np_or_dev if torch.is_tensor(X_np_or_dev) else torch.from_numpy(X_np_or_dev).to("cuda:0")
    norms = engine.row_norms(X)
    eng = engine.ShardEngine(X, norms, k, mode=MODE_PRUNE, cells=True)
    assert eng.cells_enabled
    eng.init_state()
    for s in seed:
        eng.pick_forced(int(s))
    eng.run_picks(k - len(seed))
    ctl = eng.check_status()
    assert ctl.n_sel == k
    return eng, norms


@pytest.mark.parametrize("N,D,k", [(33, 64, 20), (1000, 32, 128), (4097, 128, 300), (3000, 192, 64), (2500, 256, 200),
                                   (1500, 512, 64), (900, 1024, 48), (1200, 100, 64), (16383, 128, 512), (300, 4, 300)])
@pytest.mark.parametrize("graph", [True, False])
def test_cells_match_oracle(N, D, k, graph, monkeypatch):
    if not graph and N > 3000:
        pytest.skip("eager launches are covered by the small shapes")
    X = gaussian_mixture(N, D, 8, seed=N + D)
    eng, norms = cells_engine(X, k, monkeypatch, graph=graph)
    assert eng._cells is not None and eng.read_cells_meta().n_cells >= 3      # the index was really used
    assert_matches_oracle(eng, X, norms.cpu().numpy(), k)


def test_cells_with_duplicates_and_seeds(monkeypatch):
    """Exact duplicates (h = 0 rows, zero and slightly negative distances) and seeded first picks."""
    X = with_duplicates(clustered_jitter(3000, 16, seed=5), 600, seed=9)
    eng, norms = cells_engine(X, 1500, monkeypatch, seed=(17, 2000, 123))
    assert_matches_oracle(eng, X, norms.cpu().numpy(), 1500, seed=(17, 2000, 123))


def test_cells_forced_pick_in_the_middle(monkeypatch):
    """A forced pick while the index is live goes through the scan kernel; the index is rebuilt."""
    X = gaussian_mixture(5000, 64, 8, seed=3)
    for key, val in EAGER.items():
        monkeypatch.setenv(key, val)
    Xd = torch.from_numpy(X).to("cuda:0")
    norms = engine.row_norms(Xd)
    runs = []
    for cells in (True, False):
        eng = engine.ShardEngine(Xd, norms, 200, mode=MODE_PRUNE, cells=cells)
        eng.init_state()
        eng.pick_forced(0)
        eng.run_picks(60)
        eng.pick_forced(4321)
        eng.run_picks(138)
        assert eng.check_status().n_sel == 200
        runs.append(eng)
    a, b = runs
    assert torch.equal(a.selected, b.selected) and torch.equal(a.eps.view(torch.int32), b.eps.view(torch.int32))
    assert torch.equal(a.h.view(torch.int32), b.h.view(torch.int32)) and torch.equal(a.voronoi, b.voronoi)


@pytest.mark.parametrize("name", ["ref_script_8192x32", "uneven_16383x128", "c1_20000x64", "dups_3000x16", "mix_2500x256"])
def test_cells_reproduce_reference_golden(name, monkeypatch):
    from tests.test_oracle_golden import load_case
    z, X = load_case(name)
    K = int(z["K"])
    eng, norms = cells_engine(X, K, monkeypatch, seed=tuple(int(s) for s in z["seeds"]))
    n = X.shape[0]
    np.testing.assert_array_equal(eng.selected.cpu().numpy(), z["selected"])
    np.testing.assert_array_equal(bits(eng.eps.cpu().numpy()), bits(z["eps"]))
    np.testing.assert_array_equal(bits(eng.h[:n].cpu().numpy()), bits(z["h"]))
    np.testing.assert_array_equal(eng.voronoi[:n].cpu().numpy(), z["voronoi"])


@pytest.mark.parametrize("wname,n_rows", [("c3", 2_000_000), ("c2", 5_000_000), ("c4", 400_000)])
def test_cells_reproduce_reference_on_device_generated_workloads(wname, n_rows, monkeypatch):
    """Default knobs on the scaled benchmark workloads against the reference's own picks, and the
    final h / voronoi against the scan kernels."""
    from coresets_b200.synth import WORKLOADS, MixtureSource, scaled
    ref = np.load(GOLDEN / f"midsize_{wname}_{n_rows}_selected.npy")
    K = ref.shape[0]
    X = MixtureSource(scaled(WORKLOADS[wname], n_rows, k=K)).rows(0, n_rows, torch.device("cuda:0"))
    eng, norms = cells_engine(X, K, monkeypatch, env={})
    np.testing.assert_array_equal(eng.selected.cpu().numpy(), ref)
    plain = engine.ShardEngine(X, norms, K, mode=MODE_PRUNE)
    plain.init_state()
    plain.pick_forced(0)
    plain.run_picks(K - 1)
    assert torch.equal(plain.h.view(torch.int32), eng.h.view(torch.int32))
    assert torch.equal(plain.voronoi, eng.voronoi)
    assert torch.equal(plain.eps.view(torch.int32), eng.eps.view(torch.int32))


def test_cells_full_size_single_gpu_config():
    """The whole 20M x 256, k = 10 000 run through the public fps_cuda against the list the
    reference's fps_sharded produced on the same device-generated rows (tests/golden/fullsize_c2.npz)."""
    import coresets_b200
    from coresets_b200.synth import WORKLOADS, MixtureSource
    free, _ = torch.cuda.mem_get_info()
    if free < 30e9:
        pytest.skip("needs 30 GB of device memory")
    z = np.load(GOLDEN / "fullsize_c2.npz")
    w = WORKLOADS["c2"]
    assert int(z["rows"]) == w.n_rows and int(z["k"]) == w.k
    X = MixtureSource(w).rows(0, w.n_rows, torch.device("cuda:0"))
    sel, eps = coresets_b200.fps_cuda(X, w.k, return_epsilons=True)
    np.testing.assert_array_equal(sel.cpu().numpy(), z["selected"].astype(np.int64))
    np.testing.assert_array_equal(bits(eps.cpu().numpy()), bits(z["eps"]))


@pytest.mark.parametrize("sizes", [[1000, 1003], [0, 700, 0, 650], [333] * 7 + [340]])
def test_cells_multi_rank_kernels_on_one_device(sizes, monkeypatch):
    """world_size > 1 on ONE device (the all-gather replaced by copies): ranks with an index, ranks
    without (empty shards), index rebuilt at several pick counts; against the oracle's sharded run."""
    import oracle
    monkeypatch.setenv("CORESETS_B200_CELLS_MIN_ROWS", "1")
    N, k, D = sum(sizes), 150, 64
    X_np = with_duplicates(gaussian_mixture(N, D, 8, seed=N), 50, seed=1)
    dev = torch.device("cuda:0")
    W = len(sizes)
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).tolist()
    X = torch.from_numpy(X_np).to(dev)
    norms = engine.row_norms(X)
    engs = []
    for r in range(W):
        e = engine.ShardEngine(X[offs[r] : offs[r] + sizes[r]].contiguous(), norms[offs[r] : offs[r] + sizes[r]].contiguous(),
                               k, shard_offset=offs[r], world_size=W, mode=MODE_PRUNE, cells=True)
        assert e.cells_enabled == (sizes[r] > 0)
        e.init_state()
        engs.append(e)
    first = N // 2
    for e in engs:
        e.force_pick(first)
    for i in range(k):
        allp = torch.stack([e.pack_local for e in engs])
        for e in engs:
            e.pack_all.copy_(allp)
        for e in engs:
            e.commit()
            if e.cells_enabled and i >= 4:
                if i in (4, 7, 12, 33, 80):
                    e.n_host = i
                    e._build_cells()
                st = e._stream()
                e.native.cells_select(e.state, e._cells, st)
                e.native.fps_step_cells(e.state, e._cells, st)
            else:
                e.step()
    o_sel, o_eps, o_h, o_v = oracle.fps_sharded(X_np, norms.cpu().numpy(), k, sizes, first=first)
    for r, e in enumerate(engs):
        assert e.check_status().n_sel == k
        np.testing.assert_array_equal(e.selected.cpu().numpy(), o_sel)
        np.testing.assert_array_equal(bits(e.eps.cpu().numpy()), bits(o_eps))
        n = sizes[r]
        np.testing.assert_array_equal(bits(e.h[:n].cpu().numpy()), bits(o_h[offs[r] : offs[r] + n]))
        np.testing.assert_array_equal(e.voronoi[:n].cpu().numpy().astype(np.int64), o_v[offs[r] : offs[r] + n])


@pytest.mark.parametrize("N,D,k", [(4097, 128, 300), (5000, 64, 200), (2500, 256, 120)])
def test_cells_queue_overflow(N, D, k, monkeypatch):
    """A queue of the minimum size (one tile): most rows that need a distance do not fit and are
    finished by the scanning kernel itself; the result must not change."""
    monkeypatch.setenv("CORESETS_B200_CELLS_QUEUE", "256")
    X = gaussian_mixture(N, D, 8, seed=N + D)
    eng, norms = cells_engine(X, k, monkeypatch)
    assert_matches_oracle(eng, X, norms.cpu().numpy(), k)
