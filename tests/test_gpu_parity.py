"""Parity of the sm_100a kernels with the oracle, through the C ABI (ctypes -> libcoresets_b200.so).

Bar: bit-exact.  `selected` identical; `h`, `epsilons` compared as raw 32-bit patterns; `voronoi`
equal.  Norms are an input of both sides (the reference takes them from torch), so both get the
same float32 vector computed by torch on the GPU.
"""
import importlib

import numpy as np
import pytest
import torch

import oracle
from coresets_b200 import _native, engine
from coresets_b200._native import MODE_DENSE, MODE_PRUNE
from tests.data import clustered_jitter, gaussian_mixture, with_duplicates

pytestmark = pytest.mark.gpu
fps_mod = importlib.import_module("coresets_b200.cuda.fps")


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.int32)


def run_engine(X_np, k, *, mode=MODE_PRUNE, seed=(0,), graph=True, monkeypatch=None):
    dev = torch.device("cuda:0")
    X = torch.from_numpy(X_np).to(dev)
    norms = engine.row_norms(X)
    if monkeypatch is not None:
        monkeypatch.setenv("CORESETS_B200_GRAPH", "1" if graph else "0")
    X32, element_order = engine.engine_matrix(X)
    eng = engine.ShardEngine(X32, norms, k, mode=mode, element_order=element_order)
    eng.init_state()
    for s in seed:
        eng.pick_forced(int(s))
    eng.run_picks(k - len(seed))
    ctl = eng.check_status()
    assert ctl.n_sel == k
    return eng, norms.cpu().numpy()


def assert_matches_oracle(eng, X_np, norms_np, k, seed=(0,)):
    with oracle.element_order(X_np.dtype != np.float32):
        o_sel, o_eps, o_h, o_v = oracle.fps_cuda(X_np.astype(np.float32), norms_np, k, seed=np.asarray(seed, dtype=np.int64))
    N = X_np.shape[0]
    np.testing.assert_array_equal(eng.selected.cpu().numpy(), o_sel)
    np.testing.assert_array_equal(bits(eng.eps.cpu().numpy()), bits(o_eps))
    np.testing.assert_array_equal(bits(eng.h[:N].cpu().numpy()), bits(o_h))
    np.testing.assert_array_equal(eng.voronoi[:N].cpu().numpy().astype(np.int64), o_v)


SHAPES = [
    # N, D, k          what it exercises
    (1, 4, 1),          # a single row
    (31, 8, 31),        # less than one 32-row tile, every row selected
    (33, 64, 20),       # tile + 1 ragged row; D = 64 leaves lanes 16..31 without a chunk
    (1000, 32, 128),
    (4097, 128, 300),   # one chunk per lane, exact
    (3000, 192, 64),    # 1.5 chunks per lane (guarded second chunk)
    (2500, 256, 200),   # two chunks per lane
    (1500, 512, 64),
    (900, 1024, 48),    # eight chunks per lane
    (700, 1028, 40),    # D % 4 == 0 but wider than the register path: generic kernel
    (300, 1032, 41),    # the same with a bound table whose length is not a multiple of four
    (1200, 100, 64),    # D % 4 == 0, 25 chunks
    (800, 50, 64),      # D % 4 != 0: the reference's scalar dot
    (600, 3, 40),
    (16383, 128, 512),  # the reference's uneven-shard determinism config (N = 16383, D = 128)
]


@pytest.mark.parametrize("N,D,k", SHAPES)
def test_fps_matches_oracle_prune(N, D, k):
    X = gaussian_mixture(N, D, 8, seed=N + D)
    eng, norms = run_engine(X, k)
    assert_matches_oracle(eng, X, norms, k)


@pytest.mark.parametrize("N,D,k", [(33, 64, 20), (1000, 32, 128), (4097, 128, 300), (3000, 192, 64), (2500, 256, 200),
                                   (900, 1024, 48), (1200, 100, 64), (20000, 36, 100), (130, 128, 130),
                                   (300, 1032, 41)])
def test_fps_matches_oracle_prune_inline(N, D, k):
    """Prune mode with the rows evaluated where the scan meets them (no queue)."""
    from coresets_b200._native import MODE_PRUNE_INLINE
    X = gaussian_mixture(N, D, 8, seed=N + D)
    eng, norms = run_engine(X, k, mode=MODE_PRUNE_INLINE)
    assert_matches_oracle(eng, X, norms, k)


@pytest.mark.parametrize("N,D,k", [(130, 128, 130), (257, 64, 257), (5000, 16, 700), (40000, 8, 300), (12345, 48, 400)])
def test_fps_matches_oracle_prune_more_shapes(N, D, k):
    """Queue edge cases: every row selected, partial last super-tile, many rows per batch."""
    X = with_duplicates(gaussian_mixture(N, D, 8, seed=N + D), min(50, N // 4), seed=1)
    eng, norms = run_engine(X, k)
    assert_matches_oracle(eng, X, norms, k)


DENSE_SHAPES = [(33, 64, 20), (4097, 128, 300), (2500, 256, 100), (800, 50, 64), (900, 1024, 48), (3000, 192, 64),
                (1200, 100, 64), (1000, 32, 128), (16383, 128, 256), (700, 1028, 40), (5, 128, 5), (20000, 36, 100),
                (1500, 512, 64), (31, 8, 31), (1002, 64, 40), (258, 48, 30), (300, 1032, 41)]


@pytest.mark.parametrize("N,D,k", DENSE_SHAPES)
def test_dense_mode_is_bit_identical(N, D, k):
    """Dense mode (X streamed through the TMA ring where the row width allows it)."""
    X = gaussian_mixture(N, D, 8, seed=N + D)
    eng, norms = run_engine(X, k, mode=MODE_DENSE)
    assert_matches_oracle(eng, X, norms, k)


@pytest.mark.parametrize("dtype", ["float16", "float64"])
@pytest.mark.parametrize("N,D,k", [(3000, 128, 200), (1500, 50, 64), (2000, 64, 100), (900, 1024, 40)])
@pytest.mark.parametrize("mode", [MODE_PRUNE, MODE_DENSE])
def test_float16_and_float64_inputs(dtype, N, D, k, mode):
    """Inputs the reference sums element-wise after a cast to float (_shared.cuh:55-58)."""
    from tests.data import as_dtype
    X = as_dtype(gaussian_mixture(N, D, 8, seed=N + D), dtype)
    eng, norms = run_engine(X, k, mode=mode)
    assert_matches_oracle(eng, X, norms, k)


@pytest.mark.parametrize("N,D,k", [(3000, 128, 200), (1501, 50, 64), (2000, 7, 100), (600, 1028, 40), (777, 1, 30),
                                   # dense mode: the bulk-copy ring over half rows, every width bucket and ragged last tiles
                                   (4099, 8, 60), (5001, 32, 80), (2050, 64, 64), (1501, 72, 64), (3003, 200, 50),
                                   (1290, 256, 64), (777, 512, 40), (530, 520, 30), (431, 1024, 40), (40000, 128, 64), (3, 16, 3)])
@pytest.mark.parametrize("mode", [MODE_PRUNE, MODE_DENSE])
def test_half_rows_read_in_place_equal_the_converted_matrix(N, D, k, mode, monkeypatch):
    """float16 rows on the device are read where they lie (CS_F_X_HALF), odd row widths and
    therefore 2-byte aligned rows included; same bits as the run over a float32 copy.  Dense mode
    with rows of whole 16-byte units streams them through the bulk-copy ring (fps_step_tma_half_kernel)."""
    from tests.data import as_dtype
    X = as_dtype(gaussian_mixture(N, D, 8, seed=N + D), "float16")
    a, norms = run_engine(X, k, mode=mode)
    assert a.X.dtype == torch.float16 and a.half_rows
    monkeypatch.setenv("CORESETS_B200_NATIVE_HALF", "0")
    b, _ = run_engine(X, k, mode=mode)
    assert b.X.dtype == torch.float32 and not b.half_rows
    assert torch.equal(a.selected, b.selected) and torch.equal(a.eps.view(torch.int32), b.eps.view(torch.int32))
    assert torch.equal(a.h.view(torch.int32), b.h.view(torch.int32)) and torch.equal(a.voronoi, b.voronoi)
    assert torch.equal(a.X_sel.view(torch.int32), b.X_sel.view(torch.int32))
    assert_matches_oracle(a, X, norms, k)


@pytest.mark.parametrize("D", [128, 72, 1024])
def test_half_ring_with_a_centre_that_is_no_half(D):
    """The half-row dense kernel multiplies halves directly when the centre is representable in
    half (always, when it was committed from half rows); a centre table written otherwise takes the
    widening path.  Both against the float32 kernels on the same perturbed centre."""
    from tests.data import as_dtype
    N = 3000
    Xh = torch.from_numpy(as_dtype(gaussian_mixture(N, D, 8, seed=N + D), "float16")).cuda()
    norms = engine.row_norms(Xh)
    engs = []
    for X in (Xh, Xh.to(torch.float32)):
        e = engine.ShardEngine(X, norms, 8, mode=MODE_DENSE, element_order=True)
        e.init_state()
        e.force_pick(5)
        for i in range(6):
            e.commit()
            if i % 2 == 1:
                e.X_sel[i, ::3] += 1.0e-5          # not a half any more
            e.step()
        e.check_status()
        engs.append(e)
    a, b = engs
    assert a.half_rows and not b.half_rows
    assert torch.equal(a.h.view(torch.int32), b.h.view(torch.int32)) and torch.equal(a.voronoi, b.voronoi)
    assert torch.equal(a.selected[:6], b.selected[:6])


@pytest.mark.parametrize("N,D,k,share", [(6000, 64, 600, 0.12), (5000, 128, 300, 0.5), (3000, 256, 200, 0.02)])
def test_half_rows_leave_the_ring_for_the_pruned_scan(N, D, k, share, monkeypatch):
    """Product mode over float16 rows: the bulk-copy ring while a pick still evaluates a large
    share of the rows, then the pruned scan; the switch (a host decision between picks) changes no bit."""
    from tests.data import as_dtype
    monkeypatch.setenv("CORESETS_B200_CELLS_MIN_ROWS", "1")
    monkeypatch.setenv("CORESETS_B200_EARLY_DENSE_PICKS", "3")
    monkeypatch.setenv("CORESETS_B200_HALF_RING_SHARE", str(share))
    X = as_dtype(gaussian_mixture(N, D, 8, seed=N + D), "float16")
    eng, norms = run_engine(X, k)
    assert eng.half_ring and eng._ring_until > 3          # some stretches ran on the ring ...
    if share >= 0.5:
        assert eng._ring_off                              # ... and the scan took over
    assert_matches_oracle(eng, X, norms, k)
    monkeypatch.setenv("CORESETS_B200_HALF_RING_SHARE", "0")
    plain, _ = run_engine(X, k)
    assert not plain.half_ring
    assert torch.equal(plain.selected, eng.selected) and torch.equal(plain.h.view(torch.int32), eng.h.view(torch.int32))


@pytest.mark.parametrize("sizes,D", [([1000, 1003], 64), ([0, 700, 0, 650], 50), ([301, 299, 2, 300], 129)])
@pytest.mark.parametrize("mode", [MODE_PRUNE, MODE_DENSE])
def test_half_rows_multi_rank_kernels_on_one_device(sizes, D, mode):
    """Half rows with world_size > 1: the candidate row travels widened to float32 (multi.cu:245)."""
    from tests.data import as_dtype
    N, k = sum(sizes), 100
    X = as_dtype(with_duplicates(gaussian_mixture(N, D, 8, seed=N + D), 20, seed=2), "float16")
    engs, norms, offs = _emulate_ranks(X, sizes, k, first=3, mode=mode)
    assert all(e.half_rows for e in engs)
    with oracle.element_order():
        o_sel, o_eps, o_h, o_v = oracle.fps_sharded(X.astype(np.float32), norms, k, sizes, first=3)
    for r, e in enumerate(engs):
        assert e.check_status().n_sel == k
        np.testing.assert_array_equal(e.selected.cpu().numpy(), o_sel)
        np.testing.assert_array_equal(bits(e.eps.cpu().numpy()), bits(o_eps))
        n = sizes[r]
        np.testing.assert_array_equal(bits(e.h[:n].cpu().numpy()), bits(o_h[offs[r] : offs[r] + n]))
        np.testing.assert_array_equal(e.voronoi[:n].cpu().numpy().astype(np.int64), o_v[offs[r] : offs[r] + n])


def test_fps_cuda_accepts_float16_and_float64():
    from tests.data import as_dtype
    import coresets_b200
    Xf = gaussian_mixture(2000, 96, 8, seed=5)
    for dtype in ("float16", "float64"):
        X = as_dtype(Xf, dtype)
        Xd = torch.from_numpy(X).cuda()
        sel = coresets_b200.fps_cuda(Xd, 150)
        norms = (Xd * Xd).sum(dim=1).to(torch.float32).cpu().numpy()
        with oracle.element_order():
            o_sel, _, _, _ = oracle.fps_cuda(X.astype(np.float32), norms, 150)
        np.testing.assert_array_equal(sel.cpu().numpy(), o_sel)
    with pytest.raises(ValueError):
        coresets_b200.fps_cuda(torch.zeros(10, 4, dtype=torch.bfloat16, device="cuda"), 2)


@pytest.mark.parametrize("N,D,k", [(4097, 128, 300), (2500, 256, 100), (900, 1024, 48), (20000, 36, 100)])
def test_dense_mode_with_plain_loads_is_bit_identical(N, D, k):
    from coresets_b200._native import MODE_DENSE_LDG
    X = gaussian_mixture(N, D, 8, seed=N + D)
    eng, norms = run_engine(X, k, mode=MODE_DENSE_LDG)
    assert_matches_oracle(eng, X, norms, k)


def test_reference_parity_script_shape():
    # data and sizes of the reference's own parity script: 8192 x 32, K = 2048, seed 42
    X = clustered_jitter(8192, 32, seed=42)
    eng, norms = run_engine(X, 2048)
    assert_matches_oracle(eng, X, norms, 2048)


def test_exact_ties_take_the_smallest_index():
    X = with_duplicates(clustered_jitter(3000, 16, seed=5), 600, seed=9)
    eng, norms = run_engine(X, 1500)
    assert_matches_oracle(eng, X, norms, 1500)


def test_all_rows_identical():
    X = np.ones((200, 8), dtype=np.float32)
    eng, norms = run_engine(X, 200)
    assert_matches_oracle(eng, X, norms, 200)
    assert eng.selected.cpu().tolist() == list(range(200))


def test_seed_picks_and_eager_equals_graph(monkeypatch):
    X = gaussian_mixture(5000, 64, 8, seed=3)
    seed = (17, 4000, 123)
    e1, norms = run_engine(X, 200, seed=seed, graph=True, monkeypatch=monkeypatch)
    assert_matches_oracle(e1, X, norms, 200, seed=seed)
    e2, _ = run_engine(X, 200, seed=seed, graph=False, monkeypatch=monkeypatch)
    assert torch.equal(e1.selected, e2.selected)
    assert torch.equal(e1.h.view(torch.int32), e2.h.view(torch.int32))


def test_public_fps_cuda_api():
    X_np = gaussian_mixture(6000, 128, 16, seed=1)
    X = torch.from_numpy(X_np).cuda()
    sel = fps_mod.fps(X, 256)
    assert sel.is_cuda and sel.dtype == torch.int64 and sel.shape == (256,)
    norms = engine.row_norms(X).cpu().numpy()
    o_sel, _, _, _ = oracle.fps_cuda(X_np, norms, 256)
    np.testing.assert_array_equal(sel.cpu().numpy(), o_sel)
    sel2 = fps_mod.fps(X, 64, seed=torch.tensor([5, 9]))
    o2, _, _, _ = oracle.fps_cuda(X_np, norms, 64, seed=np.array([5, 9]))
    np.testing.assert_array_equal(sel2.cpu().numpy(), o2)
    with pytest.raises(ValueError):
        fps_mod.fps(X.cpu(), 4)
    with pytest.raises(ValueError):
        fps_mod.fps(X, 0)


def test_prune_evaluates_fewer_rows_than_dense():
    X = gaussian_mixture(20000, 64, 16, seed=0)
    dev = torch.device("cuda:0")
    Xd = torch.from_numpy(X).to(dev)
    norms = engine.row_norms(Xd)
    live = {}
    for mode in (MODE_PRUNE, MODE_DENSE):
        eng = engine.ShardEngine(Xd, norms, 300, mode=mode)
        eng.init_state()
        eng.pick_forced(0)
        eng.run_picks(298)
        eng.exchange(); eng.commit(); eng.step()
        live[mode] = eng.read_ctl().live_rows
    assert live[MODE_DENSE] == 20000 - 300
    assert 0 < live[MODE_PRUNE] < live[MODE_DENSE] // 2


def test_capacity_overrun_sets_status_not_memory():
    X = gaussian_mixture(500, 16, 4, seed=2)
    eng, _ = run_engine(X, 10)
    eng.run_picks(3)  # beyond cap: kernels refuse, status word records it
    with pytest.raises(RuntimeError, match="centre table"):
        eng.check_status()


def test_row_norms_chunked_is_bitwise_the_plain_expression(monkeypatch):
    X = torch.randn(300_000, 64, device="cuda")
    plain = (X * X).sum(dim=1)
    monkeypatch.setattr(engine, "_NORM_CHUNK_ELEMS", 64 * 70_000)
    chunked = engine.row_norms(X)
    assert torch.equal(plain.view(torch.int32), chunked.view(torch.int32))


def _emulate_ranks(X_np, sizes, k, first=0, mode=MODE_PRUNE):
    """world_size > 1 kernels on ONE device: W engines, the all-gather replaced by copies."""
    dev = torch.device("cuda:0")
    W = len(sizes)
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).tolist()
    X = torch.from_numpy(X_np).to(dev)
    norms = engine.row_norms(X)
    X, element_order = engine.engine_matrix(X)
    engs = []
    for r in range(W):
        Xl = X[offs[r] : offs[r] + sizes[r]].contiguous()
        nl = norms[offs[r] : offs[r] + sizes[r]].contiguous()
        e = engine.ShardEngine(Xl, nl, k, shard_offset=offs[r], world_size=W, mode=mode, element_order=element_order)
        e.init_state()
        engs.append(e)

    def gather():
        allp = torch.stack([e.pack_local for e in engs])
        for e in engs:
            e.pack_all.copy_(allp)

    for e in engs:
        e.force_pick(first)
    for i in range(k):
        gather()
        for e in engs:
            e.commit()
            e.step()
    return engs, norms.cpu().numpy(), offs


@pytest.mark.parametrize("sizes", [[1000, 1003], [0, 700, 0, 650], [333] * 7 + [340], [5, 2000]])
def test_multi_rank_kernels_on_one_device(sizes):
    N, k = sum(sizes), 150
    X = with_duplicates(gaussian_mixture(N, 64, 8, seed=N), 50, seed=1)
    first = N // 2
    engs, norms, offs = _emulate_ranks(X, sizes, k, first=first)
    o_sel, o_eps, o_h, o_v = oracle.fps_sharded(X, norms, k, sizes, first=first)
    for r, e in enumerate(engs):
        assert e.check_status().n_sel == k
        np.testing.assert_array_equal(e.selected.cpu().numpy(), o_sel)
        np.testing.assert_array_equal(bits(e.eps.cpu().numpy()), bits(o_eps))
        n = sizes[r]
        np.testing.assert_array_equal(bits(e.h[:n].cpu().numpy()), bits(o_h[offs[r] : offs[r] + n]))
        np.testing.assert_array_equal(e.voronoi[:n].cpu().numpy().astype(np.int64), o_v[offs[r] : offs[r] + n])
        assert torch.equal(e.X_sel, engs[0].X_sel)


@pytest.mark.parametrize("sizes,D", [([1000, 1003], 64), ([0, 700, 0, 650], 128), ([301, 299, 2, 300], 256)])
def test_multi_rank_kernels_dense_mode(sizes, D):
    """The dense kernel (bulk-copy ring) publishing candidates for world_size > 1."""
    N, k = sum(sizes), 100
    X = with_duplicates(gaussian_mixture(N, D, 8, seed=N + D), 20, seed=2)
    engs, norms, offs = _emulate_ranks(X, sizes, k, first=3, mode=MODE_DENSE)
    o_sel, o_eps, o_h, o_v = oracle.fps_sharded(X, norms, k, sizes, first=3)
    for r, e in enumerate(engs):
        assert e.check_status().n_sel == k
        np.testing.assert_array_equal(e.selected.cpu().numpy(), o_sel)
        np.testing.assert_array_equal(bits(e.eps.cpu().numpy()), bits(o_eps))
        n = sizes[r]
        np.testing.assert_array_equal(bits(e.h[:n].cpu().numpy()), bits(o_h[offs[r] : offs[r] + n]))
        np.testing.assert_array_equal(e.voronoi[:n].cpu().numpy().astype(np.int64), o_v[offs[r] : offs[r] + n])


def test_large_shard_properties():
    """Benchmark-sized shard (the 8-GPU share of the 300M x 128 config: 37.5M rows, 19.2 GB)
    checked through size-independent properties: unique picks, non-increasing radii, dense and
    prune modes agreeing, and for sampled rows h == distance to the centre voronoi names, bitwise
    in the reference's arithmetic."""
    from coresets_b200.synth import WORKLOADS, MixtureSource, scaled
    w = scaled(WORKLOADS["c3"], 37_500_000, k=96)
    dev = torch.device("cuda:0")
    X = MixtureSource(w).rows(0, w.n_rows, dev)
    norms = engine.row_norms(X)
    out = {}
    for mode in (MODE_PRUNE, MODE_DENSE):
        eng = engine.ShardEngine(X, norms, w.k, mode=mode)
        eng.init_state()
        eng.pick_forced(0)
        eng.run_picks(w.k - 1)
        eng.check_status()
        out[mode] = eng
    a, b = out[MODE_PRUNE], out[MODE_DENSE]
    assert torch.equal(a.selected, b.selected)
    assert torch.equal(a.h.view(torch.int32), b.h.view(torch.int32))
    assert torch.equal(a.voronoi, b.voronoi)
    sel = a.selected.cpu().numpy()
    assert len(set(sel.tolist())) == w.k
    eps = a.eps.cpu().numpy().astype(np.float64)
    assert np.isinf(eps[0]) and np.all(eps[2:] <= eps[1:-1] * (1 + 1e-5))
    g = torch.Generator().manual_seed(0)
    rows = torch.randint(0, w.n_rows, (2048,), generator=g)
    Xs = X[rows.to(dev)].cpu().numpy()
    hs = a.h[rows.to(dev)].cpu().numpy()
    vs = a.voronoi[rows.to(dev)].cpu().numpy()
    ns = norms[rows.to(dev)].cpu().numpy()
    Xsel = a.X_sel.cpu().numpy()
    nsel = a.norms_sel.cpu().numpy()
    for j in range(rows.numel()):
        if hs[j] < 0:
            continue
        dot = np.float32(oracle.warp_dot(Xs[j], Xsel[vs[j]]))
        d = np.float32(np.float32(ns[j] + nsel[vs[j]]) - np.float32(dot + dot))
        assert bits(d) == bits(hs[j])
    # the nearest centre in float64 agrees with voronoi up to rounding
    d64 = ((Xs[:256, None, :].astype(np.float64) - Xsel[None].astype(np.float64)) ** 2).sum(-1)
    near = d64.min(axis=1)
    mine = d64[np.arange(256), vs[:256]]
    assert np.all(mine <= near * (1 + 1e-4) + 1e-6)


# ---- golden vectors written by the reference's own CUDA extension on a B200 ----------------------
from pathlib import Path  # noqa: E402

GOLDEN = Path(__file__).resolve().parent / "golden"
GOLDEN_CASES = sorted(p.stem for p in GOLDEN.glob("*.npz") if p.stem != "cpu_fps_c1" and not p.stem.startswith(("acc", "fullsize", "torch_")))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_engine_reproduces_reference_golden(name):
    from tests.test_oracle_golden import load_case
    z, X = load_case(name)
    K = int(z["K"])
    seeds = tuple(int(s) for s in z["seeds"])
    eng, norms = run_engine(X, K, seed=seeds)
    np.testing.assert_array_equal(bits(norms), bits(z["norms"]))      # torch norms, same GPU type
    np.testing.assert_array_equal(eng.selected.cpu().numpy(), z["selected"])
    np.testing.assert_array_equal(bits(eng.eps.cpu().numpy()), bits(z["eps"]))
    np.testing.assert_array_equal(bits(eng.h[: X.shape[0]].cpu().numpy()), bits(z["h"]))
    np.testing.assert_array_equal(eng.voronoi[: X.shape[0]].cpu().numpy(), z["voronoi"])


@pytest.mark.parametrize("wname,n_rows", [("c3", 2_000_000), ("c2", 5_000_000), ("c4", 400_000), ("c3", 37_500_000)])
def test_engine_reproduces_reference_on_device_generated_workloads(wname, n_rows):
    """`selected` of the reference's fps_cuda on scaled-down benchmark workloads (matrices
    generated on the device, so only a B200 with this torch build regenerates them)."""
    from coresets_b200.synth import WORKLOADS, MixtureSource, scaled
    ref = np.load(GOLDEN / f"midsize_{wname}_{n_rows}_selected.npy")
    K = ref.shape[0]
    w = scaled(WORKLOADS[wname], n_rows, k=K)
    X = MixtureSource(w).rows(0, n_rows, torch.device("cuda:0"))
    sel = fps_mod.fps(X, K)
    np.testing.assert_array_equal(sel.cpu().numpy(), ref)


# ---- peer-store exchange (CS_XCHG_PEER) emulated on one device ------------------------------------
def _peer_engines(X_np, sizes, k, timeout_ms=2000, monkeypatch=None):
    """W engines on ONE device wired for the peer exchange: every 'rank' gets a window in local
    memory and all windows are visible to all engines.  Launch order guarantees that a candidate is
    published before any kernel waits for it, so no kernel ever waits on a later launch."""
    from coresets_b200._native import XCHG_PEER
    dev = torch.device("cuda:0")
    W = len(sizes)
    offs = np.concatenate([[0], np.cumsum(sizes)[:-1]]).tolist()
    X = torch.from_numpy(X_np).to(dev)
    norms = engine.row_norms(X)
    native = _native.get_native()
    words = native.xchg_window_words(W, X.shape[1])
    wins = [torch.zeros(words, dtype=torch.int32, device=dev) for _ in range(W)]
    if monkeypatch is not None:
        monkeypatch.setenv("CORESETS_B200_XCHG_TIMEOUT_MS", str(timeout_ms))
    engs = []
    for r in range(W):
        Xl = X[offs[r] : offs[r] + sizes[r]].contiguous()
        nl = norms[offs[r] : offs[r] + sizes[r]].contiguous()
        e = engine.ShardEngine(Xl, nl, k, shard_offset=offs[r], world_size=W)
        e.rank, e.xchg, e.window = r, XCHG_PEER, wins[r]
        e.peer_ptrs = [w.data_ptr() for w in wins]
        e.state = e._make_state()
        e.init_state()
        engs.append(e)
    return engs, norms.cpu().numpy(), offs, wins


@pytest.mark.parametrize("sizes", [[1000, 1003], [0, 700, 0, 650], [333] * 7 + [340]])
def test_peer_exchange_kernels_on_one_device(sizes, monkeypatch):
    N, k = sum(sizes), 120
    X = with_duplicates(gaussian_mixture(N, 64, 8, seed=N), 50, seed=1)
    first = N // 3
    engs, norms, offs, _ = _peer_engines(X, sizes, k, monkeypatch=monkeypatch)
    for e in engs:
        e.force_pick(first)                 # every rank publishes ...
    for i in range(k):
        for e in engs:
            e.commit()                      # ... before any rank consumes
        for e in engs:
            e.step()
    o_sel, o_eps, o_h, o_v = oracle.fps_sharded(X, norms, k, sizes, first=first)
    for r, e in enumerate(engs):
        ctl = e.check_status()
        assert ctl.n_sel == k and ctl.xseq == k + 1
        np.testing.assert_array_equal(e.selected.cpu().numpy(), o_sel)
        np.testing.assert_array_equal(bits(e.eps.cpu().numpy()), bits(o_eps))
        n = sizes[r]
        np.testing.assert_array_equal(bits(e.h[:n].cpu().numpy()), bits(o_h[offs[r] : offs[r] + n]))


@pytest.mark.parametrize("half_rows", [False, True])
def test_dense_pipe_wait_times_out_with_a_status(half_rows, monkeypatch):
    """The bulk-copy ring of dense mode (float32 rows, half rows) with a producer that starts no
    copy (test hook): the consumers' bounded mbarrier wait gives up, the status word says so,
    nothing faults and the context stays usable."""
    from coresets_b200._native import F_TEST_STALL_PIPE
    monkeypatch.setenv("CORESETS_B200_XCHG_TIMEOUT_MS", "40")
    dev = torch.device("cuda:0")
    X = torch.from_numpy(gaussian_mixture(5000, 128, 4, seed=1)).to(dev)
    if half_rows:
        X = X.to(torch.float16)
    eng = engine.ShardEngine(X, engine.row_norms(X), 8, mode=MODE_DENSE, element_order=half_rows)
    eng._extra_flags = F_TEST_STALL_PIPE
    eng.state = eng._make_state()
    eng.init_state()
    eng.force_pick(0)
    eng.commit()
    eng.step()
    with pytest.raises(RuntimeError, match="bulk copy"):
        eng.check_status()
    assert int(torch.ones(4, device="cuda").sum().item()) == 4
    # the same engine without the hook works
    eng._extra_flags = 0
    eng.state = eng._make_state()
    eng.init_state()
    eng.pick_forced(0)
    eng.run_picks(5)
    assert eng.check_status().n_sel == 6


def test_peer_exchange_wait_times_out_with_a_status(monkeypatch):
    """A peer that never publishes: the bounded wait gives up, the status word says so, the
    context stays usable."""
    X = gaussian_mixture(600, 32, 4, seed=4)
    engs, _, _, _ = _peer_engines(X, [300, 300], 8, timeout_ms=40, monkeypatch=monkeypatch)
    e0 = engs[0]
    e0.force_pick(5)          # rank 1 stays silent
    e0.commit()
    with pytest.raises(RuntimeError, match="timed out waiting for a peer"):
        e0.check_status()
    # the device still answers
    assert int(torch.ones(4, device="cuda").sum().item()) == 4


# ---- fused multi-state step ("lanes") -------------------------------------------------------------
@pytest.mark.parametrize("N,D,L", [(5000, 128, 4), (3001, 64, 2), (2000, 256, 3), (1500, 1024, 2), (4000, 32, 8),
                                   (900, 50, 3)])
@pytest.mark.parametrize("lane_mode", ["prune", "inline", "dense"])
def test_lanes_step_equals_separate_steps(N, D, L, lane_mode):
    """L states with different histories share X: one cs_fps_step_lanes call (per-lane deferred-row
    steps in prune mode, ONE fused pass over X in the inline and dense modes) must leave every
    state exactly where its own cs_fps_step leaves it (h bits, voronoi, next key, pick counter),
    several steps in a row."""
    from coresets_b200._native import MODE_PRUNE_INLINE
    lanes_mode = {"prune": MODE_PRUNE, "inline": MODE_PRUNE_INLINE, "dense": MODE_DENSE}[lane_mode]
    dev = torch.device("cuda:0")
    X = torch.from_numpy(gaussian_mixture(N, D, 8, seed=N + D + L)).to(dev)
    norms = engine.row_norms(X)

    def make_set():
        engs = []
        for l in range(L):
            e = engine.ShardEngine(X, norms, 64)
            e.init_state()
            e.pick_forced((37 * l + 5) % N)
            e.run_picks(3 * l)                       # lane l has 1 + 3l centres
            engs.append(e)
        return engs

    fused, apart = make_set(), make_set()
    for _ in range(5):
        for e in fused:
            e.exchange(); e.commit()
        engine.ShardEngine.step_lanes(fused, mode=lanes_mode)
        for e in apart:
            e.exchange(); e.commit(); e.step()
        for a, b in zip(fused, apart):
            ca, cb = a.check_status(), b.check_status()
            assert ca.n_sel == cb.n_sel and list(ca.key) == list(cb.key)
            assert torch.equal(a.h.view(torch.int32), b.h.view(torch.int32))
            assert torch.equal(a.voronoi, b.voronoi)
    for a, b in zip(fused, apart):
        assert torch.equal(a.selected[: a.check_status().n_sel], b.selected[: b.check_status().n_sel])


def test_more_centres_than_the_shared_bound_table():
    """k above 16384: the bound table no longer fits the 64 KB shared-memory stage, the tail of
    the look-ups goes to global memory; picks must stay the oracle's."""
    N, D, k = 30000, 8, 17000
    X = gaussian_mixture(N, D, 8, seed=77)
    eng, norms = run_engine(X, k)
    assert_matches_oracle(eng, X, norms, k)


# ---- exact selection (the bisect early exit of the single-GPU accretion driver) -------------------
@pytest.mark.parametrize("n", [1, 2, 255, 4096, 100_003, 3_000_000])
def test_kth_largest_live_matches_a_sort(n):
    """cs_select_kth_largest against torch.sort / torch.kthvalue on h with selected rows (-1),
    zeros of both signs, duplicates, +inf and a wide range of magnitudes."""
    g = torch.Generator(device="cpu").manual_seed(n)
    h = torch.rand(n, generator=g) ** 4 * 1e4
    h[torch.rand(n, generator=g) < 0.2] = -1.0                  # selected rows
    h[torch.rand(n, generator=g) < 0.05] = 0.0
    h[torch.rand(n, generator=g) < 0.02] = -0.0
    h[torch.rand(n, generator=g) < 0.1] = 3.25                  # heavy duplicates
    if n > 10:
        h[7] = float("inf")
        h[3] = 1e-30
    dev = torch.device("cuda:0")
    X = torch.zeros((n, 4), device=dev)
    eng = engine.ShardEngine(X, torch.zeros(n, device=dev), 1)
    eng.h.copy_(h.to(dev))
    live = torch.sort(h[h >= 0]).values
    n_alive = int(live.numel())
    ks = sorted({1, 2, 3, n_alive // 2, n_alive - 1, n_alive, n_alive + 1, 0, 17, 1000} )
    for k in ks:
        val, cnt = eng.kth_largest_live(k)
        assert cnt == n_alive
        if 1 <= k <= n_alive:
            want = float(live[n_alive - k])
            assert val == want, (k, val, want)
            if n_alive - k + 1 >= 1:
                assert val == float(torch.kthvalue(h[h >= 0], n_alive - k + 1).values)
        else:
            assert val is None
