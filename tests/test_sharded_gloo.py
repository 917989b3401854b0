"""fps_sharded host logic at world_size > 1 on CPU: gloo ranks, oracle-backed stand-in native
library, compared with the oracle's emulation of the reference's sharded driver."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import oracle
from tests.data import clustered_jitter, with_duplicates
from tests.ports import address_in_use, free_port

ROOT = Path(__file__).resolve().parent.parent


def _run(world: int, cfg: dict, timeout: int = 240) -> None:
    for attempt in range(3):
        port = free_port()
        procs = []
        for r in range(world):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r),
                       MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
            procs.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "gloo_worker.py"), json.dumps(cfg)],
                                          env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        outs = []
        try:
            for p in procs:
                o, _ = p.communicate(timeout=timeout)
                outs.append(o)
        finally:
            for p in procs:
                if p.poll() is None:
                    p.kill()
        if any(p.returncode != 0 for p in procs) and address_in_use(outs) and attempt < 2:
            continue                                   # the rendezvous port was taken: another one
        break
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} failed:\n{outs[r][-3000:]}"


def _norms(X):
    import torch
    t = torch.from_numpy(X)
    return (t * t).sum(dim=1).numpy()


@pytest.mark.parametrize("sizes,k,seed", [
    ([300, 301], 64, None),            # remainder on the last rank
    ([0, 257], 40, 5),                 # an empty shard publishes "nothing"
    ([128, 128, 131], 48, 200),        # three ranks, seeded first pick owned by rank 1
])
def test_fps_sharded_matches_oracle(tmp_path, sizes, k, seed):
    N = sum(sizes)
    X = with_duplicates(clustered_jitter(N, 16, seed=7), 20, seed=3)
    np.save(tmp_path / "x.npy", X)
    cfg = dict(x_path=str(tmp_path / "x.npy"), sizes=sizes, k=k, seed=seed, out_dir=str(tmp_path))
    _run(len(sizes), cfg)
    o_sel, o_eps, _, _ = oracle.fps_sharded(X, _norms(X), k, sizes, first=seed or 0)
    single_sel, _, _, _ = oracle.fps_cuda(X, _norms(X), k, seed=np.array([seed or 0]))
    np.testing.assert_array_equal(o_sel, single_sel)      # the oracle itself: sharded == single
    for r in range(len(sizes)):
        sel = np.load(tmp_path / f"sel_{r}.npy")
        eps = np.load(tmp_path / f"eps_{r}.npy")
        np.testing.assert_array_equal(sel, o_sel)
        assert np.isinf(eps[0]) and eps[0] > 0
        np.testing.assert_array_equal(eps.view(np.int32), o_eps.view(np.int32))


@pytest.mark.parametrize("dtype", ["float16", "float64"])
def test_fps_sharded_float16_and_float64(tmp_path, dtype):
    """Non-float32 shards: norms in the input's dtype, rows cast to float, element-wise dots."""
    import torch
    from tests.data import as_dtype
    sizes, k = [150, 153], 48
    X = as_dtype(with_duplicates(clustered_jitter(sum(sizes), 16, seed=9), 10, seed=4), dtype)
    np.save(tmp_path / "x.npy", X)
    cfg = dict(x_path=str(tmp_path / "x.npy"), sizes=sizes, k=k, seed=None, out_dir=str(tmp_path))
    _run(2, cfg)
    t = torch.from_numpy(X)
    norms = (t * t).sum(dim=1).to(torch.float32).numpy()
    with oracle.element_order():
        o_sel, o_eps, _, _ = oracle.fps_sharded(X.astype(np.float32), norms, k, sizes)
    for r in range(2):
        np.testing.assert_array_equal(np.load(tmp_path / f"sel_{r}.npy"), o_sel)
        np.testing.assert_array_equal(np.load(tmp_path / f"eps_{r}.npy").view(np.int32), o_eps.view(np.int32))


def test_checkpoint_cadence_and_resume(tmp_path):
    sizes, k = [200, 203], 40
    X = clustered_jitter(sum(sizes), 8, seed=11)
    np.save(tmp_path / "x.npy", X)
    cfg = dict(x_path=str(tmp_path / "x.npy"), sizes=sizes, k=k, out_dir=str(tmp_path), checkpoint=True)
    _run(2, cfg)
    full = np.load(tmp_path / "sel_0.npy")
    full_eps = np.load(tmp_path / "eps_0.npy")
    # powers of two plus the last pick; ids hold k+1 entries (fps_sharded.py:269-281, 422-446)
    steps = sorted(int(p.name.split("_k")[1].split("_")[0]) for p in tmp_path.glob("ck_k*_ids.npy"))
    assert steps == [2, 4, 8, 16, 32, 39]
    for s in steps:
        ids = np.load(tmp_path / f"ck_k{s:010d}_ids.npy")
        eps = np.load(tmp_path / f"ck_k{s:010d}_eps.npy")
        assert ids.dtype == np.int64 and eps.dtype == np.float32
        np.testing.assert_array_equal(ids, full[: s + 1])
        np.testing.assert_array_equal(eps.view(np.int32), full_eps[: s + 1].view(np.int32))
    assert (tmp_path / "ck_latest.txt").read_text() == "39\n"
    # resume from pick 16 and extend to the same k: identical ids and radii
    (tmp_path / "ck_latest.txt").write_text("16\n")
    cfg2 = dict(cfg, checkpoint=False, resume=True)
    _run(2, cfg2)
    np.testing.assert_array_equal(np.load(tmp_path / "sel_1.npy"), full)
    np.testing.assert_array_equal(np.load(tmp_path / "eps_1.npy").view(np.int32), full_eps.view(np.int32))


def test_dim_mismatch_raises_on_every_rank(tmp_path):
    X = clustered_jitter(64, 8, seed=1)
    np.save(tmp_path / "x.npy", X)
    cfg = dict(x_path=str(tmp_path / "x.npy"), sizes=[32, 32], k=4, out_dir=str(tmp_path), expect_error="dim")
    _run(2, cfg)
    for r in range(2):
        assert "disagrees with peers" in (tmp_path / f"err_{r}.txt").read_text()
