"""Shard geometry and the on-disk result layout.

tests/golden/io_layout.json describes what the reference's `save_result` / `load_result` wrote for
a small result (tests/golden/make_golden_io.py ran src/coresets/io.py:40-110); this package must
write the same files, dtypes, meta.json keys in the same order and the same machine-independent
values, and raise the same exception types."""
import json
from pathlib import Path

import numpy as np
import pytest

import coresets_b200
from coresets_b200.cuda.multi.layout import ShardLayout, compute_shard_layout

GOLD = json.loads((Path(__file__).resolve().parent / "golden" / "io_layout.json").read_text())


def _outcome(fn):
    try:
        fn()
        return "ok"
    except Exception as e:  # noqa: BLE001
        return type(e).__name__


def test_result_directory_matches_the_reference(tmp_path, monkeypatch):
    for k in [k for k in __import__("os").environ if k.startswith("CORESETS_")]:
        monkeypatch.delenv(k)
    monkeypatch.setenv("CORESETS_FILL_CHUNK", "256")
    monkeypatch.setenv("CORESETS_BISECT_SEED", "1")
    sel = np.array([5, 0, 9, 3], dtype=np.int32)
    eps = np.array([np.inf, 4.0, 2.5, 1.0], dtype=np.float64)
    out = tmp_path / "run"
    coresets_b200.save_result(out, sel, epsilons=eps, n_rows=10, dim=3, backend="unit", walltime_s=1.5,
                              world_size=2, extra={"note": "x"})
    assert sorted(p.name for p in out.iterdir()) == GOLD["files"]
    meta = json.loads((out / "meta.json").read_text())
    assert list(meta.keys()) == GOLD["meta_keys"]
    assert {k: meta[k] for k in GOLD["meta_stable"]} == GOLD["meta_stable"]
    s2, e2 = np.load(out / "selected.npy"), np.load(out / "epsilons.npy")
    assert dict(dtype=str(s2.dtype), shape=list(s2.shape)) == GOLD["selected"]
    assert dict(dtype=str(e2.dtype), shape=list(e2.shape)) == GOLD["epsilons"]
    np.testing.assert_array_equal(s2, sel)
    np.testing.assert_array_equal(e2, eps.astype(np.float32))
    loaded = coresets_b200.load_result(out)
    assert sorted(loaded.keys()) == GOLD["load_keys"]
    np.testing.assert_array_equal(loaded["selected"], sel)
    assert _outcome(lambda: coresets_b200.save_result(out, sel)) == GOLD["second_save"]
    coresets_b200.save_result(out, sel, overwrite=True)
    assert sorted(p.name for p in out.iterdir()) == GOLD["files_after_overwrite_without_eps"]
    assert json.loads((out / "meta.json").read_text())["has_epsilons"] == GOLD["has_epsilons_after_overwrite"]
    assert _outcome(lambda: coresets_b200.load_result(tmp_path / "missing")) == GOLD["load_missing"]
    assert _outcome(lambda: coresets_b200.save_result(tmp_path / "bad", np.zeros((2, 2), dtype=np.int64))) == GOLD["save_2d"]
    assert _outcome(lambda: coresets_b200.save_result(tmp_path / "bad2", sel, epsilons=eps[:2])) == GOLD["save_eps_mismatch"]


def test_save_result_accepts_tensors(tmp_path):
    import torch
    out = coresets_b200.save_result(tmp_path / "t", torch.tensor([3, 1, 2]), epsilons=torch.tensor([float("inf"), 2.0, 1.0]))
    got = coresets_b200.load_result(out)
    assert got["selected"].tolist() == [3, 1, 2] and got["epsilons"].dtype == np.float32
    assert got["meta"]["K"] == 3 and got["meta"]["has_epsilons"] is True


# ---- shard geometry (src/coresets/cuda/multi/layout.py:8-50) -----------------------------------------
def linear_scan_owner(offsets, world, idx):
    """The reference's rule in words: the first rank whose successor starts beyond idx, else the last."""
    for r in range(world - 1):
        if idx < offsets[r + 1]:
            return r
    return world - 1


def test_layout_puts_the_remainder_on_the_last_rank():
    assert compute_shard_layout(16383, 4) == ([4095, 4095, 4095, 4098], [0, 4095, 8190, 12285])
    assert compute_shard_layout(10, 3) == ([3, 3, 4], [0, 3, 6])
    assert compute_shard_layout(2, 4) == ([0, 0, 0, 2], [0, 0, 0, 0])      # empty shards are legal
    assert compute_shard_layout(0, 2) == ([0, 0], [0, 0])
    assert compute_shard_layout(7, 1) == ([7], [0])
    for bad in (0, -1):
        with pytest.raises(ValueError):
            compute_shard_layout(5, bad)


def test_owner_of_equals_the_reference_linear_scan():
    for n in (0, 1, 2, 5, 16, 33, 100):
        for world in (1, 2, 3, 4, 7, 8):
            sizes, offsets = compute_shard_layout(n, world)
            for rank in range(world):
                lay = ShardLayout(rank=rank, world_size=world, sizes=sizes, offsets=offsets)
                assert lay.N_global == n and lay.N_shard == sizes[rank] and lay.shard_offset == offsets[rank]
                for idx in range(-2, n + 3):
                    assert lay.owner_of(idx) == linear_scan_owner(offsets, world, idx), (n, world, idx)
                if sizes[rank]:
                    assert lay.to_local(offsets[rank]) == 0
