"""Accretion host logic on CPU against golden vectors written by the REFERENCE's own drivers
(tests/golden/make_golden_accrete_cpu.py runs src/coresets/cuda/accrete.py and
src/coresets/cuda/multi/sharded.py on CPU tensors with the oracle as their kernel extension).
Here the package's drivers run on the oracle-backed stand-in native library; index lists and the
per-commit trace (values and separations bit for bit) must be identical."""
import importlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from coresets_b200 import _native
from tests.fake_native import FakeNative
from tests.golden.make_golden_accrete_cpu import CASES, PHASES, make_case, read_trace
from tests.test_sharded_gloo import _run

GOLDEN = Path(__file__).resolve().parent / "golden"
acc_mod = importlib.import_module("coresets_b200.cuda.accrete")


@pytest.fixture()
def fake_native(monkeypatch):
    monkeypatch.setattr(_native, "_native", FakeNative())
    monkeypatch.setattr(acc_mod, "_REQUIRE_CUDA", False)
    for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
        monkeypatch.delenv(k, raising=False)
    yield


@pytest.mark.parametrize("name", [n for n, c in CASES.items() if "n_target" not in c])
def test_single_gpu_driver_matches_reference(fake_native, name, tmp_path):
    c = CASES[name]
    z = np.load(GOLDEN / f"accrete_cpu_{name}.npz")
    X, order = make_case(c)
    np.testing.assert_array_equal(order, z["anchor_order"])
    Xt = torch.from_numpy(X)
    tr = str(tmp_path / "trace.tsv")
    got = acc_mod.accrete(Xt[: c["n_anchor"]], Xt[c["n_anchor"] :], torch.from_numpy(order), c["max_k"],
                          verbose=False, trace_path=tr)
    np.testing.assert_array_equal(got.numpy(), z["single"])
    mine = read_trace(tr)
    for key in ("trace_phase", "trace_pos", "trace_idx"):
        np.testing.assert_array_equal(mine[key], z[key])
    # values and running separations: every bit (hex floats in the trace)
    np.testing.assert_array_equal(mine["trace_val"].view(np.int64), z["trace_val"].view(np.int64))
    np.testing.assert_array_equal(mine["trace_sep"].view(np.int64), z["trace_sep"].view(np.int64))


@pytest.mark.parametrize("world", [1, 2])
def test_sharded_driver_matches_reference(tmp_path, world):
    cases = []
    for name, c in CASES.items():
        X, order = make_case(c)
        np.save(tmp_path / f"{name}_x.npy", X)
        np.save(tmp_path / f"{name}_o.npy", order)
        base = dict(x_path=str(tmp_path / f"{name}_x.npy"), order_path=str(tmp_path / f"{name}_o.npy"),
                    n_anchor=c["n_anchor"], max_k=c["max_k"], n_target=c.get("n_target"))
        cases.append(dict(base, name=f"{name}_plain"))
        cases.append(dict(base, name=f"{name}_knobs", env={"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"}))
        # fused probe lanes forced on (they need long simulations by default): same list as without
        cases.append(dict(base, name=f"{name}_lanes", env={"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256",
                                                          "CORESETS_LANES_MIN_STEPS": "4"}))
        # knobs that change the probe schedule (and, on one case, the reference's list itself)
        cases.append(dict(base, name=f"{name}_deep", env={"CORESETS_BISECT_SEED": "1", "CORESETS_BISECT_GALLOP_DEEP": "1",
                                                         "CORESETS_FILL_CHUNK": "64"}))
        cases.append(dict(base, name=f"{name}_nolazy", env={"CORESETS_BISECT_SEED": "1", "CORESETS_LAZY_FORWARD": "0"}))
        if "n_target" not in c:
            # the replicated entry (whole matrix on every rank): the reference's three drivers give one list
            # (its tests/test_determinism.py), so the sharded driver's golden list applies
            cases.append(dict(base, name=f"{name}_repl", replicated=True))
    _run(world, dict(mode="accrete", cases=cases, out_dir=str(tmp_path)), timeout=900)
    for name in CASES:
        z = np.load(GOLDEN / f"accrete_cpu_{name}.npz")
        for r in range(world):
            np.testing.assert_array_equal(np.load(tmp_path / f"{name}_plain_{r}.npy"), z[f"sharded_w{world}"])
            np.testing.assert_array_equal(np.load(tmp_path / f"{name}_knobs_{r}.npy"), z[f"sharded_w{world}_knobs"])
            np.testing.assert_array_equal(np.load(tmp_path / f"{name}_lanes_{r}.npy"), z[f"sharded_w{world}_knobs"])
            np.testing.assert_array_equal(np.load(tmp_path / f"{name}_deep_{r}.npy"), z[f"sharded_w{world}_deep"])
            np.testing.assert_array_equal(np.load(tmp_path / f"{name}_nolazy_{r}.npy"), z[f"sharded_w{world}_nolazy"])
            if "n_target" not in CASES[name]:
                np.testing.assert_array_equal(np.load(tmp_path / f"{name}_repl_{r}.npy"), z[f"sharded_w{world}"])


def test_accrete_validation(fake_native):
    X = torch.zeros(8, 4)
    with pytest.raises(ValueError, match="empty"):
        acc_mod.accrete(X[:0], X, torch.arange(0), 2, verbose=False)
    with pytest.raises(ValueError, match="mismatch"):
        acc_mod.accrete(X, torch.zeros(8, 5), torch.arange(8), 2, verbose=False)


def test_checkpoint_files_match_the_reference_and_resume_reproduces_the_run(tmp_path):
    """Layer checkpoints of the sharded driver (`<prefix>_kKK.npy`, `_kKK_sep.npy`, `_latest.txt`,
    `_seeds.npy`; src/coresets/cuda/multi/sharded.py:493-549, 754-775) against the files the
    reference wrote for the same run (tests/golden/make_golden_accrete_ckpt.py), then a resume
    from the last but one layer.  This package resumes by replaying the stored picks through the
    same kernels, so the resumed list equals the uninterrupted one; the reference rebuilds its
    state with a matrix product and its own resumed list differs from its own full run on this
    case (kept in the fixture as `resumed`)."""
    from tests.golden.make_golden_accrete_ckpt import CASE, EVERY, KNOBS
    z = np.load(GOLDEN / "accrete_cpu_ckpt.npz")
    c = CASES[CASE]
    X, order = make_case(c)
    np.save(tmp_path / "x.npy", X)
    np.save(tmp_path / "o.npy", order)
    base = dict(x_path=str(tmp_path / "x.npy"), order_path=str(tmp_path / "o.npy"), n_anchor=c["n_anchor"],
                max_k=c["max_k"], env=KNOBS)
    _run(1, dict(mode="accrete", out_dir=str(tmp_path),
                 cases=[dict(base, name="full", checkpoint="ck", checkpoint_every=EVERY)]), timeout=600)
    full = np.load(tmp_path / "full_0.npy")
    np.testing.assert_array_equal(full, z["full"])
    names = sorted(p.name for p in tmp_path.iterdir() if p.name.startswith("ck_"))
    assert names == [str(n) for n in z["names"]]
    for n in names:
        want = z["file:" + n]
        if n.endswith(".npy"):
            got = np.load(tmp_path / n)
            assert got.dtype == want.dtype and got.shape == want.shape, n
            np.testing.assert_array_equal(got.view(np.int64) if got.dtype == np.float64 else got,
                                          want.view(np.int64) if want.dtype == np.float64 else want, err_msg=n)
        else:
            assert (tmp_path / n).read_text() == str(want), n
    top = c["max_k"]
    for n in names:
        if f"_k{top:02d}" in n:
            (tmp_path / n).unlink()
    (tmp_path / "ck_latest.txt").write_text(f"{top - 1}\n")
    _run(1, dict(mode="accrete", out_dir=str(tmp_path), cases=[dict(base, name="again", resume="ck")]), timeout=600)
    np.testing.assert_array_equal(np.load(tmp_path / "again_0.npy"), full)
    assert not np.array_equal(z["resumed"], z["full"])      # the reference's own resume is not reproducible here


@pytest.mark.parametrize("world", [1, 2])
def test_sharded_driver_trace_matches_the_reference(tmp_path, world):
    """Per-commit trace of the sharded driver (forward / replay / fill lines with value and
    running separation, bit for bit) against the reference's own one-rank trace; the trace does not
    depend on the number of ranks."""
    from tests.golden.make_golden_accrete_traces import KNOB_SETS, TRACE_CASES
    z = np.load(GOLDEN / "accrete_cpu_sharded_traces.npz")
    cases = []
    for name in TRACE_CASES:
        c = CASES[name]
        X, order = make_case(c)
        np.save(tmp_path / f"{name}_x.npy", X)
        np.save(tmp_path / f"{name}_o.npy", order)
        for tag, env in KNOB_SETS.items():
            cases.append(dict(x_path=str(tmp_path / f"{name}_x.npy"), order_path=str(tmp_path / f"{name}_o.npy"),
                              n_anchor=c["n_anchor"], max_k=c["max_k"], name=f"{name}_{tag}", env=env, trace=True))
    _run(world, dict(mode="accrete", cases=cases, out_dir=str(tmp_path)), timeout=900)
    for name in TRACE_CASES:
        for tag in KNOB_SETS:
            mine = read_trace(str(tmp_path / f"{name}_{tag}_trace_0.tsv"))
            for key in ("trace_phase", "trace_pos", "trace_idx"):
                np.testing.assert_array_equal(mine[key], z[f"{name}:{tag}:{key}"], err_msg=f"{name} {tag} {key}")
            for key in ("trace_val", "trace_sep"):
                np.testing.assert_array_equal(mine[key].view(np.int64), z[f"{name}:{tag}:{key}"].view(np.int64),
                                              err_msg=f"{name} {tag} {key}")
