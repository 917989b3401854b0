"""One chained-run scenario driven through an `io` module (the reference's or this package's) and
the normalised description of everything it leaves on disk.  Used by
tests/golden/make_golden_io_run.py (reference side) and tests/test_io_run.py (this package)."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

_CLOCK_KEYS = {"created_at", "finished_at", "git_commit"}


def _mask(obj):
    if isinstance(obj, dict):
        return {k: ("<masked>" if k in _CLOCK_KEYS else _mask(v)) for k, v in obj.items()}
    if isinstance(obj, list):
        return [_mask(v) for v in obj]
    return obj


def describe_tree(root: Path) -> dict:
    """Every file under ``root``: JSON parsed (key order kept, clock / commit values masked), .npy as
    dtype + values, text verbatim."""
    out = {}
    for p in sorted(root.rglob("*")):
        if p.is_dir():
            continue
        rel = str(p.relative_to(root))
        if p.suffix == ".json":
            text = p.read_text()
            obj = json.loads(text)
            out[rel] = {"keys": list(obj.keys()), "value": _mask(obj), "ends_with_newline": text.endswith("\n"),
                        "indent2": text.startswith("{\n  \"")}
        elif p.suffix == ".npy":
            a = np.load(p)
            out[rel] = {"dtype": str(a.dtype), "shape": list(a.shape), "values": a.tolist()}
        else:
            out[rel] = {"text": p.read_text()}
    return out


def run_scenario(io, root: Path) -> dict:
    """Returns ``{"tree": ..., "calls": ...}``: the directory description and what the calls returned or raised."""
    calls = {}

    def attempt(name, fn):
        try:
            calls[name] = fn()
        except Exception as e:  # noqa: BLE001
            calls[name] = f"raises {type(e).__name__}"

    run_dir = io.init_run(root, "runA", target_K=64, feature_dim=8, description="two chained steps")
    calls["init_run"] = str(Path(run_dir).relative_to(root))
    attempt("init_run_again", lambda: str(io.init_run(root, "runA", target_K=1, feature_dim=1)))
    calls["src_a"] = io.register_source(root, "runA", "set_a", path="/data/a.npy", n_rows=1000, sha256="ab12")
    calls["src_b"] = io.register_source(root, "runA", "set_b", n_rows=500, extra={"units": "eV"})
    calls["src_a_again"] = io.register_source(root, "runA", "set_a", n_rows=7)
    calls["manifest_sources"] = _mask(io.read_manifest(root, "runA"))["data_sources"]

    core0 = np.array([3, 1, 4, 15, 9], dtype=np.int64)
    prov0 = np.zeros(5, dtype=io.PROVENANCE_DTYPE)
    prov0["source_id"] = [0, 0, 1, 1, 0]
    prov0["source_row"] = [3, 1, 0, 11, 9]
    s0 = io.save_step(root, "runA", "seed", coreset=core0, provenance=prov0,
                      stats=io.StepStats(max_k=3, n_anchor=5, n_candidates=0, walltime_s=1.25),
                      started_at="2020-01-01T00:00:00+00:00")
    calls["step0_dir"] = Path(s0).name
    with io.open_per_level(s0) as wr:
        wr.write(1, 2, 3.5, 1.25, 0.0, 0.125)
        wr.write(2, 4, 1.0 / 3.0, 1e-12, 123456789.125, 10.0)
    io.append_per_level(root, "runA", "seed", k=3, size=5, sep=2.0, cov=0.5, rel_gap=1e-3, walltime_s=0.5)

    core1 = np.arange(7, dtype=np.int64)
    s1 = io.save_step(root, "runA", "grow", coreset=core1,
                      stats=io.StepStats(max_k=4, n_anchor=5, n_candidates=20, walltime_s=2.0, peak_mem_gb=1.5,
                                         max_rel_gap=0.01, parents=("seed",), candidate_sources=("set_b",)))
    calls["step1_dir"] = Path(s1).name
    io.append_per_level(root, "runA", "001_grow", k=4, size=7, sep=1.5, cov=0.75, rel_gap=0.0, walltime_s=2.0)
    # a failed step does not move LATEST; an explicit index is honoured; a re-run of a name wins look-ups
    s2 = io.save_step(root, "runA", "grow", coreset=core1[:3],
                      stats=io.StepStats(max_k=4, n_anchor=5, n_candidates=20, walltime_s=0.1, success=False))
    calls["step2_dir"] = Path(s2).name
    s7 = io.save_step(root, "runA", "late", coreset=core1[:2],
                      stats=io.StepStats(max_k=1, n_anchor=2, n_candidates=0, walltime_s=0.0), step_idx=7)
    calls["step7_dir"] = Path(s7).name
    calls["list_steps"] = io.list_steps(root, "runA")
    calls["latest_coreset"] = io.load_latest(root, "runA")["coreset"].tolist()
    calls["latest_dir"] = io.load_latest(root, "runA")["dir"].name
    by_name = io.load_step(root, "runA", "grow")
    calls["load_grow_dir"] = by_name["dir"].name
    calls["load_grow_prov_is_none"] = by_name["provenance"] is None
    calls["load_seed_prov"] = io.load_step(root, "runA", "000_seed")["provenance"].tolist()
    calls["load_seed_meta_keys"] = list(io.load_step(root, "runA", "seed")["meta"].keys())
    attempt("load_missing_step", lambda: io.load_step(root, "runA", "nope"))
    attempt("save_step_bad_dtype", lambda: io.save_step(root, "runA", "x", coreset=core0.astype(np.int32),
                                                        stats=io.StepStats(1, 1, 1, 0.0)))
    attempt("save_step_bad_prov_shape", lambda: io.save_step(root, "runA", "x", coreset=core0, provenance=prov0[:2],
                                                             stats=io.StepStats(1, 1, 1, 0.0)))
    attempt("save_step_bad_prov_dtype", lambda: io.save_step(root, "runA", "x", coreset=core0,
                                                             provenance=np.zeros(5, dtype=np.int64),
                                                             stats=io.StepStats(1, 1, 1, 0.0)))
    attempt("save_step_no_run", lambda: io.save_step(root, "ghost", "x", coreset=core0, stats=io.StepStats(1, 1, 1, 0.0)))
    io.init_run(root, "runB", target_K=8, feature_dim=2)
    attempt("load_latest_empty_run", lambda: io.load_latest(root, "runB"))
    calls["list_steps_empty"] = io.list_steps(root, "runB")
    io.init_run(root, "runB", target_K=9, feature_dim=3, overwrite=True)
    calls["overwritten_target"] = io.read_manifest(root, "runB")["target_K"]
    return {"tree": describe_tree(Path(root)), "calls": calls}
