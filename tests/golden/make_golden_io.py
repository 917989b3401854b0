"""Golden description of the reference's result directory.

    python tests/golden/make_golden_io.py --reference <reference checkout>

Runs the reference's `save_result` / `load_result` (src/coresets/io.py:40-110) on a small result
and records what a reader of the directory depends on: the file names, the array dtypes and
shapes, the key order of meta.json and the values that do not depend on the machine or the clock.
Writes tests/golden/io_layout.json.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
from pathlib import Path

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
    a = ap.parse_args()
    sys.path.insert(0, str(Path(a.reference) / "src"))
    import coresets
    for k in [k for k in os.environ if k.startswith("CORESETS_")]:
        del os.environ[k]
    os.environ["CORESETS_FILL_CHUNK"] = "256"
    os.environ["CORESETS_BISECT_SEED"] = "1"
    sel = np.array([5, 0, 9, 3], dtype=np.int32)
    eps = np.array([np.inf, 4.0, 2.5, 1.0], dtype=np.float64)
    rec = {}
    with tempfile.TemporaryDirectory() as d:
        out = Path(d) / "run"
        coresets.save_result(out, sel, epsilons=eps, n_rows=10, dim=3, backend="unit", walltime_s=1.5,
                             world_size=2, extra={"note": "x"})
        rec["files"] = sorted(p.name for p in out.iterdir())
        meta = json.loads((out / "meta.json").read_text())
        rec["meta_keys"] = list(meta.keys())
        stable = ("schema", "K", "n_rows", "dim", "backend", "world_size", "walltime_s", "has_epsilons", "knobs", "note")
        rec["meta_stable"] = {k: meta[k] for k in stable if k in meta}
        s2, e2 = np.load(out / "selected.npy"), np.load(out / "epsilons.npy")
        rec["selected"] = dict(dtype=str(s2.dtype), shape=list(s2.shape))
        rec["epsilons"] = dict(dtype=str(e2.dtype), shape=list(e2.shape))
        loaded = coresets.load_result(out)
        rec["load_keys"] = sorted(loaded.keys())
        try:
            coresets.save_result(out, sel)
            rec["second_save"] = "ok"
        except Exception as e:  # noqa: BLE001
            rec["second_save"] = type(e).__name__
        coresets.save_result(out, sel, overwrite=True)
        rec["files_after_overwrite_without_eps"] = sorted(p.name for p in out.iterdir())
        rec["has_epsilons_after_overwrite"] = json.loads((out / "meta.json").read_text())["has_epsilons"]
        try:
            coresets.load_result(Path(d) / "missing")
            rec["load_missing"] = "ok"
        except Exception as e:  # noqa: BLE001
            rec["load_missing"] = type(e).__name__
        try:
            coresets.save_result(Path(d) / "bad", np.zeros((2, 2), dtype=np.int64))
            rec["save_2d"] = "ok"
        except Exception as e:  # noqa: BLE001
            rec["save_2d"] = type(e).__name__
        try:
            coresets.save_result(Path(d) / "bad2", sel, epsilons=eps[:2])
            rec["save_eps_mismatch"] = "ok"
        except Exception as e:  # noqa: BLE001
            rec["save_eps_mismatch"] = type(e).__name__
    path = Path(__file__).parent / "io_layout.json"
    path.write_text(json.dumps(rec, indent=1) + "\n")
    print(json.dumps(rec, indent=1))


if __name__ == "__main__":
    main()
