"""Golden description of the reference's chained-run files (manifest, steps, per-level log).

    python tests/golden/make_golden_io_run.py --reference <reference checkout>

Drives the reference's own `coresets.io` (src/coresets/io.py:162-490) through the scenario in
tests/io_run_scenario.py and writes what it left on disk, and what each call returned or raised,
to tests/golden/io_run.json (clock values and the commit hash masked).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"), required=not os.environ.get("CORESETS_REFERENCE_ROOT"))
    a = ap.parse_args()
    sys.path.insert(0, str(Path(a.reference) / "src"))
    import coresets.io as ref_io
    from tests.io_run_scenario import run_scenario
    with tempfile.TemporaryDirectory() as d:
        rec = run_scenario(ref_io, Path(d))
    path = Path(__file__).parent / "io_run.json"
    path.write_text(json.dumps(rec, indent=1) + "\n")
    print(f"wrote {path}: {len(rec['tree'])} files, {len(rec['calls'])} calls")


if __name__ == "__main__":
    main()
