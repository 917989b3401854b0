"""The chained-run files (manifest, step directories, LATEST, per-level log) against the golden
description written from the reference's own io module (tests/golden/make_golden_io_run.py)."""
import json
from pathlib import Path

from coresets_b200 import io
from tests.io_run_scenario import run_scenario

GOLDEN = Path(__file__).parent / "golden" / "io_run.json"


def test_run_directory_matches_the_reference(tmp_path):
    want = json.loads(GOLDEN.read_text())
    got = json.loads(json.dumps(run_scenario(io, tmp_path)))
    assert list(got["tree"].keys()) == list(want["tree"].keys())
    for rel, w in want["tree"].items():
        assert got["tree"][rel] == w, rel
    assert got["calls"] == want["calls"]


def test_reference_names_are_exported():
    import coresets_b200
    for name in ("init_run", "register_source", "read_manifest", "StepStats", "save_step", "load_step", "load_latest",
                 "list_steps", "open_per_level", "append_per_level", "PROVENANCE_DTYPE", "SCHEMA_VERSION"):
        assert hasattr(coresets_b200.io, name), name
