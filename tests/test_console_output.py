"""What the accretion drivers print with ``verbose=True, profile=True`` against the reference's own
console output (tests/golden/verbose_*.txt, written by tests/golden/make_golden_verbose.py with
every wall-clock figure masked): the level tables, the per-block / per-probe log lines of the
sharded driver (probe order, `mid`, `sim_fill`, verdicts, `best_m`) and the profile block."""
import contextlib
import importlib
import io
from pathlib import Path

import torch

from coresets_b200 import _native
from tests.fake_native import FakeNative
from tests.golden.make_golden_accrete_cpu import CASES, make_case
from tests.golden.make_golden_verbose import CASE, CASE_KNOBS, KNOBS, mask

GOLDEN = Path(__file__).resolve().parent / "golden"


def _setup(monkeypatch, case=CASE, knobs=None):
    monkeypatch.setattr(_native, "_native", FakeNative())
    for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK", "CORESETS_LAZY_FORWARD", "CORESETS_BISECT_GALLOP_DEEP"):
        monkeypatch.delenv(k, raising=False)
    for k, v in (knobs or {}).items():
        monkeypatch.setenv(k, v)
    c = CASES[case]
    X, order = make_case(c)
    return c, torch.from_numpy(X), torch.from_numpy(order)


def test_single_driver_console_output(monkeypatch):
    acc = importlib.import_module("coresets_b200.cuda.accrete")
    monkeypatch.setattr(acc, "_REQUIRE_CUDA", False)
    c, X, order = _setup(monkeypatch)
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        acc.accrete(X[: c["n_anchor"]], X[c["n_anchor"] :], order, c["max_k"], verbose=True, profile=True)
    assert mask(buf.getvalue()) == (GOLDEN / "verbose_single.txt").read_text()


import pytest


@pytest.mark.parametrize("case,knobs,golden,profile", [(CASE, None, "verbose_sharded.txt", True),
                                                       (CASE_KNOBS, KNOBS, "verbose_sharded_knobs.txt", False)])
def test_sharded_driver_console_output(monkeypatch, case, knobs, golden, profile):
    import torch.distributed as dist
    from tests.ports import free_port
    sh = importlib.import_module("coresets_b200.cuda.multi.sharded")
    monkeypatch.setattr(sh, "_REQUIRE_CUDA", False)
    c, X, order = _setup(monkeypatch, case, knobs)
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    monkeypatch.setenv("MASTER_PORT", str(free_port()))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            sh.accrete_voronoi_multi_sharded(X, 0, 1, c["n_anchor"], X.shape[0], [X.shape[0]], order,
                                             max_k=c["max_k"], verbose=True, profile=profile)
    finally:
        dist.destroy_process_group()
    got, want = mask(buf.getvalue()), (GOLDEN / golden).read_text()
    assert got.splitlines() == want.splitlines()
