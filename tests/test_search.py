"""The bisect searches (coresets_b200/cuda/search.py) against the reference's own probe sequences
(tests/golden/search_probes.json, written by tests/golden/make_golden_search.py from
src/coresets/cuda/multi/_base.py:735-809) and through the properties the reference tests state
(tests/test_bisect_search.py): equal answers for every monotone predicate and seed, the floor at
zero, no probe of m = 0, few probes when the answer is near the seed."""
import json
from pathlib import Path

import pytest

from coresets_b200.cuda import search

GOLDEN = Path(__file__).resolve().parent / "golden" / "search_probes.json"


def recording(t, n, probes):
    def pred(m):
        assert 0 <= m <= n, f"probe {m} outside [0, {n}]"
        probes.append(m)
        return m <= t
    return pred


def brute(t, n):
    return max([m for m in range(0, n + 1) if m <= t], default=0)


def test_probe_sequences_match_the_reference():
    cases = json.loads(GOLDEN.read_text())
    assert len(cases) > 500
    for c in cases:
        probes = []
        pred = recording(c["t"], c["n"], probes)
        got = search.binary_search(pred, c["n"]) if c["kind"] == "binary" else search.largest_true(pred, c["n"], c["seed"])
        assert got == c["answer"], c
        assert probes == c["probes"], c


def test_both_searches_agree_with_brute_force_for_every_seed():
    checks = 0
    for n in range(0, 40):
        for t in range(-1, n + 1):
            want = brute(t, n)
            assert search.binary_search(recording(t, n, []), n) == want
            for seed in range(-3, n + 4):
                assert search.largest_true(recording(t, n, []), n, seed) == want, (n, t, seed)
                checks += 1
    assert checks > 20_000


def test_nothing_viable_gives_zero():
    for n in range(0, 20):
        assert search.binary_search(lambda m: False, n) == 0
        for seed in range(0, n + 2):
            assert search.largest_true(lambda m: False, n, seed) == 0


def test_walk_from_seed_zero_never_probes_zero():
    """m = 0 cannot move the floor, so a walk that starts there must not spend a simulation on it."""
    for n in range(0, 60):
        for t in range(-1, n + 1):
            probes = []
            assert search.largest_true(recording(t, n, probes), n, 0) == brute(t, n)
            assert 0 not in probes, (n, t, probes)


@pytest.mark.parametrize("n", [4096, 16384])
def test_answer_next_to_the_seed_costs_a_handful_of_probes(n):
    """The regime the seed exists for: the previous layer's answer is close to this one's."""
    import math
    for t in (0, 1, 3, 9, 30):
        for seed in (t, t + 1, max(t - 1, 0)):
            probes = []
            assert search.largest_true(recording(t, n, probes), n, seed) == t
            false_probes = [m for m in probes if m > t]
            assert len(probes) <= 4 and len(false_probes) <= 2, (t, seed, probes)
            plain = []
            search.binary_search(recording(t, n, plain), n)
            assert len(plain) >= math.floor(math.log2(n))      # what the seed saves


def test_small_upward_drift_costs_one_false_probe():
    """A false probe runs a whole simulated fill, so when the answer lies less than the linear
    walk length above the seed, exactly one probe may come out false (the one that ends the walk)."""
    n = 4096
    for seed in range(0, 33):
        for drift in range(0, search.GALLOP_LINEAR):
            t = seed + drift
            probes = []
            assert search.largest_true(recording(t, n, probes), n, seed) == t
            assert sum(1 for m in probes if m > t) == 1, (seed, drift, probes)
    for seed in range(1, 33):                      # downward drift: the walk ends on a true probe
        for drift in range(1, min(search.GALLOP_LINEAR, seed) + 1):
            t = seed - drift
            probes = []
            assert search.largest_true(recording(t, n, probes), n, seed) == t
            assert probes[-1] <= t or len(probes) <= drift + 2


def test_walk_constants():
    assert isinstance(search.GALLOP_MAX_SEED, int) and search.GALLOP_MAX_SEED > 0
    assert isinstance(search.GALLOP_LINEAR, int) and search.GALLOP_LINEAR > 0
