"""Golden probe sequences of the reference's bisect searches.

    python tests/golden/make_golden_search.py --reference <reference checkout>

Imports `MultiGPUAccrete._binary_search` / `_largest_true`
(src/coresets/cuda/multi/_base.py:735-809) and records, for monotone predicates `m <= t` on
[0, n], the answer and the exact sequence of probes; every probe of a real run costs a simulated
FPS fill, so the sequence (not only the answer) is part of the behaviour to keep.  Writes
tests/golden/search_probes.json.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
    a = ap.parse_args()
    sys.path.insert(0, str(Path(a.reference) / "src"))
    from coresets.cuda.multi._base import MultiGPUAccrete
    cases = []
    for n in (0, 1, 2, 3, 7, 16, 33, 100, 1024, 5000):
        thresholds = sorted({-1, 0, 1, 2, n // 3, n // 2, n - 1, n} & set(range(-1, n + 1)))
        for t in thresholds:
            probes = []

            def pred(m, probes=probes, t=t):
                probes.append(m)
                return m <= t

            ans = MultiGPUAccrete._binary_search(pred, n)
            cases.append(dict(kind="binary", n=n, t=t, answer=ans, probes=list(probes)))
            for seed in sorted({-2, 0, 1, 2, 5, t, t + 1, t - 1, 2 * max(t, 0), n, n + 3, 17, 32}):
                probes = []

                def pred2(m, probes=probes, t=t):
                    probes.append(m)
                    return m <= t

                ans = MultiGPUAccrete._largest_true(pred2, n, seed)
                cases.append(dict(kind="seeded", n=n, t=t, seed=seed, answer=ans, probes=list(probes)))
    out = Path(__file__).parent / "search_probes.json"
    out.write_text(json.dumps(cases, separators=(",", ":")))
    print(f"{len(cases)} cases -> {out}")


if __name__ == "__main__":
    main()
