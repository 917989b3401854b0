"""Golden console output of the reference's accretion drivers (verbose + profile).

    python tests/golden/make_golden_verbose.py --reference <reference checkout>

Runs `accrete` (src/coresets/cuda/accrete.py) and the one-rank `accrete_voronoi_multi_sharded`
(src/coresets/cuda/multi/sharded.py) on CPU tensors with the oracle as kernel extension and keeps
what they print, with every wall-clock figure replaced by `T` (see `mask`).  Writes
tests/golden/verbose_single.txt, verbose_sharded.txt and verbose_sharded_knobs.txt (the seeded
walk: CORESETS_BISECT_SEED=1 CORESETS_FILL_CHUNK=256 on a second case).
"""
from __future__ import annotations

import argparse
import contextlib
import io
import os
import re
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests.golden.make_golden_accrete_cpu import CASES, make_case, setup_reference  # noqa: E402

CASE = "jitter_1024x8_k128"
CASE_KNOBS = "mix_3000x16_k256_fps"
KNOBS = {"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"}


def mask(text: str) -> str:
    """Replace every wall-clock figure by `T`: the time column of a level row (column 5 in the
    single-GPU table, the last column in the sharded one), `0.035s  ( 29.5%)` in the profile,
    `(bisect 0.0s`, `(0.0s)` after a probe, `block_bisect=     0.0s  fill=     0.0s`."""
    out = []
    for line in text.splitlines():
        line = re.sub(r"\d+\.\d+s\s+\(\s*\d+\.\d+%\)", "Ts (P%)", line)
        line = re.sub(r"\(bisect \d+\.\d+s", "(bisect Ts", line)
        line = re.sub(r"\(\d+\.\d+s\)", "(Ts)", line)
        line = re.sub(r"(block_bisect|fill)=\s*\d+\.\d+s", r"\1=Ts", line)
        cells = line.split("|")
        if len(cells) == 9 and cells[0].strip().isdigit():
            if re.search(r"e[-+]\d+|inf", cells[8]):      # single-GPU table: rel_gap is the last column
                cells[5] = " T "
            else:                                       # sharded table: the layer time is
                cells[8] = " T"
            line = "|".join(cells)
        out.append(line.rstrip())
    return "\n".join(out) + "\n"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
    a = ap.parse_args()
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29593")
    dist.init_process_group("gloo", rank=0, world_size=1)
    setup_reference(a.reference)
    from coresets.cuda.accrete import accrete
    from coresets.cuda.multi.sharded import accrete_voronoi_multi_sharded
    c = CASES[CASE]
    X, order = make_case(c)
    Xt = torch.from_numpy(X)
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        accrete(Xt[: c["n_anchor"]], Xt[c["n_anchor"] :], torch.from_numpy(order), c["max_k"], verbose=True, profile=True)
    (Path(__file__).parent / "verbose_single.txt").write_text(mask(buf.getvalue()))
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        accrete_voronoi_multi_sharded(Xt, 0, 1, c["n_anchor"], X.shape[0], [X.shape[0]], torch.from_numpy(order),
                                      max_k=c["max_k"], verbose=True, profile=True)
    (Path(__file__).parent / "verbose_sharded.txt").write_text(mask(buf.getvalue()))
    # the seeded walk with lazy forward and chunked fill on a second case
    c2 = CASES[CASE_KNOBS]
    X2, order2 = make_case(c2)
    os.environ.update(KNOBS)
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        accrete_voronoi_multi_sharded(torch.from_numpy(X2), 0, 1, c2["n_anchor"], X2.shape[0], [X2.shape[0]],
                                      torch.from_numpy(order2), max_k=c2["max_k"], verbose=True, profile=False)
    (Path(__file__).parent / "verbose_sharded_knobs.txt").write_text(mask(buf.getvalue()))
    dist.destroy_process_group()
    print(mask(buf.getvalue()))


if __name__ == "__main__":
    main()
