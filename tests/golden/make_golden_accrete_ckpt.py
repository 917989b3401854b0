"""Golden checkpoint files of the reference's sharded accretion driver.

    python tests/golden/make_golden_accrete_ckpt.py --reference <reference checkout>

Runs `accrete_voronoi_multi_sharded` (src/coresets/cuda/multi/sharded.py) in a one-rank gloo
group on CPU tensors with the oracle as kernel extension (tests/golden/ref_ext_cpu.py), with
`checkpoint_path` and a mid-layer cadence, and records every file it wrote (name -> array or
text) plus the list a `resume_from` run returns.  Writes tests/golden/accrete_cpu_ckpt.npz.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests.golden.make_golden_accrete_cpu import CASES, make_case, setup_reference  # noqa: E402

CASE = "jitter_1024x8_k128"
KNOBS = {"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"}
EVERY = 24


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
    a = ap.parse_args()
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29591")
    dist.init_process_group("gloo", rank=0, world_size=1)
    setup_reference(a.reference)
    from coresets.cuda.multi.sharded import accrete_voronoi_multi_sharded
    c = CASES[CASE]
    X, order = make_case(c)
    os.environ.update(KNOBS)
    Xl = torch.from_numpy(X)
    rec = {}
    with tempfile.TemporaryDirectory() as d:
        prefix = str(Path(d) / "ck")
        full = accrete_voronoi_multi_sharded(Xl, 0, 1, c["n_anchor"], X.shape[0], [X.shape[0]], torch.from_numpy(order),
                                             max_k=c["max_k"], verbose=False, checkpoint_path=prefix,
                                             checkpoint_every=EVERY)
        rec["full"] = full.numpy().astype(np.int64)
        names = sorted(p.name for p in Path(d).iterdir())
        rec["names"] = np.array(names)
        for n in names:
            p = Path(d) / n
            rec["file:" + n] = np.load(p) if n.endswith(".npy") else np.array(p.read_text())
        # resume from the last complete layer below the top: drop the top layer's files first
        top = c["max_k"]
        for n in names:
            if f"_k{top:02d}" in n:
                (Path(d) / n).unlink()
        (Path(d) / "ck_latest.txt").write_text(f"{top - 1}\n")
        resumed = accrete_voronoi_multi_sharded(Xl, 0, 1, c["n_anchor"], X.shape[0], [X.shape[0]], torch.from_numpy(order),
                                                max_k=c["max_k"], verbose=False, resume_from=prefix)
        rec["resumed"] = resumed.numpy().astype(np.int64)
    dist.destroy_process_group()
    print("files:", names)
    print("resume equals full run:", bool(np.array_equal(rec["full"], rec["resumed"])))
    np.savez_compressed(Path(__file__).parent / "accrete_cpu_ckpt.npz", **rec)


if __name__ == "__main__":
    main()
