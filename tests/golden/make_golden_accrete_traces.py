"""Golden per-commit traces of the reference's SHARDED accretion driver.

    python tests/golden/make_golden_accrete_traces.py --reference <reference checkout>

`accrete_voronoi_multi_sharded(..., trace_path=...)` (src/coresets/cuda/multi/sharded.py) in a
one-rank gloo group on CPU tensors with the oracle as kernel extension; one trace per case and
knob set (default; CORESETS_BISECT_SEED=1 CORESETS_FILL_CHUNK=256, whose lazy forward commits
fewer forward picks).  Writes tests/golden/accrete_cpu_sharded_traces.npz with the columns of
every trace (phase, position, index, value and separation as float64 bit patterns).
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

from tests.golden.make_golden_accrete_cpu import CASES, make_case, read_trace, setup_reference  # noqa: E402

TRACE_CASES = ("jitter_1024x8_k128", "mix_3000x16_k256_fps")
KNOB_SETS = {"plain": {}, "knobs": {"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"}}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
    a = ap.parse_args()
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29595")
    dist.init_process_group("gloo", rank=0, world_size=1)
    setup_reference(a.reference)
    from coresets.cuda.multi.sharded import accrete_voronoi_multi_sharded
    rec = {}
    with tempfile.TemporaryDirectory() as d:
        for name in TRACE_CASES:
            c = CASES[name]
            X, order = make_case(c)
            for tag, env in KNOB_SETS.items():
                for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
                    os.environ.pop(k, None)
                os.environ.update(env)
                tr = str(Path(d) / f"{name}_{tag}.tsv")
                accrete_voronoi_multi_sharded(torch.from_numpy(X), 0, 1, c["n_anchor"], X.shape[0], [X.shape[0]],
                                              torch.from_numpy(order), max_k=c["max_k"], verbose=False, trace_path=tr)
                for field, arr in read_trace(tr).items():
                    rec[f"{name}:{tag}:{field}"] = arr
                print(name, tag, len(rec[f"{name}:{tag}:trace_idx"]), "lines")
    dist.destroy_process_group()
    np.savez_compressed(Path(__file__).parent / "accrete_cpu_sharded_traces.npz", **rec)


if __name__ == "__main__":
    main()
