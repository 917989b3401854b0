"""Golden lists of the reference's plain-torch accretion backend.

    python tests/golden/make_golden_torch_accrete.py --reference <reference checkout>

Runs the reference's own `coresets.pytorch.accrete` (src/coresets/pytorch/accrete.py:12-247) on CPU,
one thread, on small seeded cases from tests/data.py and writes tests/golden/torch_accrete.npz (one
index list per case, plus the printed table of one case).
"""
from __future__ import annotations

import argparse
import contextlib
import io
import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

CASES = {
    "jitter_1200x8_k7": dict(gen="jitter", N=1200, D=8, n_anchor=500, max_k=7),
    "mix_2000x16_k8": dict(gen="mix", N=2000, D=16, n_anchor=900, max_k=8),
    "mix_600x5_auto": dict(gen="mix", N=600, D=5, n_anchor=200, max_k=None),
}


def case_inputs(c: dict):
    from tests.data import clustered_jitter, gaussian_mixture
    X = clustered_jitter(c["N"], c["D"], seed=7) if c["gen"] == "jitter" else gaussian_mixture(c["N"], c["D"], 6, seed=c["N"])
    na = c["n_anchor"]
    rng = np.random.default_rng(c["N"])
    order = rng.permutation(na).astype(np.int64)
    return torch.from_numpy(X[:na]), torch.from_numpy(X[na:]), torch.from_numpy(order)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
    a = ap.parse_args()
    sys.path.insert(0, str(Path(a.reference) / "src"))
    from coresets.pytorch import accrete
    torch.set_num_threads(1)
    rec = {}
    for name, c in CASES.items():
        Xa, Xc, order = case_inputs(c)
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            out = accrete(Xa, Xc, order, torch.arange(Xc.shape[0]), max_k=c["max_k"], verbose=True)
        rec[name] = out.numpy().astype(np.int64)
        rec[name + "_table"] = np.array(buf.getvalue())
        print(name, out.shape[0], out[:6].tolist())
    np.savez_compressed(Path(__file__).parent / "torch_accrete.npz", **rec)


if __name__ == "__main__":
    main()
