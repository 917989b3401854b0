"""Golden vectors of the reference's CPU backend: run where the reference checkout is importable.

    python tests/golden/make_golden_cpu.py --reference <reference checkout>

Writes tests/golden/cpu_fps_c1.npz: outputs of the reference's own ``coresets.fps``
(src/coresets/pytorch/fps.py:32-73) on the 20 000 x 64, 16-component, k = 512 case.  Inputs are
regenerated from tests/data.py; float32 throughout, one thread (the MKL sgemv result is
independent of the thread count for this shape, the test checks `selected` exactly and the
radii to 1e-6 relative).
"""
import argparse
import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from tests.data import gaussian_mixture  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
a = ap.parse_args()
sys.path.insert(0, str(Path(a.reference) / "src"))
from coresets import fps  # noqa: E402

torch.set_num_threads(1)
X = gaussian_mixture(20000, 64, 16, seed=0)
sel, eps, h, v = fps(torch.from_numpy(X), 512)
np.savez_compressed(Path(__file__).parent / "cpu_fps_c1.npz", selected=sel.numpy(), eps=eps.numpy(),
                    hausdorff_max=np.float32(h.max().item()), voronoi=v.numpy().astype(np.int16))
print("wrote cpu_fps_c1.npz", sel[:6].tolist(), float(eps[1]), float(eps[-1]), float(h.max()))
