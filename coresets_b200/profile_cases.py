"""Small fixed runs for profiling the kernels under ncu (the commands quoted in profiles/*.md).

    python -m coresets_b200.profile_cases cells <workload> <rows> <k>   fps_cuda to k picks, single launches
                                                                         (no CUDA graphs): cell-index kernels
    python -m coresets_b200.profile_cases dense <workload> <rows>       six dense picks: the bulk-copy kernel
    python -m coresets_b200.profile_cases dense16 <workload> <rows>     the same over float16 rows

Rows are the first <rows> of the named synthetic workload (coresets_b200/synth.py), generated on
the device.
"""
from __future__ import annotations

import os
import sys


def main(argv) -> None:
    what, wname, rows = argv[0], argv[1], int(argv[2])
    if what == "cells":
        os.environ["CORESETS_B200_GRAPH"] = "0"
    import torch
    from . import engine, fps_cuda
    from ._native import MODE_DENSE
    from .synth import WORKLOADS, MixtureSource, scaled
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    k = int(argv[3]) if what == "cells" else 16
    X = MixtureSource(scaled(WORKLOADS[wname], rows, k=k)).rows(0, rows, dev)
    if what == "cells":
        sel = fps_cuda(X, k)
        torch.cuda.synchronize()
        print("done", wname, rows, k, sel[-3:].tolist())
    elif what in ("dense", "dense16"):
        if what == "dense16":
            X = X.to(torch.float16)
        eng = engine.ShardEngine(X, engine.row_norms(X), k, mode=MODE_DENSE, element_order=what == "dense16")
        eng.init_state()
        eng.pick_forced(0)
        for _ in range(6):
            eng.exchange()
            eng.commit()
            eng.step()
        eng.check_status()
        print("done", wname, rows)
    else:
        raise SystemExit(__doc__)


if __name__ == "__main__":
    main(sys.argv[1:])
