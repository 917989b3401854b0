"""Golden lists of the reference's REPLICATED multi-GPU accretion driver, written on GPUs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29543 tests/golden/make_golden_replicated_gpu.py --out <dir>

Runs the reference's own `accrete_voronoi_multi` (src/coresets/cuda/multi/replicated.py:252-308: the
whole matrix on every rank; oracle/_ref holds its kernels built for cc 10.0) on the float32 cases of
make_golden_gpu.py, and this package's entry of the same name beside it.  Rank 0 writes
<dir>/acc_replicated.npz (one index list per case).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle" / "_ref" / "site"))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(ROOT / "golden_out"))
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from tests.golden.make_golden_gpu import ACCRETE_CASES, accrete_case_matrix, load_reference
    coresets, _ = load_reference()
    from coresets.cuda.multi import accrete_voronoi_multi as ref_replicated
    from coresets_b200.cuda.multi import accrete_voronoi_multi as my_replicated
    golden = ROOT / "tests" / "golden"
    rec, report = {}, {}
    for name, c in ACCRETE_CASES.items():
        if c.get("dtype", "float32") != "float32":
            continue
        X = torch.from_numpy(accrete_case_matrix(c)).to(dev)
        na = c["n_anchor"]
        order = torch.from_numpy(np.load(golden / f"{name}.npz")["anchor_order"]).to(dev)
        ref = ref_replicated(X[:na], X[na:], order, rank, world, max_k=c["max_k"], verbose=False)
        mine = my_replicated(X[:na], X[na:], order, rank, world, max_k=c["max_k"], verbose=False)
        rec[name] = ref.cpu().numpy().astype(np.int64)
        report[name] = dict(n=int(ref.shape[0]), engine_equal=bool(torch.equal(ref, mine)),
                            equals_reference_sharded=bool(np.array_equal(rec[name], np.load(golden / f"{name}.npz")["sharded_plain"])))
        dist.barrier()
    if rank == 0:
        out = Path(a.out)
        out.mkdir(parents=True, exist_ok=True)
        np.savez_compressed(out / "acc_replicated.npz", **rec)
        print("[replicated]", json.dumps(report), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
