"""Golden index list of the accretion benchmark case (anchors + candidates x 256, seeded knobs) written
by the reference's own `accrete_sharded` (oracle/_ref) on B200s, with this package run beside it.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29542 tests/golden/make_golden_accrete_fullsize.py \
        --anchors 5000000 --candidates 5000000 --max-k 12 --out <dir>

Rows come from coresets_b200.synth.accretion_sources (device generator, seeded per block): the
global matrix is cat(anchors, candidates) sharded contiguously; `anchor_order` is the first
2^max_k picks of FPS over the anchors, computed in the run.  Both implementations run with
CORESETS_FILL_CHUNK=256 CORESETS_BISECT_SEED=1, the knobs of the benchmark case.  Rank 0 writes
    <dir>/accrete_<anchors>_<candidates>_k<max_k>.npz   anchor_order, selected (int32) + sizes
and prints one JSON line with the wall time of both.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle" / "_ref" / "site"))

KNOBS = {"CORESETS_FILL_CHUNK": "256", "CORESETS_BISECT_SEED": "1"}


def shard_rows(n_anchor: int, n_cand: int, rank: int, world: int, dev):
    """This rank's rows of cat(anchors, candidates) and how many of them are anchors."""
    from coresets_b200.cuda.multi.layout import compute_shard_layout
    from coresets_b200.synth import accretion_sources
    _, _, stacked = accretion_sources(n_anchor, n_cand)
    sizes, offsets = compute_shard_layout(n_anchor + n_cand, world)
    X = stacked.rows(offsets[rank], sizes[rank], dev)
    n_anchor_local = max(0, min(n_anchor - offsets[rank], sizes[rank]))
    return X, n_anchor_local


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--anchors", type=int, required=True)
    ap.add_argument("--candidates", type=int, required=True)
    ap.add_argument("--max-k", type=int, required=True)
    ap.add_argument("--out", default=str(ROOT / "golden_out"))
    ap.add_argument("--skip-reference", action="store_true", help="compare with the existing golden file instead")
    ap.add_argument("--golden-dir", default="", help="where the existing golden file lies (default: --out)")
    ap.add_argument("--exchanges", default="nccl")
    a = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29542")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    os.environ.update(KNOBS)

    import coresets_b200
    X, n_anchor_local = shard_rows(a.anchors, a.candidates, rank, world, dev)
    torch.cuda.synchronize(dev)
    t0 = time.time()
    order, _ = coresets_b200.fps_sharded(X[:n_anchor_local], min(1 << a.max_k, a.anchors), verbose=False)
    torch.cuda.synchronize(dev)
    rec = dict(anchors=a.anchors, candidates=a.candidates, dim=int(X.shape[1]), max_k=a.max_k, world=world,
               knobs=KNOBS, anchor_order_s=round(time.time() - t0, 2))
    out = Path(a.out)
    gold_path = out / f"accrete_{a.anchors}_{a.candidates}_k{a.max_k}.npz"

    if a.skip_reference:
        ref = np.load(Path(a.golden_dir or a.out) / gold_path.name)["selected"].astype(np.int64)
    else:
        from tests.golden.make_golden_gpu import load_reference
        coresets, _ = load_reference()
        dist.barrier()
        torch.cuda.synchronize(dev)
        t0 = time.time()
        r = coresets.accrete_sharded(X, order, a.anchors, max_k=a.max_k, verbose=False)
        torch.cuda.synchronize(dev)
        dist.barrier()
        rec["reference_s"] = round(time.time() - t0, 2)
        ref = r.cpu().numpy().astype(np.int64)
        if rank == 0:
            out.mkdir(parents=True, exist_ok=True)
            np.savez_compressed(gold_path, anchor_order=order.cpu().numpy().astype(np.int32),
                                selected=ref.astype(np.int32), anchors=a.anchors, candidates=a.candidates,
                                max_k=a.max_k, world=world)
        torch.cuda.empty_cache()

    for xchg in [x for x in a.exchanges.split(",") if x]:
        if xchg == "p2p" and world == 1:
            continue
        os.environ["CORESETS_B200_EXCHANGE"] = xchg
        dist.barrier()
        torch.cuda.synchronize(dev)
        t0 = time.time()
        mine = coresets_b200.accrete_sharded(X, order, a.anchors, max_k=a.max_k, verbose=False)
        torch.cuda.synchronize(dev)
        dist.barrier()
        rec[f"engine_{xchg}_s"] = round(time.time() - t0, 2)
        m = mine.cpu().numpy()
        rec[f"engine_{xchg}_equal"] = bool(m.shape == ref.shape and np.array_equal(m, ref))
        rec["n_selected"] = int(ref.shape[0])
    if rank == 0:
        print("[accrete-fullsize]", json.dumps(rec), flush=True)
        out.mkdir(parents=True, exist_ok=True)
        (out / f"accrete_{a.anchors}_{a.candidates}_k{a.max_k}_w{world}.json").write_text(json.dumps(rec, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
