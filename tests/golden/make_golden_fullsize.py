"""Golden `selected` / `epsilons` of the benchmark configurations at FULL size, written by the
reference's own `fps_sharded` (oracle/_ref: the reference's kernels compiled for cc 10.0 plus its
Python package) on B200s, with this package's `fps_sharded` run beside it on the same device rows.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29541 tests/golden/make_golden_fullsize.py --config c3 --out <dir>
    python tests/golden/make_golden_fullsize.py --config c2 --out <dir>            (one GPU)

The reference is valid up to 2^27 rows per GPU (32-bit warp index, src/coresets/cuda/kernels/warp.cu:21)
and needs a second N_local x D temporary for its norms (src/coresets/cuda/multi/fps_sharded.py:90):
c3 (300M x 128) needs 4 or 8 GPUs, c4 (40M x 1024) at least 2, c2 (20M x 256) runs on one.
Rows come from coresets_b200/synth.py (device generator, seeded per 2^18-row block), so the same
bytes are regenerated on any B200 at any world size.  Rank 0 writes
    <dir>/fullsize_<config>.npz     selected (int32), eps (float32), plus rows / dim / k / world
and prints one JSON line per run with the wall time of both implementations.
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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["c2", "c3", "c4"])
    ap.add_argument("--rows", type=int, default=0, help="scale the row count down (dry runs)")
    ap.add_argument("--k", type=int, default=0, help="override the number of picks (dry runs)")
    ap.add_argument("--out", default=str(ROOT / "golden_out"))
    ap.add_argument("--exchanges", default="nccl,p2p", help="exchanges of this package to run beside the reference")
    ap.add_argument("--skip-reference", action="store_true",
                    help="compare this package with an existing fullsize_<config>.npz (in --golden-dir) instead of "
                         "running the reference; a smaller --k compares a prefix")
    ap.add_argument("--golden-dir", default="", help="where the existing golden file lies (default: --out)")
    a = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    import coresets_b200
    from coresets_b200.cuda.multi.layout import compute_shard_layout
    from coresets_b200.synth import WORKLOADS, MixtureSource, scaled

    w = WORKLOADS[a.config]
    if a.rows or a.k:
        w = scaled(w, a.rows or w.n_rows, k=a.k or min(w.k, a.rows or w.n_rows))
    sizes, offsets = compute_shard_layout(w.n_rows, world)
    t0 = time.time()
    X = torch.empty((sizes[rank], w.dim), dtype=torch.float32, device=dev)
    MixtureSource(w).fill(X, offsets[rank])
    torch.cuda.synchronize(dev)
    t_gen = time.time() - t0
    out = Path(a.out)
    gold_path = out / f"fullsize_{a.config}.npz"
    rec = dict(config=a.config, rows=w.n_rows, dim=w.dim, k=w.k, world=world, rows_per_gpu=max(sizes),
               generate_s=round(t_gen, 2))

    if a.skip_reference:
        z = np.load(Path(a.golden_dir or a.out) / gold_path.name)
        if int(z["rows"]) != w.n_rows:
            raise SystemExit(f"{gold_path.name} is for {int(z['rows'])} rows, this run has {w.n_rows}")
        ref_sel, ref_eps = z["selected"].astype(np.int64)[: w.k], z["eps"][: w.k]
    else:
        from tests.golden.make_golden_gpu import load_reference
        coresets, _ = load_reference()
        dist.barrier()
        torch.cuda.synchronize(dev)
        t0 = time.time()
        r_sel, r_eps = coresets.fps_sharded(X, w.k, verbose=False)
        torch.cuda.synchronize(dev)
        dist.barrier()
        rec["reference_s"] = round(time.time() - t0, 2)
        rec["reference_picks_per_s"] = round(w.k / (time.time() - t0), 1)
        ref_sel = r_sel.cpu().numpy().astype(np.int64)
        ref_eps = r_eps.cpu().numpy().astype(np.float32)
        del r_sel, r_eps
        torch.cuda.empty_cache()
        if rank == 0:
            out.mkdir(parents=True, exist_ok=True)
            np.savez_compressed(gold_path, selected=ref_sel.astype(np.int32), eps=ref_eps, rows=w.n_rows, dim=w.dim,
                                k=w.k, world=world)

    for xchg in [x for x in a.exchanges.split(",") if x]:
        if xchg == "p2p" and world == 1:
            continue
        os.environ["CORESETS_B200_EXCHANGE"] = xchg
        dist.barrier()
        torch.cuda.synchronize(dev)
        t0 = time.time()
        sel, eps = coresets_b200.fps_sharded(X, w.k, verbose=False)
        torch.cuda.synchronize(dev)
        dist.barrier()
        dt = time.time() - t0
        mine = sel.cpu().numpy()
        same = bool(np.array_equal(mine, ref_sel))
        first_diff = int(np.argmax(mine != ref_sel)) if not same else -1
        eps_bits = bool(np.array_equal(eps.numpy().view(np.int32), ref_eps.view(np.int32)))
        rec[f"engine_{xchg}_s"] = round(dt, 2)
        rec[f"engine_{xchg}_picks_per_s"] = round(w.k / dt, 1)
        rec[f"engine_{xchg}_selected_equal"] = same
        rec[f"engine_{xchg}_eps_bits_equal"] = eps_bits
        rec[f"engine_{xchg}_first_diff"] = first_diff
        del sel, eps
        torch.cuda.empty_cache()
    if rank == 0:
        print("[fullsize]", json.dumps(rec), flush=True)
        out.mkdir(parents=True, exist_ok=True)
        (out / f"fullsize_{a.config}_w{world}.json").write_text(json.dumps(rec, indent=1))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
