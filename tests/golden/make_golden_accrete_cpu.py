"""Golden vectors for the accretion drivers, produced by the REFERENCE's own Python drivers.

    python tests/golden/make_golden_accrete_cpu.py --reference <reference checkout>

The reference's `accrete` (src/coresets/cuda/accrete.py) and `accrete_voronoi_multi_sharded`
(src/coresets/cuda/multi/sharded.py) are run on CPU tensors with the oracle standing in for their
CUDA extension (tests/golden/ref_ext_cpu.py).  Writes tests/golden/accrete_cpu_<case>.npz with the
returned index lists and the per-commit trace (phase, position, index, value, separation) of the
single-GPU driver.  The sharded driver runs in a one-rank and a two-rank gloo group, with default
knobs, with CORESETS_BISECT_SEED=1 CORESETS_FILL_CHUNK=256, with the deep gallop
(CORESETS_BISECT_GALLOP_DEEP=1, CORESETS_FILL_CHUNK=64) and with CORESETS_LAZY_FORWARD=0.
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests.data import clustered_jitter, gaussian_mixture  # noqa: E402

PHASES = {"forward": 0, "replay": 1, "fill": 2}

CASES = {
    "jitter_1024x8_k128": dict(gen="jitter", N=1024, D=8, max_k=7, n_anchor=512, order="arange"),
    "jitter_4096x32_k512": dict(gen="jitter", N=4096, D=32, max_k=9, n_anchor=2048, order="arange"),
    "mix_3000x16_k256_fps": dict(gen="mix", N=3000, D=16, max_k=8, n_anchor=1200, order="fps"),
    "mix_1501x12_target200": dict(gen="mix", N=1501, D=12, max_k=8, n_anchor=700, order="fps", n_target=200),
}


def make_case(c: dict):
    if c["gen"] == "jitter":
        X = clustered_jitter(c["N"], c["D"], seed=42)
    else:
        X = gaussian_mixture(c["N"], c["D"], 12, seed=c["N"])
    na = c["n_anchor"]
    if c["order"] == "arange":
        order = np.arange(na, dtype=np.int64)
    else:
        import oracle
        Xa = np.ascontiguousarray(X[:na])
        order, _, _, _ = oracle.fps_cuda(Xa, oracle.row_norms_f32(Xa), na)
    return X, order


def read_trace(path: str):
    rows = [l.rstrip("\n").split("\t") for l in open(path)]
    return dict(
        trace_phase=np.array([PHASES[r[0]] for r in rows], dtype=np.int8),
        trace_pos=np.array([int(r[1]) for r in rows], dtype=np.int32),
        trace_idx=np.array([int(r[2]) for r in rows], dtype=np.int64),
        trace_val=np.array([float.fromhex(r[3]) for r in rows], dtype=np.float64),
        trace_sep=np.array([float.fromhex(r[4]) for r in rows], dtype=np.float64),
    )


def setup_reference(ref_root: str):
    sys.path.insert(0, str(Path(ref_root) / "src"))
    from tests.golden import ref_ext_cpu
    ref_ext_cpu.install()
    import coresets.cuda.multi.sharded as sh
    sh._validate_inputs = lambda *a, **k: None      # only rejects CPU tensors here; inputs are valid by construction


def run_sharded(X, order, c, world, rank, knobs: dict):
    import torch.distributed as dist
    from coresets.cuda.multi.layout import compute_shard_layout
    from coresets.cuda.multi.sharded import accrete_voronoi_multi_sharded
    for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK", "CORESETS_BISECT_GALLOP_DEEP", "CORESETS_LAZY_FORWARD"):
        os.environ.pop(k, None)
    os.environ.update(knobs)
    sizes, offs = compute_shard_layout(X.shape[0], world)
    Xl = torch.from_numpy(np.ascontiguousarray(X[offs[rank] : offs[rank] + sizes[rank]]))
    out = accrete_voronoi_multi_sharded(Xl, rank, world, c["n_anchor"], X.shape[0], sizes, torch.from_numpy(order),
                                        max_k=c["max_k"], n_target=c.get("n_target"), verbose=False)
    for k in knobs:
        os.environ.pop(k, None)
    return out.numpy().astype(np.int64)


def worker(ref_root: str, out_dir: str):
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    setup_reference(ref_root)
    for name, c in CASES.items():
        X, order = make_case(c)
        res = run_sharded(X, order, c, world, rank, {})
        res2 = run_sharded(X, order, c, world, rank, {"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"})
        res3 = run_sharded(X, order, c, world, rank, {"CORESETS_BISECT_SEED": "1", "CORESETS_BISECT_GALLOP_DEEP": "1",
                                                      "CORESETS_FILL_CHUNK": "64"})
        res4 = run_sharded(X, order, c, world, rank, {"CORESETS_BISECT_SEED": "1", "CORESETS_LAZY_FORWARD": "0"})
        if rank == 0:
            np.savez(Path(out_dir) / f"w{world}_{name}.npz", plain=res, knobs=res2, deep=res3, nolazy=res4)
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
    ap.add_argument("--worker-out", default=None)
    a = ap.parse_args()
    if a.worker_out:
        worker(a.reference, a.worker_out)
        return
    tmp = tempfile.mkdtemp()
    for world in (1, 2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        procs = [subprocess.Popen([sys.executable, __file__, "--reference", a.reference, "--worker-out", tmp],
                                  env=dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                                           MASTER_PORT=str(port), OMP_NUM_THREADS="2")) for r in range(world)]
        for p in procs:
            assert p.wait() == 0
    setup_reference(a.reference)
    from coresets.cuda.accrete import accrete
    for name, c in CASES.items():
        X, order = make_case(c)
        rec = dict(config=json.dumps(c), anchor_order=order)
        if "n_target" not in c:
            Xt = torch.from_numpy(X)
            tr = os.path.join(tmp, f"{name}.tsv")
            single = accrete(Xt[: c["n_anchor"]], Xt[c["n_anchor"] :], torch.from_numpy(order), c["max_k"],
                             verbose=False, trace_path=tr).numpy().astype(np.int64)
            rec["single"] = single
            rec.update(read_trace(tr))
        for world in (1, 2):
            z = np.load(Path(tmp) / f"w{world}_{name}.npz")
            rec[f"sharded_w{world}"] = z["plain"]
            rec[f"sharded_w{world}_knobs"] = z["knobs"]
            rec[f"sharded_w{world}_deep"] = z["deep"]
            rec[f"sharded_w{world}_nolazy"] = z["nolazy"]
        same = all(np.array_equal(rec["sharded_w1"], rec[k]) for k in rec if k.startswith("sharded_"))
        if "single" in rec:
            same = same and np.array_equal(rec["single"], rec["sharded_w1"])
        print(f"[accrete golden] {name}: {len(rec['sharded_w1'])} ids, all reference variants identical: {same}")
        np.savez_compressed(Path(__file__).parent / f"accrete_cpu_{name}.npz", **rec)


if __name__ == "__main__":
    main()
