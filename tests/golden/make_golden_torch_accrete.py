"""Golden lists of the reference's plain-torch accretion backend.

    python tests/golden/make_golden_torch_accrete.py --reference <reference checkout>

Runs the reference's own `coresets.pytorch.accrete` (src/coresets/pytorch/accrete.py:12-247) on CPU,
one thread, on small seeded cases from tests/data.py, and its `accrete_distributed`
(src/coresets/pytorch/accrete_distributed.py:12-237) on the same cases in a two-rank gloo group, and
writes tests/golden/torch_accrete.npz (per case: the index list and the printed table of the single
run, the index list of the distributed run as `<case>_dist`).
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


def split_rows(Xa, Xc, rank: int, world: int):
    """This rank's slice of cat(anchors, candidates): equal parts, the remainder on the last rank."""
    X = torch.cat([Xa, Xc], dim=0)
    base = X.shape[0] // world
    lo = rank * base
    hi = X.shape[0] if rank == world - 1 else lo + base
    return X[lo:hi].contiguous()


def dist_worker(reference: str, out_dir: str) -> None:
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, str(Path(reference) / "src"))
    from coresets.pytorch import accrete_distributed
    torch.set_num_threads(1)
    rec = {}
    for name, c in CASES.items():
        Xa, Xc, order = case_inputs(c)
        out = accrete_distributed(split_rows(Xa, Xc, rank, world), order, Xa.shape[0], rank, world, max_k=c["max_k"],
                                  verbose=False)
        rec[name + "_dist"] = out.numpy().astype(np.int64)
    if rank == 0:
        np.savez(Path(out_dir) / "dist.npz", **rec)
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CORESETS_REFERENCE_ROOT"),
                    required=not os.environ.get("CORESETS_REFERENCE_ROOT"), help="the reference checkout (or set CORESETS_REFERENCE_ROOT)")
    ap.add_argument("--dist-worker-out", default=None)
    a = ap.parse_args()
    if a.dist_worker_out:
        dist_worker(a.reference, a.dist_worker_out)
        return
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
    import socket
    import subprocess
    import tempfile
    tmp = tempfile.mkdtemp()
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    procs = [subprocess.Popen([sys.executable, __file__, "--reference", a.reference, "--dist-worker-out", tmp],
                              env=dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port)))
             for r in range(2)]
    for p in procs:
        assert p.wait() == 0
    z = np.load(Path(tmp) / "dist.npz")
    for k in z.files:
        rec[k] = z[k]
        print(k, "equal to the single run:", bool(np.array_equal(z[k], rec[k[:-5]])))
    np.savez_compressed(Path(__file__).parent / "torch_accrete.npz", **rec)


if __name__ == "__main__":
    main()
