"""Worker of the multi-GPU test (one process per GPU, NCCL).  Run by tests/test_gpu_multi.py."""
from __future__ import annotations

import datetime
import json
import os
import sys
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> None:
    cfg = json.loads(sys.argv[1])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=int(cfg.get("pg_timeout", 150))))
    import oracle
    from coresets_b200 import engine, fps_cuda, fps_sharded
    from tests.data import gaussian_mixture, with_duplicates

    failures = []
    if cfg.get("mode") == "accrete":
        failures = accrete_mode(cfg, rank, world, dev)
        cfg = dict(cfg, cases=[])
    for case in cfg["cases"]:
        N, D, k, seed = case["N"], case["D"], case["k"], case.get("seed")
        X_np = with_duplicates(gaussian_mixture(N, D, 8, seed=N + D), 30, seed=2)
        sizes = case["sizes"]
        offs = [sum(sizes[:r]) for r in range(world)]
        X_local = torch.from_numpy(np.ascontiguousarray(X_np[offs[rank] : offs[rank] + sizes[rank]])).to(dev)
        sel, eps = fps_sharded(X_local, k, seed=seed, verbose=False)
        # norms exactly as every rank computed them for its own shard
        norms = np.concatenate([
            engine.row_norms(torch.from_numpy(np.ascontiguousarray(X_np[offs[r] : offs[r] + sizes[r]])).to(dev)).cpu().numpy()
            if sizes[r] > 0 else np.zeros(0, np.float32) for r in range(world)])
        o_sel, o_eps, _, _ = oracle.fps_sharded(X_np, norms, k, sizes, first=seed or 0)
        if not np.array_equal(sel.cpu().numpy(), o_sel):
            failures.append(f"{case}: selected differs from the oracle on rank {rank}")
        if not np.array_equal(eps.numpy().view(np.int32), o_eps.view(np.int32)):
            failures.append(f"{case}: epsilons differ on rank {rank}")
        if sizes[rank] == N:                # this rank holds everything: compare with single-GPU fps_cuda too
            one = fps_cuda(X_local, k, seed=None if seed is None else torch.tensor([seed]))
            if not torch.equal(one, sel):
                failures.append(f"{case}: fps_sharded != fps_cuda")
        dist.barrier()
    out = Path(cfg["out_dir"]) / f"result_{rank}.json"
    out.write_text(json.dumps({"failures": failures}))
    dist.barrier()
    dist.destroy_process_group()


def accrete_mode(cfg, rank, world, dev):
    """accrete_sharded over NCCL ranks against the golden lists written by the reference on a B200."""
    import coresets_b200
    from coresets_b200.cuda.multi.layout import compute_shard_layout
    from tests.data import clustered_jitter, gaussian_mixture
    from tests.golden.make_golden_gpu import ACCRETE_CASES, accrete_case_matrix
    golden = ROOT / "tests" / "golden"
    failures = []
    for name, c in ACCRETE_CASES.items():
        z = np.load(golden / f"{name}.npz")
        X_np = accrete_case_matrix(c)
        sizes, offs = compute_shard_layout(c["N"], world)
        Xl = torch.from_numpy(np.ascontiguousarray(X_np[offs[rank] : offs[rank] + sizes[rank]])).to(dev)
        order = torch.from_numpy(z["anchor_order"]).to(dev)
        for tag, env in (("plain", {}), ("knobs", {"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"})):
            for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
                os.environ.pop(k, None)
            os.environ.update(env)
            res = coresets_b200.accrete_sharded(Xl, order, c["n_anchor"], max_k=c["max_k"], verbose=False)
            if not np.array_equal(res.cpu().numpy(), z[f"sharded_{tag}"]):
                nd = int((res.cpu().numpy() != z[f"sharded_{tag}"]).sum())
                failures.append(f"{name}/{tag}: {nd} ids differ from the reference on rank {rank} (world {world})")
        for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
            os.environ.pop(k, None)
        dist.barrier()
    return failures


if __name__ == "__main__":
    try:
        main()
    except BaseException:  # a rank that dies must not leave its peers waiting in a collective
        traceback.print_exc()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1)
