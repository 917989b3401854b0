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
    if cfg.get("mode") == "resume":
        failures = resume_mode(cfg, rank, world, dev)
        cfg = dict(cfg, cases=[])
    for case in cfg["cases"]:
        N, D, k, seed = case["N"], case["D"], case["k"], case.get("seed")
        X_np = with_duplicates(gaussian_mixture(N, D, 8, seed=N + D), 30, seed=2)
        other_dtype = case.get("dtype", "float32") != "float32"      # float16: summed element-wise, rows read in place
        if other_dtype:
            X_np = X_np.astype(case["dtype"])
        sizes = case["sizes"]
        offs = [sum(sizes[:r]) for r in range(world)]
        X_local = torch.from_numpy(np.ascontiguousarray(X_np[offs[rank] : offs[rank] + sizes[rank]])).to(dev)
        sel, eps = fps_sharded(X_local, k, seed=seed, verbose=False)
        # norms exactly as every rank computed them for its own shard
        norms = np.concatenate([
            engine.row_norms(torch.from_numpy(np.ascontiguousarray(X_np[offs[r] : offs[r] + sizes[r]])).to(dev)).cpu().numpy()
            if sizes[r] > 0 else np.zeros(0, np.float32) for r in range(world)])
        with oracle.element_order(other_dtype):
            o_sel, o_eps, _, _ = oracle.fps_sharded(X_np.astype(np.float32), norms, k, sizes, first=seed or 0)
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


def resume_mode(cfg, rank, world, dev):
    """fps_sharded with checkpoints, then resume_from to a larger k (file names and cadence as
    src/coresets/cuda/multi/fps_sharded.py:269-281, 422-446): ids and radii of the resumed run must
    equal the uninterrupted run's and the oracle's, bit for bit."""
    import oracle
    from coresets_b200 import engine, fps_sharded
    from tests.data import gaussian_mixture, with_duplicates
    failures = []
    out = Path(cfg["out_dir"])
    N, D, k_ck, k_full, every = cfg["N"], cfg["D"], cfg["k_ck"], cfg["k_full"], cfg["every"]
    X_np = with_duplicates(gaussian_mixture(N, D, 8, seed=N + D), 30, seed=2)
    base = N // world
    sizes = [base] * (world - 1) + [N - base * (world - 1)]
    offs = [sum(sizes[:r]) for r in range(world)]
    X_local = torch.from_numpy(np.ascontiguousarray(X_np[offs[rank] : offs[rank] + sizes[rank]])).to(dev)
    prefix = str(out / "ck")
    sel_a, eps_a = fps_sharded(X_local, k_ck, checkpoint_path=prefix, checkpoint_every=every, verbose=False)
    dist.barrier()
    if rank == 0:
        steps = sorted(int(p.name.split("_k")[1].split("_")[0]) for p in out.glob("ck_k*_ids.npy"))
        want = sorted(set(range(every, k_ck, every)) | {k_ck - 1})
        if steps != want:
            failures.append(f"checkpoint steps {steps} != {want}")
        if (out / "ck_latest.txt").read_text() != f"{k_ck - 1}\n":
            failures.append("latest.txt does not name the last pick")
        ids = np.load(out / f"ck_k{k_ck - 1:010d}_ids.npy")
        if ids.dtype != np.int64 or not np.array_equal(ids, sel_a.cpu().numpy()):
            failures.append("final checkpoint ids differ from the returned picks")
    dist.barrier()
    sel_b, eps_b = fps_sharded(X_local, k_full, resume_from=prefix, verbose=False)
    sel_c, eps_c = fps_sharded(X_local, k_full, verbose=False)
    if not torch.equal(sel_b, sel_c):
        failures.append(f"resumed picks differ from the uninterrupted run on rank {rank}")
    if not np.array_equal(eps_b.numpy().view(np.int32), eps_c.numpy().view(np.int32)):
        failures.append(f"resumed radii differ from the uninterrupted run on rank {rank}")
    norms = np.concatenate([
        engine.row_norms(torch.from_numpy(np.ascontiguousarray(X_np[offs[r] : offs[r] + sizes[r]])).to(dev)).cpu().numpy()
        for r in range(world)])
    o_sel, o_eps, _, _ = oracle.fps_sharded(X_np, norms, k_full, sizes, first=0)
    if not np.array_equal(sel_b.cpu().numpy(), o_sel) or not np.array_equal(eps_b.numpy().view(np.int32), o_eps.view(np.int32)):
        failures.append(f"resumed run differs from the oracle on rank {rank}")
    dist.barrier()
    return failures


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
        if Xl.dtype == torch.float32:
            # the replicated entry (whole matrix on every rank) against the reference's replicated driver
            # (tests/golden/acc_replicated.npz), or its sharded list where that file has no such case
            rep = golden / "acc_replicated.npz"
            want = np.load(rep)[name] if rep.is_file() and name in np.load(rep).files else z["sharded_plain"]
            Xf = torch.from_numpy(X_np).to(dev)
            na = c["n_anchor"]
            res = coresets_b200.cuda.multi.accrete_voronoi_multi(Xf[:na], Xf[na:], order, rank, world, max_k=c["max_k"],
                                                                 verbose=False)
            if not np.array_equal(res.cpu().numpy(), want):
                failures.append(f"{name}/replicated: ids differ from the reference on rank {rank} (world {world})")
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
