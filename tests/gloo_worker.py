"""Worker process of the world_size > 1 CPU tests (gloo).  Run by tests/test_sharded_gloo.py."""
from __future__ import annotations

import importlib
import json
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> None:
    cfg = json.loads(sys.argv[1])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from coresets_b200 import _native
    from tests.fake_native import FakeNative
    _native.set_native_for_tests(FakeNative())
    sharded_mod = importlib.import_module("coresets_b200.cuda.multi.fps_sharded")
    sharded_mod._REQUIRE_CUDA = False

    if cfg.get("mode") == "accrete":
        return accrete_mode(cfg, rank, world)
    X = np.load(cfg["x_path"])
    sizes = cfg["sizes"]
    off = sum(sizes[:rank])
    X_local = torch.from_numpy(np.ascontiguousarray(X[off : off + sizes[rank]]))
    out = Path(cfg["out_dir"])
    try:
        if cfg.get("expect_error"):
            try:
                sharded_mod.fps_sharded(X_local if not (cfg["expect_error"] == "dim" and rank == 1)
                                        else X_local[:, :-1].contiguous(), cfg["k"], verbose=False)
            except ValueError as e:
                (out / f"err_{rank}.txt").write_text(str(e))
            return
        kwargs = dict(seed=cfg.get("seed"), verbose=cfg.get("verbose", False))
        if cfg.get("checkpoint"):
            kwargs.update(checkpoint_path=str(out / "ck"), checkpoint_every=cfg.get("checkpoint_every", 0))
        if cfg.get("resume"):
            kwargs.update(resume_from=str(out / "ck"))
        sel, eps = sharded_mod.fps_sharded(X_local, cfg["k"], **kwargs)
        assert sel.dtype == torch.int64 and eps.dtype == torch.float32 and eps.device.type == "cpu"
        np.save(out / f"sel_{rank}.npy", sel.numpy())
        np.save(out / f"eps_{rank}.npy", eps.numpy())
    finally:
        dist.barrier()
        dist.destroy_process_group()


def accrete_mode(cfg, rank, world) -> None:
    """accrete_voronoi_multi_sharded over gloo ranks for the cases of a golden file."""
    sh = importlib.import_module("coresets_b200.cuda.multi.sharded")
    sh._REQUIRE_CUDA = False
    from coresets_b200.cuda.multi.layout import compute_shard_layout
    out = Path(cfg["out_dir"])
    try:
        for case in cfg["cases"]:
            for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK", "CORESETS_LANES_MIN_STEPS", "CORESETS_BISECT_GALLOP_DEEP",
                      "CORESETS_LAZY_FORWARD"):
                os.environ.pop(k, None)
            os.environ.update(case.get("env", {}))
            X = np.load(case["x_path"])
            order = np.load(case["order_path"])
            sizes, offs = compute_shard_layout(X.shape[0], world)
            Xl = torch.from_numpy(np.ascontiguousarray(X[offs[rank] : offs[rank] + sizes[rank]]))
            kw = {}
            if case.get("checkpoint"):
                kw.update(checkpoint_path=str(out / case["checkpoint"]), checkpoint_every=case.get("checkpoint_every", 0))
            if case.get("resume"):
                kw.update(resume_from=str(out / case["resume"]))
            if case.get("trace"):
                kw.update(trace_path=str(out / f"{case['name']}_trace_{rank}.tsv"))
            if case.get("replicated"):      # every rank holds the whole matrix (accrete_voronoi_multi)
                from coresets_b200.cuda.multi import accrete_voronoi_multi
                na = case["n_anchor"]
                res = accrete_voronoi_multi(torch.from_numpy(X[:na]), torch.from_numpy(X[na:]), torch.from_numpy(order),
                                            rank, world, max_k=case["max_k"], verbose=False)
            else:
                res = sh.accrete_voronoi_multi_sharded(
                    Xl, rank, world, case["n_anchor"], X.shape[0], sizes, torch.from_numpy(order),
                    max_k=case["max_k"], n_target=case.get("n_target"), verbose=False, **kw)
            assert res.dtype == torch.int64
            np.save(out / f"{case['name']}_{rank}.npy", res.numpy())
    finally:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
