"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own CUDA path on a GPU.

Needs (all git-ignored, produced on a machine that has the reference checkout):
  oracle/_ref/site/   `pip install --no-deps --target oracle/_ref/site <reference checkout>`
  oracle/_ref/build/  `python oracle/build_ref.py --reference <reference checkout>` (the reference's kernels, its own flags)

Run on a B200:   python tests/golden/make_golden_gpu.py --out <output directory>
then copy the produced *.npz next to this file.  Each file holds the inputs that cannot be
regenerated bit-exactly elsewhere (the float32 row norms torch computed on the GPU) and the
reference's outputs: `selected` from its public `fps_cuda`, `selected`/`epsilons` from its
`fps_sharded` (one-rank NCCL group), and `h` / `voronoi` / `eps` from a transparent re-run of
its driver loop (`voronoi_step` + `argmax_cuda`, src/coresets/cuda/fps.py:105-128) that must
reproduce `fps_cuda`'s picks.  X itself is regenerated from tests/data.py (numpy, seeded).
"""
from __future__ import annotations

import argparse
import importlib.machinery
import importlib.util
import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle" / "_ref" / "site"))

from tests import data as tdata  # noqa: E402

CASES = [
    # name, generator, kwargs, K, seeds
    ("ref_script_8192x32", "clustered_jitter", dict(N=8192, D=32, seed=42), 2048, None),
    ("mix_4097x128", "gaussian_mixture", dict(N=4097, D=128, n_comp=8, seed=4225), 300, None),
    ("mix_2500x256", "gaussian_mixture", dict(N=2500, D=256, n_comp=8, seed=2756), 200, None),
    ("mix_900x1024", "gaussian_mixture", dict(N=900, D=1024, n_comp=8, seed=1924), 48, None),
    ("mix_33x64", "gaussian_mixture", dict(N=33, D=64, n_comp=8, seed=97), 20, None),
    ("mix_800x50", "gaussian_mixture", dict(N=800, D=50, n_comp=8, seed=850), 64, None),
    ("uneven_16383x128", "gaussian_mixture", dict(N=16383, D=128, n_comp=8, seed=16511), 512, None),
    ("c1_20000x64", "gaussian_mixture", dict(N=20000, D=64, n_comp=16, seed=0), 512, None),
    ("dups_3000x16", "dups", dict(N=3000, D=16, seed=5), 1500, None),
    ("seeded_5000x64", "gaussian_mixture", dict(N=5000, D=64, n_comp=8, seed=3), 200, [17, 4000, 123]),
    # float16 / float64 inputs (the reference's AT_DISPATCH_FLOATING_TYPES_AND_HALF, warp.cu:167)
    ("f16_2500x128", "gaussian_mixture", dict(N=2500, D=128, n_comp=8, seed=11), 200, None, "float16"),
    ("f16_800x50", "gaussian_mixture", dict(N=800, D=50, n_comp=8, seed=12), 64, None, "float16"),
    ("f64_1500x64", "gaussian_mixture", dict(N=1500, D=64, n_comp=8, seed=13), 128, None, "float64"),
    ("f64_1200x256", "gaussian_mixture", dict(N=1200, D=256, n_comp=8, seed=14), 100, [5, 900], "float64"),
]


def make_x(gen: str, kw: dict, dtype: str = "float32") -> np.ndarray:
    if gen == "dups":
        X = tdata.with_duplicates(tdata.clustered_jitter(kw["N"], kw["D"], seed=kw["seed"]), 600, seed=9)
    else:
        X = getattr(tdata, gen)(**kw)
    return tdata.as_dtype(X, dtype)


def load_reference():
    so = ROOT / "oracle" / "_ref" / "build" / "coreset_kernels.so"
    loader = importlib.machinery.ExtensionFileLoader("coreset_kernels", str(so))
    spec = importlib.util.spec_from_loader("coreset_kernels", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    import coresets.cuda.extension as ext
    ext._extension = mod
    ext._compiled = True
    import coresets
    return coresets, mod


def transparent_run(coresets, ext, X, K, seeds):
    """The reference's fps() loop with its state kept (src/coresets/cuda/fps.py:34-128)."""
    from coresets.cuda._internal import voronoi_step
    dev = X.device
    N, D = X.shape
    norms = (X * X).sum(dim=1).to(torch.float32)
    h = torch.full((N,), float("inf"), dtype=torch.float32, device=dev)
    v = torch.zeros(N, dtype=torch.int64, device=dev)
    X_sel = torch.empty((K, D), dtype=X.dtype, device=dev)
    norms_sel = torch.empty(K, dtype=torch.float32, device=dev)
    dSL = torch.empty(K, dtype=torch.float32, device=dev)
    d_idx = torch.empty(1, dtype=torch.int32, device=dev)
    d_val = torch.empty(1, dtype=torch.float32, device=dev)
    nb = int(ext.MAX_ARGMAX_BLOCKS)
    bv = torch.empty(nb, dtype=torch.float32, device=dev)
    bi = torch.empty(nb, dtype=torch.int32, device=dev)
    sel = np.empty(K, dtype=np.int64)
    eps = np.full(K, np.inf, dtype=np.float32)
    seeds = [0] if seeds is None else list(seeds)
    for i, s in enumerate(seeds):
        sel[i] = s
        voronoi_step(X, norms, h, v, X_sel, norms_sel, dSL, d_idx, int(s), i)
    for i in range(len(seeds), K):
        ext.argmax_cuda(h, bv, bi, d_val, d_idx, N)
        idx = int(d_idx.item())
        sel[i] = idx
        eps[i] = float(d_val.item())
        voronoi_step(X, norms, h, v, X_sel, norms_sel, dSL, d_idx, idx, i)
    return sel, eps, norms.cpu().numpy(), h.cpu().numpy(), v.cpu().numpy().astype(np.int32)


def compare_with_engine(name, X, K, seeds, sel_ref, eps_ref, h_ref, v_ref):
    """Side-by-side run of this repository's engine on the same device tensor (diagnostic)."""
    from coresets_b200 import engine
    norms = engine.row_norms(X)
    X32, element_order = engine.engine_matrix(X.contiguous())
    eng = engine.ShardEngine(X32, norms, K, element_order=element_order)
    eng.init_state()
    for s_ in ([0] if seeds is None else seeds):
        eng.pick_forced(int(s_))
    eng.run_picks(K - (1 if seeds is None else len(seeds)))
    eng.check_status()
    N = X.shape[0]
    ok_sel = np.array_equal(eng.selected.cpu().numpy(), sel_ref)
    ok_h = np.array_equal(eng.h[:N].cpu().numpy().view(np.int32), h_ref.view(np.int32))
    ok_v = np.array_equal(eng.voronoi[:N].cpu().numpy(), v_ref)
    ok_e = np.array_equal(eng.eps.cpu().numpy().view(np.int32), eps_ref.view(np.int32))
    print(f"[compare] {name}: selected={ok_sel} h_bits={ok_h} voronoi={ok_v} eps_bits={ok_e}", flush=True)


def midsize_compare(coresets, dev, out):
    """Reference vs engine on larger device-generated matrices: identical picks, wall time of both."""
    import json
    import time
    from coresets_b200 import engine
    from coresets_b200.synth import WORKLOADS, MixtureSource, scaled
    results = []
    for wname, n_rows, K in (("c3", 2_000_000, 2000), ("c2", 5_000_000, 1000), ("c4", 400_000, 500),
                             ("c3", 37_500_000, 1024)):
        w = scaled(WORKLOADS[wname], n_rows, k=K)
        X = MixtureSource(w).rows(0, n_rows, dev)
        torch.cuda.synchronize()
        t0 = time.time()
        ref_sel = coresets.fps_cuda(X, K)
        torch.cuda.synchronize()
        t_ref = time.time() - t0
        t0 = time.time()
        norms = engine.row_norms(X)
        eng = engine.ShardEngine(X, norms, K)
        eng.init_state()
        eng.pick_forced(0)
        eng.run_picks(K - 1)
        eng.check_status()
        torch.cuda.synchronize()
        t_new = time.time() - t0
        same = bool(torch.equal(ref_sel, eng.selected))
        ndiff = int((ref_sel != eng.selected).sum().item())
        rec = dict(workload=wname, n_rows=n_rows, dim=w.dim, K=K, identical=same, n_diff=ndiff,
                   reference_fps_cuda_s=t_ref, engine_s=t_new,
                   reference_picks_per_s=K / t_ref, engine_picks_per_s=K / t_new)
        print("[midsize]", json.dumps(rec), flush=True)
        results.append(rec)
        np.save(out / f"midsize_{wname}_{n_rows}_selected.npy", ref_sel.cpu().numpy())
        del X, norms, eng
        torch.cuda.empty_cache()
    (out / "midsize_compare.json").write_text(json.dumps(results, indent=1))


ACCRETE_CASES = {
    # the reference's own determinism configs (tests/slurm/test_determinism.sh:43-46), scaled K
    "acc_8192x32_k2048": dict(gen="jitter", N=8192, D=32, max_k=11, n_anchor=4096, order="arange"),
    "acc_16383x128_k1024": dict(gen="jitter", N=16383, D=128, max_k=10, n_anchor=8191, order="arange"),
    "acc_mix_20000x64_k512_fps": dict(gen="mix", N=20000, D=64, max_k=9, n_anchor=8000, order="fps"),
    # float16 input: element-wise sums in the kernels, reconstruct product in float16.  (float64 has
    # no case: the reference's reconstruct step stops with a dtype error from torch's index_put, and
    # on the clustered-jitter matrix in float16 its invariant check reports a gross violation.)
    "acc_f16_4000x32_k256": dict(gen="mix", N=4000, D=32, max_k=8, n_anchor=1500, order="arange", dtype="float16"),
}


def accrete_case_matrix(c: dict) -> np.ndarray:
    """The matrix of an accretion case, regenerated from tests/data.py (numpy, seeded)."""
    X = (tdata.clustered_jitter(c["N"], c["D"], seed=42) if c["gen"] == "jitter"
         else tdata.gaussian_mixture(c["N"], c["D"], 12, seed=c["N"]))
    return tdata.as_dtype(X, c.get("dtype", "float32"))


def accrete_goldens(coresets, dev, out, compare, only=""):
    """Reference `accrete` and one-rank `accrete_sharded` (default knobs and
    CORESETS_BISECT_SEED=1 CORESETS_FILL_CHUNK=256) on the GPU; index lists + the single-GPU trace."""
    from tests.golden.make_golden_accrete_cpu import read_trace
    import time
    for name, c in ACCRETE_CASES.items():
        if only and only not in name:
            continue
        X = torch.from_numpy(accrete_case_matrix(c)).to(dev)
        na = c["n_anchor"]
        if c["order"] == "arange":
            order = torch.arange(na, dtype=torch.long, device=dev)
        else:
            order = coresets.fps_cuda(X[:na].contiguous(), na)
        tr = str(out / f"{name}.tsv")
        t0 = time.time()
        try:
            single = coresets.accrete(X[:na], X[na:], order, c["max_k"], verbose=False, trace_path=tr)
        except RuntimeError as e:      # the reference's own invariant check can reject low-precision inputs
            print(f"[golden] {name}: the reference raised: {str(e)[:200]}", flush=True)
            continue
        torch.cuda.synchronize()
        t_single = time.time() - t0
        rec = dict(anchor_order=order.cpu().numpy(), single=single.cpu().numpy().astype(np.int64), **read_trace(tr))
        times = {"reference_accrete_s": t_single}
        for tag, env in (("plain", {}), ("knobs", {"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"})):
            for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
                os.environ.pop(k, None)
            os.environ.update(env)
            t0 = time.time()
            res = coresets.accrete_sharded(X, order, na, max_k=c["max_k"], verbose=False)
            torch.cuda.synchronize()
            times[f"reference_accrete_sharded_{tag}_s"] = time.time() - t0
            rec[f"sharded_{tag}"] = res.cpu().numpy().astype(np.int64)
        for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
            os.environ.pop(k, None)
        np.savez_compressed(out / f"{name}.npz", **rec)
        msg = {k_: bool(np.array_equal(rec["single"], rec[k_])) for k_ in ("sharded_plain", "sharded_knobs")}
        print(f"[golden] {name}: {len(rec['single'])} ids; reference variants equal to single: {msg}; {times}", flush=True)
        if compare:
            import coresets_b200
            t0 = time.time()
            mine = coresets_b200.accrete(X[:na], X[na:], order, c["max_k"], verbose=False)
            torch.cuda.synchronize()
            t_mine = time.time() - t0
            ms = coresets_b200.accrete_sharded(X, order, na, max_k=c["max_k"], verbose=False)
            os.environ.update({"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"})
            mk = coresets_b200.accrete_sharded(X, order, na, max_k=c["max_k"], verbose=False)
            for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
                os.environ.pop(k, None)
            print(f"[compare] {name}: accrete={bool(np.array_equal(mine.cpu().numpy(), rec['single']))} "
                  f"sharded={bool(np.array_equal(ms.cpu().numpy(), rec['sharded_plain']))} "
                  f"sharded_knobs={bool(np.array_equal(mk.cpu().numpy(), rec['sharded_knobs']))} "
                  f"engine_accrete_s={t_mine:.2f} reference_accrete_s={t_single:.2f}", flush=True)


def midsize_accrete_compare(coresets, dev, out):
    """Reference vs engine accretion on a larger device-generated matrix (no fixture: evidence of
    identical lists and the wall time of both)."""
    import json
    import time
    import coresets_b200
    from coresets_b200.synth import Workload, MixtureSource
    results = []
    for n_anchor, n_cand, dim, max_k in ((400_000, 400_000, 64, 11), (1_000_000, 1_000_000, 128, 10)):
        wa = Workload("acc_anchor", n_anchor, dim, 32, 11, 0)
        wc = Workload("acc_cand", n_cand, dim, 48, 12, 0, mean_scale=6.0)
        X = torch.cat([MixtureSource(wa).rows(0, n_anchor, dev), MixtureSource(wc).rows(0, n_cand, dev)])
        order = coresets_b200.fps_cuda(X[:n_anchor].contiguous(), 2 ** max_k)
        rec = dict(n_anchor=n_anchor, n_cand=n_cand, dim=dim, max_k=max_k)
        for tag, env in (("plain", {}), ("knobs", {"CORESETS_BISECT_SEED": "1", "CORESETS_FILL_CHUNK": "256"})):
            for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
                os.environ.pop(k, None)
            os.environ.update(env)
            torch.cuda.synchronize(); t0 = time.time()
            ref = coresets.accrete_sharded(X, order, n_anchor, max_k=max_k, verbose=False)
            torch.cuda.synchronize(); t_ref = time.time() - t0
            t0 = time.time()
            mine = coresets_b200.accrete_sharded(X, order, n_anchor, max_k=max_k, verbose=False)
            torch.cuda.synchronize(); t_new = time.time() - t0
            rec[f"{tag}_identical"] = bool(torch.equal(ref, mine))
            rec[f"{tag}_reference_s"] = round(t_ref, 2)
            rec[f"{tag}_engine_s"] = round(t_new, 2)
        for k in ("CORESETS_BISECT_SEED", "CORESETS_FILL_CHUNK"):
            os.environ.pop(k, None)
        print("[midsize-accrete]", json.dumps(rec), flush=True)
        results.append(rec)
        del X
        torch.cuda.empty_cache()
    (out / "midsize_accrete_compare.json").write_text(json.dumps(results, indent=1))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(ROOT / "golden_out"))
    ap.add_argument("--compare", action="store_true", help="also run this repository's engine side by side")
    ap.add_argument("--cases", default="", help="only the FPS and accretion cases whose name contains this text")
    a = ap.parse_args()
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    coresets, ext = load_reference()
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    torch.cuda.set_device(0)
    dist.init_process_group("nccl", rank=0, world_size=1)
    dev = torch.device("cuda:0")
    for name, gen, kw, K, seeds, *rest in CASES:
        if a.cases and a.cases not in name:
            continue
        dtype = rest[0] if rest else "float32"
        X_np = make_x(gen, kw, dtype)
        X = torch.from_numpy(X_np).to(dev)
        seed_t = None if seeds is None else torch.tensor(seeds, dtype=torch.long)
        sel_api = coresets.fps_cuda(X, K, seed=seed_t).cpu().numpy().astype(np.int64)
        sel, eps, norms, h, v = transparent_run(coresets, ext, X, K, seeds)
        assert np.array_equal(sel, sel_api), f"{name}: transparent loop diverged from fps_cuda"
        rec = dict(generator=gen, K=K, dtype=dtype, selected=sel_api, eps=eps, norms=norms, h=h, voronoi=v,
                   seeds=np.asarray(seeds if seeds is not None else [0], dtype=np.int64),
                   **{f"gen_{k}": v_ for k, v_ in kw.items()})
        if seeds is None or len(seeds) == 1:
            s_sel, s_eps = coresets.fps_sharded(X, K, seed=None if seeds is None else int(seeds[0]), verbose=False)
            rec["sharded_selected"] = s_sel.cpu().numpy().astype(np.int64)
            rec["sharded_eps"] = s_eps.numpy().astype(np.float32)
            assert np.array_equal(rec["sharded_selected"], sel_api), f"{name}: fps_sharded != fps_cuda"
        np.savez_compressed(out / f"{name}.npz", **rec)
        print(f"[golden] {name}: K={K} first={sel_api[:5].tolist()} last={sel_api[-3:].tolist()}", flush=True)
        if a.compare:
            compare_with_engine(name, X, K, seeds, sel_api, eps, h, v)
    if a.cases:
        accrete_goldens(coresets, dev, out, a.compare, only=a.cases)
        dist.destroy_process_group()
        return
    accrete_goldens(coresets, dev, out, a.compare)
    if a.compare:
        midsize_accrete_compare(coresets, dev, out)
        midsize_compare(coresets, dev, out)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
