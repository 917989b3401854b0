"""Benchmark of the farthest-point-sampling hot path.

    python bench.py --gpus 1 --steps K --warmup W            (one process)
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...                       (the reference's CPU `fps`)

A "step" is ONE FPS pick over the resident matrix: the bound kernel plus the fused
distance / min-update / arg-max kernel on every rank, plus the candidate all-gather when N > 1.
The headline line is measured in DENSE mode (every live row's distance is evaluated each pick --
the bandwidth-bound pass the roofline is about, and what the reference's CPU `fps` does); the
`prune` object reports the default product mode (triangle-bound skip through the cell index,
identical picks).

Workload: the 300M x 128 fp32 mixture ("c3"), rows split over the ranks with
compute_shard_layout (strong scaling).  Inputs are synthetic, generated on the device from
(seed, row block).  X is far larger than the 126 MB L2, so no flush is needed between steps.
Every pick the bench makes on c3 starts from row 0, so the picks are a prefix of the full
k = 16384 run: `parity` compares them with the list the reference's own fps_sharded produced at
full size (tests/golden/fullsize_c3.npz).  `configs` adds the other benchmark configurations
(c2 on one GPU, c4 split over the ranks, the accretion case c5 on two or more GPUs), each with its
own dense-kernel roofline, product-mode picks/s and parity against its golden list.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "fps_picks_per_s"
UNIT = "picks/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=24)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--rows", type=int, default=0, help="override the workload's global row count")
    ap.add_argument("--prune-picks", type=int, default=1000, help="picks run before the prune-mode timing")
    ap.add_argument("--dense-kernel", default="tma", choices=["tma", "ldg"],
                    help="dense mode: X through the TMA ring (default) or plain 128-bit loads")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-prune", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the c2 / c4 / c5 legs")
    ap.add_argument("--configs", default="c2,c4,c5", help="which of the other configurations to run")
    ap.add_argument("--c5-rows", type=int, default=0, help="accretion leg: anchors = candidates = this many rows (0 = 50M from 4 GPUs on, the pinned 5M case below)")
    ap.add_argument("--c5-max-k", type=int, default=14)
    ap.add_argument("--cpu-rows", type=int, default=32_000_000, help="rows of the CPU reference's sample")
    ap.add_argument("--no-ref-cuda", action="store_true", help="reference arm: skip the reference's own CUDA fps")
    return ap.parse_args()


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons for one GPU while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.rows = []
        self.proc = None
        try:
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            ident = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={ident}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=3)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            f = [x.strip() for x in r.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_max(x: float, device) -> float:
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return x


def barrier_sync(device):
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()
    torch.cuda.synchronize(device)


GOLDEN = ROOT / "tests" / "golden"


def parity_with_golden(selected, name: str, rows: int, first_pick: int = 0) -> dict:
    """Compare picks (a prefix of the run from `first_pick`) with the list the reference wrote at
    FULL size for this configuration; None-valued `equal` when no such list applies."""
    path = GOLDEN / f"fullsize_{name}.npz"
    if not path.is_file():
        return {"checked": 0, "equal": None, "golden": None, "why": f"no {path.name} in tests/golden"}
    z = np.load(path)
    if int(z["rows"]) != rows or first_pick != 0:
        return {"checked": 0, "equal": None, "golden": path.name,
                "why": f"the golden list is for {int(z['rows'])} rows from row 0; this run has {rows} rows"}
    mine = np.asarray(selected.detach().cpu().numpy() if hasattr(selected, "detach") else selected, dtype=np.int64)
    n = min(mine.shape[0], int(z["selected"].shape[0]))
    equal = bool(np.array_equal(mine[:n], z["selected"][:n].astype(np.int64)))
    out = {"checked": n, "equal": equal, "golden": f"tests/golden/{path.name}",
           "written_by": f"the reference's fps_sharded at world size {int(z['world'])}"}
    if not equal:
        out["first_difference"] = int(np.argmax(mine[:n] != z["selected"][:n]))
    return out


# ------------------------------------------------------------------------------------- CPU arms
def cpu_reference_fn():
    """The reference's own CPU `fps` when its package travelled with the repo (oracle/_ref/site),
    else the port in oracle/cpu_fps.py."""
    site = ROOT / "oracle" / "_ref" / "site"
    if (site / "coresets" / "pytorch" / "fps.py").is_file():
        sys.path.insert(0, str(site))
        try:
            from coresets.pytorch.fps import fps as ref_fps
            return ref_fps, "reference"
        except Exception:
            pass
    from oracle.cpu_fps import fps as port_fps
    return port_fps, "port"


def cpu_arm(w, rows: int, steps: int, warmup: int) -> dict:
    """The reference's CPU `fps` on a bounded sample: the first `rows` rows of the workload (the CPU
    `fps` keeps an N x D temporary beside X, so the full 153.6 GB matrix does not fit the host).
    A dense pick is one matrix-vector product over X, linear in the rows: the full-size figure is
    the sample's scaled by rows / n_rows and is labelled as extrapolated."""
    from coresets_b200.synth import MixtureSource, scaled
    fn, kind = cpu_reference_fn()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    try:
        import psutil
        fit = int(psutil.virtual_memory().available * 0.3 // (w.dim * 4))
    except Exception:
        fit = rows
    rows = max(1, min(rows, w.n_rows, fit))
    X = MixtureSource(scaled(w, rows)).rows(0, rows, torch.device("cpu"))
    fn(X, max(warmup, 2))                       # TorchScript / BLAS warm-up, untimed
    t0 = time.perf_counter()
    fn(X, steps)
    dt = time.perf_counter() - t0
    sample_rate = steps / dt
    scale = rows / w.n_rows
    return {"value": sample_rate * scale, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"{steps} dense picks on the first {rows} rows of {w.name} ({w.dim} cols) in {dt:.2f} s = "
                      f"{sample_rate:.2f} picks/s on the sample",
            "extrapolated": scale != 1.0, "scale_factor": scale, "sample_rows": rows,
            "sample_picks_per_s": sample_rate, "ms_per_step_sample": 1e3 * dt / steps}


def reference_cuda_leg(w, shard_rows: int, picks_before: int, steps: int) -> dict:
    """The reference's own CUDA `fps_cuda` (its kernels built for cc 10.0 under oracle/_ref) on the
    first `shard_rows` rows of the workload -- the 8-GPU share of the headline configuration, the
    most one GPU can hold for the reference (2^27 rows, plus its N x D norms temporary).  Its API
    is one call per run, so the rate of picks picks_before .. picks_before + steps is the
    difference of two calls."""
    so = ROOT / "oracle" / "_ref" / "build" / "coreset_kernels.so"
    if not (so.is_file() and torch.cuda.is_available()):
        return {"unavailable": "needs a GPU and the reference's extension under oracle/_ref (oracle/build_ref.py)"}
    try:
        sys.path.insert(0, str(ROOT / "oracle" / "_ref" / "site"))
        from tests.golden.make_golden_gpu import load_reference
        from coresets_b200.synth import MixtureSource, scaled
        coresets, _ = load_reference()
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(0)
        rows = min(shard_rows, w.n_rows)
        X = MixtureSource(scaled(w, rows)).rows(0, rows, dev)
        coresets.fps_cuda(X, 8)                                   # context, allocator
        torch.cuda.synchronize()
        t = []
        for k in (picks_before, picks_before + steps):
            t0 = time.perf_counter()
            sel = coresets.fps_cuda(X, k)
            torch.cuda.synchronize()
            t.append(time.perf_counter() - t0)
        return {"what": f"reference fps_cuda on the first {rows} rows of {w.name}, row 0 first",
                "rows": rows, "picks_before": picks_before, "steps": steps,
                "value": steps / max(t[1] - t[0], 1e-9), "unit": UNIT,
                "whole_call_s": t[1], "whole_call_picks": picks_before + steps,
                "whole_call_picks_per_s": (picks_before + steps) / t[1],
                "selected_tail": [int(v) for v in sel[-3:].tolist()]}
    except Exception as ex:  # the CPU line must still print
        return {"unavailable": f"{type(ex).__name__}: {str(ex)[:200]}"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from coresets_b200.synth import WORKLOADS, scaled
    w = WORKLOADS[args.workload]
    if args.rows:
        w = scaled(w, args.rows, k=w.k)
    steps = max(args.steps, 1)
    cb = cpu_arm(w, args.cpu_rows, steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_step_sample"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "extrapolated": cb["extrapolated"], "scale_factor": cb["scale_factor"],
        "ms_per_step_what": "the SAMPLE's own time per pick (what this run really executed); value = the sample's "
                            "picks/s x scale_factor",
        "config": {"workload": f"{w.name}: {w.describe}", "rows": w.n_rows, "dim": w.dim, "mode": "dense (reference CPU fps)",
                   "sample_rows": cb["sample_rows"]},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not args.no_ref_cuda:
        line["cuda"] = reference_cuda_leg(w, SHARD_ROWS, 1 + args.prune_picks, steps)
    print(json.dumps(line), flush=True)


SHARD_ROWS = 37_500_000      # the 8-GPU share of c3: the largest shard the reference's CUDA path takes on one GPU


# ------------------------------------------------------------------------------------- GPU arm
def timed_region(fn, device) -> float:
    """Device time of fn() in ms: barrier + synchronize on both sides, max over the ranks."""
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier_sync(device)
    ev0.record()
    fn()
    ev1.record()
    barrier_sync(device)
    return dist_max(ev0.elapsed_time(ev1), device)


def dense_leg(eng, K: int, W: int, device, extra: int):
    """W warm-up picks, then EXACTLY K timed dense picks, launched one by one with an event on
    either side of every step kernel: the per-kernel durations come from inside the timed region, so
    the kernel time can never exceed the step that contains it.  `extra` more picks after the region
    widen the per-kernel sample.  Returns (ms of the K picks, kernel ms list of the region, kernel ms
    list of region + extra, commit ms list, exchange ms list)."""
    def picks(n, rec):
        for _ in range(n):
            a, b, c, d = (torch.cuda.Event(enable_timing=True) for _ in range(4))
            a.record()
            eng.exchange()
            b.record()
            eng.commit()
            c.record()
            eng.step()
            d.record()
            rec.append((a, b, c, d))

    picks(W, [])
    region, after = [], []
    ms_total = timed_region(lambda: picks(K, region), device)
    picks(extra, after)
    torch.cuda.synchronize(device)
    kern = [c.elapsed_time(d) for _, _, c, d in region]
    kern_all = kern + [c.elapsed_time(d) for _, _, c, d in after]
    commit = [b.elapsed_time(c) for _, b, c, _ in region + after]
    xchg = [a.elapsed_time(b) for a, b, _, _ in region + after]
    return ms_total, kern, kern_all, commit, xchg


def roofline_of(kern_region, kern_all, rows_per_launch: int, dim: int, device, dense_kernel: str) -> dict:
    kern_ms = dist_max(statistics.mean(kern_region), device)
    algo_bytes = rows_per_launch * (4 * dim + 8)
    achieved = algo_bytes / (kern_ms / 1e3) / 1e9
    peak, peak_kind = peaks()
    # DRAM traffic per row from the ncu captures under profiles/ (dram__bytes_read + write of one launch
    # divided by its rows; traffic grows in proportion to the rows of a launch)
    per_row = {("tma", 128): 526.8, ("ldg", 128): 525.3, ("tma", 256): 1038.0, ("tma", 1024): 4117.7}.get((dense_kernel, dim))
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_kind": peak_kind, "traffic": rows_per_launch * per_row if per_row else None,
            "traffic_source": (f"ncu dram__bytes_read+write of one launch on a 4-8 GB case at D = {dim} ({per_row} B/row, "
                               "profiles/), scaled by rows" if per_row
                               else f"no ncu capture of the dense kernel at D = {dim} under profiles/"),
            "kernel": ("fps_step_tma_kernel (dense, cp.async.bulk ring)" if dense_kernel == "tma"
                       else "fps_step_kernel (dense, LDG.128)"),
            "kernel_ms": kern_ms, "kernel_ms_median": statistics.median(kern_all), "kernel_launches_timed": len(kern_all),
            "kernel_ms_what": "mean over the launches INSIDE the timed region (events around each step kernel); "
                              "median over those plus the launches that follow",
            "algorithmic_bytes_per_launch": algo_bytes}


def prune_leg(X, norms, cap, off, world, picks_before: int, K: int, device, cells: bool) -> dict:
    """Product mode (triangle-bound skip): a fresh run from row 0, `picks_before` picks untimed,
    then K timed.  cells=True is the default path (cell index), False the full scan of h / voronoi."""
    from coresets_b200 import engine
    from coresets_b200._native import MODE_PRUNE
    eng = engine.ShardEngine(X, norms, cap, shard_offset=off, world_size=world, mode=MODE_PRUNE, cells=cells)
    eng.init_state()
    eng.pick_forced(0)
    eng.run_picks(picks_before - 1)
    eng.prepare(K)
    ms = timed_region(lambda: eng.run_picks(K), device)
    ctl = eng.check_status()
    out = {"value": K / (ms / 1e3), "unit": UNIT, "ms_per_step": ms / K, "picks_before": picks_before,
           "live_rows_last_step_rank0": int(ctl.live_rows), "rows_rank0": int(X.shape[0]),
           "path": "cell index" if eng.cells_enabled else "full scan"}
    if eng.cells_enabled:
        out["index_builds"] = [{"at_pick": a, "visited_share": s} for a, s in eng.cells_log]
    return out, eng


def run_ours(args):
    from coresets_b200 import _native, engine
    from coresets_b200._native import MODE_DENSE, MODE_DENSE_LDG
    from coresets_b200.cuda.multi.layout import compute_shard_layout
    from coresets_b200.synth import WORKLOADS, MixtureSource, scaled

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    native = _native.get_native()
    sms = native.device_check()

    w = WORKLOADS[args.workload]
    if args.rows:
        w = scaled(w, args.rows, k=w.k)
    sizes, offsets = compute_shard_layout(w.n_rows, world)
    n_local, off = sizes[rank], offsets[rank]
    K, W = max(args.steps, 1), max(args.warmup, 0)
    extra = max(0, 50 - K)
    do_prune = not args.no_prune

    need = n_local * (w.dim * 4 + 28) + (2 << 30)
    free_b, _ = torch.cuda.mem_get_info(device)
    if need > free_b:
        raise SystemExit(f"rank {rank}: needs {need/1e9:.1f} GB of device memory, {free_b/1e9:.1f} GB free")

    t_gen = time.time()
    X = torch.empty((n_local, w.dim), dtype=torch.float32, device=device)
    MixtureSource(w).fill(X, off)
    norms = engine.row_norms(X)
    torch.cuda.synchronize(device)
    t_gen = time.time() - t_gen

    # ---- headline: dense picks, inputs resident in HBM -------------------------------------------
    dense_mode = MODE_DENSE if args.dense_kernel == "tma" else MODE_DENSE_LDG
    cap = 1 + W + K + extra + 8
    eng = engine.ShardEngine(X, norms, cap, shard_offset=off, world_size=world, mode=dense_mode)
    eng.init_state()
    eng.pick_forced(0)
    sampler = ClockSampler(local) if rank == 0 else None
    ms_total, kern, kern_all, commit_ms, xchg_ms = dense_leg(eng, K, W, device, extra)
    clocks = sampler.stop() if sampler else None
    eng.check_status()
    value = K / (ms_total / 1e3)
    roofline = roofline_of(kern, kern_all, max(sizes), w.dim, device, args.dense_kernel)
    roofline["live_rows_last_launch_rank0"] = int(eng.read_ctl().live_rows)
    parity = {"dense": parity_with_golden(eng.selected[: 1 + W + K + extra], w.name, w.n_rows)}
    eng = None

    # ---- default product mode ---------------------------------------------------------------------
    prune = None
    shard = None
    if do_prune:
        pcap = 1 + args.prune_picks + K + 8
        prune, peng = prune_leg(X, norms, pcap, off, world, 1 + args.prune_picks, K, device, cells=True)
        parity["prune"] = parity_with_golden(peng.selected[: 1 + args.prune_picks + K], w.name, w.n_rows)
        peng = None
        torch.cuda.empty_cache()
        scan, seng = prune_leg(X, norms, pcap, off, world, 1 + args.prune_picks, K, device, cells=False)
        prune["full_scan"] = {k: scan[k] for k in ("value", "ms_per_step", "path")}
        seng = None
        torch.cuda.empty_cache()
        if world == 1 and n_local > SHARD_ROWS:
            # the shard the reference's own CUDA path can take on one GPU (see --impl reference, `cuda`)
            Xs, ns = X[:SHARD_ROWS], norms[:SHARD_ROWS]
            shard, sheng = prune_leg(Xs, ns, pcap, 0, 1, 1 + args.prune_picks, K, device, cells=True)
            shard["what"] = f"product mode on the first {SHARD_ROWS} rows of {w.name}, row 0 first (one GPU)"
            sheng = Xs = ns = None
            torch.cuda.empty_cache()
    parity["equal"] = (None if any(p["equal"] is None for p in parity.values())
                       else all(p["equal"] for p in parity.values()))
    parity["checked"] = sum(p["checked"] for p in parity.values() if isinstance(p, dict))

    # ---- end to end through the public API: host X -> device -> picks -> host -----------------
    e2e = None
    if not args.no_e2e:
        norms = None
        torch.cuda.empty_cache()
        try:
            e2e = run_e2e(args, X, w, world, rank, device, K, W, off)
        except Exception as ex:  # the headline line must still print
            e2e = {"value": None, "unit": UNIT, "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                   "error": f"{type(ex).__name__}: {str(ex)[:200]}"}
    X = norms = None
    torch.cuda.empty_cache()

    configs = None
    if not args.no_configs:
        configs = {}
        for name in [c for c in args.configs.split(",") if c]:
            try:
                configs[name] = run_config(name, args, world, rank, device, K, W)
            except Exception as ex:
                configs[name] = {"error": f"{type(ex).__name__}: {str(ex)[:300]}"}
            torch.cuda.empty_cache()

    cpu_b = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_b = cpu_arm(w, args.cpu_rows, 24, 3)

    if rank == 0:
        n_prune = (2 * (1 + args.prune_picks + K) if do_prune else 0)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{w.name}: {w.describe}", "rows": w.n_rows, "dim": w.dim,
                       "rows_per_gpu": max(sizes), "mode": "dense", "first_pick": 0,
                       "l2": "inputs (>= 19 GB per GPU) exceed the 126 MB L2; no flush",
                       "exchange": ("none" if world == 1 else
                                    "peer stores over NVLink + flag wait, fused into the two kernels"
                                    if engine.exchange_mode() == "p2p" else
                                    "one NCCL all-gather of (4+D) words per rank per pick"),
                       "generate_s": round(t_gen, 2), "sms": sms},
            "roofline": roofline,
            "step_breakdown_ms": {"fps_step": roofline["kernel_ms"], "commit_bound": statistics.mean(commit_ms),
                                  "exchange": statistics.mean(xchg_ms) if world > 1 else 0.0},
            "parity": parity, "prune": prune, "shard_37m": shard, "e2e": e2e, "configs": configs,
            "cpu_baseline": cpu_b, "clocks": clocks,
            "gpu_launches": 2 * K,
            "gpu_launches_what": "commit_bound_kernel + the dense step kernel per timed pick; the other legs launch their own",
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


class HostMatrix:
    """Host-side copy of a rank's rows in ordinary (pageable) memory, moved to and from the device
    through a ring of eight page-locked 64 MiB staging buffers: the CPU copy of the next chunks
    overlaps the DMA of the earlier ones (measured on the GPU box: 43 GB/s against 38 GB/s with two
    1 GiB buffers; the DMA alone reaches 55 GB/s, the 16-core CPU copy 40-57 GB/s).  This is how a
    user's large numpy array reaches the device; page-locking the whole matrix is not attempted
    (153.6 GB of locked pages starve a 196 GB host)."""
    RING_BYTES = 64 << 20
    RING_SLOTS = 8

    def __init__(self, X: torch.Tensor, try_pinned: bool = False):
        """``try_pinned``: keep the rows in page-locked memory outright (one DMA, no staging copy)
        when the allocation succeeds; used when the matrix is a small part of the host's memory."""
        self.shape, self.dtype = tuple(X.shape), X.dtype
        self.pinned = False
        self.host = None
        if try_pinned:
            try:
                self.host = torch.empty(self.shape, dtype=self.dtype, pin_memory=True)
                self.pinned = True
            except RuntimeError:
                torch.cuda.synchronize(X.device)
                self.host = None
        if self.host is None:
            self.host = torch.empty(self.shape, dtype=self.dtype)
        rows = max(1, self.RING_BYTES // max(1, self.shape[1] * 4))
        self.ring = [] if self.pinned else [torch.empty((rows, self.shape[1]), dtype=self.dtype, pin_memory=True)
                                            for _ in range(self.RING_SLOTS)]
        self._move(X, to_device=False)

    def _move(self, X: torch.Tensor, to_device: bool) -> None:
        if self.pinned:
            (X.copy_(self.host, non_blocking=True) if to_device else self.host.copy_(X, non_blocking=True))
            if not to_device:
                torch.cuda.synchronize(X.device)
            return
        rows = self.ring[0].shape[0]
        slots = len(self.ring)
        evs = [None] * slots
        n = self.shape[0]
        pending = None
        for i, a in enumerate(range(0, n, rows)):
            b = min(a + rows, n)
            buf = self.ring[i % slots]
            if evs[i % slots] is not None:
                evs[i % slots].synchronize()
            if to_device:
                buf[: b - a].copy_(self.host[a:b])
                X[a:b].copy_(buf[: b - a], non_blocking=True)
            else:
                if pending is not None:          # drain the previous chunk while this one flies
                    pa, pb, pbuf, pev = pending
                    pev.synchronize()
                    self.host[pa:pb].copy_(pbuf[: pb - pa])
                buf[: b - a].copy_(X[a:b], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
            evs[i % slots] = ev
            if not to_device:
                pending = (a, b, buf, ev)
        if not to_device and pending is not None:
            pa, pb, pbuf, pev = pending
            pev.synchronize()
            self.host[pa:pb].copy_(pbuf[: pb - pa])

    def upload(self, X: torch.Tensor) -> None:
        self._move(X, to_device=True)


def host_memory_available() -> int:
    """Bytes this process group may still use: the smaller of the machine's available memory and the
    head-room under the cgroup limit (a container can be capped far below the machine)."""
    import psutil
    avail = psutil.virtual_memory().available
    try:
        limit = Path("/sys/fs/cgroup/memory.max").read_text().strip()
        used = int(Path("/sys/fs/cgroup/memory.current").read_text().strip())
        if limit != "max":
            avail = min(avail, int(limit) - used)
    except Exception:
        pass
    return int(avail)


def run_e2e(args, X, w, world, rank, device, K, W, off):
    """One complete job through the PUBLIC API from HOST rows: H2D of the rank's rows, then
    ``coresets_b200.fps_cuda`` (one GPU) / ``fps_sharded`` (several) for K picks -- its validation,
    norms, state set-up, graph capture and the picks themselves -- then the D2H read of the result.
    The one-off upload is charged in full to the K picks."""
    import coresets_b200
    n_local, dim = X.shape
    nbytes = n_local * dim * 4
    avail = host_memory_available()
    share = max(1, min(world, torch.cuda.device_count()))
    # all ranks of this node together (rows + 0.5 GiB of staging buffers each) must leave 16 GiB free
    ok = torch.tensor([1 if (nbytes + (2 << 30)) * share + (16 << 30) < avail else 0], device=device)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        return {"value": None, "unit": UNIT, "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                "skipped": f"host memory: {nbytes/1e9:.1f} GB per rank needed, {avail/1e9:.1f} GB available"}
    # torchrun pins OMP_NUM_THREADS=1; the pageable -> page-locked copies want this rank's share of the cores
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // share))
    # Page-lock the rows outright when all ranks' matrices together are a small part of the host's
    # memory (the 8-GPU split of the headline config on a 1 TB host); otherwise stage.  A single
    # page-locked allocation of 96 GB failed on the 196 GB single-GPU host, 48 GB worked.
    pin = torch.tensor([1 if (nbytes <= (40 << 30) and nbytes * share <= 0.2 * avail) else 0], device=device)
    if world > 1:
        dist.all_reduce(pin, op=dist.ReduceOp.MIN)
    hm = HostMatrix(X, try_pinned=bool(int(pin.item())))
    torch.cuda.synchronize(device)

    def job(k):
        if world == 1:
            sel, eps = coresets_b200.fps_cuda(X, k, return_epsilons=True)
            return sel.cpu(), eps.cpu()
        sel, eps = coresets_b200.fps_sharded(X, k, verbose=False)
        return sel.cpu(), eps

    job(max(W, 2))                               # untimed: library load, allocator, NCCL channels
    X.zero_()
    barrier_sync(device)
    t0 = time.perf_counter()
    hm.upload(X)
    torch.cuda.synchronize(device)
    t1 = time.perf_counter()
    sel, eps = job(K)
    torch.cuda.synchronize(device)
    t2 = time.perf_counter()
    barrier_sync(device)
    load_ms = dist_max(1e3 * (t1 - t0), device)
    total_ms = dist_max(1e3 * (t2 - t0), device)
    k_job = w.k
    par = parity_with_golden(sel, w.name, w.n_rows)
    return {"value": K / (total_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": nbytes * world / K,
            "d2h_bytes_per_step": 12.0, "load_ms": load_ms, "api_call_ms": total_ms - load_ms,
            "api": "coresets_b200.fps_cuda" if world == 1 else "coresets_b200.fps_sharded",
            "host_memory": "page-locked" if hm.pinned else "pageable, staged through eight 64 MiB page-locked buffers",
            "h2d_gb_per_s": nbytes / 1e9 / (load_ms / 1e3), "parity": par,
            "full_job_estimate": {"value": k_job / (load_ms / 1e3 + (total_ms - load_ms) / 1e3 * k_job / K), "unit": UNIT,
                                  "how": f"derived, not measured: the same upload plus the API call's time scaled from {K} to "
                                         f"the config's k={k_job} picks (an upper bound of the time: the first picks are the "
                                         "most expensive ones)"},
            "what": f"one job of {K} picks through the public API (default product mode): host rows -> device "
                    f"({nbytes/1e9:.1f} GB per rank), validation, norms, state, graph capture, {K} picks, read-back of "
                    f"selected / epsilons; wall clock, max over ranks; the whole upload is charged to the {K} picks"}


def run_config(name, args, world, rank, device, K, W):
    """The other benchmark configurations, each on fresh device rows: dense-kernel roofline at the
    configuration's row width, product-mode picks/s, parity with the golden list."""
    from coresets_b200 import engine
    from coresets_b200._native import MODE_DENSE
    from coresets_b200.cuda.multi.layout import compute_shard_layout
    from coresets_b200.synth import WORKLOADS, MixtureSource
    if name == "c5":
        return run_accretion_config(args, world, rank, device)
    w = WORKLOADS[name]
    if name == "c2" and world > 1:
        return {"skipped": "the single-GPU configuration runs at N = 1 only"}
    sizes, offsets = compute_shard_layout(w.n_rows, world)
    n_local, off = sizes[rank], offsets[rank]
    free_b, _ = torch.cuda.mem_get_info(device)
    ok = torch.tensor([1 if n_local * (w.dim * 4 + 12) + (1 << 30) < free_b else 0], device=device)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0:
        return {"skipped": f"{n_local * w.dim * 4 / 1e9:.1f} GB of rows per GPU do not fit beside the state "
                           f"({free_b / 1e9:.1f} GB free)"}
    X = torch.empty((n_local, w.dim), dtype=torch.float32, device=device)
    MixtureSource(w).fill(X, off)
    norms = engine.row_norms(X)
    extra = max(0, 50 - K)
    eng = engine.ShardEngine(X, norms, 1 + W + K + extra + 8, shard_offset=off, world_size=world, mode=MODE_DENSE)
    eng.init_state()
    eng.pick_forced(0)
    ms_total, kern, kern_all, _, _ = dense_leg(eng, K, W, device, extra)
    eng.check_status()
    roof = roofline_of(kern, kern_all, max(sizes), w.dim, device, "tma")
    par = {"dense": parity_with_golden(eng.selected[: 1 + W + K + extra], name, w.n_rows)}
    eng = None
    picks_before = 1 + min(args.prune_picks, w.k // 4)
    prune, peng = prune_leg(X, norms, picks_before + K + 8, off, world, picks_before, K, device, cells=True)
    par["prune"] = parity_with_golden(peng.selected[: picks_before + K], name, w.n_rows)
    peng = None
    return {"workload": f"{w.name}: {w.describe}", "rows": w.n_rows, "dim": w.dim, "k": w.k, "rows_per_gpu": max(sizes),
            "dense": {"value": K / (ms_total / 1e3), "unit": UNIT, "ms_per_step": ms_total / K},
            "roofline": roof, "prune": prune, "parity": par}


def accretion_case(n_rows: int, max_k: int, world: int, rank: int, device) -> dict:
    """One run of the public ``accrete_sharded`` on n_rows anchors + n_rows candidates x 256 with
    CORESETS_FILL_CHUNK=256 CORESETS_BISECT_SEED=1; anchor_order by FPS over the anchors in the run."""
    import coresets_b200
    from coresets_b200.cuda.multi.layout import compute_shard_layout
    from coresets_b200.synth import accretion_sources
    _, _, stacked = accretion_sources(n_rows, n_rows)
    sizes, offsets = compute_shard_layout(2 * n_rows, world)
    knobs = {"CORESETS_FILL_CHUNK": "256", "CORESETS_BISECT_SEED": "1"}
    saved = {k: os.environ.get(k) for k in knobs}
    os.environ.update(knobs)
    try:
        X = stacked.rows(offsets[rank], sizes[rank], device)
        n_anchor_local = max(0, min(n_rows - offsets[rank], sizes[rank]))
        barrier_sync(device)
        t0 = time.perf_counter()
        order, _ = coresets_b200.fps_sharded(X[:n_anchor_local], min(1 << max_k, n_rows), verbose=False)
        torch.cuda.synchronize(device)
        t_order = time.perf_counter() - t0
        barrier_sync(device)
        t0 = time.perf_counter()
        sel = coresets_b200.accrete_sharded(X, order, n_rows, max_k=max_k, verbose=False)
        torch.cuda.synchronize(device)
        barrier_sync(device)
        t_acc = dist_max(time.perf_counter() - t0, device)
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
    out = {"workload": f"{n_rows} anchors + {n_rows} candidates x 256, max_k = {max_k}, knobs {knobs}",
           "rows": 2 * n_rows, "dim": 256, "max_k": max_k, "rows_per_gpu": max(sizes), "n_selected": int(sel.shape[0]),
           "anchor_order_s": t_order, "accrete_sharded_s": t_acc, "value": int(sel.shape[0]) / t_acc, "unit": "committed picks/s"}
    gold = GOLDEN / f"accrete_{n_rows}_{n_rows}_k{max_k}.npz"
    if gold.is_file():
        z = np.load(gold)
        out["parity"] = {"checked": int(z["selected"].shape[0]), "golden": f"tests/golden/{gold.name}",
                         "written_by": f"the reference's accrete_sharded at world size {int(z['world'])}",
                         "equal": bool(np.array_equal(sel.cpu().numpy(), z["selected"].astype(np.int64)))}
    else:
        out["parity"] = {"checked": 0, "equal": None, "why": f"no {gold.name} in tests/golden"}
    return out


def run_accretion_config(args, world, rank, device):
    """The accretion configuration through the public ``accrete_sharded`` (two or more GPUs): wall
    clock to the final layer at full size, and the same call on the largest case for which the
    reference's own list is committed (its run at full size costs more GPU time than a round has)."""
    if world < 2:
        return {"skipped": "the accretion configuration is quoted on 2, 4 and 8 GPUs"}
    if world < 4 and not args.c5_rows:
        # 50 M rows per GPU: several minutes of wall clock for this leg alone; --c5-rows 50000000 runs it
        out = {"skipped": "the full-size run takes part from 4 GPUs on (4 GPUs: 249 s); --c5-rows forces it"}
        out["pinned_case"] = accretion_case(5_000_000, 12, world, rank, device)
        return out
    out = accretion_case(args.c5_rows or 50_000_000, args.c5_max_k, world, rank, device)
    torch.cuda.empty_cache()
    if out["parity"]["equal"] is None:
        out["pinned_case"] = accretion_case(5_000_000, 12, world, rank, device)
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
