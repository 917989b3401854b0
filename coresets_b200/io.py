"""Result files: ``selected.npy`` (int64), ``epsilons.npy`` (float32), ``meta.json``.

Byte-compatible with the layout the reference writes in ``save_result`` / ``load_result``
(src/coresets/io.py:40-110): same file names, dtypes, meta keys in the same order, two-space
indented JSON with a trailing newline, every file written to ``<name>.tmp`` and renamed.

Chained runs (src/coresets/io.py:128-490): a run directory holds ``manifest.json`` (target size,
feature width, registered data sources), one ``NNN_<step>`` directory per accretion step with
``coreset.npy`` (int64), optional ``provenance.npy`` (structured ``source_id`` uint16 /
``source_row`` int64), ``step.json`` and an optional ``per_level.tsv``, and a ``LATEST`` file naming
the last successful step.  Same names, key order, number formats and atomic writes.
"""
from __future__ import annotations

import datetime as _dt
import json
import os
import re
import shutil
import subprocess
from dataclasses import dataclass, field
from pathlib import Path
from typing import List, Optional, Sequence, Union

import numpy as np

from ._version import __version__

PathLike = Union[str, os.PathLike]
KNOB_PREFIX = "CORESETS_"
RESULT_SCHEMA = "coresets.result/1"
SCHEMA_VERSION = 1
# one record per coreset entry: which registered source the row came from, and its row there
PROVENANCE_DTYPE = np.dtype([("source_id", np.uint16), ("source_row", np.int64)])


def active_knobs() -> dict:
    """Every set ``CORESETS_*`` environment variable, sorted by name (io.py:31-37)."""
    return {k: os.environ[k] for k in sorted(os.environ) if k.startswith(KNOB_PREFIX)}


def _as_numpy(x) -> np.ndarray:
    return x.detach().cpu().numpy() if hasattr(x, "detach") else np.asarray(x)


def _replace_into(path: Path, writer) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    writer(tmp)
    os.replace(tmp, path)


def _write_npy(path: Path, arr: np.ndarray) -> None:
    def w(tmp: Path) -> None:
        with open(tmp, "wb") as f:  # an open handle keeps numpy from appending ".npy"
            np.save(f, arr, allow_pickle=False)
    _replace_into(path, w)


def _write_json(path: Path, obj: dict) -> None:
    _replace_into(path, lambda tmp: tmp.write_text(json.dumps(obj, indent=2, sort_keys=False) + "\n"))


def _head_commit(where: Path) -> Optional[str]:
    try:
        r = subprocess.run(["git", "rev-parse", "HEAD"], cwd=str(where), capture_output=True,
                           text=True, timeout=2)
    except (FileNotFoundError, subprocess.TimeoutExpired):
        return None
    return r.stdout.strip() if r.returncode == 0 else None


def save_result(
    out_dir: PathLike,
    selected,
    *,
    epsilons=None,
    n_rows: Optional[int] = None,
    dim: Optional[int] = None,
    backend: str = "",
    walltime_s: Optional[float] = None,
    world_size: int = 1,
    extra: Optional[dict] = None,
    overwrite: bool = False,
) -> Path:
    """Write one result directory; refuses to replace an existing ``selected.npy`` unless
    ``overwrite=True`` (``FileExistsError``); shapes are validated with ``ValueError``."""
    out = Path(out_dir)
    sel = np.ascontiguousarray(_as_numpy(selected), dtype=np.int64)
    if sel.ndim != 1:
        raise ValueError(f"selected must be 1-D, got shape {sel.shape}")
    out.mkdir(parents=True, exist_ok=True)
    target = out / "selected.npy"
    if target.exists() and not overwrite:
        raise FileExistsError(f"{target} exists, pass overwrite=True")
    _write_npy(target, sel)

    if epsilons is not None:
        eps = np.asarray(_as_numpy(epsilons), dtype=np.float32)
        if eps.shape != sel.shape:
            raise ValueError(f"epsilons shape {eps.shape} != selected shape {sel.shape}")
        _write_npy(out / "epsilons.npy", eps)

    meta = {
        "schema": RESULT_SCHEMA,
        "K": int(sel.shape[0]),
        "n_rows": None if n_rows is None else int(n_rows),
        "dim": None if dim is None else int(dim),
        "backend": backend,
        "world_size": int(world_size),
        "walltime_s": None if walltime_s is None else float(walltime_s),
        "has_epsilons": epsilons is not None,
        "knobs": active_knobs(),
        "git_commit": _head_commit(Path(__file__).parent),
        "coresets_version": __version__,
        "written_at": _dt.datetime.now(_dt.timezone.utc).isoformat(timespec="seconds"),
    }
    if extra:
        meta.update(extra)
    _write_json(out / "meta.json", meta)
    return out


def load_result(out_dir: PathLike) -> dict:
    """Return ``{"selected", "epsilons" (or None), "meta" (or {})}`` (io.py:99-110)."""
    out = Path(out_dir)
    eps_path, meta_path = out / "epsilons.npy", out / "meta.json"
    return {
        "selected": np.load(out / "selected.npy"),
        "epsilons": np.load(eps_path) if eps_path.is_file() else None,
        "meta": json.loads(meta_path.read_text()) if meta_path.is_file() else {},
    }


# ---- chained runs: manifest, steps, per-level log (src/coresets/io.py:128-490) ------------------
_STEP_NAME = re.compile(r"^(\d{3,})_(.+)$")
_LEVEL_COLUMNS = ("k", "size", "sep", "cov", "rel_gap", "walltime_s")


def _utc_now() -> str:
    return _dt.datetime.now(_dt.timezone.utc).isoformat(timespec="seconds")


def _write_text(path: Path, text: str) -> None:
    _replace_into(path, lambda tmp: tmp.write_text(text))


class _Run:
    """One run directory ``<results_root>/<run_name>``."""

    def __init__(self, results_root: PathLike, run_name: str):
        self.dir = Path(results_root) / run_name
        self.manifest_path = self.dir / "manifest.json"

    def manifest(self) -> dict:
        return json.loads(self.manifest_path.read_text())

    def steps(self) -> List[tuple]:
        """``(index, bare name, directory)`` of every step directory, in name order."""
        found = []
        for p in self.dir.iterdir():
            m = _STEP_NAME.match(p.name) if p.is_dir() else None
            if m:
                found.append((int(m.group(1)), m.group(2), p))
        return sorted(found, key=lambda t: t[2].name)

    def find(self, name: str) -> Path:
        """A step by its directory name, else by its bare name (the last one when re-run)."""
        if (self.dir / name).is_dir():
            return self.dir / name
        hits = [p for _, bare, p in self.steps() if bare == name]
        if not hits:
            raise FileNotFoundError(f"no step matching {name!r} in {self.dir}")
        return hits[-1]


def init_run(results_root: PathLike, run_name: str, *, target_K: int, feature_dim: int,
             description: str = "", overwrite: bool = False) -> Path:
    """Create the run directory with an empty manifest (io.py:162-196); an existing run is kept
    (``FileExistsError``) unless ``overwrite=True`` wipes it."""
    run = _Run(results_root, run_name)
    if run.dir.exists():
        if not overwrite:
            raise FileExistsError(f"run already exists: {run.dir}. Pass overwrite=True to wipe.")
        shutil.rmtree(run.dir)
    run.dir.mkdir(parents=True)
    _write_json(run.manifest_path, {
        "schema_version": SCHEMA_VERSION,
        "run_name": run_name,
        "description": description,
        "target_K": int(target_K),
        "feature_dim": int(feature_dim),
        "data_sources": {},
        "git_commit": _head_commit(Path.cwd()),
        "created_at": _utc_now(),
    })
    return run.dir


def register_source(results_root: PathLike, run_name: str, source_name: str, *, path: Optional[PathLike] = None,
                    n_rows: Optional[int] = None, sha256: Optional[str] = None, extra: Optional[dict] = None) -> int:
    """Id of a data source in the manifest (the uint16 of ``provenance.npy``); a name seen before
    keeps its id, a new one gets the next free id (io.py:198-230)."""
    run = _Run(results_root, run_name)
    manifest = run.manifest()
    sources = manifest["data_sources"]
    if source_name not in sources:
        entry = {"id": 1 + max((int(s["id"]) for s in sources.values()), default=-1),
                 "path": None if path is None else str(path),
                 "n_rows": None if n_rows is None else int(n_rows),
                 "sha256": sha256}
        entry.update(extra or {})
        sources[source_name] = entry
        _write_json(run.manifest_path, manifest)
    return int(sources[source_name]["id"])


def read_manifest(results_root: PathLike, run_name: str) -> dict:
    return _Run(results_root, run_name).manifest()


@dataclass
class StepStats:
    """What ``step.json`` records about a step besides its arrays (io.py:258-269)."""
    max_k: int
    n_anchor: int
    n_candidates: int
    walltime_s: float
    peak_mem_gb: float = 0.0
    max_rel_gap: float = 0.0
    success: bool = True
    parents: Sequence[str] = field(default_factory=tuple)
    candidate_sources: Sequence[str] = field(default_factory=tuple)


def save_step(results_root: PathLike, run_name: str, step_name: str, *, coreset: np.ndarray,
              provenance: Optional[np.ndarray] = None, stats: StepStats, started_at: Optional[str] = None,
              step_idx: Optional[int] = None) -> Path:
    """Write ``NNN_<step_name>/`` (``NNN`` = next free index unless given) and, when the step
    succeeded, point ``LATEST`` at it (io.py:272-341)."""
    if coreset.ndim != 1 or coreset.dtype != np.int64:
        raise ValueError(f"coreset must be 1-D int64; got shape={coreset.shape}, dtype={coreset.dtype}")
    if provenance is not None:
        if provenance.dtype != PROVENANCE_DTYPE:
            raise ValueError(f"provenance must have dtype {PROVENANCE_DTYPE}; got {provenance.dtype}")
        if provenance.shape != coreset.shape:
            raise ValueError(f"provenance shape {provenance.shape} != coreset shape {coreset.shape}")
    run = _Run(results_root, run_name)
    if not run.manifest_path.is_file():
        raise FileNotFoundError(f"no manifest at {run.dir}; call init_run first.")
    if step_idx is None:
        step_idx = 1 + max((idx for idx, _, _ in run.steps()), default=-1)
    step_dir = run.dir / f"{step_idx:03d}_{step_name}"
    step_dir.mkdir(parents=True, exist_ok=True)
    _write_npy(step_dir / "coreset.npy", coreset)
    if provenance is not None:
        _write_npy(step_dir / "provenance.npy", provenance)
    _write_json(step_dir / "step.json", {
        "name": step_name,
        "step_idx": int(step_idx),
        "parents": list(stats.parents),
        "candidate_sources": list(stats.candidate_sources),
        "max_k": int(stats.max_k),
        "n_anchor": int(stats.n_anchor),
        "n_candidates": int(stats.n_candidates),
        "coreset_size": int(coreset.shape[0]),
        "walltime_s": float(stats.walltime_s),
        "peak_mem_gb": float(stats.peak_mem_gb),
        "max_rel_gap": float(stats.max_rel_gap),
        "success": bool(stats.success),
        "started_at": started_at,
        "finished_at": _utc_now(),
    })
    if stats.success:                      # a failed step leaves LATEST where it was
        _write_text(run.dir / "LATEST", step_dir.name + "\n")
    return step_dir


def load_step(results_root: PathLike, run_name: str, step_name_or_dir: str) -> dict:
    """``{"coreset", "provenance" (or None), "meta", "dir"}`` of one step (io.py:353-375)."""
    step_dir = _Run(results_root, run_name).find(step_name_or_dir)
    prov = step_dir / "provenance.npy"
    return {"coreset": np.load(step_dir / "coreset.npy"),
            "provenance": np.load(prov) if prov.is_file() else None,
            "meta": json.loads((step_dir / "step.json").read_text()),
            "dir": step_dir}


def load_latest(results_root: PathLike, run_name: str) -> dict:
    """The step ``LATEST`` names (io.py:378-388)."""
    run = _Run(results_root, run_name)
    marker = run.dir / "LATEST"
    if not marker.is_file():
        raise FileNotFoundError(f"no LATEST at {run.dir}; run has no completed steps")
    return load_step(results_root, run_name, marker.read_text().strip())


def list_steps(results_root: PathLike, run_name: str) -> List[str]:
    """Step directory names, sorted (io.py:391-401)."""
    return [p.name for _, _, p in _Run(results_root, run_name).steps()]


def _level_line(k: int, size: int, sep: float, cov: float, rel_gap: float, walltime_s: float) -> str:
    return f"{k}\t{size}\t{sep:.10g}\t{cov:.10g}\t{rel_gap:.10g}\t{walltime_s:.6f}\n"


class _PerLevelWriter:
    """Line-buffered ``per_level.tsv`` of a step, flushed per row so it can be tailed (io.py:440-470)."""

    def __init__(self, path: Path) -> None:
        self.path = path
        self._fh = open(path, "w", buffering=1)
        self._fh.write("\t".join(_LEVEL_COLUMNS) + "\n")

    def write(self, k: int, size: int, sep: float, cov: float, rel_gap: float, walltime_s: float) -> None:
        self._fh.write(_level_line(k, size, sep, cov, rel_gap, walltime_s))
        self._fh.flush()

    def close(self) -> None:
        if not self._fh.closed:
            self._fh.close()

    def __enter__(self) -> "_PerLevelWriter":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def open_per_level(step_dir: PathLike) -> _PerLevelWriter:
    """Start (truncate) ``<step_dir>/per_level.tsv`` and return its writer (io.py:436-437)."""
    return _PerLevelWriter(Path(step_dir) / "per_level.tsv")


def append_per_level(results_root: PathLike, run_name: str, step_name_or_dir: str, *, k: int, size: int,
                     sep: float, cov: float, rel_gap: float, walltime_s: float) -> None:
    """Append one row to a step's ``per_level.tsv``, writing the header first when the file is new
    (io.py:473-490)."""
    path = _Run(results_root, run_name).find(step_name_or_dir) / "per_level.tsv"
    fresh = not path.is_file()
    with open(path, "a", buffering=1) as fh:
        if fresh:
            fh.write("\t".join(_LEVEL_COLUMNS) + "\n")
        fh.write(_level_line(k, size, sep, cov, rel_gap, walltime_s))
