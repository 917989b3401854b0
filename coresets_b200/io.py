"""Result files: ``selected.npy`` (int64), ``epsilons.npy`` (float32), ``meta.json``.

Byte-compatible with the layout the reference writes in ``save_result`` / ``load_result``
(src/coresets/io.py:40-110): same file names, dtypes, meta keys in the same order, two-space
indented JSON with a trailing newline, every file written to ``<name>.tmp`` and renamed.
The reference's run-manifest / step bookkeeping (io.py:128-490) is outside the accelerated
path and is not part of this module.
"""
from __future__ import annotations

import datetime as _dt
import json
import os
import subprocess
from pathlib import Path
from typing import Optional, Union

import numpy as np

from ._version import __version__

PathLike = Union[str, os.PathLike]
KNOB_PREFIX = "CORESETS_"
RESULT_SCHEMA = "coresets.result/1"


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
