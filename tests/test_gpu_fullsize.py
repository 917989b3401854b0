"""Full-size benchmark configurations against the lists the reference's own `fps_sharded` /
`accrete_sharded` wrote on B200s (tests/golden/fullsize_*.npz, accrete_*_k*.npz; generator scripts
tests/golden/make_golden_fullsize.py and make_golden_accrete_fullsize.py).

Farthest-point sampling is chaotic -- one differing bit in an early pick changes every later one --
so a prefix does not pin a run; these tests run the whole k.  The picks do not depend on the
world size, so each test uses every visible GPU (one process per GPU over NCCL) and also runs on a
single one when the rows fit its memory.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.ports import address_in_use, free_port

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"


def _run(script: str, args, world: int, timeout: int, extra_env=None):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    for attempt in range(3):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()), str(ROOT / "tests" / "golden" / script), *args]
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, cwd=str(ROOT), env=env)
        if res.returncode != 0 and address_in_use([res.stdout, res.stderr]) and attempt < 2:
            continue                                   # the rendezvous port was taken: another one
        break
    assert res.returncode == 0, (res.stdout + res.stderr)[-3000:]
    return res.stdout


def _world_for(bytes_total: float) -> int:
    """Largest power-of-two world size the box offers, provided the rows fit."""
    n = torch.cuda.device_count()
    world = 1
    while world * 2 <= min(n, 8):
        world *= 2
    free, _ = torch.cuda.mem_get_info()
    if bytes_total / world * 1.06 + 8e9 > free:
        pytest.skip(f"{bytes_total / world / 1e9:.0f} GB of rows per GPU do not fit {free / 1e9:.0f} GB")
    return world


@pytest.mark.parametrize("config,k_env", [("c2", None), ("c3", None), ("c4", "CORESETS_TEST_C4_PICKS")])
def test_full_size_fps_matches_reference(config, k_env, tmp_path):
    """`fps_sharded` of this package to the configuration's full k (c4: its first 1024 picks unless
    CORESETS_TEST_C4_PICKS says otherwise -- every pick of that configuration reads all 164 GB)
    against `selected` / `epsilons` of the reference's own run."""
    from coresets_b200.synth import WORKLOADS
    gold = GOLDEN / f"fullsize_{config}.npz"
    if not gold.is_file():
        pytest.skip(f"{gold.name} not generated yet")
    w = WORKLOADS[config]
    world = _world_for(w.n_rows * w.dim * 4.0)
    args = ["--config", config, "--out", str(tmp_path), "--skip-reference", "--golden-dir", str(GOLDEN),
            "--exchanges", "nccl,p2p" if world > 1 else "nccl"]
    if k_env:
        args += ["--k", os.environ.get(k_env, "1024")]
    out = _run("make_golden_fullsize.py", args, world, timeout=1500)
    rec = json.loads((tmp_path / f"fullsize_{config}_w{world}.json").read_text())
    for xchg in (["nccl", "p2p"] if world > 1 else ["nccl"]):
        assert rec[f"engine_{xchg}_selected_equal"], (xchg, rec)
        assert rec[f"engine_{xchg}_eps_bits_equal"], (xchg, rec)
    print(out[-600:])


@pytest.mark.parametrize("anchors,max_k", [(2_000_000, 11), (5_000_000, 12)])
def test_accretion_matches_reference(anchors, max_k, tmp_path):
    """`accrete_sharded` (CORESETS_FILL_CHUNK=256 CORESETS_BISECT_SEED=1) on anchors + candidates x 256
    against the reference's list; the 2M case was written on one GPU, the 5M case on two."""
    gold = GOLDEN / f"accrete_{anchors}_{anchors}_k{max_k}.npz"
    if not gold.is_file():
        pytest.skip(f"{gold.name} not generated yet")
    world = _world_for(2 * anchors * 256 * 4.0 * 2.5)
    _run("make_golden_accrete_fullsize.py",
         ["--anchors", str(anchors), "--candidates", str(anchors), "--max-k", str(max_k), "--out", str(tmp_path),
          "--skip-reference", "--golden-dir", str(GOLDEN)], world, timeout=900)
    rec = json.loads((tmp_path / f"accrete_{anchors}_{anchors}_k{max_k}_w{world}.json").read_text())
    assert rec["engine_nccl_equal"], rec
