"""fps_sharded over real NCCL ranks (one process per GPU) against the oracle's emulation of the
reference's sharded driver.  With one visible GPU only the world_size = 1 group is exercised."""
import json
import os
import subprocess
import time
import sys
from pathlib import Path

import pytest
import torch

from tests.ports import address_in_use, free_port

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _launch(world: int, cfg: dict, timeout: int = 420, extra_env=None) -> None:
    for attempt in range(3):
        port = free_port()
        procs = []
        for r in range(world):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r),
                       MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", **(extra_env or {}))
            procs.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "nccl_worker.py"), json.dumps(cfg)],
                                          env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        outs = []
        deadline = time.time() + timeout
        for p in procs:
            try:
                o, _ = p.communicate(timeout=max(1.0, deadline - time.time()))
            except subprocess.TimeoutExpired:
                p.kill()
                o, _ = p.communicate()
                o = (o or "") + "\n[killed after timeout]"
            outs.append(o)
        if any(p.returncode != 0 for p in procs) and address_in_use(outs) and attempt < 2:
            continue                                   # the rendezvous port was taken: another one
        break
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} failed:\n{outs[r][-3000:]}"
    for r in range(world):
        res = json.loads((Path(cfg["out_dir"]) / f"result_{r}.json").read_text())
        assert res["failures"] == [], res["failures"]


def _cases(world: int):
    def split(N, uneven=False, empty=False):
        base = N // world
        sizes = [base] * (world - 1) + [N - base * (world - 1)]
        if empty and world > 1:
            sizes = [0] + [N // (world - 1)] * (world - 2) + [N - (N // (world - 1)) * (world - 2)]
        return sizes
    return [
        dict(N=16383, D=128, k=300, sizes=split(16383)),           # uneven shards (remainder on the last rank)
        dict(N=6000, D=64, k=200, sizes=split(6000), seed=4321),   # seeded first pick
        dict(N=5001, D=256, k=96, sizes=split(5001, empty=True)),  # an empty shard when world > 1
        dict(N=3000, D=50, k=64, sizes=split(3000)),               # D % 4 != 0
        # float16 rows read in place; with the eager knobs below each rank leaves the dense ring for
        # the pruned scan at its own pick count
        dict(N=8000, D=64, k=400, sizes=split(8000), dtype="float16"),
    ]


def test_fps_sharded_nccl_world1(tmp_path):
    _launch(1, dict(cases=_cases(1), out_dir=str(tmp_path)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fps_sharded_nccl_multi(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _launch(world, dict(cases=_cases(world), out_dir=str(tmp_path)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fps_sharded_peer_exchange_multi(tmp_path, world):
    """Same cases with the candidates exchanged by peer stores over NVLink instead of NCCL."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _launch(world, dict(cases=_cases(world), out_dir=str(tmp_path)),
            extra_env={"CORESETS_B200_EXCHANGE": "p2p", "CORESETS_B200_XCHG_TIMEOUT_MS": "5000"})


CELLS_EAGER = {"CORESETS_B200_CELLS_MIN_ROWS": "1", "CORESETS_B200_CELLS_FIRST_BUILD": "3", "CORESETS_B200_CELLS_GROWTH": "1.4",
               "CORESETS_B200_EARLY_DENSE_PICKS": "2", "CORESETS_B200_CELLS_GIVE_UP_SHARE": "2.0",
               "CORESETS_B200_CELLS_PROBE_PICKS": "5", "CORESETS_B200_CELLS_LIVE_GATE": "2.0"}


def test_fps_sharded_cell_index_world1(tmp_path):
    """The cell index inside fps_sharded (tiny indexes, rebuilt often) on a one-rank NCCL group."""
    _launch(1, dict(cases=_cases(1), out_dir=str(tmp_path)), extra_env=CELLS_EAGER)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("xchg", ["nccl", "p2p"])
def test_fps_sharded_cell_index_multi(tmp_path, world, xchg):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _launch(world, dict(cases=_cases(world), out_dir=str(tmp_path)),
            extra_env=dict(CELLS_EAGER, CORESETS_B200_EXCHANGE=xchg, CORESETS_B200_XCHG_TIMEOUT_MS="5000"))


def test_fps_sharded_checkpoint_resume_world1(tmp_path):
    """Checkpoint cadence, file names, and resume to a larger k through the graph-replayed forced
    picks, on a one-rank NCCL group (runs on a single GPU)."""
    _launch(1, dict(mode="resume", N=6000, D=64, k_ck=150, k_full=260, every=40, out_dir=str(tmp_path)))


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("xchg", ["nccl", "p2p"])
def test_fps_sharded_checkpoint_resume_multi(tmp_path, world, xchg):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _launch(world, dict(mode="resume", N=6001, D=128, k_ck=150, k_full=260, every=40, out_dir=str(tmp_path)),
            extra_env={"CORESETS_B200_EXCHANGE": xchg, "CORESETS_B200_XCHG_TIMEOUT_MS": "5000"})
