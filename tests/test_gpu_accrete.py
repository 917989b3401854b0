"""Accretion on the GPU against golden lists written by the reference's own CUDA `accrete` /
`accrete_sharded` on a B200 (tests/golden/make_golden_gpu.py), including the per-commit trace."""
import importlib
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _cases():
    from tests.golden.make_golden_gpu import ACCRETE_CASES
    return {n: c for n, c in ACCRETE_CASES.items() if (GOLDEN / f"{n}.npz").is_file()}


def test_accrete_golden_files_present():
    assert len(_cases()) >= 4


@pytest.mark.parametrize("name", ["acc_8192x32_k2048", "acc_16383x128_k1024", "acc_mix_20000x64_k512_fps",
                                  "acc_f16_4000x32_k256"])
def test_accrete_matches_reference(name, tmp_path):
    import coresets_b200
    from tests.golden.make_golden_accrete_cpu import read_trace
    from tests.golden.make_golden_gpu import accrete_case_matrix
    c = _cases()[name]
    z = np.load(GOLDEN / f"{name}.npz")
    X = torch.from_numpy(accrete_case_matrix(c)).cuda()
    na = c["n_anchor"]
    order = torch.from_numpy(z["anchor_order"]).cuda()
    if c["order"] == "fps":   # the anchor ordering itself is the reference's fps_cuda output
        np.testing.assert_array_equal(coresets_b200.fps_cuda(X[:na].contiguous(), na).cpu().numpy(), z["anchor_order"])
    tr = str(tmp_path / "t.tsv")
    got = coresets_b200.accrete(X[:na], X[na:], order, c["max_k"], verbose=False, trace_path=tr)
    assert got.is_cuda and got.dtype == torch.int64
    np.testing.assert_array_equal(got.cpu().numpy(), z["single"])
    mine = read_trace(tr)
    for key in ("trace_phase", "trace_pos", "trace_idx"):
        np.testing.assert_array_equal(mine[key], z[key])
    np.testing.assert_array_equal(mine["trace_val"].view(np.int64), z["trace_val"].view(np.int64))
    np.testing.assert_array_equal(mine["trace_sep"].view(np.int64), z["trace_sep"].view(np.int64))


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_accrete_sharded_matches_reference(tmp_path, world):
    from tests.test_gpu_multi import _launch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _launch(world, dict(mode="accrete", cases=[], out_dir=str(tmp_path)), timeout=1500)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_accrete_sharded_peer_exchange_matches_reference(tmp_path, world):
    from tests.test_gpu_multi import _launch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _launch(world, dict(mode="accrete", cases=[], out_dir=str(tmp_path)), timeout=1500,
            extra_env={"CORESETS_B200_EXCHANGE": "p2p", "CORESETS_B200_XCHG_TIMEOUT_MS": "5000"})


def test_float16_gross_violation_is_reported_like_the_reference():
    """On the clustered-jitter matrix in float16 the reference's own invariant check aborts
    (`accrete`, 6000 x 64, 3000 anchors, max_k = 9, run on a B200): "sep > cov violated at level
    k=9 (size=512): sep=5.66210904e-01, cov=5.69710191e-01, rel_gap=-1.225e-02".  The same input
    must fail here at the same layer with the same numbers (they depend on every bit of h)."""
    import coresets_b200
    from tests.data import as_dtype, clustered_jitter
    X = torch.from_numpy(as_dtype(clustered_jitter(6000, 64, seed=42), "float16")).cuda()
    order = torch.arange(3000, dtype=torch.long, device="cuda")
    with pytest.raises(RuntimeError) as ei:
        coresets_b200.accrete(X[:3000], X[3000:], order, 9, verbose=False)
    msg = str(ei.value)
    assert "accrete: sep > cov violated at level k=9 (size=512)" in msg
    assert "sep=5.66210904e-01, cov=5.69710191e-01, rel_gap=-1.225e-02" in msg
    assert msg.endswith("Gross violation, not float noise.")


def test_accrete_sharded_fused_lanes_match_reference(tmp_path):
    """The one-pass-over-X lanes kernel on the real driver: dense mode routes cs_fps_step_lanes to
    fps_step_lanes_kernel, CORESETS_LANES_MIN_STEPS=1 makes every seeded walk start with lanes; the
    lists must be the ones the reference's accrete_sharded wrote (default knobs and
    CORESETS_BISECT_SEED=1 CORESETS_FILL_CHUNK=256)."""
    from tests.test_gpu_multi import _launch
    _launch(1, dict(mode="accrete", cases=[], out_dir=str(tmp_path)), timeout=1500,
            extra_env={"CORESETS_B200_MODE": "dense", "CORESETS_LANES_MIN_STEPS": "1"})


SIM_CELLS = {"CORESETS_B200_CELLS_SIM_MIN_ROWS": "1", "CORESETS_B200_CELLS_SIM_MIN_STEPS": "1",
             "CORESETS_B200_CELLS_MIN_ROWS": "1", "CORESETS_B200_CELLS_FIRST_BUILD": "3", "CORESETS_B200_CELLS_GROWTH": "1.4",
             "CORESETS_B200_EARLY_DENSE_PICKS": "2", "CORESETS_B200_CELLS_GIVE_UP_SHARE": "2.0",
             "CORESETS_B200_CELLS_PROBE_PICKS": "5", "CORESETS_B200_CELLS_LIVE_GATE": "2.0"}


@pytest.mark.parametrize("name", ["acc_8192x32_k2048", "acc_mix_20000x64_k512_fps"])
def test_accrete_probes_through_the_cell_index(name, tmp_path, monkeypatch):
    """Single-GPU accretion with every bisect probe forced through the cell index (built per probe
    from the reconstructed state, tiny and rebuilt often): lists and traces must stay the reference's."""
    for k, v in SIM_CELLS.items():
        monkeypatch.setenv(k, v)
    test_accrete_matches_reference(name, tmp_path)


def test_accrete_sharded_probes_through_the_cell_index(tmp_path):
    """The sharded driver (default knobs and seeded walk with lanes) with probes on the cell index."""
    from tests.test_gpu_multi import _launch
    _launch(1, dict(mode="accrete", cases=[], out_dir=str(tmp_path)), timeout=1500,
            extra_env=dict(SIM_CELLS, CORESETS_LANES_MIN_STEPS="1"))


@pytest.mark.parametrize("world", [2, 4])
def test_accrete_sharded_probes_through_the_cell_index_multi(tmp_path, world):
    from tests.test_gpu_multi import _launch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _launch(world, dict(mode="accrete", cases=[], out_dir=str(tmp_path)), timeout=1500,
            extra_env=dict(SIM_CELLS, CORESETS_LANES_MIN_STEPS="1"))


@pytest.mark.parametrize("name", ["acc_8192x32_k2048", "acc_mix_20000x64_k512_fps"])
def test_accrete_with_the_forward_walk_on_the_host(name, tmp_path, monkeypatch):
    """The forward walk runs on the device by default (cs_pool_pick + CS_RULE_STOP_NONPOS, replayed
    from graphs); the per-pick host loop it replaces must give the same lists and traces."""
    monkeypatch.setenv("CORESETS_B200_DEVICE_FORWARD", "0")
    test_accrete_matches_reference(name, tmp_path)


def test_restricted_run_stops_when_the_pool_runs_dry():
    """run_restricted on a pool smaller than the request: it commits the pool's rows in greedy
    order, stops by itself, reports `dry`, and leaves the engine usable for free picks."""
    from coresets_b200 import engine
    from tests.data import gaussian_mixture
    X = torch.from_numpy(gaussian_mixture(3000, 32, 6, seed=1)).cuda()
    norms = engine.row_norms(X)
    eng = engine.ShardEngine(X, norms, 64)
    eng.init_state()
    eng.pick_forced(5)
    pool = torch.tensor([10, 11, 12, 5, 2000, 2500], dtype=torch.long, device="cuda")
    made, dry = eng.run_restricted(pool, 4)
    assert (made, dry) == (4, False)
    made2, dry2 = eng.run_restricted(pool, 10)
    assert dry2 and made2 == 1                      # one unselected row was left; row 5 was the seed
    picked = eng.selected[:6].tolist()
    assert picked[0] == 5 and sorted(picked[1:]) == [10, 11, 12, 2000, 2500]
    # greedy order: every pick had the largest h of the rows still unselected in the pool
    ref = engine.ShardEngine(X, norms, 64)
    ref.init_state()
    ref.pick_forced(5)
    left = {10, 11, 12, 2000, 2500}
    for want in picked[1:]:
        h = ref.h.cpu()
        best = max(left, key=lambda r: (float(h[r]), -r))
        assert best == want
        ref.pick_forced(best, float(h[best]))
        left.remove(best)
    assert torch.equal(ref.h.view(torch.int32), eng.h.view(torch.int32))
    eng.scan()
    eng.run_picks(3)
    assert eng.check_status().n_sel == 9
