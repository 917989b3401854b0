"""The allocation-free step entry point, `cs_fps_step_noalloc`, against the regular `cs_fps_step`.

Some hosts of the library cannot allocate device memory while they run (they own the whole HBM
through an arena of their own, or their policy forbids driver allocations on the request path),
so this entry point keeps its scratch in a fixed array inside the library.  The test drives both
entry points through the C ABI from the same starting state, on two picks in a row, and demands
bit-identical `h`, identical `voronoi`, the same arg-max key and the same live-row count.  It is
collected last on purpose and must pass both alone and after every other test.
"""
import numpy as np
import pytest
import torch

from coresets_b200 import _native, engine
from coresets_b200._native import MODE_DENSE, MODE_PRUNE
from tests.data import gaussian_mixture

pytestmark = pytest.mark.gpu


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


@pytest.mark.parametrize("N,D,mode", [(5000, 128, MODE_PRUNE), (3001, 64, MODE_DENSE), (2000, 50, MODE_PRUNE),
                                      (1500, 2048, MODE_PRUNE), (2000, 50, MODE_DENSE)])
def test_noalloc_step_matches_regular_step_twice_in_a_row(N, D, mode):
    dev = torch.device("cuda:0")
    native = _native.get_native()
    X = torch.from_numpy(gaussian_mixture(N, D, 8, seed=N + D)).to(dev)
    norms = engine.row_norms(X)
    eng = engine.ShardEngine(X, norms, 64, mode=mode)
    eng.init_state()
    eng.pick_forced(0)
    eng.run_picks(9)                       # some history so that the bounds prune real rows
    out_key = torch.zeros(1, dtype=torch.int64, device=dev)
    out_live = torch.zeros(1, dtype=torch.int64, device=dev)
    for _ in range(2):                     # two calls in a row share the library's scratch
        eng.exchange()
        eng.commit()                       # centre i and its bounds are now in the engine's tables
        i = eng.read_ctl().n_sel
        h2, v2 = eng.h.clone(), eng.voronoi.clone()
        eng.step()                         # regular entry point on the engine's own buffers
        ctl = eng.read_ctl()
        native.fps_step_noalloc(
            X.data_ptr(), norms.data_ptr(), h2.data_ptr(), v2.data_ptr(), N, D, 0,
            eng.X_sel[i].data_ptr(), float(eng.norms_sel[i].item()),
            eng.dSL.data_ptr() if i > 0 else None, i, mode,
            out_key.data_ptr(), out_live.data_ptr(), _stream(dev))
        torch.cuda.synchronize(dev)
        assert torch.equal(h2.view(torch.int32), eng.h.view(torch.int32))
        assert torch.equal(v2, eng.voronoi)
        assert int(out_key.item()) & 0xFFFFFFFFFFFFFFFF == int(ctl.key[ctl.n_sel & 1])
        assert int(out_live.item()) == int(ctl.live_rows)


def test_noalloc_first_centre_and_size_limit():
    dev = torch.device("cuda:0")
    native = _native.get_native()
    N, D = 1000, 32
    X = torch.from_numpy(gaussian_mixture(N, D, 4, seed=9)).to(dev)
    norms = engine.row_norms(X)
    eng = engine.ShardEngine(X, norms, 4)
    eng.init_state()
    eng.force_pick(7)
    eng.commit()
    h2, v2 = eng.h.clone(), eng.voronoi.clone()
    eng.step()
    key = torch.zeros(1, dtype=torch.int64, device=dev)
    native.fps_step_noalloc(X.data_ptr(), norms.data_ptr(), h2.data_ptr(), v2.data_ptr(), N, D, 0,
                            X[7].data_ptr(), float(norms[7].item()), None, 0, MODE_PRUNE,
                            key.data_ptr(), None, _stream(dev))
    torch.cuda.synchronize(dev)
    assert torch.equal(h2.view(torch.int32), eng.h.view(torch.int32)) and torch.equal(v2, eng.voronoi)
    # wider than the fixed scratch: refused with a clear error, nothing launched
    with pytest.raises(_native.NativeError, match="CS_NOALLOC_MAX_D"):
        native.fps_step_noalloc(X.data_ptr(), norms.data_ptr(), h2.data_ptr(), v2.data_ptr(), 1, 4100, 0,
                                X.data_ptr(), 0.0, None, 0, MODE_PRUNE, key.data_ptr(), None, _stream(dev))
