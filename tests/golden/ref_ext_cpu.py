"""Run the REFERENCE's own Python accretion drivers on CPU tensors.

The reference's drivers (src/coresets/cuda/accrete.py, src/coresets/cuda/multi/sharded.py) reach
their kernels through `get_ext()`.  This module provides a stand-in for that extension whose every
function is the CPU oracle's restatement of the corresponding kernel, and patches it into the
reference package, so the reference's control flow (blocks, bisect, reconstruct, replay, fill)
runs unchanged here without a GPU.  Used only by tests/golden/make_golden_accrete_cpu.py to write
fixtures; needs the reference checkout on sys.path.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle  # noqa: E402


def _np(t):
    return t.detach().numpy()


class OracleExt:
    MAX_ARGMAX_BLOCKS = 1024

    # ---- kernels/commit.cu, warp.cu, argmax.cu ------------------------------------------------
    def commit_center_cuda(self, X, norms, X_sel, norms_sel, h_m, voronoi_m, d_out_idx, n_sel):
        i = int(d_out_idx[0])
        norms_sel[n_sel] = norms[i]
        h_m[i] = -1.0
        voronoi_m[i] = n_sel
        X_sel[n_sel] = X[i]

    def fps_update_cuda(self, X, norms, x_new, h, v, norm_new_t, sel_idx):
        if X.shape[0]:
            oracle.fps_update(_np(X), _np(norms), _np(x_new), float(norm_new_t[0]), _np(h), _np(v), sel_idx)

    def voronoi_update_cuda(self, X, norms, x_new, dSL, h, v, norm_new_t, sel_idx):
        if X.shape[0]:
            oracle.voronoi_update(_np(X), _np(norms), _np(x_new), float(norm_new_t[0]), _np(dSL), _np(h), _np(v), sel_idx)

    def compute_dSL_quarter_cuda(self, X_sel, norms_sel, dSL, n_sel):
        if n_sel > 0:
            dSL[:n_sel] = torch.from_numpy(oracle.dsl_quarter(_np(X_sel[: n_sel + 1]), _np(norms_sel[: n_sel + 1]), n_sel))

    def argmax_cuda(self, h, block_vals, block_idxs, d_out_val, d_out_idx, N):
        val, idx = oracle.argmax(_np(h[:N]))
        d_out_val[0] = float(val)
        d_out_idx[0] = idx

    # ---- kernels/simulate.cu ---------------------------------------------------------------------
    def simulate_fps_voronoi(self, X, norms, h_m, voronoi_m, X_sel_init, norms_sel_init, sep, points_left,
                             full_fraction, *scratch):
        ok, steps, _ = oracle.simulate(_np(X), _np(norms), _np(h_m), _np(voronoi_m), _np(X_sel_init),
                                       _np(norms_sel_init), sep, points_left)
        return ok, steps

    # ---- kernels/multi.cu, sharded path ------------------------------------------------------------
    def pack_argmax_with_row_cuda(self, X_local, norms_local, d_out_val, d_out_idx, shard_offset, pack):
        li = int(d_out_idx[0])
        valid = 0 <= li < X_local.shape[0]
        pack[0] = d_out_val[0]
        pack.view(torch.int32)[1] = (li + shard_offset) if valid else -1
        pack[2] = norms_local[li] if valid else 0.0
        pack[3:] = X_local[li] if valid else 0.0

    def fill_pack_with_row_neg_inf_cuda(self, pack, D):
        pack[0] = float("-inf")
        pack.view(torch.int32)[1] = -1
        pack[2:] = 0.0

    def simulate_fps_voronoi_multi_sharded(self, X_local, norms_local, h, v, X_sel, norms_sel, X_sel_init,
                                           norms_sel_init, block_vals, block_idxs, d_out_val, d_out_idx, pack,
                                           gather, dSL, d_sep, d_viable, mask, sep, points_left, shard_offset,
                                           N_shard, world_size, pg):
        """Host loop of multi.cu:428-528 with the all-gather done through torch.distributed."""
        D = X_local.shape[1]
        stride = 3 + D
        n_init = X_sel_init.shape[0]
        sep = np.float32(sep)
        viable = False
        n_sel = n_init

        def gather_local():
            if N_shard > 0:
                self.argmax_cuda(h, None, None, d_out_val, d_out_idx, N_shard)
                self.pack_argmax_with_row_cuda(X_local, norms_local, d_out_val, d_out_idx, shard_offset, pack)
            else:
                self.fill_pack_with_row_neg_inf_cuda(pack, D)
            dist.all_gather_into_tensor(gather, pack)
            return gather.view(world_size, stride)

        for step in range(points_left):
            g = gather_local()
            best_val, best_idx, best_r = np.float32(-np.inf), np.iinfo(np.int64).max, -1
            for r in range(world_size):
                val = np.float32(g[r, 0].item())
                idx = int(g.view(torch.int32)[r, 1].item())
                if val > best_val or (val == best_val and idx < best_idx):
                    best_val, best_idx, best_r = val, idx, r
            if best_idx == np.iinfo(np.int64).max:
                best_idx = -1
            if sep > best_val or best_val <= 0 or best_idx < 0:
                viable = True
            if best_val > 0 and best_val < sep:
                sep = best_val
            if best_idx >= 0 and best_r >= 0:
                norms_sel[n_sel] = g[best_r, 2]
                local = best_idx - shard_offset
                if 0 <= local < N_shard:
                    h[local] = -1.0
                    v[local] = n_sel
                X_sel[n_sel] = g[best_r, 3:]
            if n_sel > 0:
                self.compute_dSL_quarter_cuda(X_sel, norms_sel, dSL, n_sel)
                self.voronoi_update_cuda(X_local, norms_local, X_sel[n_sel], dSL[:n_sel], h, v,
                                         norms_sel[n_sel : n_sel + 1], n_sel)
            else:
                self.fps_update_cuda(X_local, norms_local, X_sel[0], h, v, norms_sel[0:1], 0)
            n_sel += 1
            if (step + 1) % 16 == 0 and viable:
                return True, step + 1
        g = gather_local()
        if sep > np.float32(g[:, 0].max().item()):
            viable = True
        return viable, points_left


def install() -> OracleExt:
    """Patch the stand-in into every reference module that imported the loader by name."""
    import importlib
    ext = OracleExt()
    torch.cuda.mem_get_info = lambda device=None: (1 << 40, 1 << 40)      # resolve_max_k on a CPU box
    for name in ("coresets.cuda.extension", "coresets.cuda.accrete", "coresets.cuda.fps",
                 "coresets.cuda._internal.voronoi_step", "coresets.cuda._internal.bisect",
                 "coresets.cuda.multi.sharded", "coresets.cuda.multi.fps_sharded",
                 "coresets.cuda.multi.replicated"):
        mod = importlib.import_module(name)
        if hasattr(mod, "get_ext"):
            mod.get_ext = lambda: ext
        if hasattr(mod, "ensure_compiled"):
            mod.ensure_compiled = lambda: None
    return ext
