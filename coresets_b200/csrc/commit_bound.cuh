// Kernel A of a pick: resolve the winner, commit it as the next centre, compute the triangle bounds.
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_COMMIT_BOUND_CUH
#define CORESETS_B200_COMMIT_BOUND_CUH

namespace {

// ---- kernel A: resolve + commit + triangle bounds ------------------------------------------
__global__ void __launch_bounds__(kThreads) commit_bound_kernel(const cs_state s, const unsigned rules) {
    pdl_enter();
    extern __shared__ __align__(16) float s_cen[];
    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    if (ctl->halt) return;                                 // a restricted run that ran dry
    if (i >= s.cap) {
        if (blockIdx.x == 0 && threadIdx.x == 0) ctl->status = ST_CAPACITY;
        return;
    }
    const uint32_t* packs = await_candidates(s, ctl);
    const Winner w = resolve_winner(s, ctl, i, packs);
    const float val = key_val(w.key);
    const int64_t gidx = key_idx(w.key);
    const int D = s.D;
    if (rules == CS_RULE_STOP_NONPOS && (gidx < 0 || val <= 0.0f)) {
        // every block reaches the same verdict from the same candidates; nothing is committed
        if (blockIdx.x == 0 && threadIdx.x == 0) ctl->halt = 1;
        return;
    }

    if (blockIdx.x == 0) {
        if (threadIdx.x == 0) {
            if (s.selected) s.selected[i] = gidx;
            if (s.eps) s.eps[i] = val;
            ctl->last_val = val;
            ctl->last_idx = (int)gidx;
            ctl->key[(i + 1) & 1] = 0;     // slot the coming step kernel reduces into
            ctl->live_rows = 0;
            if (rules == CS_RULE_SIM_SINGLE) {            // commit.cu:41-51
                float sep = ctl->sep;
                if (sep > val) ctl->viable = 1;
                if (val < sep) ctl->sep = val;
                ctl->steps += 1;
            } else if (rules == CS_RULE_SIM_SHARDED) {    // multi.cu:331-340
                float sep = ctl->sep;
                if (sep > val || val <= 0.0f || gidx < 0) ctl->viable = 1;
                if (val > 0.0f && val < sep) ctl->sep = val;
                ctl->steps += 1;
            }
            if (gidx >= 0) {
                s.norms_sel[i] = w.norm;
                int64_t l = gidx - s.shard_offset;
                if (l >= 0 && l < s.N_local) {            // owner marks the row (commit.cu:16-18)
                    s.h[l] = -1.0f;
                    s.voronoi[l] = i;
                }
            }
        }
        if (gidx >= 0) {
            float* dst = s.X_sel + (int64_t)i * D;
            for (int c = threadIdx.x; c < D; c += blockDim.x) dst[c] = winner_elem(s, w, c);
        }
    }
    if (gidx < 0 || i == 0) return;

    // dSL_quarter[v] = |X_sel[v] - x_new|^2 / 4 for every old centre (commit.cu:69-102)
    for (int c = threadIdx.x; c < D; c += blockDim.x) s_cen[c] = winner_elem(s, w, c);
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int nw = gridDim.x * kWarps;
    for (int v = gw; v < i; v += nw) {
        float dot = warp_dot_generic(s.X_sel + (int64_t)v * D, s_cen, D, lane, (s.flags & CS_F_ELEMENT_ORDER) != 0);
        if (lane == 0) s.dSL_quarter[v] = __fmul_rn(sq_dist(s.norms_sel[v], w.norm, dot), 0.25f);
    }
}

}  // namespace

#endif  // CORESETS_B200_COMMIT_BOUND_CUH
