// Kernel B for several states that share one pass over X (bisect probes).
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_STEP_LANES_CUH
#define CORESETS_B200_STEP_LANES_CUH

namespace {

// ---- several probes in one pass over X ("lanes") ------------------------------------------------
// L independent states (own h, voronoi, centre table, control block) share X and norms.  A warp
// owns tiles of 32 consecutive rows; lane j of the warp holds, for every state, h / voronoi of row
// base + j and that state's predicate.  A row is loaded ONCE if any state needs its distance and
// is dotted with every interested state's centre (centres in shared memory), with exactly the
// arithmetic of fps_step_kernel, so every state ends bit-identical to a separate cs_fps_step.
struct LaneSet {
    cs_state s[CS_MAX_LANES];
};

template <int L, int CPL>
__global__ void __launch_bounds__(kThreads, 2) fps_step_lanes_kernel(const LaneSet ls, const unsigned mode) {
    extern __shared__ __align__(16) float s_cen[];           // [L][D]
    __shared__ u64 s_keys[L][kWarps];
    __shared__ int s_last;
    const int D = ls.s[0].D;
    const int d4 = D >> 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool dense = (mode & CS_MODE_DENSE) != 0;

    Ctl* ctl[L];
    int pick[L];
    float nn[L];
    bool on[L];
#pragma unroll
    for (int l = 0; l < L; ++l) {
        ctl[l] = reinterpret_cast<Ctl*>(ls.s[l].ctl);
        pick[l] = ctl[l]->n_sel;
        on[l] = pick[l] < ls.s[l].cap;
        if (!on[l] && blockIdx.x == 0 && threadIdx.x == 0) ctl[l]->status = ST_CAPACITY;
        nn[l] = on[l] ? ls.s[l].norms_sel[pick[l]] : 0.0f;
        if (on[l]) {
            const float* cg = ls.s[l].X_sel + (int64_t)pick[l] * D;
            for (int c = threadIdx.x; c < D; c += blockDim.x) s_cen[l * D + c] = cg[c];
        }
    }
    __syncthreads();

    const int64_t N = ls.s[0].N_local;
    const int n32 = (int)N;
    const int tiles = (int)((N + 31) >> 5);
    const int nw = (int)gridDim.x * kWarps;
    const float4* X4 = reinterpret_cast<const float4*>(ls.s[0].X);
    const float* norms = ls.s[0].norms;
    const float kNegInf = __uint_as_float(0xff800000u);
    float best_h[L];
    int best_row[L];
#pragma unroll
    for (int l = 0; l < L; ++l) { best_h[l] = kNegInf; best_row[l] = -1; }

    for (int t = (int)blockIdx.x * kWarps + warp; t < tiles; t += nw) {
        const int row = (t << 5) + lane;
        const bool valid = row < n32;
        float hq[L];
        bool up[L];
        unsigned m[L];
        unsigned uni = 0;
#pragma unroll
        for (int l = 0; l < L; ++l) {
            hq[l] = (valid && on[l]) ? ls.s[l].h[row] : kNegInf;
            const bool live = !(hq[l] < 0.0f);                              // warp.cu:28-30, 75-77
            up[l] = live;
            if (live && pick[l] > 0) {
                const int v = ls.s[l].voronoi[row];
                up[l] = !(__ldg(ls.s[l].dSL_quarter + v) >= hq[l]);         // warp.cu:80-82
            }
            m[l] = __ballot_sync(kFull, dense ? live : up[l]);
            uni |= m[l];
        }
        float dots[L];
#pragma unroll
        for (int l = 0; l < L; ++l) dots[l] = 0.0f;
        constexpr int RB = CPL >= 4 ? 1 : (4 / CPL);        // rows whose loads are in flight together
        while (uni) {
            int rows[RB];
            float4 a[RB][CPL];
#pragma unroll
            for (int b = 0; b < RB; ++b) {
                rows[b] = uni ? (__ffs(uni) - 1) : -1;
                uni &= uni - 1;
            }
#pragma unroll
            for (int b = 0; b < RB; ++b) {
                if (rows[b] >= 0) {
                    const float4* rp = X4 + ((int64_t)(t << 5) + rows[b]) * (int64_t)d4 + lane;
#pragma unroll
                    for (int c = 0; c < CPL; ++c)
                        if (lane + 32 * c < d4) a[b][c] = ld_stream4(rp + 32 * c);
                }
            }
#pragma unroll
            for (int b = 0; b < RB; ++b) {
                if (rows[b] < 0) continue;
#pragma unroll
                for (int l = 0; l < L; ++l) {
                    if (!((m[l] >> rows[b]) & 1u)) continue;                // warp-uniform
                    const float4* c4 = reinterpret_cast<const float4*>(s_cen + l * D);
                    float p = 0.0f;
#pragma unroll
                    for (int c = 0; c < CPL; ++c)
                        if (lane + 32 * c < d4) p = __fadd_rn(p, chunk_dot(a[b][c], c4[lane + 32 * c]));
                    p = warp_tree_sum(p);
                    if (lane == rows[b]) dots[l] = p;
                }
            }
        }
        const float nrow = valid ? __ldg(norms + row) : 0.0f;
#pragma unroll
        for (int l = 0; l < L; ++l) {
            if (up[l]) {
                const float d = sq_dist(nrow, nn[l], dots[l]);
                if (d < hq[l]) {
                    hq[l] = d;
                    ls.s[l].h[row] = d;
                    ls.s[l].voronoi[row] = pick[l];
                }
            }
            if (hq[l] > best_h[l]) { best_h[l] = hq[l]; best_row[l] = row; }   // rows come in order
        }
    }

#pragma unroll
    for (int l = 0; l < L; ++l) {
        u64 k = best_row[l] >= 0 ? make_key(best_h[l], ls.s[l].shard_offset + best_row[l]) : 0;
        k = warp_max_key(k);
        if (lane == 0) s_keys[l][warp] = k;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int l = 0; l < L; ++l) {
            u64 bk = 0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) bk = s_keys[l][w] > bk ? s_keys[l][w] : bk;
            if (bk && on[l]) atomicMax(&ctl[l]->key[(pick[l] + 1) & 1], bk);
        }
        __threadfence();
        s_last = (atomicAdd(&ctl[0]->ticket, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
#pragma unroll
    for (int l = 0; l < L; ++l) {
        if (!on[l]) continue;
        const u64 k = *reinterpret_cast<volatile u64*>(&ctl[l]->key[(pick[l] + 1) & 1]);
        if (ls.s[l].world_size > 1) publish_candidate(ls.s[l], ctl[l], k, key_idx(k) - ls.s[l].shard_offset);
        __syncthreads();
        if (threadIdx.x == 0) ctl[l]->n_sel = pick[l] + 1;
    }
    if (threadIdx.x == 0) ctl[0]->ticket = 0;
}

}  // namespace

#endif  // CORESETS_B200_STEP_LANES_CUH
