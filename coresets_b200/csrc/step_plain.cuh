// Kernel B with plain loads: fused distance, min-update and arg-max (inline prune walk, dense with 128-bit loads, any row width).
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_STEP_PLAIN_CUH
#define CORESETS_B200_STEP_PLAIN_CUH

namespace {

// ---- kernel B: fused distance + min-update + arg-max ---------------------------------------
// A warp owns super-tiles of 128 consecutive rows: lane j holds h / voronoi of rows base+4j..4j+3
// (one 16-byte load each, coalesced), the warp then walks the rows that need a distance, RB rows
// per batch so that RB * CPL 16-byte loads per lane are in flight, every row read with one fully coalesced
// 512-byte (or wider) request.  CPL = float4 chunks per lane = ceil(D / 128); CPL == 0 is the
// generic path (any D, centre in shared memory).
// Rows of at most 64 floats (d4 <= 16) fill only half of a warp-wide request in the reference's lane
// mapping.  Here the two half-warps take two different rows at once: lanes 0-15 row A, lanes
// 16-31 row B.  The reference's tree adds p[j+16] (always 0 for such rows) at its first level and
// then reduces within 16 lanes; the same is done per half-warp, so every bit is kept.
__device__ __forceinline__ void tile_rows_half(const float4* __restrict__ X4, const int64_t base, const int d4,
                                               unsigned m, const float4 cen_h, const int lane, float& mydot) {
    constexpr int PB = kInflight;            // row PAIRS whose loads are in flight together
    const int sub = lane & 15;
    const bool hi = lane >= 16;
    while (m) {
        int ra[PB], rb[PB];
        float4 a[PB];
#pragma unroll
        for (int b = 0; b < PB; ++b) {
            ra[b] = m ? (__ffs(m) - 1) : -1;
            m &= m - 1;
            rb[b] = m ? (__ffs(m) - 1) : -1;
            m &= m - 1;
        }
#pragma unroll
        for (int b = 0; b < PB; ++b) {
            const int r = hi ? rb[b] : ra[b];
            if (r >= 0 && sub < d4) a[b] = ld_stream4(X4 + (base + (int64_t)r * kRowsPerLane) * (int64_t)d4 + sub);
        }
#pragma unroll
        for (int b = 0; b < PB; ++b) {
            if (ra[b] < 0) continue;                       // warp-uniform
            const int r = hi ? rb[b] : ra[b];
            float p = 0.0f;
            if (r >= 0 && sub < d4) p = __fadd_rn(p, chunk_dot(a[b], cen_h));
            p = __fadd_rn(p, 0.0f);                        // level 16 of the tree: the partner lane holds 0
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) p = __fadd_rn(p, __shfl_xor_sync(kFull, p, off));
            const float pa = __shfl_sync(kFull, p, 0), pb = __shfl_sync(kFull, p, 16);
            if (lane == ra[b]) mydot = pa;
            if (lane == rb[b]) mydot = pb;
        }
    }
}

template <int CPL, bool FULL>
__device__ __forceinline__ void tile_rows(const float4* __restrict__ X4, const int64_t base,
                                          const int d4, unsigned m, const float4 (&cen)[CPL ? CPL : 1],
                                          const int lane, float& mydot) {
    // bit r of m stands for row base + kRowsPerLane * r (lane r's sub-row)
    constexpr int RB = CPL >= kInflight ? 1 : (kInflight / (CPL ? CPL : 1));
    while (m) {
        int rows[RB];
        float4 a[RB][CPL ? CPL : 1];
#pragma unroll
        for (int b = 0; b < RB; ++b) {
            rows[b] = m ? (__ffs(m) - 1) : -1;
            m &= m - 1;                       // m == 0 stays 0
        }
#pragma unroll
        for (int b = 0; b < RB; ++b) {
            if (rows[b] >= 0) {
                const float4* rp = X4 + (base + (int64_t)rows[b] * kRowsPerLane) * (int64_t)d4 + lane;
#pragma unroll
                for (int c = 0; c < CPL; ++c)
                    if (FULL || lane + 32 * c < d4) a[b][c] = ld_stream4(rp + 32 * c);
            }
        }
#pragma unroll
        for (int b = 0; b < RB; ++b) {
            if (rows[b] >= 0) {
                float p = 0.0f;
#pragma unroll
                for (int c = 0; c < CPL; ++c)
                    if (FULL || lane + 32 * c < d4) p = __fadd_rn(p, chunk_dot(a[b][c], cen[c]));
                p = warp_tree_sum(p);
                if (lane == rows[b]) mydot = p;
            }
        }
    }
}

template <int CPL, bool FULL, bool HALF>
__global__ void __launch_bounds__(kThreads, CS_MIN_BLOCKS) fps_step_kernel(const cs_state s, const unsigned mode,
                                                                           const int n_bound_smem) {
    pdl_enter();
    // dynamic shared memory: the first n_bound_smem triangle bounds (the per-row bound lookup is
    // then a shared-memory read instead of an L2 round trip), then the centre on the generic path
    extern __shared__ __align__(16) float s_dyn[];
    float* s_dsl = s_dyn;
    float* s_cen = s_dyn + ((n_bound_smem + 3) & ~3);            // 16-byte aligned: read as float4 chunks
    __shared__ u64 s_keys[kWarps];
    __shared__ unsigned s_live[kWarps];
    __shared__ int s_last;

    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    if (ctl->halt) return;                                       // a restricted run that ran dry
    if (i >= s.cap) {
        if (blockIdx.x == 0 && threadIdx.x == 0) ctl->status = ST_CAPACITY;
        return;
    }
    const int D = s.D;
    const bool element_order = (s.flags & CS_F_ELEMENT_ORDER) != 0;   // generic path only
    const int d4 = D >> 2;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const bool first = (i == 0);                 // slot 0 uses the dense kernel (voronoi_step.py:40-43)
    const bool dense = (mode & CS_MODE_DENSE) != 0;
    const float nn = s.norms_sel[i];
    const float* cen_g = s.X_sel + (int64_t)i * D;

    float4 cen[CPL ? CPL : 1];
    if (CPL) {
        const float4* c4 = reinterpret_cast<const float4*>(cen_g);
#pragma unroll
        for (int c = 0; c < (CPL ? CPL : 1); ++c)
            cen[c] = (FULL || lane + 32 * c < d4) ? c4[lane + 32 * c] : make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        for (int c = threadIdx.x; c < D; c += blockDim.x) s_cen[c] = cen_g[c];
    }
    float4 cen_h = make_float4(0.f, 0.f, 0.f, 0.f);      // half-warp mapping: chunk (lane & 15)
    if (HALF && (lane & 15) < d4) cen_h = reinterpret_cast<const float4*>(cen_g)[lane & 15];
    const int nb = i < n_bound_smem ? i : n_bound_smem;
    for (int c = threadIdx.x; c < nb; c += blockDim.x) s_dsl[c] = s.dSL_quarter[c];
    __syncthreads();

    const int64_t N = s.N_local;
    constexpr int R = kRowsPerLane;
    const int n32 = (int)N;                                  // local rows fit 31 bits (validated)
    const int tiles = (int)((N + (32 * R - 1)) >> kTileShift);
    const int whole_tiles = (int)(N >> kTileShift);          // super-tiles whose rows all exist
    const int nw = (int)gridDim.x * kWarps;
    const float4* X4 = reinterpret_cast<const float4*>(s.X);
    const bool vec_ok = ((((uintptr_t)s.h) | ((uintptr_t)s.voronoi) | ((uintptr_t)s.norms)) & 15u) == 0;
    const float kNegInf = __uint_as_float(0xff800000u);
    // Per-lane running arg-max as (value, local row); the 64-bit key is built once at the end.
    // NaN never wins (comparisons are false), -0.0 == +0.0, as in argmax_better.
    float best_h = kNegInf;
    int best_row = -1;
    unsigned live_cnt = 0;

    // ---- full treatment of one super-tile: predicate, row walk, update, arg-max ---------------
    // Lane j owns rows r0 .. r0+R-1 (one vector load each for h and voronoi, coalesced).  Rows
    // past the end read as -inf: not live, never above the running maximum.
    auto full_tile = [&](const int t) {
        const int r0 = (t << kTileShift) + R * lane;
        float hq[R];
        int vq[R];
        if (vec_ok && t < whole_tiles) {
            if (R == 4) {
                const float4 a = *reinterpret_cast<const float4*>(s.h + r0);
                hq[0] = a.x; hq[1] = a.y; hq[R - 2] = a.z; hq[R - 1] = a.w;
                if (!first) {
                    const int4 b = *reinterpret_cast<const int4*>(s.voronoi + r0);
                    vq[0] = b.x; vq[1] = b.y; vq[R - 2] = b.z; vq[R - 1] = b.w;
                }
            } else {
                const float2 a = *reinterpret_cast<const float2*>(s.h + r0);
                hq[0] = a.x; hq[1] = a.y;
                if (!first) {
                    const int2 b = *reinterpret_cast<const int2*>(s.voronoi + r0);
                    vq[0] = b.x; vq[1] = b.y;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < R; ++j) {
                const bool in = r0 + j < n32;
                hq[j] = in ? s.h[r0 + j] : kNegInf;
                vq[j] = (in && !first) ? s.voronoi[r0 + j] : 0;
            }
        }
        bool up[R], need[R];
        bool any_need = false;
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const bool live = !(hq[j] < 0.0f);                             // warp.cu:28-30, 75-77
            up[j] = live;
            if (!first && live) {
                const float b = (vq[j] < nb) ? s_dsl[vq[j]] : __ldg(s.dSL_quarter + vq[j]);
                up[j] = !(b >= hq[j]);                                     // warp.cu:80-82
            }
            need[j] = dense ? live : up[j];
            any_need |= need[j];
        }
        if (__any_sync(kFull, any_need)) {                   // most super-tiles need nothing in prune mode
        const int64_t base = (int64_t)t << kTileShift;
        float dots[R];
#pragma unroll
        for (int j = 0; j < R; ++j) dots[j] = 0.0f;
#pragma unroll 1
        for (int j = 0; j < R; ++j) {        // one copy of the row walk, not R (register budget)
            bool nj = need[0];
#pragma unroll
            for (int q = 1; q < R; ++q) nj = (j == q) ? need[q] : nj;
            const unsigned mj = __ballot_sync(kFull, nj);
            if (!mj) continue;
            live_cnt += __popc(mj);
            float dj = 0.0f;
            if (CPL) {
                if (HALF) tile_rows_half(X4, base + j, d4, mj, cen_h, lane, dj);
                else tile_rows<CPL, FULL>(X4, base + j, d4, mj, cen, lane, dj);
            } else {
                unsigned mm = mj;
                while (mm) {
                    const int r = __ffs(mm) - 1;
                    mm &= mm - 1;
                    const int64_t xr = base + j + (int64_t)r * kRowsPerLane;
                    float p = (s.flags & CS_F_X_HALF)
                                  ? warp_dot_half(reinterpret_cast<const __half*>(s.X) + xr * (int64_t)D, s_cen, D, lane)
                                  : warp_dot_generic(s.X + xr * (int64_t)D, s_cen, D, lane, element_order);
                    if (lane == r) dj = p;
                }
            }
#pragma unroll
            for (int q = 0; q < R; ++q) dots[q] = (j == q) ? dj : dots[q];
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
            if (up[j]) {
                const float d = sq_dist(__ldg(s.norms + r0 + j), nn, dots[j]);
                if (d < hq[j]) {
                    hq[j] = d;
                    s.h[r0 + j] = d;
                    s.voronoi[r0 + j] = i;
                }
            }
        }
        }
        // running arg-max: a lane meets its rows in increasing order, so a strict '>' keeps the
        // smallest row among equal values; the row is resolved only on improvement
        float tmax = hq[0];
#pragma unroll
        for (int j = 1; j < R; ++j) tmax = fmaxf(tmax, hq[j]);
        if (tmax > best_h) {
            best_h = tmax;
#pragma unroll
            for (int j = R - 1; j >= 0; --j) best_row = (hq[j] == tmax) ? r0 + j : best_row;
        }
    };

    for (int t = (int)blockIdx.x * kWarps + warp; t < tiles; t += nw) full_tile(t);
    u64 best = best_row >= 0 ? make_key(best_h, s.shard_offset + best_row) : 0;

    best = warp_max_key(best);
    if (lane == 0) { s_keys[warp] = best; s_live[warp] = live_cnt; }
    __syncthreads();
    const int slot = (i + 1) & 1;
    if (threadIdx.x == 0) {
        u64 bk = 0;
        unsigned lv = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) { bk = s_keys[w] > bk ? s_keys[w] : bk; lv += s_live[w]; }
        if (bk) atomicMax(&ctl->key[slot], bk);
        if (lv) atomicAdd(&ctl->live_rows, (u64)lv);
        __threadfence();
        const unsigned tk = atomicAdd(&ctl->ticket, 1u);
        s_last = (tk == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;

    // last block to finish: publish this rank's candidate and advance the pick counter
    __threadfence();
    const u64 k = *reinterpret_cast<volatile u64*>(&ctl->key[slot]);
    if (s.world_size > 1) publish_candidate(s, ctl, k, key_idx(k) - s.shard_offset);
    if (threadIdx.x == 0) {
        ctl->ticket = 0;
        ctl->n_sel = i + 1;
    }
}

}  // namespace

#endif  // CORESETS_B200_STEP_PLAIN_CUH
