// Dense mode over IEEE-half rows (CS_F_X_HALF): the bulk-copy ring of step_tma.cuh moving 2 bytes per
// element, with the dot products summed in the reference's element order for half inputs.
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_STEP_TMA_HALF_CUH
#define CORESETS_B200_STEP_TMA_HALF_CUH

namespace {

// The reference's half instantiation widens every element and lets lane l run one fma chain over
// the elements l, l + 32, l + 64, ... before the xor-shuffle tree (_shared.cuh:52-58).  Here a
// stage of the ring holds whole half rows; lane l reads exactly those elements from shared memory
// (32 consecutive halves per warp-wide load, conflict-free) and RB rows are reduced together:
//
// tree_pack combines two rows' partial sums in ONE shuffle of one level of the tree.  Lanes whose
// bit `off` is clear keep row a, the others row b; each receives its partner's value of the row it
// keeps, so a lane holds a[l] + a[l ^ off] or b[l] + b[l ^ off] -- the very addition the tree of a
// single row performs at that level (both partners of the plain tree hold the same sum afterwards,
// so nothing is lost by keeping it in half of the lanes).
__device__ __forceinline__ float tree_pack(const float a, const float b, const int off, const int lane) {
    const bool up = (lane & off) != 0;
    const float keep = up ? b : a, send = up ? a : b;
    return __fadd_rn(keep, __shfl_xor_sync(kFull, send, off));
}

// Sums of RB rows (RB = 2, 4 or 8).  Returns, in EVERY lane, the complete sum of row
// `rowsel(lane)`, where rowsel picks bit 4 of the lane as bit 0 of the row, bit 3 as bit 1, bit 2 as
// bit 2 (as far as RB has bits).
template <int RB>
__device__ __forceinline__ float tree_rows(const float (&acc)[RB], const int lane) {
    float v;
    if (RB == 8) {
        const float a = tree_pack(acc[0], acc[1], 16, lane), b = tree_pack(acc[2], acc[3], 16, lane);
        const float c = tree_pack(acc[4], acc[5], 16, lane), d = tree_pack(acc[6], acc[7], 16, lane);
        const float e = tree_pack(a, b, 8, lane), f = tree_pack(c, d, 8, lane);
        v = tree_pack(e, f, 4, lane);
    } else if (RB == 4) {
        const float a = tree_pack(acc[0], acc[1], 16, lane), b = tree_pack(acc[2], acc[3], 16, lane);
        v = tree_pack(a, b, 8, lane);
        v = __fadd_rn(v, __shfl_xor_sync(kFull, v, 4));
    } else {
        v = tree_pack(acc[0], acc[1], 16, lane);
        v = __fadd_rn(v, __shfl_xor_sync(kFull, v, 8));
        v = __fadd_rn(v, __shfl_xor_sync(kFull, v, 4));
    }
    v = __fadd_rn(v, __shfl_xor_sync(kFull, v, 2));
    v = __fadd_rn(v, __shfl_xor_sync(kFull, v, 1));
    return v;
}
// A lane that holds the sum of row r of a batch (see tree_rows).
template <int RB>
__device__ __forceinline__ int tree_lane_of(const int r) {
    return ((r & 1) << 4) | (((r >> 1) & 1) << 3) | (((r >> 2) & 1) << 2);
}

// d = a * b + c with a and b IEEE halves, rounded once: what __fmaf_rn gives for the widened
// values, without the two conversions.  (No flush-to-zero form exists and none is needed: products
// of halves are multiples of 2^-48, so are all their partial sums, and no subnormal float can appear.)
__device__ __forceinline__ float fma_half(const __half a, const __half b, float c) {
    asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(c) : "h"(__half_as_ushort(a)), "h"(__half_as_ushort(b)));
    return c;
}

// One half from shared memory, by its shared-window address (an explicit ld.shared: the rows reach
// these functions through pointers whose address space the compiler need not know).
__device__ __forceinline__ __half lds_half(const uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __ushort_as_half(v);
}

// Sums of RB rows against the centre: rows_h points at element `lane` of the batch's first row.
// FULL: D == 32 J, no lane is ever out of the row.  MIXED: the centre is exactly representable in
// half (it is whenever it was committed from half rows) and the fma takes both operands as halves;
// otherwise the float centre is re-read from global memory (`cen`, the centre's row of X_sel).
template <int J, int RB, bool FULL, bool MIXED>
__device__ __forceinline__ float batch_rows(const __half* __restrict__ rows_h, const int D, const float* __restrict__ cen,
                                            const __half (&cenh)[J], const int lane) {
    float acc[RB];
    const uint32_t a0 = smem_u32(rows_h), row_bytes = 2u * (uint32_t)D;
#pragma unroll
    for (int b = 0; b < RB; ++b) acc[b] = 0.0f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
        if (FULL || lane + 32 * j < D) {
            __half x[RB];
#pragma unroll
            for (int b = 0; b < RB; ++b) x[b] = lds_half(a0 + (uint32_t)b * row_bytes + 64u * j);
#pragma unroll
            for (int b = 0; b < RB; ++b)
                acc[b] = MIXED ? fma_half(x[b], cenh[j], acc[b]) : __fmaf_rn(__half2float(x[b]), __ldg(cen + lane + 32 * j), acc[b]);
        }
    }
    return tree_rows<RB>(acc, lane);
}

// Wide rows (J > 8): the float centre stays in registers and every element is widened -- a second
// copy of the centre as halves, or a re-read per element, costs more than the conversions
// (2 M x 1024: 0.61 ms this way, 0.80 ms with the half centre spilling out of 96 registers).
template <int J, int RB>
__device__ __forceinline__ float batch_rows_wide(const __half* __restrict__ rows_h, const int D, const float (&cen)[J],
                                                 const int lane) {
    float acc[RB];
    const uint32_t a0 = smem_u32(rows_h), row_bytes = 2u * (uint32_t)D;
#pragma unroll
    for (int b = 0; b < RB; ++b) acc[b] = 0.0f;
#pragma unroll
    for (int j = 0; j < J; ++j) {
        if (lane + 32 * j < D) {
            __half x[RB];
#pragma unroll
            for (int b = 0; b < RB; ++b) x[b] = lds_half(a0 + (uint32_t)b * row_bytes + 64u * j);
#pragma unroll
            for (int b = 0; b < RB; ++b) acc[b] = __fmaf_rn(__half2float(x[b]), cen[j], acc[b]);
        }
    }
    return tree_rows<RB>(acc, lane);
}

// J = elements per lane (D <= 32 J), RB = rows reduced together (rows of a tile per consumer warp is a
// multiple of RB, at most 32), S stages, W consumer warps, B blocks per SM.
template <int J, int RB, int S, int W, int B>
__global__ void __launch_bounds__((W + 1) * 32, B) fps_step_tma_half_kernel(const cs_state s, const int tile_rows) {
    extern __shared__ __align__(128) unsigned char s_tile[];
    __shared__ uint64_t s_full[S], s_empty[S];
    __shared__ u64 s_keys[W];
    __shared__ unsigned s_live[W];
    __shared__ int s_last, s_abort;

    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    if (ctl->halt) return;
    if (i >= s.cap) {
        if (blockIdx.x == 0 && threadIdx.x == 0) ctl->status = ST_CAPACITY;
        return;
    }
    const int D = s.D;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool first = (i == 0);
    const float nn = s.norms_sel[i];
    const int64_t N = s.N_local;
    const int n32 = (int)N;
    const __half* Xh = reinterpret_cast<const __half*>(s.X);
    const int x_bytes = tile_rows * D * 2;                       // D is a multiple of 8: whole 16-byte units
    const int stage_bytes = x_bytes + 3 * tile_rows * 4;
    const unsigned long long pipe_limit_ns =
        (unsigned long long)(s.xchg_timeout_ms > 0 ? s.xchg_timeout_ms : 10000) * 1000000ull;
    const bool stall_for_test = (s.flags & CS_F_TEST_STALL_PIPE) != 0;
    const int ntiles = (int)((N + tile_rows - 1) / tile_rows);
    const int rpw = tile_rows / W;

    if (threadIdx.x == 0) {
        for (int q = 0; q < S; ++q) { mbar_init(&s_full[q], 1); mbar_init(&s_empty[q], W); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    float best_h = __uint_as_float(0xff800000u);
    int best_row = -1;
    unsigned live_cnt = 0;

    int issued = 0;
    if (warp == W) {
        // ---- producer (one lane): keep S tiles in flight; every wait bounded ----------------------
        if (lane == 0) {
            int n = 0;
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++n, issued = n) {
                const int q = n % S;
                if (n >= S && !mbar_wait(&s_empty[q], (uint32_t)((n / S) - 1) & 1u, pipe_limit_ns)) {
                    ctl->status = ST_PIPE_TIMEOUT;
                    s_abort = 1;
                    break;
                }
                if (*(volatile int*)&s_abort || stall_for_test) break;
                const int64_t row0 = (int64_t)t * tile_rows;
                const int rows = (int)((N - row0) < tile_rows ? (N - row0) : tile_rows);
                const int rows4 = rows & ~3;
                unsigned char* st = s_tile + (size_t)q * stage_bytes;
                float* sh = reinterpret_cast<float*>(st + x_bytes);
                int* sv = reinterpret_cast<int*>(sh + tile_rows);
                float* sn = sh + 2 * tile_rows;
                for (int r = rows4; r < rows; ++r) {
                    sh[r] = s.h[row0 + r];
                    sv[r] = s.voronoi[row0 + r];
                    sn[r] = s.norms[row0 + r];
                }
                const uint32_t xb = (uint32_t)rows * (uint32_t)D * 2u, mb = (uint32_t)rows4 * 4u;
                mbar_expect_tx(&s_full[q], xb + 3u * mb);
                bulk_load(st, Xh + row0 * (int64_t)D, xb, &s_full[q]);
                if (mb) {
                    bulk_load(sh, s.h + row0, mb, &s_full[q]);
                    bulk_load(sv, s.voronoi + row0, mb, &s_full[q]);
                    bulk_load(sn, s.norms + row0, mb, &s_full[q]);
                }
            }
        }
    } else {
        // ---- consumers ------------------------------------------------------------------------------
        constexpr bool kNarrow = J <= 8;                     // see batch_rows_wide
        constexpr int JH = kNarrow ? J : 1, JF = kNarrow ? 1 : J;
        const float* cen = s.X_sel + (int64_t)i * D;
        __half cenh[JH];
        float cenf[JF];
        bool exact = true;
        if constexpr (kNarrow) {
#pragma unroll
            for (int j = 0; j < J; ++j) {
                const float c = (lane + 32 * j < D) ? cen[lane + 32 * j] : 0.0f;
                cenh[j] = __float2half_rn(c);
                exact = exact && (__half2float(cenh[j]) == c);
            }
            cenf[0] = 0.0f;
        } else {
#pragma unroll
            for (int j = 0; j < J; ++j) cenf[j] = (lane + 32 * j < D) ? cen[lane + 32 * j] : 0.0f;
            cenh[0] = __float2half_rn(0.0f);
        }
        // the same centre in every warp of every block: one verdict for the whole launch
        const bool mixed = __all_sync(kFull, exact);
        const bool full = (D == 32 * J);
        int n = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++n) {
            const int q = n % S;
            if (!__all_sync(kFull, mbar_wait(&s_full[q], (uint32_t)(n / S) & 1u, pipe_limit_ns))) {
                if (lane == 0) { ctl->status = ST_PIPE_TIMEOUT; s_abort = 1; }
                break;
            }
            const unsigned char* st = s_tile + (size_t)q * stage_bytes;
            const float* sh = reinterpret_cast<const float*>(st + x_bytes);
            const int* sv = reinterpret_cast<const int*>(sh + tile_rows);
            const float* sn = sh + 2 * tile_rows;
            const int slot_row = warp * rpw + lane;              // lane j < rpw owns this row of the tile
            const int row = t * tile_rows + slot_row;
            const bool valid = lane < rpw && row < n32;
            float hq = valid ? sh[slot_row] : __uint_as_float(0xff800000u);
            const bool live = !(hq < 0.0f) && valid;
            float bound = 0.0f, nrow = 0.0f;
            if (live) {
                if (!first) bound = __ldg(s.dSL_quarter + sv[slot_row]);
                nrow = sn[slot_row];
            }
            const unsigned m = __ballot_sync(kFull, live);
            // the statistic counts the rows the reference's test would have evaluated (warp.cu:80-82):
            // the host leaves this kernel for the pruned scan once that share is small
            live_cnt += __popc(__ballot_sync(kFull, live && (first || !(bound >= hq))));
            const __half* rows_h = reinterpret_cast<const __half*>(st) + (size_t)(warp * rpw) * D + lane;
            float mydot = 0.0f;
            // RB rows at a time, dead ones included (their sums are dropped): no branch inside a batch.
            // A row of the tile that lies beyond N holds what an earlier tile left there; it is read
            // and never used.
            for (int base = 0; base < rpw; base += RB) {
                if (((m >> base) & ((1u << RB) - 1u)) == 0u) continue;
                const __half* bh = rows_h + (size_t)base * D;
                float v;
                if constexpr (kNarrow) {
                    if (!mixed) v = batch_rows<J, RB, false, false>(bh, D, cen, cenh, lane);
                    else if (full) v = batch_rows<J, RB, true, true>(bh, D, cen, cenh, lane);
                    else v = batch_rows<J, RB, false, true>(bh, D, cen, cenh, lane);
                } else {
                    v = batch_rows_wide<J, RB>(bh, D, cenf, lane);
                }
                const int r = lane - base;
                const float mine = __shfl_sync(kFull, v, tree_lane_of<RB>(r & (RB - 1)));
                if (r >= 0 && r < RB) mydot = mine;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[q]);
            if (live && (first || !(bound >= hq))) {
                const float d = sq_dist(nrow, nn, mydot);
                if (d < hq) {
                    hq = d;
                    s.h[row] = d;
                    s.voronoi[row] = i;
                }
            }
            if (hq > best_h) { best_h = hq; best_row = row; }
        }
    }

    u64 best = best_row >= 0 ? make_key(best_h, s.shard_offset + best_row) : 0;
    best = warp_max_key(best);
    if (lane == 0 && warp < W) { s_keys[warp] = best; s_live[warp] = live_cnt; }
    __syncthreads();
    if (s_abort && warp == W && lane == 0) {
        // a wait ran out: let the copies still in flight land before the shared memory is released
        for (int q = 0; q < S && q < issued; ++q)
            (void)mbar_wait(&s_full[q], (uint32_t)((issued - 1 - q) / S) & 1u, pipe_limit_ns);
    }
    const int slot = (i + 1) & 1;
    if (threadIdx.x == 0) {
        u64 bk = 0;
        unsigned lv = 0;
#pragma unroll
        for (int w = 0; w < W; ++w) { bk = s_keys[w] > bk ? s_keys[w] : bk; lv += s_live[w]; }
        if (bk) atomicMax(&ctl->key[slot], bk);
        if (lv) atomicAdd(&ctl->live_rows, (u64)lv);
        __threadfence();
        s_last = (atomicAdd(&ctl->ticket, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const u64 k = *reinterpret_cast<volatile u64*>(&ctl->key[slot]);
    if (s.world_size > 1) publish_candidate(s, ctl, k, key_idx(k) - s.shard_offset);
    if (threadIdx.x == 0) {
        ctl->ticket = 0;
        ctl->n_sel = i + 1;
    }
}

}  // namespace

#endif  // CORESETS_B200_STEP_TMA_HALF_CUH
