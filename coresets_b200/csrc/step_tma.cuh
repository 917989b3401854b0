// Kernel B of dense mode: X, h, voronoi and norms through a cp.async.bulk + mbarrier ring.
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_STEP_TMA_CUH
#define CORESETS_B200_STEP_TMA_CUH

namespace {

// ---- dense mode through the TMA engine -------------------------------------------------------------
// Every live row is read in dense mode, so X can be streamed by bulk asynchronous copies
// (cp.async.bulk, the 1-D TMA path: rows are contiguous, no tensor map needed) into a ring of
// shared-memory stages, with the copies of several stages in flight while the consumer warps work:
// memory-level parallelism no longer depends on registers or occupancy.  One producer warp issues
// the copies and arms the "full" mbarriers with the byte count; the consumer warps wait on
// "full", take their rows of the tile from shared memory (512-byte conflict-free reads), run the
// same per-row arithmetic as fps_step_kernel, and release the stage through the "empty" mbarrier.
// Every wait is bounded; a wait that runs out sets status = 4 and the block drains and leaves.
// Ring shapes per row width, found by measurement on B200: one block per SM with 160-200 KB of
// copies in flight; narrow rows need sixteen consumer warps to keep up with the ring.
struct RingCfg { int stages, blocks, tile_bytes, warps; };   // stages, blocks per SM, bytes of X per stage, consumer warps
constexpr RingCfg kRingNarrow{3, 1, 65536, 16};   // D <= 64
constexpr RingCfg kRingMid{3, 1, 65536, 8};       // 64 < D <= 128
constexpr RingCfg kRingWide{5, 1, 40960, 8};      // 128 < D <= 1024
constexpr int kTmaMaxWarps = 16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
// Bounded wait on a phase of an mbarrier: gives up after limit_ns of wall time (checked every 64
// polls) and returns false.
__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, unsigned long long limit_ns) {
    if (mbar_try(b, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int it = 0; it < 64; ++it)
            if (mbar_try(b, parity)) return true;
        if (global_ns() - t0 > limit_ns) return false;
    }
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* b) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(b)) : "memory");
}

template <int CPL, int S, bool HALF, int W, int B>
__global__ void __launch_bounds__((W + 1) * 32, B) fps_step_tma_kernel(const cs_state s, const int tile_rows) {
    // S stages; a stage holds the tile's rows of X, then their h, voronoi and norm words
    extern __shared__ __align__(128) unsigned char s_tile[];
    __shared__ uint64_t s_full[S], s_empty[S];
    __shared__ u64 s_keys[W];
    __shared__ unsigned s_live[W];
    __shared__ int s_last, s_abort;

    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    if (ctl->halt) return;                                       // a restricted run that ran dry
    if (i >= s.cap) {
        if (blockIdx.x == 0 && threadIdx.x == 0) ctl->status = ST_CAPACITY;
        return;
    }
    const int D = s.D, d4 = D >> 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool first = (i == 0);
    const float nn = s.norms_sel[i];
    const int64_t N = s.N_local;
    const int n32 = (int)N;
    const int x_bytes = tile_rows * D * 4;
    const int stage_bytes = x_bytes + 3 * tile_rows * 4;
    const unsigned long long pipe_limit_ns =
        (unsigned long long)(s.xchg_timeout_ms > 0 ? s.xchg_timeout_ms : 10000) * 1000000ull;
    const bool stall_for_test = (s.flags & CS_F_TEST_STALL_PIPE) != 0;   // the producer starts no copy
    const int ntiles = (int)((N + tile_rows - 1) / tile_rows);
    const int rpw = tile_rows / W;                           // rows of a tile per consumer warp (<= 32)

    if (threadIdx.x == 0) {
        for (int q = 0; q < S; ++q) { mbar_init(&s_full[q], 1); mbar_init(&s_empty[q], W); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    float best_h = __uint_as_float(0xff800000u);
    int best_row = -1;
    unsigned live_cnt = 0;

    int issued = 0;                                               // producer: tiles whose copies were started
    if (warp == W) {
        // ---- producer: keep S tiles in flight -----------------------------------------------------
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
                const int rows4 = rows & ~3;                       // a bulk copy moves multiples of 16 bytes
                unsigned char* st = s_tile + (size_t)q * stage_bytes;
                float* sh = reinterpret_cast<float*>(st + x_bytes);
                int* sv = reinterpret_cast<int*>(sh + tile_rows);
                float* sn = sh + 2 * tile_rows;
                for (int r = rows4; r < rows; ++r) {               // the last tile's odd rows, by plain loads
                    sh[r] = s.h[row0 + r];
                    sv[r] = s.voronoi[row0 + r];
                    sn[r] = s.norms[row0 + r];
                }
                const uint32_t xb = (uint32_t)rows * (uint32_t)D * 4u, mb = (uint32_t)rows4 * 4u;
                mbar_expect_tx(&s_full[q], xb + 3u * mb);          // release: the plain stores above are visible
                bulk_load(st, s.X + row0 * (int64_t)D, xb, &s_full[q]);
                if (mb) {
                    bulk_load(sh, s.h + row0, mb, &s_full[q]);
                    bulk_load(sv, s.voronoi + row0, mb, &s_full[q]);
                    bulk_load(sn, s.norms + row0, mb, &s_full[q]);
                }
            }
        }
    } else {
        // ---- consumers ------------------------------------------------------------------------------
        const int sub = HALF ? (lane & 15) : lane;
        const bool hi = HALF && lane >= 16;
        float4 cen[CPL];
        {
            const float4* c4 = reinterpret_cast<const float4*>(s.X_sel + (int64_t)i * D);
#pragma unroll
            for (int c = 0; c < CPL; ++c)
                cen[c] = (sub + 32 * c < d4) ? c4[sub + 32 * c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        int n = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++n) {
            const int q = n % S;
            if (!__all_sync(kFull, mbar_wait(&s_full[q], (uint32_t)(n / S) & 1u, pipe_limit_ns))) {   // warp-uniform verdict
                if (lane == 0) { ctl->status = ST_PIPE_TIMEOUT; s_abort = 1; }
                break;
            }
            const unsigned char* st = s_tile + (size_t)q * stage_bytes;
            const float* sh = reinterpret_cast<const float*>(st + x_bytes);
            const int* sv = reinterpret_cast<const int*>(sh + tile_rows);
            const float* sn = sh + 2 * tile_rows;
            // lane j < rpw owns row (t * tile_rows + warp * rpw + j)
            const int slot_row = warp * rpw + lane;
            const int row = t * tile_rows + slot_row;
            const bool valid = lane < rpw && row < n32;
            float hq = valid ? sh[slot_row] : __uint_as_float(0xff800000u);
            const bool live = !(hq < 0.0f) && valid;                          // warp.cu:28-30, 75-77
            float bound = 0.0f, nrow = 0.0f;
            if (live) {
                if (!first) bound = __ldg(s.dSL_quarter + sv[slot_row]);      // used after the dot products
                nrow = sn[slot_row];
            }
            unsigned m = __ballot_sync(kFull, live);
            live_cnt += __popc(m);
            const float4* tile4 = reinterpret_cast<const float4*>(st) + (warp * rpw) * d4;
            float mydot = 0.0f;
            // Rows are taken in batches whose arithmetic is free of branches, so that the shuffle
            // chains of a batch overlap: an empty slot of the last batch re-reads row 0 and its sum
            // is dropped (no lane equals -1).
            if (HALF) {
                constexpr int PB = 4;                                          // row pairs per batch
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
                        a[b] = tile4[(r < 0 ? 0 : r) * d4 + (sub < d4 ? sub : 0)];
                    }
#pragma unroll
                    for (int b = 0; b < PB; ++b) {
                        float p = 0.0f;
                        if (sub < d4) p = __fadd_rn(p, chunk_dot(a[b], cen[0]));
                        p = __fadd_rn(p, 0.0f);                                // level 16 of the tree: the partner holds 0
#pragma unroll
                        for (int off = 8; off > 0; off >>= 1) p = __fadd_rn(p, __shfl_xor_sync(kFull, p, off));
                        const float pa = __shfl_sync(kFull, p, 0), pb = __shfl_sync(kFull, p, 16);
                        if (lane == ra[b]) mydot = pa;
                        if (lane == rb[b]) mydot = pb;
                    }
                }
            } else {
                constexpr int RBS = CPL >= 8 ? 1 : 8 / CPL;                    // rows read from the stage together
                while (m) {
                    int rows[RBS];
                    float4 a[RBS][CPL];
#pragma unroll
                    for (int b = 0; b < RBS; ++b) {
                        rows[b] = m ? (__ffs(m) - 1) : -1;
                        m &= m - 1;
                    }
#pragma unroll
                    for (int b = 0; b < RBS; ++b) {
                        const int r = rows[b] < 0 ? 0 : rows[b];
#pragma unroll
                        for (int c = 0; c < CPL; ++c)
                            a[b][c] = tile4[r * d4 + (lane + 32 * c < d4 ? lane + 32 * c : 0)];
                    }
#pragma unroll
                    for (int b = 0; b < RBS; ++b) {
                        float p = 0.0f;
#pragma unroll
                        for (int c = 0; c < CPL; ++c)
                            if (lane + 32 * c < d4) p = __fadd_rn(p, chunk_dot(a[b][c], cen[c]));
                        p = warp_tree_sum(p);
                        if (lane == rows[b]) mydot = p;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_empty[q]);                        // the stage may be refilled
            if (live && (first || !(bound >= hq))) {                        // warp.cu:80-82
                const float d = sq_dist(nrow, nn, mydot);
                if (d < hq) {
                    hq = d;
                    s.h[row] = d;
                    s.voronoi[row] = i;
                }
            }
            if (hq > best_h) { best_h = hq; best_row = row; }               // rows come in order per lane
        }
    }

    u64 best = best_row >= 0 ? make_key(best_h, s.shard_offset + best_row) : 0;
    best = warp_max_key(best);
    if (lane == 0 && warp < W) { s_keys[warp] = best; s_live[warp] = live_cnt; }
    __syncthreads();
    if (s_abort && warp == W && lane == 0) {
        // a wait ran out: let the copies that may still be in flight land before the block's
        // shared memory is released (each wait bounded): the last tile started on stage q was
        // number q + S * floor((issued - 1 - q) / S), whose phase parity is waited for
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

#endif  // CORESETS_B200_STEP_TMA_CUH
