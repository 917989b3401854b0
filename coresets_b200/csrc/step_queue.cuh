// Kernel B of the default prune mode: streamed scan, warp-private row queues, branch-free batches.
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_STEP_QUEUE_CUH
#define CORESETS_B200_STEP_QUEUE_CUH

namespace {

// ---- prune mode with deferred rows -------------------------------------------------------------------
// In prune mode few rows pass the triangle test and they are scattered, so walking them where
// they are met leaves a warp with one or two row loads in flight and a long dependent chain per
// super-tile.  Here the scan and the distance work are decoupled: a warp streams h / voronoi of
// its super-tiles (four of them in flight through asynchronous copies), applies the test, and pushes the rows that
// need a distance onto a warp-private queue in shared memory; whenever the queue holds a full
// batch, the batch is evaluated branch-free with all of its row loads in flight.  The arithmetic
// per row, the update rule and the arg-max order are those of fps_step_kernel, so the bits match.
constexpr int kQueueCap = 160;           // a batch remainder (< 16) plus one super-tile (128), padded
constexpr int kScanDepth = 4;            // super-tiles of h / voronoi in flight per warp (cp.async ring; 3-4 measured best)
constexpr int kScanRingFloats = kWarps * kScanDepth * 256;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int CPL, bool FULL, bool HALF>
__global__ void __launch_bounds__(kThreads, CPL == 0 ? 2 : CS_MIN_BLOCKS) fps_step_queue_kernel(const cs_state s, const int n_bound_smem) {
    pdl_enter();
    static_assert(kRowsPerLane == 4, "the deferred-row kernel reads four rows per lane");
    // dynamic shared memory: the scan ring (per warp and slot 128 h, then 128 voronoi words), the
    // first n_bound_smem triangle bounds, then (CPL == 0, the path for any row width and for the
    // element-wise summation order) the centre
    extern __shared__ __align__(16) float s_dyn[];
    float (*s_ring)[kScanDepth][256] = reinterpret_cast<float (*)[kScanDepth][256]>(s_dyn);
    float* s_dsl = s_dyn + kScanRingFloats;
    float* s_cen = s_dsl + ((n_bound_smem + 3) & ~3);            // 16-byte aligned: read as float4 chunks
    __shared__ int2 s_queue[kWarps][kQueueCap];                  // (local row, bits of its h)
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
    const int D = s.D, d4 = D >> 2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = HALF ? (lane & 15) : lane;
    const bool hi = HALF && lane >= 16;
    const bool first = (i == 0);
    const float nn = s.norms_sel[i];
    float4 cen[CPL ? CPL : 1];
    if (CPL) {
        const float4* c4 = reinterpret_cast<const float4*>(s.X_sel + (int64_t)i * D);
#pragma unroll
        for (int c = 0; c < (CPL ? CPL : 1); ++c)
            cen[c] = (FULL || sub + 32 * c < d4) ? c4[sub + 32 * c] : make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
        const float* cen_g = s.X_sel + (int64_t)i * D;
        for (int c = threadIdx.x; c < D; c += blockDim.x) s_cen[c] = cen_g[c];
    }
    // chunked order needs whole 16-byte chunks and is what float32 inputs get (_shared.cuh:41-50)
    const bool chunked = (D & 3) == 0 && !(s.flags & CS_F_ELEMENT_ORDER);
    const bool half_rows = (s.flags & CS_F_X_HALF) != 0;
    const int nb = i < n_bound_smem ? i : n_bound_smem;
    // voronoi <= i (the row committed for this pick carries i itself), so with i inside the staged
    // table every look-up stays within the block's shared memory
    const bool all_bounds_staged = i < n_bound_smem;
    for (int c = threadIdx.x; c < nb; c += blockDim.x) s_dsl[c] = s.dSL_quarter[c];
    __syncthreads();

    const int64_t N = s.N_local;
    const int n32 = (int)N;
    const int tiles = (int)((N + 127) >> 7);
    const int whole_tiles = (int)(N >> 7);
    const int nw = (int)gridDim.x * kWarps;
    const float4* X4 = reinterpret_cast<const float4*>(s.X);
    const bool vec_ok = ((((uintptr_t)s.h) | ((uintptr_t)s.voronoi)) & 15u) == 0;
    const float kNegInf = __uint_as_float(0xff800000u);
    float best_h = kNegInf;
    int best_row = -1;
    unsigned live_cnt = 0;
    int2* q = s_queue[warp];
    int qn = 0;                                                  // entries waiting (warp-uniform)
    constexpr int BS = HALF ? 16 : (CPL == 0 ? 4 : (CPL >= 8 ? 1 : 8 / CPL));     // rows of a batch

    // ---- one batch: entries q[base .. base+cnt), cnt <= BS; lane b < cnt finishes entry b --------
    auto run_batch = [&](const int base, const int cnt) {
        float mydot = 0.0f;
        if (CPL == 0) {
            // any row width: the lanes stride over the row, four rows side by side
            int rows[4];
            float acc[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                rows[b] = q[base + (b < cnt ? b : cnt - 1)].x;
                acc[b] = 0.0f;
            }
            if (chunked) {
                const float4* c4 = reinterpret_cast<const float4*>(s_cen);
#pragma unroll 2
                for (int c = lane; c < d4; c += 32) {
                    const float4 cc = c4[c];
                    float4 a[4];
#pragma unroll
                    for (int b = 0; b < 4; ++b) a[b] = ld_stream4(X4 + (int64_t)rows[b] * d4 + c);
#pragma unroll
                    for (int b = 0; b < 4; ++b) acc[b] = __fadd_rn(acc[b], chunk_dot(a[b], cc));
                }
            } else if (half_rows) {
                const __half* Xh = reinterpret_cast<const __half*>(s.X);
#pragma unroll 4
                for (int c = lane; c < D; c += 32) {                 // _shared.cuh:52-58: one fma per element
                    __half a[4];
#pragma unroll
                    for (int b = 0; b < 4; ++b) a[b] = __ldcs(Xh + (int64_t)rows[b] * D + c);
                    const float cc = s_cen[c];
#pragma unroll
                    for (int b = 0; b < 4; ++b) acc[b] = __fmaf_rn(__half2float(a[b]), cc, acc[b]);
                }
            } else {
#pragma unroll 2
                for (int c = lane; c < D; c += 32) {                 // _shared.cuh:52-58: one fma per element
                    float a[4];
#pragma unroll
                    for (int b = 0; b < 4; ++b) a[b] = __ldcs(s.X + (int64_t)rows[b] * D + c);
                    const float cc = s_cen[c];
#pragma unroll
                    for (int b = 0; b < 4; ++b) acc[b] = __fmaf_rn(a[b], cc, acc[b]);
                }
            }
            __syncwarp();
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float p = warp_tree_sum(acc[b]);
                if (lane == b) mydot = p;
            }
        } else if (HALF) {
            float4 a[8];
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                int e = 2 * b + (hi ? 1 : 0);
                e = e < cnt ? e : cnt - 1;                       // an empty slot repeats the last entry
                const int r = q[base + e].x;
                a[b] = ld_stream4(X4 + (int64_t)r * d4 + (sub < d4 ? sub : 0));
            }
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                float p = 0.0f;
                if (sub < d4) p = __fadd_rn(p, chunk_dot(a[b], cen[0]));
                p = __fadd_rn(p, 0.0f);                          // level 16 of the tree: the partner holds 0
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) p = __fadd_rn(p, __shfl_xor_sync(kFull, p, off));
                const float pa = __shfl_sync(kFull, p, 0), pb = __shfl_sync(kFull, p, 16);
                if (lane == 2 * b) mydot = pa;
                if (lane == 2 * b + 1) mydot = pb;
            }
        } else {
            float4 a[BS][CPL ? CPL : 1];
#pragma unroll
            for (int b = 0; b < BS; ++b) {
                const int r = q[base + (b < cnt ? b : cnt - 1)].x;
                const float4* rp = X4 + (int64_t)r * d4;
#pragma unroll
                for (int c = 0; c < (CPL ? CPL : 1); ++c)
                    a[b][c] = ld_stream4(rp + ((FULL || lane + 32 * c < d4) ? lane + 32 * c : 0));
            }
#pragma unroll
            for (int b = 0; b < BS; ++b) {
                float p = 0.0f;
#pragma unroll
                for (int c = 0; c < (CPL ? CPL : 1); ++c)
                    if (FULL || lane + 32 * c < d4) p = __fadd_rn(p, chunk_dot(a[b][c], cen[c]));
                p = warp_tree_sum(p);
                if (lane == b) mydot = p;
            }
        }
        if (lane < cnt) {
            const int2 e = q[base + lane];
            const int row = e.x;
            float hq = __int_as_float(e.y);
            const float d = sq_dist(__ldg(s.norms + row), nn, mydot);
            if (d < hq) {
                hq = d;
                s.h[row] = d;
                s.voronoi[row] = i;
            }
            // deferred rows come out of order: the full tie rule
            if (hq > best_h || (hq == best_h && row < best_row)) { best_h = hq; best_row = row; }
        }
        __syncwarp();
    };

    // h / voronoi of the next kScanDepth super-tiles of this warp travel through a warp-private ring
    // of asynchronous 16-byte copies; a lane reads back exactly the bytes it copied itself, so the
    // per-thread wait is the only synchronisation.  The ragged last super-tile is loaded directly.
    auto issue_tile = [&](const int t, const int slot) {
        if (vec_ok && t < whole_tiles) {
            const int r0 = (t << 7) + 4 * lane;
            cp_async16(&s_ring[warp][slot][4 * lane], s.h + r0);
            if (!first) cp_async16(&s_ring[warp][slot][128 + 4 * lane], s.voronoi + r0);
        }
        cp_async_commit();                                       // one group per slot, empty or not
    };
    auto take_tile = [&](const int t, const int slot, float (&hq)[4], int (&vq)[4]) {
        const int r0 = (t << 7) + 4 * lane;
        if (vec_ok && t < whole_tiles) {
            const float4 a = *reinterpret_cast<const float4*>(&s_ring[warp][slot][4 * lane]);
            hq[0] = a.x; hq[1] = a.y; hq[2] = a.z; hq[3] = a.w;
            if (!first) {
                const int4 b = *reinterpret_cast<const int4*>(&s_ring[warp][slot][128 + 4 * lane]);
                vq[0] = b.x; vq[1] = b.y; vq[2] = b.z; vq[3] = b.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bool in = r0 + j < n32;
                hq[j] = in ? s.h[r0 + j] : kNegInf;              // rows past the end: not live, never the maximum
                vq[j] = (in && !first) ? s.voronoi[r0 + j] : 0;
            }
        }
    };

    auto scan_tile = [&](const int t, float (&hq)[4], int (&vq)[4]) {
        if (t >= tiles) return;
        const int r0 = (t << 7) + 4 * lane;
        unsigned need = 0;
        if (first) {
#pragma unroll
            for (int j = 0; j < 4; ++j) need |= !(hq[j] < 0.0f) ? (1u << j) : 0u;   // warp.cu:28-30
        } else if (all_bounds_staged) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // a selected row (h = -1) reads some bound too; the live test keeps it out
                const float b = s_dsl[vq[j]];
                need |= (!(hq[j] < 0.0f) && !(b >= hq[j])) ? (1u << j) : 0u;         // warp.cu:75-82
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = (vq[j] < nb) ? s_dsl[vq[j]] : __ldg(s.dSL_quarter + vq[j]);
                need |= (!(hq[j] < 0.0f) && !(b >= hq[j])) ? (1u << j) : 0u;
            }
        }
        // rows that keep their h compete for the arg-max now (rows of a lane come in increasing
        // order here, so '>' keeps the smallest row among equal values)
        if (need == 0u) {
            const float tmax = fmaxf(fmaxf(hq[0], hq[1]), fmaxf(hq[2], hq[3]));
            if (tmax > best_h) {
                best_h = tmax;
#pragma unroll
                for (int j = 3; j >= 0; --j) best_row = (hq[j] == tmax) ? r0 + j : best_row;
            }
        } else {
            float tmax = kNegInf;
#pragma unroll
            for (int j = 0; j < 4; ++j) tmax = fmaxf(tmax, (need >> j) & 1u ? kNegInf : hq[j]);
            if (tmax > best_h) {
                best_h = tmax;
#pragma unroll
                for (int j = 3; j >= 0; --j) best_row = (!((need >> j) & 1u) && hq[j] == tmax) ? r0 + j : best_row;
            }
        }
        if (!__any_sync(kFull, need != 0u)) return;
        // append this lane's rows behind those of the lower lanes
        const int c = __popc(need);
        int pre = c;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(kFull, pre, off);
            if (lane >= off) pre += o;
        }
        const int total = __shfl_sync(kFull, pre, 31);
        int w = qn + pre - c;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if ((need >> j) & 1u) q[w++] = make_int2(r0 + j, __float_as_int(hq[j]));
        qn += total;
        live_cnt += (unsigned)total;
        __syncwarp();
        while (qn >= BS) {
            qn -= BS;
            run_batch(qn, BS);
        }
    };

    {
        const int t0 = (int)blockIdx.x * kWarps + warp;
#pragma unroll
        for (int p = 0; p < kScanDepth; ++p) issue_tile(t0 + p * nw, p);
        int n = 0;
        for (int t = t0; t < tiles; t += nw, ++n) {
            const int slot = n % kScanDepth;
            cp_async_wait<kScanDepth - 1>();                     // the oldest group has landed
            float hq[4];
            int vq[4] = {0, 0, 0, 0};
            take_tile(t, slot, hq, vq);
            issue_tile(t + kScanDepth * nw, slot);               // refill the slot just read
            scan_tile(t, hq, vq);
        }
        cp_async_wait<0>();
    }
    if (qn > 0) run_batch(0, qn);

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

#endif  // CORESETS_B200_STEP_QUEUE_CUH
