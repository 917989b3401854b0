// Cell index: rows grouped by the centre that owned them when the index was built, so that a pick
// reads only the cells whose rows can change.  Part of the single translation unit fps_kernels.cu.
#ifndef CORESETS_B200_CELLS_CUH
#define CORESETS_B200_CELLS_CUH

namespace {

constexpr int kCellTile = CS_CELL_TILE;      // slots of one warp-tile; segments are whole tiles
constexpr int kCellChunk = kCellTile;            // slots a block takes at a time: one tile, 32 per warp
constexpr int kCellWorkSmem = 1024;          // work-list entries the step kernel stages in shared memory
constexpr int kCellBinsSmem = 48 * 1024;     // cells whose counters fit the scatter kernel's shared memory

struct CellsMeta {
    int n_cells;
    int n_work;
    int n_chunks;
    int total_slots;
    u64 visited_slots;
    u64 picks;
    unsigned q_count;       // rows queued for evaluation by the pick in flight
    unsigned q_inline;      // rows evaluated by the scan kernel itself because the queue was full
};
static_assert(sizeof(CellsMeta) <= CS_CELLS_META_BYTES, "cells meta too large");
static_assert(sizeof(cs_cells_meta_view) == CS_CELLS_META_BYTES, "cs_cells_meta_view must span the meta block");

// ---- build ---------------------------------------------------------------------------------------
// 1. histogram of voronoi (and the copy cell0 = voronoi), 2. tile-aligned segment offsets,
// 3. scatter of (row, h, voronoi) into the segments, 4. padding of the segment tails,
// 5. per-cell arg-max keys, 6. per-cell h0.  The order of rows inside a segment is whatever the
// atomics give: no result depends on it (keys carry the row index for ties).

// One atomic per distinct cell of a warp instead of one per lane.
__device__ __forceinline__ void warp_hist_add(int* hist, const int v, const bool valid) {
    const unsigned act = __ballot_sync(kFull, valid);
    if (!valid) return;
    const unsigned peers = __match_any_sync(act, v);
    const int lane = threadIdx.x & 31;
    if ((__ffs(peers) - 1) == lane) atomicAdd(hist + v, __popc(peers));
}

__global__ void __launch_bounds__(kThreads) cells_hist_kernel(const cs_state s, const cs_cells c) {
    extern __shared__ int s_bin[];
    const Ctl* ctl = reinterpret_cast<const Ctl*>(s.ctl);
    const int n = ctl->n_sel;
    const bool smem_ok = n <= kCellBinsSmem;
    if (smem_ok) {
        for (int a = threadIdx.x; a < n; a += blockDim.x) s_bin[a] = 0;
        __syncthreads();
    }
    int* hist = smem_ok ? s_bin : c.seg_count;
    const int64_t N = s.N_local;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t n_round = (N + 31) & ~(int64_t)31;               // whole warps take part in the votes
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n_round; r += stride) {
        const bool valid = r < N;
        const int v = valid ? s.voronoi[r] : 0;
        if (valid) c.cell0[r] = v;
        warp_hist_add(hist, v, valid);
    }
    if (smem_ok) {
        __syncthreads();
        for (int a = threadIdx.x; a < n; a += blockDim.x) {
            const int q = s_bin[a];
            if (q) atomicAdd(c.seg_count + a, q);
        }
    }
}

// Single block: seg_start = running sum of the counts rounded up to whole tiles.
__global__ void __launch_bounds__(1024) cells_offsets_kernel(const cs_state s, const cs_cells c) {
    __shared__ int s_part[1024];
    const Ctl* ctl = reinterpret_cast<const Ctl*>(s.ctl);
    CellsMeta* m = reinterpret_cast<CellsMeta*>(c.meta);
    const int n = ctl->n_sel;
    const int per = (n + 1023) / 1024;
    const int lo = threadIdx.x * per, hi = min(n, lo + per);
    int sum = 0;
    for (int a = lo; a < hi; ++a) sum += (c.seg_count[a] + kCellTile - 1) & ~(kCellTile - 1);
    s_part[threadIdx.x] = sum;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {                      // inclusive scan of the partial sums
        const int t = threadIdx.x >= off ? s_part[threadIdx.x - off] : 0;
        __syncthreads();
        s_part[threadIdx.x] += t;
        __syncthreads();
    }
    int run = threadIdx.x ? s_part[threadIdx.x - 1] : 0;
    for (int a = lo; a < hi; ++a) {
        c.seg_start[a] = run;
        c.cursor[a] = run;
        c.seg_key[a] = 0;
        run += (c.seg_count[a] + kCellTile - 1) & ~(kCellTile - 1);
    }
    if (threadIdx.x == 1023) {
        c.seg_start[n] = s_part[1023];
        m->n_cells = n;
        m->n_work = 0;
        m->n_chunks = 0;
        m->total_slots = s_part[1023];
        m->visited_slots = 0;
        m->picks = 0;
    }
}

// A block takes `rows_per_block` consecutive rows at a time: count them per cell in shared memory,
// reserve each cell's range with one global atomic, then place the rows.
__global__ void __launch_bounds__(kThreads) cells_scatter_kernel(const cs_state s, const cs_cells c, const int rows_per_block) {
    extern __shared__ int s_bin[];
    const Ctl* ctl = reinterpret_cast<const Ctl*>(s.ctl);
    const int n = ctl->n_sel;
    const int64_t N = s.N_local;
    const bool smem_ok = n <= kCellBinsSmem;
    const int64_t n_blocks = (N + rows_per_block - 1) / rows_per_block;
    for (int64_t b = blockIdx.x; b < n_blocks; b += gridDim.x) {
        const int64_t r0 = b * rows_per_block;
        const int cnt = (int)min((int64_t)rows_per_block, N - r0);
        if (smem_ok) {
            for (int a = threadIdx.x; a < n; a += blockDim.x) s_bin[a] = 0;
            __syncthreads();
            for (int k = threadIdx.x; k < cnt; k += blockDim.x) atomicAdd(&s_bin[s.voronoi[r0 + k]], 1);
            __syncthreads();
            for (int a = threadIdx.x; a < n; a += blockDim.x) {
                const int q = s_bin[a];
                if (q) s_bin[a] = atomicAdd(c.cursor + a, q);        // the bin now holds the next free slot
            }
            __syncthreads();
            for (int k = threadIdx.x; k < cnt; k += blockDim.x) {
                const int64_t r = r0 + k;
                const int v = s.voronoi[r];
                const int pos = atomicAdd(&s_bin[v], 1);
                c.perm[pos] = (int)r;
                c.hp[pos] = s.h[r];
                c.vp[pos] = v;
            }
            __syncthreads();
        } else {
            for (int k = threadIdx.x; k < cnt; k += blockDim.x) {
                const int64_t r = r0 + k;
                const int v = s.voronoi[r];
                const int pos = atomicAdd(c.cursor + v, 1);
                c.perm[pos] = (int)r;
                c.hp[pos] = s.h[r];
                c.vp[pos] = v;
            }
        }
    }
}

// One warp per cell: the slots between the cell's rows and the next tile boundary hold nothing.
__global__ void __launch_bounds__(kThreads) cells_pad_kernel(const cs_state s, const cs_cells c) {
    const Ctl* ctl = reinterpret_cast<const Ctl*>(s.ctl);
    const int n = ctl->n_sel;
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * kWarps + (threadIdx.x >> 5), nw = gridDim.x * kWarps;
    for (int a = gw; a < n; a += nw) {
        const int lo = c.seg_start[a] + c.seg_count[a], hi = c.seg_start[a + 1];
        for (int p = lo + lane; p < hi; p += 32) {
            c.perm[p] = -1;
            c.hp[p] = __uint_as_float(0xff800000u);
            c.vp[p] = 0;
        }
    }
}

// One warp per tile: largest key of the tile into its cell's key.  Every tile holds at least one
// row, and every row of a segment carries the segment's cell in vp at build time.
__global__ void __launch_bounds__(kThreads) cells_keys_kernel(const cs_state s, const cs_cells c) {
    const CellsMeta* m = reinterpret_cast<const CellsMeta*>(c.meta);
    const int tiles = m->total_slots / kCellTile;
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * kWarps + (threadIdx.x >> 5), nw = gridDim.x * kWarps;
    for (int t = gw; t < tiles; t += nw) {
        u64 best = 0;
        int cell = -1;
#pragma unroll
        for (int j = 0; j < kCellTile / 32; ++j) {
            const int p = t * kCellTile + j * 32 + lane;
            const int row = c.perm[p];
            if (row >= 0) {
                const u64 k = make_key(c.hp[p], s.shard_offset + row);
                best = k > best ? k : best;
                cell = c.vp[p];
            }
        }
        best = warp_max_key(best);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) cell = max(cell, __shfl_xor_sync(kFull, cell, off));
        if (lane == 0 && cell >= 0 && best) atomicMax(reinterpret_cast<u64*>(c.seg_key) + cell, best);
    }
}

__global__ void cells_h0_kernel(const cs_state s, const cs_cells c) {
    const Ctl* ctl = reinterpret_cast<const Ctl*>(s.ctl);
    const int n = ctl->n_sel;
    for (int a = blockIdx.x * blockDim.x + threadIdx.x; a < n; a += gridDim.x * blockDim.x)
        c.seg_h0[a] = key_val(c.seg_key[a]);
}

// ---- per pick: which cells to visit ------------------------------------------------------------------
// Cell A (centre c_A, rows r that were within sqrt(h0) of c_A when the index was built) needs no
// visit for the new centre c when every row provably keeps its h.  In exact arithmetic
//   |r - c| >= |c_A - c| - |r - c_A|,
// and the computed squared distances differ from the exact ones by at most e = g * (sum of the two
// squared norms) (g bounds the rounding of norms, dot product and the final subtraction).  With
//   a = sqrt(4 * dSL_quarter[A] - e1)   a lower bound of |c_A - c|,
//   b = sqrt(max(h0, 0) + e2)           an upper bound of |r - c_A| for every row of the cell,
// a > b and (a - b)^2 - e3 >= (largest live h of the cell) imply that the distance the kernel would
// compute for any row of the cell is >= that row's h, i.e. the reference's update `d < h` cannot
// fire.  Rows the reference itself would evaluate and leave unchanged are thus skipped as well;
// rows that could change are never skipped.  Everything in double.
__device__ __forceinline__ bool cell_can_skip(const double dsl, const double h0, const double hmax, const double nA,
                                              const double ni, const double nr, const double g) {
    if (!(hmax >= 0.0)) return true;                       // no live row in the cell
    const double e1 = g * (nA + ni) + 1e-30, e2 = g * (nr + nA) + 1e-30, e3 = g * (nr + ni) + 1e-30;
    const double a2 = 4.0 * dsl - e1;
    if (!(a2 > 0.0)) return false;
    const double a = sqrt(a2), b = sqrt(fmax(h0, 0.0) + e2);
    if (!(a > b)) return false;
    const double t = a - b;
    return t * t - e3 >= hmax;
}

// Single block.  Writes the list of visited cells with running chunk counts, clears their keys (the
// step kernel rebuilds them) and seeds the next pick's arg-max key with the best key among the cells
// that are NOT visited.
__global__ void __launch_bounds__(1024) cells_select_kernel(const cs_state s, const cs_cells c, const double g) {
    pdl_enter();
    __shared__ int s_cells[1024], s_chunks[1024];
    __shared__ u64 s_best[32];
    __shared__ u64 s_slots[32];
    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    CellsMeta* m = reinterpret_cast<CellsMeta*>(c.meta);
    const int i = ctl->n_sel;
    if (i >= s.cap) return;                                // the step kernel reports the overflow
    const int n = m->n_cells;
    const int64_t wl = (int64_t)ctl->last_idx - s.shard_offset;
    const int win_cell = (ctl->last_idx >= 0 && wl >= 0 && wl < s.N_local) ? c.cell0[wl] : -1;
    const double ni = (double)s.norms_sel[i], nr = (double)c.row_norm_max;
    const int per = (n + 1023) / 1024;                     // <= 64 while cap <= 65536
    const int lo = threadIdx.x * per, hi = min(n, lo + per);
    unsigned long long visit = 0;
    int n_cells = 0, n_chunks = 0;
    u64 best = 0, slots = 0;
    for (int a = lo; a < hi; ++a) {
        const u64 k = c.seg_key[a];
        const int len = c.seg_start[a + 1] - c.seg_start[a];
        bool v = false;
        if (len > 0) {
            v = (a == win_cell) || !cell_can_skip((double)s.dSL_quarter[a], (double)c.seg_h0[a], (double)key_val(k),
                                                  (double)s.norms_sel[a], ni, nr, g);
        }
        if (v) {
            visit |= 1ull << (a - lo);
            ++n_cells;
            n_chunks += (len + kCellChunk - 1) / kCellChunk;
            slots += (u64)len;
        } else {
            best = k > best ? k : best;
        }
    }
    s_cells[threadIdx.x] = n_cells;
    s_chunks[threadIdx.x] = n_chunks;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
        const int t0 = threadIdx.x >= off ? s_cells[threadIdx.x - off] : 0;
        const int t1 = threadIdx.x >= off ? s_chunks[threadIdx.x - off] : 0;
        __syncthreads();
        s_cells[threadIdx.x] += t0;
        s_chunks[threadIdx.x] += t1;
        __syncthreads();
    }
    int w = s_cells[threadIdx.x] - n_cells, cum = s_chunks[threadIdx.x] - n_chunks;
    for (int a = lo; a < hi; ++a) {
        if (!((visit >> (a - lo)) & 1ull)) continue;
        const int len = c.seg_start[a + 1] - c.seg_start[a];
        cum += (len + kCellChunk - 1) / kCellChunk;
        c.work_cell[w] = a;
        c.work_cum[w] = cum;
        c.seg_key[a] = 0;
        ++w;
    }
    best = warp_max_key(best);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) slots += __shfl_xor_sync(kFull, slots, off);
    if ((threadIdx.x & 31) == 0) { s_best[threadIdx.x >> 5] = best; s_slots[threadIdx.x >> 5] = slots; }
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 bk = 0, sl = 0;
        for (int q = 0; q < 32; ++q) { bk = s_best[q] > bk ? s_best[q] : bk; sl += s_slots[q]; }
        u64* slot = &ctl->key[(i + 1) & 1];
        if (bk > *slot) *slot = bk;
        m->n_work = s_cells[1023];
        m->n_chunks = s_chunks[1023];
        m->visited_slots += sl;
        m->picks += 1;
        m->q_count = 0;
        m->q_inline = 0;
    }
}

// ---- per pick: the update over the visited cells ---------------------------------------------------
// Two kernels.  cells_scan_kernel walks the visited tiles (a warp takes a tile of kCellTile slots,
// a lane eight of them), applies the reference's predicate to every slot, feeds the rows that keep
// their h into their cell's key, and appends the rows that need a distance to ONE queue in global
// memory.  cells_eval_kernel then spreads that queue evenly over the whole grid, 32 rows per warp
// step, all row loads of a batch in flight.  The rows that pass the test are few but clustered (a
// visited cell near the new centre is live almost everywhere), which is why they are not
// evaluated where the scan meets them.  Arithmetic, update rule and tie rule are those of
// fps_step_queue_kernel.  Updates go to both copies (hp / vp by slot, h / voronoi by row).

// Dot products of the rows held by the lanes of `mask` (lane l holds `row`) with the centre, in
// branch-free batches; returns the dot of the calling lane's row (lanes outside mask: 0).
template <int CPL, bool FULL, bool HALF>
__device__ __forceinline__ float warp_dots(unsigned mask, const int row, const float4* __restrict__ X4, const int d4,
                                           const float4 (&cen)[CPL]) {
    const int lane = threadIdx.x & 31;
    const int sub = HALF ? (lane & 15) : lane;
    const bool hi = HALF && lane >= 16;
    float mydot = 0.0f;
    if (HALF) {
        constexpr int PB = 4;                                    // row pairs per batch
        while (mask) {
            int la[PB], lb[PB];
            float4 a[PB];
#pragma unroll
            for (int b = 0; b < PB; ++b) {
                la[b] = mask ? (__ffs(mask) - 1) : -1;
                mask &= mask - 1;
                lb[b] = mask ? (__ffs(mask) - 1) : -1;
                mask &= mask - 1;
            }
#pragma unroll
            for (int b = 0; b < PB; ++b) {
                const int src = hi ? lb[b] : la[b];
                const int r = __shfl_sync(kFull, row, src < 0 ? 0 : src);
                a[b] = ld_stream4(X4 + (int64_t)(r < 0 ? 0 : r) * d4 + (sub < d4 ? sub : 0));
            }
#pragma unroll
            for (int b = 0; b < PB; ++b) {
                float q = 0.0f;
                if (sub < d4) q = __fadd_rn(q, chunk_dot(a[b], cen[0]));
                q = __fadd_rn(q, 0.0f);                          // level 16 of the tree: the partner holds 0
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) q = __fadd_rn(q, __shfl_xor_sync(kFull, q, off));
                const float pa = __shfl_sync(kFull, q, 0), pb = __shfl_sync(kFull, q, 16);
                if (lane == la[b]) mydot = pa;
                if (lane == lb[b]) mydot = pb;
            }
        }
    } else {
        constexpr int BS = CPL >= 8 ? 1 : 8 / CPL;               // rows read together
        while (mask) {
            int src[BS];
            float4 a[BS][CPL];
#pragma unroll
            for (int b = 0; b < BS; ++b) {
                src[b] = mask ? (__ffs(mask) - 1) : -1;
                mask &= mask - 1;
            }
#pragma unroll
            for (int b = 0; b < BS; ++b) {
                const int r = __shfl_sync(kFull, row, src[b] < 0 ? 0 : src[b]);
                const float4* rp = X4 + (int64_t)(r < 0 ? 0 : r) * d4;
#pragma unroll
                for (int c = 0; c < CPL; ++c)
                    a[b][c] = ld_stream4(rp + ((FULL || lane + 32 * c < d4) ? lane + 32 * c : 0));
            }
#pragma unroll
            for (int b = 0; b < BS; ++b) {
                float q = 0.0f;
#pragma unroll
                for (int c = 0; c < CPL; ++c)
                    if (FULL || lane + 32 * c < d4) q = __fadd_rn(q, chunk_dot(a[b][c], cen[c]));
                q = warp_tree_sum(q);
                if (lane == src[b]) mydot = q;
            }
        }
    }
    return mydot;
}

template <int CPL, bool FULL, bool HALF>
__device__ __forceinline__ void load_centre(const cs_state& s, const int i, float4 (&cen)[CPL]) {
    const int lane = threadIdx.x & 31, d4 = s.D >> 2;
    const int sub = HALF ? (lane & 15) : lane;
    const float4* c4 = reinterpret_cast<const float4*>(s.X_sel + (int64_t)i * s.D);
#pragma unroll
    for (int c = 0; c < CPL; ++c)
        cen[c] = (FULL || sub + 32 * c < d4) ? c4[sub + 32 * c] : make_float4(0.f, 0.f, 0.f, 0.f);
}

// Keys of the lanes of one warp into the keys of their cells: one atomic per distinct cell.
__device__ __forceinline__ void warp_keys_to_cells(u64* seg_key, const u64 key, const int cell, unsigned todo) {
    while (todo) {
        const int c0 = __shfl_sync(kFull, cell, __ffs(todo) - 1);
        const unsigned grp = __ballot_sync(kFull, cell == c0) & todo;
        const u64 k = warp_max_key(((grp >> (threadIdx.x & 31)) & 1u) ? key : 0);
        if ((threadIdx.x & 31) == 0 && k) atomicMax(seg_key + c0, k);
        todo &= ~grp;
    }
}

template <int CPL, bool FULL, bool HALF>
__global__ void __launch_bounds__(kThreads, CS_MIN_BLOCKS) cells_scan_kernel(const cs_state s, const cs_cells cl) {
    pdl_enter();
    __shared__ u64 s_keys[kWarps];
    __shared__ int s_cum[kCellWorkSmem], s_cell[kCellWorkSmem];

    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    if (i >= s.cap) return;                                          // cells_eval_kernel reports it
    CellsMeta* m = reinterpret_cast<CellsMeta*>(cl.meta);
    const int n_work = m->n_work, n_tiles = m->n_chunks;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gw = blockIdx.x * kWarps + warp, nw = gridDim.x * kWarps;
    // a short work list is staged in shared memory: one round trip instead of one per search step
    const bool staged = n_work <= kCellWorkSmem;
    if (staged && (int)blockIdx.x * kWarps < n_tiles) {
        for (int k = threadIdx.x; k < n_work; k += blockDim.x) {
            s_cum[k] = __ldg(cl.work_cum + k);
            s_cell[k] = __ldg(cl.work_cell + k);
        }
    }
    __syncthreads();
    const int64_t wl = (int64_t)ctl->last_idx - s.shard_offset;
    const int win_row = (ctl->last_idx >= 0 && wl >= 0 && wl < s.N_local) ? (int)wl : -2;
    const float kNegInf = __uint_as_float(0xff800000u);
    const unsigned q_cap = (unsigned)cl.q_cap;
    u64 warp_best = 0;

    for (int t = gw; t < n_tiles; t += nw) {
        int lo = 0, hi_w = n_work - 1;                               // first running tile count above t
        while (lo < hi_w) {
            const int mid = (lo + hi_w) >> 1;
            if ((staged ? s_cum[mid] : __ldg(cl.work_cum + mid)) > t) hi_w = mid; else lo = mid + 1;
        }
        const int cell = staged ? s_cell[lo] : __ldg(cl.work_cell + lo);
        const int in_cell = t - (lo ? (staged ? s_cum[lo - 1] : __ldg(cl.work_cum + lo - 1)) : 0);
        const int tile0 = __ldg(cl.seg_start + cell) + in_cell * kCellTile;      // segments are whole tiles
        float hq[8];
        int vq[8], rq[8];
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            const int p = tile0 + g * 128 + 4 * lane;
            const float4 a = *reinterpret_cast<const float4*>(cl.hp + p);
            const int4 b = *reinterpret_cast<const int4*>(cl.vp + p);
            const int4 r = *reinterpret_cast<const int4*>(cl.perm + p);
            hq[4 * g] = a.x; hq[4 * g + 1] = a.y; hq[4 * g + 2] = a.z; hq[4 * g + 3] = a.w;
            vq[4 * g] = b.x; vq[4 * g + 1] = b.y; vq[4 * g + 2] = b.z; vq[4 * g + 3] = b.w;
            rq[4 * g] = r.x; rq[4 * g + 1] = r.y; rq[4 * g + 2] = r.z; rq[4 * g + 3] = r.w;
        }
        float bq[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (rq[j] == win_row) {                                  // the row committed for this pick
                const int p = tile0 + (j >> 2) * 128 + 4 * lane + (j & 3);
                hq[j] = -1.0f;
                vq[j] = i;
                cl.hp[p] = -1.0f;
                cl.vp[p] = i;
            }
            bq[j] = __ldg(s.dSL_quarter + vq[j]);
        }
        unsigned need = 0;
        float best_h = kNegInf;
        int best_row = -1;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const bool live = !(hq[j] < 0.0f);                       // warp.cu:75-77 (padding holds -inf)
            if (live && !(bq[j] >= hq[j])) need |= 1u << j;          // warp.cu:80-82
            else if (rq[j] >= 0 && (hq[j] > best_h || (hq[j] == best_h && rq[j] < best_row))) {
                best_h = hq[j];
                best_row = rq[j];
            }
        }
        u64 key = best_row >= 0 ? make_key(best_h, s.shard_offset + best_row) : 0;
        key = warp_max_key(key);
        if (lane == 0 && key) atomicMax(reinterpret_cast<u64*>(cl.seg_key) + cell, key);
        warp_best = key > warp_best ? key : warp_best;
        if (!__any_sync(kFull, need != 0u)) continue;
        // append this lane's rows behind those of the lower lanes
        const int cnt = __popc(need);
        int pre = cnt;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int o = __shfl_up_sync(kFull, pre, off);
            if (lane >= off) pre += o;
        }
        const int total = __shfl_sync(kFull, pre, 31);
        unsigned base = 0;
        if (lane == 0) base = atomicAdd(&m->q_count, (unsigned)total);
        base = __shfl_sync(kFull, base, 0);
        if (base + (unsigned)total <= q_cap) {
            unsigned w = base + (unsigned)(pre - cnt);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if ((need >> j) & 1u) reinterpret_cast<int2*>(cl.queue)[w++] = make_int2(tile0 + (j >> 2) * 128 + 4 * lane + (j & 3), cell);
        } else {
            // the queue is full (a bound of the caller's buffer, not of the data): this tile is
            // finished right here; its queue range stays unwritten and is skipped by the consumer
            if (lane == 0) atomicAdd(&m->q_inline, (unsigned)total);
            for (unsigned u = base + lane; u < q_cap && u < base + (unsigned)total; u += 32) reinterpret_cast<int2*>(cl.queue)[u] = make_int2(-1, -1);
            float4 cen[CPL];
            load_centre<CPL, FULL, HALF>(s, i, cen);
            const float nn = s.norms_sel[i];
            const float4* X4 = reinterpret_cast<const float4*>(s.X);
            u64 k2 = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool nd = (need >> j) & 1u;
                const unsigned mask = __ballot_sync(kFull, nd);
                const float dot = warp_dots<CPL, FULL, HALF>(mask, rq[j], X4, s.D >> 2, cen);
                if (nd) {
                    const int p = tile0 + (j >> 2) * 128 + 4 * lane + (j & 3);
                    float hh = hq[j];
                    const float d = sq_dist(__ldg(s.norms + rq[j]), nn, dot);
                    if (d < hh) {
                        hh = d;
                        cl.hp[p] = d;
                        cl.vp[p] = i;
                        s.h[rq[j]] = d;
                        s.voronoi[rq[j]] = i;
                    }
                    const u64 kk = make_key(hh, s.shard_offset + rq[j]);
                    k2 = kk > k2 ? kk : k2;
                }
            }
            k2 = warp_max_key(k2);
            if (lane == 0 && k2) atomicMax(reinterpret_cast<u64*>(cl.seg_key) + cell, k2);
            warp_best = k2 > warp_best ? k2 : warp_best;
        }
    }
    if (lane == 0) s_keys[warp] = warp_best;
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 bk = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) bk = s_keys[w] > bk ? s_keys[w] : bk;
        if (bk) atomicMax(&ctl->key[(i + 1) & 1], bk);
    }
}

template <int CPL, bool FULL, bool HALF>
__global__ void __launch_bounds__(kThreads, CS_MIN_BLOCKS) cells_eval_kernel(const cs_state s, const cs_cells cl) {
    pdl_enter();
    __shared__ u64 s_keys[kWarps];
    __shared__ int s_last;

    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    if (i >= s.cap) {
        if (blockIdx.x == 0 && threadIdx.x == 0) ctl->status = ST_CAPACITY;
        return;
    }
    const CellsMeta* m = reinterpret_cast<const CellsMeta*>(cl.meta);
    const unsigned q_cap = (unsigned)cl.q_cap;
    const unsigned reserved = m->q_count;
    // Reservations are made per tile in order of arrival.  The first one that does not fit is
    // refused, and so is every later one (their bases lie above the capacity); the scan kernel
    // finished those tiles itself and marked the part of the refused range that lies inside the
    // queue as unused (-1).
    const unsigned n_q = reserved < q_cap ? reserved : q_cap;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gw = blockIdx.x * kWarps + warp, nw = gridDim.x * kWarps;
    const float nn = s.norms_sel[i];
    float4 cen[CPL];
    load_centre<CPL, FULL, HALF>(s, i, cen);
    const float4* X4 = reinterpret_cast<const float4*>(s.X);
    u64 warp_best = 0;
    for (unsigned q0 = (unsigned)gw * 32u; q0 < n_q; q0 += (unsigned)nw * 32u) {
        const unsigned q = q0 + lane;
        int2 e = make_int2(-1, -1);
        if (q < n_q) e = reinterpret_cast<const int2*>(cl.queue)[q];
        const bool valid = e.x >= 0;
        int row = -1;
        float hq = 0.0f, nrow = 0.0f;
        if (valid) {
            row = cl.perm[e.x];
            hq = cl.hp[e.x];
            nrow = __ldg(s.norms + row);
        }
        const unsigned mask = __ballot_sync(kFull, valid);
        const float dot = warp_dots<CPL, FULL, HALF>(mask, row, X4, s.D >> 2, cen);
        u64 key = 0;
        if (valid) {
            const float d = sq_dist(nrow, nn, dot);
            if (d < hq) {
                hq = d;
                cl.hp[e.x] = d;
                cl.vp[e.x] = i;
                s.h[row] = d;
                s.voronoi[row] = i;
            }
            key = make_key(hq, s.shard_offset + row);
        }
        warp_keys_to_cells(reinterpret_cast<u64*>(cl.seg_key), key, e.y, mask);
        const u64 wk = warp_max_key(key);
        warp_best = wk > warp_best ? wk : warp_best;
    }
    if (lane == 0) s_keys[warp] = warp_best;
    __syncthreads();
    const int slot = (i + 1) & 1;
    if (threadIdx.x == 0) {
        u64 bk = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) bk = s_keys[w] > bk ? s_keys[w] : bk;
        if (bk) atomicMax(&ctl->key[slot], bk);
        __threadfence();
        s_last = (atomicAdd(&ctl->ticket, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const u64 k = *reinterpret_cast<volatile u64*>(&ctl->key[slot]);
    if (s.world_size > 1) publish_candidate(s, ctl, k, key_idx(k) - s.shard_offset);
    if (threadIdx.x == 0) {
        ctl->live_rows = (u64)n_q + (u64)m->q_inline;               // approximate above the queue's capacity
        ctl->ticket = 0;
        ctl->n_sel = i + 1;
    }
}

}  // namespace

#endif  // CORESETS_B200_CELLS_CUH
