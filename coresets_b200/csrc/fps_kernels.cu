// sm_100a kernels and C entry points of the farthest-point-sampling engine.
//
// Data layout in HBM (per rank): X [N_local, D] fp32 row-major (streamed once per pick),
// norms / h fp32 [N_local], voronoi int32 [N_local]; the committed centres X_sel [cap, D],
// norms_sel, dSL_quarter are small and L2-resident.  One pick = commit_bound_kernel (tiny) +
// fps_step_kernel (the bandwidth-bound pass over X with the arg-max fused in).
//
// Arithmetic is spelled with __fmul_rn/__fmaf_rn/__fadd_rn so that no compiler contraction or
// reassociation can change a bit; the file is compiled with -ftz=true because the reference
// builds with --use_fast_math (src/coresets/cuda/extension.py:63).
#include "coresets_b200.h"

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace {

typedef unsigned long long u64;

// Device layout of the control block; mirrors cs_ctl_view.
struct Ctl {
    u64 key[2];
    int n_sel;
    unsigned ticket;
    int status;
    int viable;
    float sep;
    int steps;
    u64 live_rows;
    float last_val;
    int last_idx;
    unsigned xseq;      // peer exchange: sequence number of this rank's last published candidate
};
static_assert(sizeof(Ctl) <= CS_CTL_BYTES, "control block too large");
static_assert(sizeof(cs_ctl_view) == CS_CTL_BYTES, "cs_ctl_view must span the control block");

enum { ST_CAPACITY = 1, ST_FORCE_NOT_OWNED = 2, ST_XCHG_TIMEOUT = 3, ST_PIPE_TIMEOUT = 4 };

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr unsigned kFull = 0xffffffffu;
#ifndef CS_RPL
#define CS_RPL 4
#endif
constexpr int kRowsPerLane = CS_RPL;     // a warp walks super-tiles of 32 * kRowsPerLane consecutive rows (4 or 2)
constexpr int kTileShift = CS_RPL == 4 ? 7 : 6;
static_assert(CS_RPL == 4 || CS_RPL == 2, "rows per lane");
#ifndef CS_INFLIGHT
#define CS_INFLIGHT 8
#endif
#ifndef CS_MIN_BLOCKS
#define CS_MIN_BLOCKS 3                  // resident blocks per SM the step kernel is compiled for
#endif
constexpr int kInflight = CS_INFLIGHT;   // independent 16-byte row loads per lane in flight

thread_local cudaError_t g_last_cuda = cudaSuccess;

// ---- order-preserving key ---------------------------------------------------------------
// Larger h wins, equal h -> smaller global index wins (argmax_better, _shared.cuh:24-27).
// key = orderable(h) << 32 | (0xFFFFFFFF - global_idx); max over keys is associative and
// commutative, so warp / block / grid / cross-rank reduction order cannot change the winner.
// key 0 means "no candidate" (empty shard; reference: (-inf, -1), multi.cu:283-292).
__device__ __forceinline__ unsigned f2ord(float h) {
    unsigned b = __float_as_uint(h);
    if (h == 0.0f) b = 0u;                 // -0.0 and +0.0 compare equal in the reference
    if (h != h) return 1u;                 // NaN never wins a reference comparison
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float ord2f(unsigned o) {
    unsigned b = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
    return __uint_as_float(b);
}
__device__ __forceinline__ u64 make_key(float h, int64_t gidx) {
    return ((u64)f2ord(h) << 32) | (u64)(0xffffffffu - (unsigned)gidx);
}
__device__ __forceinline__ float key_val(u64 k) {
    return k ? ord2f((unsigned)(k >> 32)) : __uint_as_float(0xff800000u);
}
__device__ __forceinline__ int64_t key_idx(u64 k) {
    return k ? (int64_t)(0xffffffffu - (unsigned)(k & 0xffffffffu)) : (int64_t)-1;
}
__device__ __forceinline__ u64 warp_max_key(u64 k) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        u64 o = __shfl_xor_sync(kFull, k, off);
        k = o > k ? o : k;
    }
    return k;
}

// ---- the reference's dot product ---------------------------------------------------------
// One float4 chunk: a.x*b.x + a.y*b.y + a.z*b.z + a.w*b.w as the reference's compiler
// contracts it (_shared.cuh:49): mul on .y, then fma on .x, .z, .w.
__device__ __forceinline__ float chunk_dot(const float4 a, const float4 b) {
    float t = __fmul_rn(a.y, b.y);
    t = __fmaf_rn(a.x, b.x, t);
    t = __fmaf_rn(a.z, b.z, t);
    t = __fmaf_rn(a.w, b.w, t);
    return t;
}
// The 5-round tree of warp.cu:35-37.  A xor butterfly gives every lane the value lane 0 gets
// from the reference's shfl_down tree, because fp32 addition is commutative.
__device__ __forceinline__ float warp_tree_sum(float p) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) p = __fadd_rn(p, __shfl_xor_sync(kFull, p, off));
    return p;
}
// d = norms[row] + norm_new - 2*dot (warp.cu:41-42); 2*dot is exact.
__device__ __forceinline__ float sq_dist(float n_row, float n_new, float dot) {
    return __fsub_rn(__fadd_rn(n_row, n_new), __fadd_rn(dot, dot));
}

__device__ __forceinline__ float4 ld_stream4(const float4* p) { return __ldcs(p); }

// Generic warp dot: row in global memory, centre anywhere (shared or global); any D.
__device__ __forceinline__ float warp_dot_generic(const float* __restrict__ row,
                                                  const float* __restrict__ cen, int D, int lane,
                                                  bool element_order) {
    float acc = 0.0f;
    if ((D & 3) == 0 && !element_order) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const float4* c4 = reinterpret_cast<const float4*>(cen);
        const int d4 = D >> 2;
        for (int c = lane; c < d4; c += 32) acc = __fadd_rn(acc, chunk_dot(__ldg(r4 + c), c4[c]));
    } else {
        for (int c = lane; c < D; c += 32) acc = __fmaf_rn(__ldg(row + c), cen[c], acc);
    }
    return warp_tree_sum(acc);
}

// ---- candidate exchange ---------------------------------------------------------------------
// xchg == CS_XCHG_GATHER: the candidate goes to pack_local and the caller all-gathers it.
// xchg == CS_XCHG_PEER:   the publishing block stores the candidate straight into every rank's
// exchange window over NVLink (plain peer stores) and then raises a per-rank flag with the
// sequence number; consumers spin on the flags in their OWN memory.  Window layout (32-bit words):
//   flags [2][W] padded to 64 words, then packs [2][W][stride], stride = 4 + D rounded up to 4.
// Parity = sequence number & 1.  A rank publishes sequence s+1 only after it consumed s, which
// needed every peer's s, which they published after consuming s-1: two buffers are enough.
__device__ __forceinline__ int xchg_stride(int D) { return (4 + D + 3) & ~3; }
constexpr int kFlagWords = 64;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// All threads of ONE block call this.  k == 0 publishes "nothing"; l is the local row of the key.
__device__ void publish_candidate(const cs_state& s, Ctl* ctl, const u64 k, const int64_t l) {
    const int D = s.D;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(s.X + (k ? l : 0) * (int64_t)D);
    const uint32_t norm_bits = k ? __float_as_uint(s.norms[l]) : 0u;
    if (s.xchg == CS_XCHG_GATHER) {
        uint32_t* p = s.pack_local;
        if (threadIdx.x == 0) {
            p[0] = (uint32_t)(k & 0xffffffffu);
            p[1] = (uint32_t)(k >> 32);
            p[2] = norm_bits;
            p[3] = 0u;
        }
        for (int c = threadIdx.x; c < D; c += blockDim.x) p[4 + c] = k ? src[c] : 0u;
        return;
    }
    const unsigned seq = ctl->xseq + 1u;
    const int par = (int)(seq & 1u);
    const int W = s.world_size, stride = xchg_stride(D);
    for (int q = 0; q < W; ++q) {
        uint32_t* p = s.peer_win[q] + kFlagWords + ((int64_t)par * W + s.rank) * stride;
        if (threadIdx.x == 0) {
            p[0] = (uint32_t)(k & 0xffffffffu);
            p[1] = (uint32_t)(k >> 32);
            p[2] = norm_bits;
            p[3] = 0u;
        }
        for (int c = threadIdx.x; c < D; c += blockDim.x) p[4 + c] = k ? src[c] : 0u;
    }
    __threadfence_system();              // every writer orders its stores before the barrier
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int q = 0; q < W; ++q) {
            volatile uint32_t* f = s.peer_win[q] + par * W + s.rank;
            *f = seq;
        }
        ctl->xseq = seq;
    }
}

// Thread 0 of a block waits until every rank's candidate with this rank's current sequence
// number has landed in the local window; bounded by xchg_timeout_ms, after which the status
// word records the time-out and the kernel carries on (the host reads the status).
// Returns the base of the packs to read.
__device__ const uint32_t* await_candidates(const cs_state& s, Ctl* ctl) {
    if (s.xchg == CS_XCHG_GATHER || s.world_size <= 1) return s.pack_all;
    const unsigned seq = ctl->xseq;
    const int par = (int)(seq & 1u);
    const int W = s.world_size;
    uint32_t* win = s.peer_win[s.rank];
    if (threadIdx.x == 0) {
        const unsigned long long t0 = global_ns();
        const unsigned long long limit = (unsigned long long)(s.xchg_timeout_ms > 0 ? s.xchg_timeout_ms : 10000) * 1000000ull;
        for (int r = 0; r < W; ++r) {
            volatile uint32_t* f = win + par * W + r;
            unsigned spins = 0;
            while (*f != seq) {
                if ((++spins & 0xffu) == 0 && global_ns() - t0 > limit) {
                    ctl->status = ST_XCHG_TIMEOUT;
                    break;
                }
            }
        }
        __threadfence_system();
    }
    __syncthreads();
    return win + kFlagWords + (int64_t)par * W * xchg_stride(s.D);
}

__global__ void xchg_wait_kernel(const cs_state s) {
    (void)await_candidates(s, reinterpret_cast<Ctl*>(s.ctl));
}

// ---- winner resolution shared by commit_bound and sim_final_check -------------------------
struct Winner {
    u64 key;
    const float* row;   // D floats (in X or in the gathered packs)
    float norm;
};
__device__ __forceinline__ Winner resolve_winner(const cs_state& s, const Ctl* ctl, int i, const uint32_t* packs) {
    Winner w;
    w.row = nullptr;
    w.norm = 0.0f;
    if (s.world_size <= 1) {
        w.key = ctl->key[i & 1];
        if (w.key) {
            int64_t l = key_idx(w.key) - s.shard_offset;
            w.row = s.X + l * (int64_t)s.D;
            w.norm = s.norms[l];
        }
    } else {
        const int stride = (s.xchg == CS_XCHG_PEER) ? xchg_stride(s.D) : 4 + s.D;
        w.key = 0;
        int br = -1;
        for (int r = 0; r < s.world_size; ++r) {
            const uint32_t* p = packs + (int64_t)r * stride;
            u64 k = (u64)p[0] | ((u64)p[1] << 32);
            if (k > w.key) { w.key = k; br = r; }
        }
        if (br >= 0) {
            const uint32_t* p = packs + (int64_t)br * stride;
            w.norm = __uint_as_float(p[2]);
            w.row = reinterpret_cast<const float*>(p + 4);
        }
    }
    return w;
}

// ---- kernel A: resolve + commit + triangle bounds ------------------------------------------
__global__ void __launch_bounds__(kThreads) commit_bound_kernel(const cs_state s, const unsigned rules) {
    extern __shared__ __align__(16) float s_cen[];
    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    if (i >= s.cap) {
        if (blockIdx.x == 0 && threadIdx.x == 0) ctl->status = ST_CAPACITY;
        return;
    }
    const uint32_t* packs = await_candidates(s, ctl);
    const Winner w = resolve_winner(s, ctl, i, packs);
    const float val = key_val(w.key);
    const int64_t gidx = key_idx(w.key);
    const int D = s.D;

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
            for (int c = threadIdx.x; c < D; c += blockDim.x) dst[c] = w.row[c];
        }
    }
    if (gidx < 0 || i == 0) return;

    // dSL_quarter[v] = |X_sel[v] - x_new|^2 / 4 for every old centre (commit.cu:69-102)
    for (int c = threadIdx.x; c < D; c += blockDim.x) s_cen[c] = w.row[c];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int gw = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int nw = gridDim.x * kWarps;
    for (int v = gw; v < i; v += nw) {
        float dot = warp_dot_generic(s.X_sel + (int64_t)v * D, s_cen, D, lane, (s.flags & CS_F_ELEMENT_ORDER) != 0);
        if (lane == 0) s.dSL_quarter[v] = __fmul_rn(sq_dist(s.norms_sel[v], w.norm, dot), 0.25f);
    }
}

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
                    float p = warp_dot_generic(s.X + (base + j + (int64_t)r * kRowsPerLane) * (int64_t)D, s_cen, D, lane, element_order);
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

// ---- small single-block kernels ---------------------------------------------------------------
__global__ void init_state_kernel(float* h, int32_t* v, int64_t N, Ctl* ctl) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < N; r += stride) {
        h[r] = __uint_as_float(0x7f800000u);
        v[r] = 0;
    }
    // the exchange sequence number outlives a re-initialisation: peers' flags still hold old values
    if (blockIdx.x == 0 && threadIdx.x < CS_CTL_BYTES / 4 && threadIdx.x != offsetof(Ctl, xseq) / 4)
        reinterpret_cast<uint32_t*>(ctl)[threadIdx.x] = 0u;
}

__global__ void reset_ctl_kernel(Ctl* ctl, int n_sel) {
    if (threadIdx.x < CS_CTL_BYTES / 4 && threadIdx.x != offsetof(Ctl, xseq) / 4)
        reinterpret_cast<uint32_t*>(ctl)[threadIdx.x] = 0u;
    __syncthreads();
    if (threadIdx.x == 0) ctl->n_sel = n_sel;
}

__global__ void force_pick_kernel(const cs_state s, const int64_t gidx, const float val) {
    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    const int64_t l = gidx - s.shard_offset;
    const bool owner = (l >= 0 && l < s.N_local);
    const u64 k = owner ? make_key(val, gidx) : 0;
    if (threadIdx.x == 0) {
        ctl->key[i & 1] = k;
        if (s.world_size <= 1 && !owner) ctl->status = ST_FORCE_NOT_OWNED;
    }
    if (s.world_size > 1) publish_candidate(s, ctl, k, l);
}

__global__ void sim_begin_kernel(Ctl* ctl, float sep) {
    ctl->viable = 0;
    ctl->steps = 0;
    ctl->sep = sep;
}

__global__ void sim_final_check_kernel(const cs_state s) {
    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const uint32_t* packs = await_candidates(s, ctl);
    const Winner w = resolve_winner(s, ctl, ctl->n_sel, packs);
    if (ctl->sep > key_val(w.key)) ctl->viable = 1;   // argmax.cu:152-159, multi.cu:369-384
}

// ---- arg-max only: recompute the key of the NEXT pick from the current h --------------------
// Needed whenever h was changed behind the step kernel's back (roll-back to a snapshot, a
// reconstructed bisect state) and for "global max h" queries.  Same key, same pack as fps_step.
__global__ void scan_reset_kernel(Ctl* ctl) { ctl->key[ctl->n_sel & 1] = 0; }

__global__ void __launch_bounds__(kThreads) scan_argmax_kernel(const cs_state s) {
    __shared__ u64 s_keys[kWarps];
    __shared__ int s_last;
    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int slot = ctl->n_sel & 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    u64 best = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < s.N_local; r += stride) {
        const u64 k = make_key(s.h[r], s.shard_offset + r);
        best = k > best ? k : best;
    }
    best = warp_max_key(best);
    if (lane == 0) s_keys[warp] = best;
    __syncthreads();
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
    if (threadIdx.x == 0) ctl->ticket = 0;
}

// ---- host side ---------------------------------------------------------------------------------
struct DevInfo {
    int sms = 0;
    int cc_major = 0;
    bool ok = false;
};
DevInfo device_info() {
    static thread_local int cached_dev = -1;
    static thread_local DevInfo info;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return DevInfo();
    if (dev != cached_dev) {
        DevInfo d;
        if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return DevInfo();
        if (cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return DevInfo();
        d.ok = true;
        info = d;
        cached_dev = dev;
    }
    return info;
}

// ---- exact selection: k-th largest live entry of h ---------------------------------------------
// Radix select over the bit patterns of the non-negative floats (monotone as unsigned integers;
// -0.0 counts as 0), most significant byte first.  Each pass histograms the byte under the prefix
// found so far; the last block to finish picks the bucket that holds the k-th largest.
struct SelectCtl {
    cs_select_result res;          // what the host reads
    unsigned prefix;               // leading bytes of the answer found so far
    unsigned k_rem;                // rank of the answer among the entries that share the prefix
    unsigned ticket;
    unsigned pad;
    unsigned hist[4][256];
};
static_assert(sizeof(SelectCtl) <= CS_SELECT_SCRATCH_BYTES, "selection scratch");

__global__ void select_init_kernel(SelectCtl* c, unsigned k) {
    for (int i = threadIdx.x; i < 4 * 256; i += blockDim.x) (&c->hist[0][0])[i] = 0u;
    if (threadIdx.x == 0) {
        c->res.value = 0.0f;
        c->res.valid = 0;
        c->res.n_alive = 0;
        c->prefix = 0u;
        c->k_rem = k;
        c->ticket = 0u;
    }
}

template <int PASS>
__global__ void __launch_bounds__(kThreads) select_pass_kernel(const float* __restrict__ h, const int64_t n, SelectCtl* c) {
    __shared__ unsigned s_hist[256];
    __shared__ int s_last;
    s_hist[threadIdx.x] = 0u;                          // kThreads == 256
    __syncthreads();
    if (PASS > 0 && c->res.valid == 0 && c->k_rem == 0u) return;   // pass 0 found k out of range (uniform)
    constexpr int shift = 24 - 8 * PASS;
    constexpr unsigned hi_mask = PASS == 0 ? 0u : (0xffffffffu << (32 - 8 * PASS));
    const unsigned prefix = c->prefix;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t base = (int64_t)blockIdx.x * blockDim.x; base < n; base += stride) {   // block-uniform trip count
        const int64_t r = base + threadIdx.x;
        const float v = r < n ? h[r] : -1.0f;
        const bool alive = v >= 0.0f;                  // false for selected rows (-1) and NaN
        const unsigned key = (v == 0.0f) ? 0u : __float_as_uint(v);
        const bool hit = alive && ((key & hi_mask) == prefix);
        const unsigned bin = (key >> shift) & 255u;
        // one shared-memory atomic per distinct bin of the warp
        const unsigned act = __ballot_sync(kFull, hit);
        if (hit) {
            const unsigned peers = __match_any_sync(act, bin);
            if ((int)(__ffs(peers) - 1) == (int)(threadIdx.x & 31)) atomicAdd(&s_hist[bin], (unsigned)__popc(peers));
        }
    }
    __syncthreads();
    if (s_hist[threadIdx.x]) atomicAdd(&c->hist[PASS][threadIdx.x], s_hist[threadIdx.x]);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(&c->ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) {
        const volatile unsigned* hist = c->hist[PASS];
        unsigned k = c->k_rem;
        if (PASS == 0) {
            unsigned long long total = 0;
            for (int b = 0; b < 256; ++b) total += hist[b];
            c->res.n_alive = (int64_t)total;
            if (k == 0u || (unsigned long long)k > total) k = 0u;      // out of range: later passes do nothing
        }
        if (k != 0u) {
            unsigned above = 0u;
            int b = 255;
            for (; b > 0; --b) {
                const unsigned cnt = hist[b];
                if (above + cnt >= k) break;
                above += cnt;
            }
            c->prefix = prefix | ((unsigned)b << shift);
            c->k_rem = k - above;
            if (PASS == 3) {
                c->res.value = __uint_as_float(c->prefix);
                c->res.valid = 1;
            }
        } else {
            c->k_rem = 0u;
        }
        c->ticket = 0u;
    }
}

// ---- arg-max of h over a list of rows (accretion forward loop) --------------------------------
__global__ void __launch_bounds__(kThreads) pool_argmax_kernel(const float* __restrict__ h, const int64_t* __restrict__ pool,
                                                               const int64_t n_pool, const int64_t lo, const int64_t n_local,
                                                               u64* out_key) {
    __shared__ u64 s_keys[kWarps];
    u64 best = 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n_pool; j += stride) {
        const int64_t p = pool[j];
        if (p >= lo && p < lo + n_local) {
            const u64 k = make_key(h[p - lo], p);
            best = k > best ? k : best;
        }
    }
    best = warp_max_key(best);
    if ((threadIdx.x & 31) == 0) s_keys[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 bk = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) bk = s_keys[w] > bk ? s_keys[w] : bk;
        if (bk) atomicMax(out_key, bk);
    }
}

int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda = e;
        return CS_E_LAUNCH;
    }
    return CS_OK;
}

int validate(const cs_state* s) {
    if (!s || !s->ctl || !s->X_sel || !s->norms_sel || !s->dSL_quarter) return CS_E_ARG;
    if (s->N_local < 0 || s->D <= 0 || s->cap <= 0 || s->world_size < 1 || s->shard_offset < 0) return CS_E_ARG;
    if (s->N_local > 0 && (!s->X || !s->norms || !s->h || !s->voronoi)) return CS_E_ARG;
    if (s->xchg != CS_XCHG_GATHER && s->xchg != CS_XCHG_PEER) return CS_E_ARG;
    if (s->world_size > 1 && s->xchg == CS_XCHG_GATHER && (!s->pack_local || !s->pack_all)) return CS_E_ARG;
    if (s->world_size > 1 && s->xchg == CS_XCHG_PEER) {
        if (s->world_size > CS_MAX_PEERS || s->rank < 0 || s->rank >= s->world_size) return CS_E_ARG;
        for (int r = 0; r < s->world_size; ++r)
            if (!s->peer_win[r] || ((uintptr_t)s->peer_win[r] & 15u)) return CS_E_ARG;
    }
    if (s->shard_offset + s->N_local >= (int64_t)1 << 31) return CS_E_RANGE;
    if (s->cap >= (int64_t)1 << 31) return CS_E_RANGE;
    if ((s->D & 3) == 0) {
        if (((uintptr_t)s->X | (uintptr_t)s->X_sel) & 15u) return CS_E_ALIGN;
        if (s->world_size > 1 && s->xchg == CS_XCHG_GATHER &&
            (((uintptr_t)s->pack_local | (uintptr_t)s->pack_all) & 15u)) return CS_E_ALIGN;
    }
    return CS_OK;
}

template <int CPL, bool HALF, int S, int B, int T, int W>
int launch_step_tma(const cs_state* s, cudaStream_t st, int sms) {
    static_assert(W <= kTmaMaxWarps && (W % 8) == 0, "consumer warps");
    const int D = s->D;
    int tile_rows = T / (D * 4);
    tile_rows = tile_rows > 32 * W ? 32 * W : tile_rows;   // a lane owns one row of its warp's share
    tile_rows -= tile_rows % W;                             // W is a multiple of 8: 16-byte multiples of h / voronoi / norms
    if (tile_rows < W) tile_rows = W;
    const size_t smem = (size_t)S * tile_rows * (D * 4 + 12);   // rows of X, then h / voronoi / norm words
    static thread_local size_t attr_set = 0;
    if (smem > attr_set) {
        if (cudaFuncSetAttribute(fps_step_tma_kernel<CPL, S, HALF, W, B>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) {
            g_last_cuda = cudaGetLastError();
            return CS_E_LAUNCH;
        }
        attr_set = smem;
    }
    const int64_t ntiles = (s->N_local + tile_rows - 1) / tile_rows;
    int64_t cap = (int64_t)sms * B;                         // resident blocks, each with its own ring
    int grid = (int)(ntiles < 1 ? 1 : (ntiles < cap ? ntiles : cap));
    fps_step_tma_kernel<CPL, S, HALF, W, B><<<grid, (W + 1) * 32, smem, st>>>(*s, tile_rows);
    return check_launch();
}

constexpr int kBoundSmemMax = 16384;     // triangle bounds staged in shared memory (64 KB)

template <int CPL, bool FULL, bool HALF = false>
int launch_step(const cs_state* s, unsigned mode, cudaStream_t st, int sms) {
    static thread_local size_t attr_set = 0, occ_smem = ~(size_t)0;
    static thread_local int occ_blocks = 0;
    const int n_bound = (int)(s->cap < kBoundSmemMax ? s->cap : kBoundSmemMax);
    const size_t smem = ((size_t)((n_bound + 3) & ~3) + (CPL ? 0 : (size_t)s->D)) * sizeof(float);
    if (smem > 48 * 1024 && smem > attr_set) {
        if (cudaFuncSetAttribute(fps_step_kernel<CPL, FULL, HALF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) {
            g_last_cuda = cudaGetLastError();
            return CS_E_LAUNCH;
        }
        attr_set = smem;
    }
    if (occ_smem != smem) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fps_step_kernel<CPL, FULL, HALF>, kThreads, smem) !=
                cudaSuccess || per_sm < 1) {
            g_last_cuda = cudaGetLastError();
            return CS_E_LAUNCH;
        }
        occ_blocks = per_sm;
        occ_smem = smem;
    }
    const int64_t tiles = (s->N_local + (32 * kRowsPerLane - 1)) >> kTileShift;
    int64_t want = (tiles + kWarps - 1) / kWarps;
    int64_t cap = (int64_t)sms * occ_blocks;     // persistent grid: a multiple of the SM count
    int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    fps_step_kernel<CPL, FULL, HALF><<<grid, kThreads, smem, st>>>(*s, mode, n_bound);
    return check_launch();
}

// prune mode with deferred rows (rows in whole 16-byte chunks, D <= 1024)
template <int CPL, bool FULL, bool HALF = false>
int launch_step_queue(const cs_state* s, cudaStream_t st, int sms) {
    static thread_local size_t attr_set = 0, occ_smem = ~(size_t)0;
    static thread_local int occ_blocks = 0;
    const int n_bound = (int)(s->cap < kBoundSmemMax ? s->cap : kBoundSmemMax);
    const size_t smem = ((size_t)kScanRingFloats + (size_t)((n_bound + 3) & ~3) + (CPL ? 0 : (size_t)s->D)) * sizeof(float);
    if (smem > attr_set) {
        if (cudaFuncSetAttribute(fps_step_queue_kernel<CPL, FULL, HALF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess) {
            g_last_cuda = cudaGetLastError();
            return CS_E_LAUNCH;
        }
        attr_set = smem;
    }
    if (occ_smem != smem) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fps_step_queue_kernel<CPL, FULL, HALF>, kThreads,
                                                          smem) != cudaSuccess || per_sm < 1) {
            g_last_cuda = cudaGetLastError();
            return CS_E_LAUNCH;
        }
        occ_blocks = per_sm;
        occ_smem = smem;
    }
    const int64_t tiles = (s->N_local + 127) >> 7;
    int64_t want = (tiles + kWarps - 1) / kWarps;
    int64_t cap = (int64_t)sms * occ_blocks;     // persistent grid: a multiple of the SM count
    int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    fps_step_queue_kernel<CPL, FULL, HALF><<<grid, kThreads, smem, st>>>(*s, n_bound);
    return check_launch();
}

template <int L, int CPL>
int launch_lanes_t(const LaneSet& ls, unsigned mode, cudaStream_t st, int sms) {
    const size_t smem = (size_t)L * ls.s[0].D * sizeof(float);
    static thread_local int per_sm = 0;
    if (per_sm == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fps_step_lanes_kernel<L, CPL>, kThreads, smem) !=
                cudaSuccess || per_sm < 1) {
            g_last_cuda = cudaGetLastError();
            per_sm = 0;
            return CS_E_LAUNCH;
        }
    }
    const int64_t tiles = (ls.s[0].N_local + 31) >> 5;
    int64_t want = (tiles + kWarps - 1) / kWarps;
    int64_t cap = (int64_t)sms * per_sm;
    int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    fps_step_lanes_kernel<L, CPL><<<grid, kThreads, smem, st>>>(ls, mode);
    return check_launch();
}

template <int L>
int launch_lanes_l(const LaneSet& ls, unsigned mode, cudaStream_t st, int sms) {
    const int D = ls.s[0].D;
    if (D <= 128) return launch_lanes_t<L, 1>(ls, mode, st, sms);
    if (D <= 256) return launch_lanes_t<L, 2>(ls, mode, st, sms);
    if (D <= 512) return launch_lanes_t<L, 4>(ls, mode, st, sms);
    return launch_lanes_t<L, 8>(ls, mode, st, sms);
}

int launch_lanes(const LaneSet& ls, int n, unsigned mode, cudaStream_t st, int sms) {
    switch (n) {
        case 2: return launch_lanes_l<2>(ls, mode, st, sms);
        case 3: return launch_lanes_l<3>(ls, mode, st, sms);
        case 4: return launch_lanes_l<4>(ls, mode, st, sms);
        case 5: return launch_lanes_l<5>(ls, mode, st, sms);
        case 6: return launch_lanes_l<6>(ls, mode, st, sms);
        case 7: return launch_lanes_l<7>(ls, mode, st, sms);
        case 8: return launch_lanes_l<8>(ls, mode, st, sms);
        default: return CS_E_ARG;
    }
}

}  // namespace

extern "C" {

int cs_version(void) { return CS_ABI_VERSION; }

const char* cs_error_string(int code) {
    switch (code) {
        case CS_OK: return "ok";
        case CS_E_ARG: return "invalid argument (null pointer, negative size or unknown flag)";
        case CS_E_ALIGN: return "X, X_sel and the packs must be 16-byte aligned when D is a multiple of 4";
        case CS_E_RANGE: return "global row index space or capacity must stay below 2^31";
        case CS_E_LAUNCH: return "CUDA launch failed (see cs_last_cuda_error)";
        case CS_E_DEVICE: return "no CUDA device of compute capability 10.x is current";
        case CS_E_SCRATCH: return "row length exceeds CS_NOALLOC_MAX_D, the fixed scratch of cs_fps_step_noalloc";
        default: return "unknown error code";
    }
}

const char* cs_last_cuda_error(void) { return cudaGetErrorString(g_last_cuda); }

int cs_device_check(void) {
    DevInfo d = device_info();
    if (!d.ok || d.cc_major != 10) return CS_E_DEVICE;
    return d.sms;
}

int cs_init_state(const cs_state* s, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    DevInfo d = device_info();
    if (!d.ok) return CS_E_DEVICE;
    int64_t want = (s->N_local + 1023) / 1024;
    int grid = (int)(want < 1 ? 1 : (want < (int64_t)d.sms * 8 ? want : (int64_t)d.sms * 8));
    init_state_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(s->h, s->voronoi, s->N_local,
                                                              reinterpret_cast<Ctl*>(s->ctl));
    return check_launch();
}

int cs_reset_ctl(const cs_state* s, int32_t n_sel, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    if (n_sel < 0 || n_sel > s->cap) return CS_E_ARG;
    reset_ctl_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(reinterpret_cast<Ctl*>(s->ctl), n_sel);
    return check_launch();
}

int cs_force_pick(const cs_state* s, int64_t global_idx, float val, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    if (global_idx < 0 || global_idx >= (int64_t)1 << 31) return CS_E_RANGE;
    force_pick_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(*s, global_idx, val);
    return check_launch();
}

int cs_commit_bound(const cs_state* s, uint32_t rules, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    if (rules > CS_RULE_SIM_SHARDED) return CS_E_ARG;
    DevInfo d = device_info();
    if (!d.ok) return CS_E_DEVICE;
    const size_t smem = (size_t)s->D * sizeof(float);
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(commit_bound_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess) {
            g_last_cuda = cudaGetLastError();
            return CS_E_LAUNCH;
        }
    }
    // enough warps for one centre per warp up to the capacity, at most two blocks per SM
    int64_t want = (s->cap + kWarps - 1) / kWarps;
    int64_t lim = (int64_t)d.sms * 2;
    int grid = (int)(want < 1 ? 1 : (want < lim ? want : lim));
    commit_bound_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(*s, rules);
    return check_launch();
}

int cs_fps_step(const cs_state* s, uint32_t mode, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    if (mode != CS_MODE_PRUNE && mode != CS_MODE_DENSE && mode != CS_MODE_DENSE_LDG && mode != CS_MODE_PRUNE_INLINE)
        return CS_E_ARG;
    DevInfo d = device_info();
    if (!d.ok) return CS_E_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    const int D = s->D;
    // dense mode streams X through the TMA ring when rows are whole 16-byte chunks of moderate width
    // bulk copies need 16-byte aligned sources; anything else takes the plain-load kernel
    const bool bulk_ok = (((uintptr_t)s->X | (uintptr_t)s->h | (uintptr_t)s->voronoi | (uintptr_t)s->norms) & 15u) == 0;
    const bool element_order = (s->flags & CS_F_ELEMENT_ORDER) != 0;
    if (mode == CS_MODE_DENSE && bulk_ok && !element_order && (D & 3) == 0 && D >= 32 && D <= 1024 && s->N_local > 0) {
        if (D <= 64) return launch_step_tma<1, true, kRingNarrow.stages, kRingNarrow.blocks, kRingNarrow.tile_bytes, kRingNarrow.warps>(s, st, d.sms);
        if (D <= 128) return launch_step_tma<1, false, kRingMid.stages, kRingMid.blocks, kRingMid.tile_bytes, kRingMid.warps>(s, st, d.sms);
        if (D <= 256) return launch_step_tma<2, false, kRingWide.stages, kRingWide.blocks, kRingWide.tile_bytes, kRingWide.warps>(s, st, d.sms);
        if (D <= 512) return launch_step_tma<4, false, kRingWide.stages, kRingWide.blocks, kRingWide.tile_bytes, kRingWide.warps>(s, st, d.sms);
        return launch_step_tma<8, false, kRingWide.stages, kRingWide.blocks, kRingWide.tile_bytes, kRingWide.warps>(s, st, d.sms);
    }
    const bool generic = element_order || (D & 3) != 0 || D > 1024;
    if (generic && mode == CS_MODE_PRUNE && s->N_local > 0 && D <= 16384) return launch_step_queue<0, false>(s, st, d.sms);
    if (generic) return launch_step<0, false>(s, mode, st, d.sms);
    if (mode == CS_MODE_PRUNE && s->N_local > 0) {
        switch (D) {
            case 128: return launch_step_queue<1, true>(s, st, d.sms);
            case 256: return launch_step_queue<2, true>(s, st, d.sms);
            case 512: return launch_step_queue<4, true>(s, st, d.sms);
            case 1024: return launch_step_queue<8, true>(s, st, d.sms);
            default: break;
        }
        if (D <= 64) return launch_step_queue<1, false, true>(s, st, d.sms);
        if (D < 128) return launch_step_queue<1, false>(s, st, d.sms);
        if (D < 256) return launch_step_queue<2, false>(s, st, d.sms);
        if (D < 512) return launch_step_queue<4, false>(s, st, d.sms);
        return launch_step_queue<8, false>(s, st, d.sms);
    }
    switch (D) {
        case 128: return launch_step<1, true>(s, mode, st, d.sms);
        case 256: return launch_step<2, true>(s, mode, st, d.sms);
        case 512: return launch_step<4, true>(s, mode, st, d.sms);
        case 1024: return launch_step<8, true>(s, mode, st, d.sms);
        default: break;
    }
    if (D <= 64) return launch_step<1, false, true>(s, mode, st, d.sms);    // two rows per warp-wide load
    if (D < 128) return launch_step<1, false>(s, mode, st, d.sms);
    if (D < 256) return launch_step<2, false>(s, mode, st, d.sms);
    if (D < 512) return launch_step<4, false>(s, mode, st, d.sms);
    return launch_step<8, false>(s, mode, st, d.sms);
}

int cs_sim_begin(const cs_state* s, float sep, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    sim_begin_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(reinterpret_cast<Ctl*>(s->ctl), sep);
    return check_launch();
}

int cs_sim_final_check(const cs_state* s, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    sim_final_check_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(*s);
    return check_launch();
}

int64_t cs_xchg_window_words(int32_t world_size, int32_t D) {
    if (world_size < 1 || D < 1) return CS_E_ARG;
    return (int64_t)kFlagWords + 2 * (int64_t)world_size * (int64_t)((4 + D + 3) & ~3);
}

int cs_xchg_wait(const cs_state* s, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    xchg_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(*s);
    return check_launch();
}

int cs_scan_argmax(const cs_state* s, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    DevInfo d = device_info();
    if (!d.ok) return CS_E_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    scan_reset_kernel<<<1, 1, 0, st>>>(reinterpret_cast<Ctl*>(s->ctl));
    rc = check_launch();
    if (rc) return rc;
    int64_t want = (s->N_local + 4 * kThreads - 1) / (4 * kThreads);
    int64_t lim = (int64_t)d.sms * 8;
    int grid = (int)(want < 1 ? 1 : (want < lim ? want : lim));
    scan_argmax_kernel<<<grid, kThreads, 0, st>>>(*s);
    return check_launch();
}

int cs_pool_argmax(const float* h, const int64_t* pool, int64_t n_pool, int64_t shard_offset, int64_t n_local,
                   uint64_t* out_key, cs_stream stream) {
    if (!out_key || n_pool < 0 || n_local < 0 || (n_pool > 0 && !pool) || (n_local > 0 && !h)) return CS_E_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(out_key, 0, sizeof(uint64_t), st) != cudaSuccess) {
        g_last_cuda = cudaGetLastError();
        return CS_E_LAUNCH;
    }
    if (n_pool == 0 || n_local == 0) return CS_OK;
    int64_t want = (n_pool + kThreads - 1) / kThreads;
    const int grid = (int)(want > 1024 ? 1024 : want);
    pool_argmax_kernel<<<grid, kThreads, 0, st>>>(h, pool, n_pool, shard_offset, n_local, reinterpret_cast<u64*>(out_key));
    return check_launch();
}

int cs_select_kth_largest(const float* h, int64_t n, int64_t k, void* scratch, cs_stream stream) {
    if (!scratch || n < 0 || n > 0x7fffffffLL || (n > 0 && !h)) return CS_E_ARG;
    DevInfo d = device_info();
    if (!d.ok) return CS_E_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    SelectCtl* c = reinterpret_cast<SelectCtl*>(scratch);
    const unsigned k32 = (k >= 1 && k <= n) ? (unsigned)k : 0u;       // 0 = out of range: only the count is produced
    select_init_kernel<<<1, kThreads, 0, st>>>(c, k32);
    int64_t want = (n + kThreads * 8 - 1) / (kThreads * 8);
    int64_t cap = (int64_t)d.sms * 8;
    const int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    select_pass_kernel<0><<<grid, kThreads, 0, st>>>(h, n, c);
    select_pass_kernel<1><<<grid, kThreads, 0, st>>>(h, n, c);
    select_pass_kernel<2><<<grid, kThreads, 0, st>>>(h, n, c);
    select_pass_kernel<3><<<grid, kThreads, 0, st>>>(h, n, c);
    return check_launch();
}

int cs_fps_step_lanes(const cs_state* lanes, int32_t n_lanes, uint32_t mode, cs_stream stream) {
    if (!lanes || n_lanes < 1 || n_lanes > CS_MAX_LANES) return CS_E_ARG;
    if (mode != CS_MODE_PRUNE && mode != CS_MODE_DENSE && mode != CS_MODE_PRUNE_INLINE) return CS_E_ARG;
    for (int l = 0; l < n_lanes; ++l) {
        int rc = validate(&lanes[l]);
        if (rc) return rc;
        if (lanes[l].X != lanes[0].X || lanes[l].norms != lanes[0].norms || lanes[l].N_local != lanes[0].N_local ||
            lanes[l].D != lanes[0].D || lanes[l].shard_offset != lanes[0].shard_offset || lanes[l].flags != lanes[0].flags)
            return CS_E_ARG;                   // lanes share the matrix; only their state differs
    }
    const int D = lanes[0].D;
    // Default prune mode: one deferred-row step per lane.  Sharing the pass over X pays when most
    // rows are read (dense mode); in prune mode the rows are a minor part of the traffic and the
    // per-lane kernel is several times faster than the fused walk (measured 0.43 ms against
    // 1.62 ms per lock-step pick of four lanes on 37.5 M x 128).
    // Also per lane: one lane, rows that are not 16-byte chunks, very wide rows.
    if (mode == CS_MODE_PRUNE || n_lanes == 1 || (lanes[0].flags & CS_F_ELEMENT_ORDER) || (D & 3) != 0 || D > 1024 ||
        lanes[0].N_local == 0) {
        for (int l = 0; l < n_lanes; ++l) {
            int rc = cs_fps_step(&lanes[l], mode, stream);
            if (rc) return rc;
        }
        return CS_OK;
    }
    DevInfo d = device_info();
    if (!d.ok) return CS_E_DEVICE;
    LaneSet ls;
    for (int l = 0; l < n_lanes; ++l) ls.s[l] = lanes[l];
    for (int l = n_lanes; l < CS_MAX_LANES; ++l) ls.s[l] = lanes[0];
    return launch_lanes(ls, n_lanes, mode, (cudaStream_t)stream, d.sms);
}

}  // extern "C"

// ---- allocation-free variant of the fused step -------------------------------------------------
// Some hosts of this library own every byte of device memory themselves and may not call
// cudaMalloc once they are running: a process that handed the whole HBM to its own arena when it
// started (a 150 GB matrix leaves little else), or a plug-in loaded into a service whose policy
// forbids driver allocations -- and the device-wide stall they cause -- on the request path.
// For them the scratch the step needs (the 256-byte control block plus a one-row centre table)
// lives in the fixed array below instead of in caller-allocated buffers.  Every GPU that loads
// the library holds these CS_NOALLOC_SCRATCH_BYTES until the process exits.
#define CS_NOALLOC_SCRATCH_BYTES (CS_CTL_BYTES + 256 + CS_NOALLOC_MAX_D * 4)
static __device__ __align__(256) unsigned char g_noalloc_scratch[CS_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
unsigned char* g_noalloc_ptr[kMaxDevices] = {nullptr};

// Device address of g_noalloc_scratch on the CURRENT device.  In host code the array's name is
// only a handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once per
// device while that device is current.
int noalloc_scratch(unsigned char** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return CS_E_DEVICE;
    if (!g_noalloc_ptr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            g_last_cuda = e;
            return CS_E_LAUNCH;
        }
        g_noalloc_ptr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_noalloc_ptr[dev];
    return CS_OK;
}

// The scratch keeps whatever the previous call left: zero the control block, then stage this
// call's centre (row + norm) and pick position.
__global__ void noalloc_prepare_kernel(unsigned char* scratch, const float* __restrict__ centre,
                                       const float norm_new, const int D, const int sel_pos) {
    Ctl* ctl = reinterpret_cast<Ctl*>(scratch);
    float* norm_slot = reinterpret_cast<float*>(scratch + CS_CTL_BYTES);
    float* row_slot = reinterpret_cast<float*>(scratch + CS_CTL_BYTES + 256);
    if (threadIdx.x < CS_CTL_BYTES / 4) reinterpret_cast<uint32_t*>(ctl)[threadIdx.x] = 0u;
    for (int c = threadIdx.x; c < D; c += blockDim.x) row_slot[c] = centre[c];
    __syncthreads();
    if (threadIdx.x == 0) {
        ctl->n_sel = sel_pos;
        norm_slot[0] = norm_new;
    }
}

__global__ void noalloc_publish_kernel(const unsigned char* scratch, const int sel_pos, u64* out_key,
                                       u64* out_live_rows) {
    const Ctl* ctl = reinterpret_cast<const Ctl*>(scratch);
    if (out_key) *out_key = ctl->key[(sel_pos + 1) & 1];
    if (out_live_rows) *out_live_rows = ctl->live_rows;
}

}  // namespace

extern "C" int cs_fps_step_noalloc(const float* X, const float* norms, float* h, int32_t* voronoi,
                                   int64_t N_local, int32_t D, int64_t shard_offset, const float* centre,
                                   float norm_new, const float* dSL_quarter, int32_t sel_pos, uint32_t mode,
                                   uint64_t* out_key, uint64_t* out_live_rows, cs_stream stream) {
    if (!X || !norms || !h || !voronoi || !centre || !out_key) return CS_E_ARG;
    if (N_local <= 0 || D <= 0 || sel_pos < 0 || shard_offset < 0 || mode > CS_MODE_DENSE) return CS_E_ARG;
    if (sel_pos > 0 && !dSL_quarter) return CS_E_ARG;
    if (D > CS_NOALLOC_MAX_D) return CS_E_SCRATCH;        // the centre would not fit the fixed scratch
    unsigned char* scratch = nullptr;
    int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;

    // A one-row centre table whose slot `sel_pos` is the staged row: the step kernel indexes
    // X_sel / norms_sel by the pick position, so the bases are set sel_pos rows before the slot.
    cs_state s;
    s.X = X;
    s.norms = norms;
    s.h = h;
    s.voronoi = voronoi;
    s.N_local = N_local;
    s.shard_offset = shard_offset;
    s.D = D;
    s.world_size = 1;
    const uintptr_t row_slot = (uintptr_t)(scratch + CS_CTL_BYTES + 256);
    const uintptr_t norm_slot = (uintptr_t)(scratch + CS_CTL_BYTES);
    s.X_sel = reinterpret_cast<float*>(row_slot - (uintptr_t)sel_pos * (uintptr_t)D * sizeof(float));
    s.norms_sel = reinterpret_cast<float*>(norm_slot - (uintptr_t)sel_pos * sizeof(float));
    s.dSL_quarter = const_cast<float*>(dSL_quarter ? dSL_quarter : reinterpret_cast<const float*>(norm_slot));
    s.cap = (int64_t)sel_pos + 1;
    s.selected = nullptr;
    s.eps = nullptr;
    s.ctl = scratch;
    s.pack_local = nullptr;
    s.pack_all = nullptr;
    s.rank = 0;
    s.xchg = CS_XCHG_GATHER;
    s.xchg_timeout_ms = 0;
    s.flags = 0;
    for (int r = 0; r < CS_MAX_PEERS; ++r) s.peer_win[r] = nullptr;

    noalloc_prepare_kernel<<<1, 256, 0, st>>>(scratch, centre, norm_new, D, sel_pos);
    rc = check_launch();
    if (rc) return rc;
    rc = cs_fps_step(&s, mode, stream);
    if (rc) return rc;
    noalloc_publish_kernel<<<1, 1, 0, st>>>(scratch, sel_pos, reinterpret_cast<u64*>(out_key),
                                            reinterpret_cast<u64*>(out_live_rows));
    return check_launch();
}
