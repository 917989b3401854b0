// Constants, the control block, the order-preserving arg-max key and the reference's dot product.
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_FPS_COMMON_CUH
#define CORESETS_B200_FPS_COMMON_CUH

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
    int halt;           // a restricted run found nothing positive to pick: later launches of the run do nothing
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

// First statement of every kernel of the per-pick chain.  Under a programmatic dependent launch
// the grid may already be resident while its predecessor runs: wait for the predecessor's
// completion (and the visibility of its writes) before reading anything, then let the successor
// become resident in turn.  Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float4 ld_stream4(const float4* p) { return __ldcs(p); }

// Element c of local row `row` of X as a float: float32 rows, or half rows widened on the fly.
__device__ __forceinline__ float x_elem(const cs_state& s, const int64_t row, const int c) {
    if (s.flags & CS_F_X_HALF) return __half2float(__ldg(reinterpret_cast<const __half*>(s.X) + row * (int64_t)s.D + c));
    return __ldg(s.X + row * (int64_t)s.D + c);
}

// Element-wise warp dot of a half row with the centre (one fma per element, _shared.cuh:52-58).
__device__ __forceinline__ float warp_dot_half(const __half* __restrict__ row, const float* __restrict__ cen, int D, int lane) {
    float acc = 0.0f;
    for (int c = lane; c < D; c += 32) acc = __fmaf_rn(__half2float(__ldg(row + c)), cen[c], acc);
    return warp_tree_sum(acc);
}

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

}  // namespace

#endif  // CORESETS_B200_FPS_COMMON_CUH
