// Exact k-th largest selection and the arg-max over a list of rows (accretion helpers).
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_SELECT_CUH
#define CORESETS_B200_SELECT_CUH

namespace {

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

}  // namespace

#endif  // CORESETS_B200_SELECT_CUH
