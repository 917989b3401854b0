// Single-block state kernels and the stand-alone arg-max scan.
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_SMALL_KERNELS_CUH
#define CORESETS_B200_SMALL_KERNELS_CUH

namespace {

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

__device__ __forceinline__ void force_pick_body(const cs_state& s, const int64_t gidx, const float val) {
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

__global__ void force_pick_kernel(const cs_state s, const int64_t gidx, const float val) { force_pick_body(s, gidx, val); }

// The same with the row taken from a device list at the position of the pick counter, so that a
// run of prescribed picks (a resumed checkpoint) can be replayed from a CUDA graph.
__global__ void force_pick_list_kernel(const cs_state s, const int64_t* __restrict__ list,
                                       const float* __restrict__ vals, const float val) {
    const Ctl* ctl = reinterpret_cast<const Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    if (i >= s.cap) return;                                // the commit kernel reports the overflow
    force_pick_body(s, list[i], vals ? vals[i] : val);
}

// Restricted arg-max as the next pick's candidate: largest key over the rows of `pool` this shard
// owns (one block; pools are at most a few thousand rows).
__global__ void __launch_bounds__(1024) pool_pick_kernel(const cs_state s, const int64_t* __restrict__ pool,
                                                        const int64_t* __restrict__ n_pool) {
    __shared__ u64 s_best[32];
    __shared__ u64 s_key;
    Ctl* ctl = reinterpret_cast<Ctl*>(s.ctl);
    const int i = ctl->n_sel;
    if (ctl->halt || i >= s.cap) return;
    const int64_t n = *n_pool;
    u64 best = 0;
    for (int64_t p = threadIdx.x; p < n; p += blockDim.x) {
        const int64_t g = pool[p];
        const int64_t l = g - s.shard_offset;
        if (l >= 0 && l < s.N_local) {
            const u64 k = make_key(s.h[l], g);
            best = k > best ? k : best;
        }
    }
    best = warp_max_key(best);
    if ((threadIdx.x & 31) == 0) s_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 bk = 0;
        for (int q = 0; q < (int)(blockDim.x >> 5); ++q) bk = s_best[q] > bk ? s_best[q] : bk;
        ctl->key[i & 1] = bk;
        s_key = bk;
    }
    __syncthreads();
    const u64 k = s_key;
    if (s.world_size > 1) publish_candidate(s, ctl, k, key_idx(k) - s.shard_offset);
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

}  // namespace

#endif  // CORESETS_B200_SMALL_KERNELS_CUH
