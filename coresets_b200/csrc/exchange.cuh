// Candidate exchange between ranks (gathered pack or peer stores over NVLink) and winner resolution.
// Part of the single translation unit fps_kernels.cu (included there, in order).
#ifndef CORESETS_B200_EXCHANGE_CUH
#define CORESETS_B200_EXCHANGE_CUH

namespace {

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
    // the candidate row travels as float32 bit patterns; half rows widen losslessly (multi.cu:245)
    const bool half_rows = (s.flags & CS_F_X_HALF) != 0;
    const int64_t lrow = k ? l : 0;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(s.X + (half_rows ? 0 : lrow * (int64_t)D));
    const uint32_t norm_bits = k ? __float_as_uint(s.norms[l]) : 0u;
    if (s.xchg == CS_XCHG_GATHER) {
        uint32_t* p = s.pack_local;
        if (threadIdx.x == 0) {
            p[0] = (uint32_t)(k & 0xffffffffu);
            p[1] = (uint32_t)(k >> 32);
            p[2] = norm_bits;
            p[3] = 0u;
        }
        for (int c = threadIdx.x; c < D; c += blockDim.x)
            p[4 + c] = k ? (half_rows ? __float_as_uint(x_elem(s, lrow, c)) : src[c]) : 0u;
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
        for (int c = threadIdx.x; c < D; c += blockDim.x)
            p[4 + c] = k ? (half_rows ? __float_as_uint(x_elem(s, lrow, c)) : src[c]) : 0u;
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
    const float* row;   // D floats (in X or in the gathered packs); null when the row is a half row of X
    int64_t xrow;       // local row of X when the winner is this rank's own row (world_size 1)
    float norm;
};
// Element c of the winner's row.
__device__ __forceinline__ float winner_elem(const cs_state& s, const Winner& w, const int c) {
    return w.row ? w.row[c] : x_elem(s, w.xrow, c);
}
__device__ __forceinline__ Winner resolve_winner(const cs_state& s, const Ctl* ctl, int i, const uint32_t* packs) {
    Winner w;
    w.row = nullptr;
    w.xrow = 0;
    w.norm = 0.0f;
    if (s.world_size <= 1) {
        w.key = ctl->key[i & 1];
        if (w.key) {
            int64_t l = key_idx(w.key) - s.shard_offset;
            w.row = (s.flags & CS_F_X_HALF) ? nullptr : s.X + l * (int64_t)s.D;
            w.xrow = l;
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

}  // namespace

#endif  // CORESETS_B200_EXCHANGE_CUH
