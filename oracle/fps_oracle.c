/*
 * CPU restatement of the reference's CUDA farthest-point-sampling path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package links, loads or calls this
 * file; it exists so that tests (and the CPU-baseline leg of the benchmark) can check the
 * sm_100a kernels bit for bit.  Every function names the reference source it follows
 * (paths relative to the reference project root).
 *
 * Parity status: PINNED.  tests/test_oracle_golden.py replays the golden vectors under
 * tests/golden/ (written by the reference's own CUDA extension running on a B200, see
 * tests/golden/make_golden_gpu.py) through these functions and demands identical
 * `selected`, and bit-identical `h` / `voronoi` / `epsilons`.
 *
 * Arithmetic contract.  The reference builds with `-O3 --use_fast_math`
 * (src/coresets/cuda/extension.py:63): flush-to-zero and fused multiply-add contraction,
 * no reassociation.  The expression
 *     dot += a.x*b.x + a.y*b.y + a.z*b.z + a.w*b.w            (_shared.cuh:49)
 * therefore evaluates as  t = a.y*b.y; t = fma(a.x,b.x,t); t = fma(a.z,b.z,t);
 * t = fma(a.w,b.w,t); dot = dot + t.  This file spells that sequence with fmaf() and is
 * compiled with -ffp-contract=off so the host compiler adds no contraction of its own;
 * MXCSR FTZ|DAZ are set while an oracle function runs.
 */
#include <limits.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <xmmintrin.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ---- flush-to-zero scope (nvcc --use_fast_math implies -ftz=true) ------------------ */
static unsigned ftz_enter(void) {
    unsigned old = _mm_getcsr();
    _mm_setcsr(old | 0x8040u); /* FTZ (bit 15) | DAZ (bit 6) */
    return old;
}
static void ftz_leave(unsigned old) { _mm_setcsr(old); }

/* ---- tie rule: larger value wins, equal values -> smaller index (_shared.cuh:24-27) */
static int better(float va, int64_t ia, float vb, int64_t ib) {
    return (va > vb) || (va == vb && ia < ib);
}

/*
 * One warp's dot product of a row with the new centre, then the 5-round shuffle tree.
 * Follows warp_dot (_shared.cuh:31-61) and the `__shfl_down_sync` loop that every caller
 * runs afterwards (warp.cu:35-37, commit.cu:92-94): lane l accumulates float4 chunks
 * l, l+32, ...; then p[j] += p[j+off] for off = 16,8,4,2,1.  Lane 0 holds the result.
 */
static int g_element_order = 0;

/* Inputs that were float16 / float64 take the element-wise branch of warp_dot for every D
 * (_shared.cuh:55-58: `dot += (float) row[i] * (float) c[i]`, one fma per element); the caller
 * hands this oracle the converted float rows and switches the branch here. */
ORACLE_API void oracle_set_element_order(int on) { g_element_order = on; }

static float ref_warp_dot(const float* row, const float* c, int D) {
    float p[32];
    if (D % 4 == 0 && !g_element_order) {
        const int d4 = D / 4;
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (int i = l; i < d4; i += 32) {
                const float* a = row + 4 * i;
                const float* b = c + 4 * i;
                float t = a[1] * b[1];
                t = fmaf(a[0], b[0], t);
                t = fmaf(a[2], b[2], t);
                t = fmaf(a[3], b[3], t);
                acc = acc + t;
            }
            p[l] = acc;
        }
    } else {
        /* scalar tail form (_shared.cuh:52-53): dot += x*c contracts to one fma */
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (int i = l; i < D; i += 32)
                acc = fmaf(row[i], c[i], acc);
            p[l] = acc;
        }
    }
    for (int off = 16; off > 0; off >>= 1)
        for (int j = 0; j < off; ++j)
            p[j] = p[j] + p[j + off];
    return p[0];
}

ORACLE_API float oracle_warp_dot(const float* row, const float* c, int D) {
    unsigned m = ftz_enter();
    float r = ref_warp_dot(row, c, D);
    ftz_leave(m);
    return r;
}

/* d = norms[row] + norm_new - 2*dot  (warp.cu:41-42); 2*dot is exact, so the optional
 * contraction fma(-2,dot,s) rounds identically to s - (dot+dot). */
static float ref_dist(float norm_row, float norm_new, float dot) {
    float s = norm_row + norm_new;
    return s - (dot + dot);
}

/* Dense update for the first centre: fps_update_warp_kernel (warp.cu:6-48). */
ORACLE_API void oracle_fps_update(const float* X, const float* norms, const float* x_new,
                                  float norm_new, float* h, int64_t* v, int64_t sel_idx,
                                  int64_t N, int D) {
    unsigned m = ftz_enter();
    for (int64_t r = 0; r < N; ++r) {
        float hr = h[r];
        if (hr < 0) continue; /* warp.cu:28-30 */
        float d = ref_dist(norms[r], norm_new, ref_warp_dot(X + r * (int64_t)D, x_new, D));
        if (d < hr) { h[r] = d; v[r] = sel_idx; }
    }
    ftz_leave(m);
}

/* Per-pick update with the triangle-inequality skip: voronoi_update_warp_kernel
 * (warp.cu:54-100).  Returns the number of rows whose distance was evaluated. */
ORACLE_API int64_t oracle_voronoi_update(const float* X, const float* norms, const float* x_new,
                                         float norm_new, const float* dSL_quarter, float* h,
                                         int64_t* v, int64_t sel_idx, int64_t N, int D) {
    unsigned m = ftz_enter();
    int64_t live = 0;
    for (int64_t r = 0; r < N; ++r) {
        float hr = h[r];
        if (hr < 0) continue;                    /* warp.cu:75-77 */
        if (dSL_quarter[v[r]] >= hr) continue;   /* warp.cu:80-82 */
        ++live;
        float d = ref_dist(norms[r], norm_new, ref_warp_dot(X + r * (int64_t)D, x_new, D));
        if (d < hr) { h[r] = d; v[r] = sel_idx; }
    }
    ftz_leave(m);
    return live;
}

/* Two-phase argmax (argmax.cu:11-95): accumulators start at (-1e38, INT_MAX), the tie rule
 * is a total order so the reduction shape cannot change the winner; "nothing found" is -1. */
ORACLE_API void oracle_argmax(const float* h, int64_t N, float* out_val, int32_t* out_idx) {
    float bv = -1e38f;
    int64_t bi = INT_MAX;
    for (int64_t i = 0; i < N; ++i)
        if (better(h[i], i, bv, bi)) { bv = h[i]; bi = i; }
    *out_val = bv;
    *out_idx = (bi == INT_MAX) ? -1 : (int32_t)bi;
}

/* compute_dSL_quarter_kernel (commit.cu:69-102): a quarter of the squared distance from
 * every old centre v < n_sel to the centre stored at slot n_sel. */
ORACLE_API void oracle_dsl_quarter(const float* X_sel, const float* norms_sel, float* dSL,
                                   int64_t n_sel, int D) {
    unsigned m = ftz_enter();
    const float* x_new = X_sel + n_sel * (int64_t)D;
    float norm_new = norms_sel[n_sel];
    for (int64_t r = 0; r < n_sel; ++r) {
        float dot = ref_warp_dot(X_sel + r * (int64_t)D, x_new, D);
        dSL[r] = ref_dist(norms_sel[r], norm_new, dot) * 0.25f;
    }
    ftz_leave(m);
}

/* commit_center_kernel (commit.cu:6-26) followed by the update choice of voronoi_step
 * (cuda/_internal/voronoi_step.py:9-55): dense kernel for slot 0, bound + skip kernel after. */
static void ref_voronoi_step(const float* X, const float* norms, float* h, int64_t* v,
                             float* X_sel, float* norms_sel, float* dSL, int64_t new_idx,
                             int64_t sel_pos, int64_t N, int D) {
    norms_sel[sel_pos] = norms[new_idx];
    h[new_idx] = -1.0f;
    v[new_idx] = sel_pos;
    memcpy(X_sel + sel_pos * (int64_t)D, X + new_idx * (int64_t)D, sizeof(float) * (size_t)D);
    if (sel_pos == 0) {
        oracle_fps_update(X, norms, X_sel, norms_sel[0], h, v, 0, N, D);
    } else {
        oracle_dsl_quarter(X_sel, norms_sel, dSL, sel_pos, D);
        oracle_voronoi_update(X, norms, X_sel + sel_pos * (int64_t)D, norms_sel[sel_pos], dSL, h,
                              v, sel_pos, N, D);
    }
}

/*
 * Whole single-GPU driver: fps() in src/coresets/cuda/fps.py:13-130.
 * `seed` (n_seed >= 1 indices) are committed in order first; pass {0},1 for the default.
 * Outputs: selected[k]; eps[k] (max h before each pick; eps[i < n_seed] = +inf -- the
 * reference driver returns no epsilons, the values are what its argmax kernel saw);
 * h[N], v[N] final state.  Returns 0, or -1 on bad arguments / allocation failure.
 */
ORACLE_API int oracle_fps_cuda(const float* X, const float* norms, int64_t N, int D, int64_t k,
                               const int64_t* seed, int64_t n_seed, int64_t* selected, float* eps,
                               float* h, int64_t* v) {
    if (N <= 0 || D <= 0 || k < 1 || k > N || n_seed < 1 || n_seed > k) return -1;
    float* X_sel = (float*)malloc(sizeof(float) * (size_t)k * (size_t)D);
    float* norms_sel = (float*)malloc(sizeof(float) * (size_t)k);
    float* dSL = (float*)malloc(sizeof(float) * (size_t)k);
    if (!X_sel || !norms_sel || !dSL) { free(X_sel); free(norms_sel); free(dSL); return -1; }
    for (int64_t i = 0; i < N; ++i) { h[i] = INFINITY; v[i] = 0; }
    for (int64_t i = 0; i < n_seed; ++i) {
        selected[i] = seed[i];
        eps[i] = INFINITY;
        ref_voronoi_step(X, norms, h, v, X_sel, norms_sel, dSL, seed[i], i, N, D);
    }
    for (int64_t i = n_seed; i < k; ++i) {
        float val; int32_t idx;
        oracle_argmax(h, N, &val, &idx);
        selected[i] = idx;
        eps[i] = val;
        ref_voronoi_step(X, norms, h, v, X_sel, norms_sel, dSL, idx, i, N, D);
    }
    free(X_sel); free(norms_sel); free(dSL);
    return 0;
}

/*
 * Sharded driver, W ranks emulated in one process: fps_sharded()
 * (src/coresets/cuda/multi/fps_sharded.py:21-418) with the replicated X_sel layout.
 * Per pick: every rank's local argmax (argmax.cu) packed with its global index
 * (multi.cu:249-280; empty shard -> (-inf,-1), multi.cu:283-292), then the winner is
 * `torch.argmax` over the W values = first maximum = lowest rank (fps_sharded.py:173-176).
 * sizes[W] are the contiguous shard sizes (layout.py:8-17).  eps[0] = +inf (:127-128).
 */
ORACLE_API int oracle_fps_sharded(const float* X, const float* norms, int D, int64_t k, int W,
                                  const int64_t* sizes, int64_t first, int64_t* selected,
                                  float* eps, float* h, int64_t* v) {
    int64_t N = 0;
    for (int r = 0; r < W; ++r) N += sizes[r];
    if (W < 1 || N <= 0 || k < 1 || k > N || first < 0 || first >= N) return -1;
    int64_t* off = (int64_t*)malloc(sizeof(int64_t) * (size_t)(W + 1));
    float* X_sel = (float*)malloc(sizeof(float) * (size_t)k * (size_t)D);
    float* norms_sel = (float*)malloc(sizeof(float) * (size_t)k);
    float* dSL = (float*)malloc(sizeof(float) * (size_t)k);
    if (!off || !X_sel || !norms_sel || !dSL) { free(off); free(X_sel); free(norms_sel); free(dSL); return -1; }
    off[0] = 0;
    for (int r = 0; r < W; ++r) off[r + 1] = off[r] + sizes[r];
    for (int64_t i = 0; i < N; ++i) { h[i] = INFINITY; v[i] = 0; }

    int64_t idx = first;
    eps[0] = INFINITY;
    for (int64_t i = 0; i < k; ++i) {
        if (i > 0) {
            float best = 0; int64_t best_idx = -1; int have = 0;
            for (int r = 0; r < W; ++r) {
                float val; int64_t g;
                if (sizes[r] > 0) {
                    int32_t li;
                    oracle_argmax(h + off[r], sizes[r], &val, &li);
                    g = (li >= 0) ? (int64_t)li + off[r] : -1;
                } else { val = -INFINITY; g = -1; }
                if (!have || val > best) { best = val; best_idx = g; have = 1; }
            }
            idx = best_idx;
            eps[i] = best;
        }
        selected[i] = idx;
        /* owner marks the row; X_sel/norms_sel are replicated (fps_sharded.py:181-196) */
        h[idx] = -1.0f; v[idx] = i;
        norms_sel[i] = norms[idx];
        memcpy(X_sel + i * (int64_t)D, X + idx * (int64_t)D, sizeof(float) * (size_t)D);
        if (i > 0) oracle_dsl_quarter(X_sel, norms_sel, dSL, i, D); /* replicated, same on all ranks */
        for (int r = 0; r < W; ++r) {
            if (sizes[r] == 0) continue;
            const float* Xr = X + off[r] * (int64_t)D;
            if (i == 0) {
                oracle_fps_update(Xr, norms + off[r], X_sel, norms_sel[0], h + off[r], v + off[r],
                                  0, sizes[r], D);
            } else {
                oracle_voronoi_update(Xr, norms + off[r], X_sel + i * (int64_t)D, norms_sel[i], dSL,
                                      h + off[r], v + off[r], i, sizes[r], D);
            }
        }
    }
    free(off); free(X_sel); free(norms_sel); free(dSL);
    return 0;
}

/*
 * Single-GPU bisect probe: simulate_fps_voronoi (simulate.cu:10-90).
 * Starting from (h, v) with n_init centres in X_sel_init/norms_sel_init, run up to
 * points_left picks; each step = argmax, commit_center_with_sep (commit.cu:31-64: viable if
 * sep > val; sep = min(sep, val)), bound (masked variant is result-neutral, simulate.cu:50-61),
 * update.  The host polls the flag every 16 steps (simulate.cu:77-81); after the loop one more
 * argmax and final_viable_check (argmax.cu:152-159).  h and v are updated in place.
 * Returns viable (0/1); *steps_used as the reference reports it.
 */
ORACLE_API int oracle_simulate(const float* X, const float* norms, int64_t N, int D, float* h,
                               int64_t* v, const float* X_sel_init, const float* norms_sel_init,
                               int64_t n_init, double sep_in, int64_t points_left,
                               int64_t* steps_used, float* sep_out) {
    int64_t cap = n_init + points_left + 1;
    float* X_sel = (float*)calloc((size_t)cap * (size_t)D, sizeof(float));
    float* norms_sel = (float*)calloc((size_t)cap, sizeof(float));
    float* dSL = (float*)calloc((size_t)cap, sizeof(float));
    if (!X_sel || !norms_sel || !dSL) { free(X_sel); free(norms_sel); free(dSL); return -1; }
    if (n_init > 0) {
        memcpy(X_sel, X_sel_init, sizeof(float) * (size_t)n_init * (size_t)D);
        memcpy(norms_sel, norms_sel_init, sizeof(float) * (size_t)n_init);
    }
    float sep = (float)sep_in;
    int viable = 0;
    int64_t n_sel = n_init;
    int result = -2;
    for (int64_t step = 0; step < points_left; ++step) {
        float val; int32_t idx;
        oracle_argmax(h, N, &val, &idx);
        if (sep > val) viable = 1;
        if (val < sep) sep = val;
        norms_sel[n_sel] = norms[idx];
        h[idx] = -1.0f; v[idx] = n_sel;
        memcpy(X_sel + n_sel * (int64_t)D, X + (int64_t)idx * D, sizeof(float) * (size_t)D);
        if (n_sel > 0) {
            oracle_dsl_quarter(X_sel, norms_sel, dSL, n_sel, D);
            oracle_voronoi_update(X, norms, X_sel + n_sel * (int64_t)D, norms_sel[n_sel], dSL, h, v,
                                  n_sel, N, D);
        } else {
            oracle_fps_update(X, norms, X_sel, norms_sel[0], h, v, 0, N, D);
        }
        ++n_sel;
        if ((step + 1) % 16 == 0 && viable) { *steps_used = step + 1; result = 1; break; }
    }
    if (result == -2) {
        float val; int32_t idx;
        oracle_argmax(h, N, &val, &idx);
        if (sep > val) viable = 1;
        *steps_used = points_left;
        result = viable;
    }
    if (sep_out) *sep_out = sep;
    free(X_sel); free(norms_sel); free(dSL);
    return result;
}

/*
 * Sharded bisect probe: simulate_fps_voronoi_multi_sharded (multi.cu:428-528), W ranks
 * emulated in-process over the concatenated state.  The cross-rank reduce and the
 * viability rules follow reduce_and_commit_multi_sharded_kernel (multi.cu:296-365):
 * start (-inf, INT64_MAX); viable if sep > val || val <= 0 || idx < 0; sep lowered only
 * when 0 < val < sep.  Tail check: final_viable_check_multi_sharded_kernel (:369-384).
 */
ORACLE_API int oracle_simulate_sharded(const float* X, const float* norms, int D, int W,
                                       const int64_t* sizes, float* h, int64_t* v,
                                       const float* X_sel_init, const float* norms_sel_init,
                                       int64_t n_init, double sep_in, int64_t points_left,
                                       int64_t* steps_used, float* sep_out) {
    int64_t N = 0;
    for (int r = 0; r < W; ++r) N += sizes[r];
    int64_t cap = n_init + points_left + 1;
    int64_t* off = (int64_t*)malloc(sizeof(int64_t) * (size_t)(W + 1));
    float* X_sel = (float*)calloc((size_t)cap * (size_t)D, sizeof(float));
    float* norms_sel = (float*)calloc((size_t)cap, sizeof(float));
    float* dSL = (float*)calloc((size_t)cap, sizeof(float));
    if (!off || !X_sel || !norms_sel || !dSL) { free(off); free(X_sel); free(norms_sel); free(dSL); return -1; }
    off[0] = 0;
    for (int r = 0; r < W; ++r) off[r + 1] = off[r] + sizes[r];
    if (n_init > 0) {
        memcpy(X_sel, X_sel_init, sizeof(float) * (size_t)n_init * (size_t)D);
        memcpy(norms_sel, norms_sel_init, sizeof(float) * (size_t)n_init);
    }
    float sep = (float)sep_in;
    int viable = 0;
    int64_t n_sel = n_init;
    int result = -2;
    for (int64_t step = 0; step <= points_left; ++step) {
        /* gather of per-rank (val, global idx) */
        float best_val = -INFINITY; int64_t best_idx = INT64_MAX;
        float max_val = -INFINITY;
        for (int r = 0; r < W; ++r) {
            float val; int64_t g;
            if (sizes[r] > 0) {
                int32_t li;
                oracle_argmax(h + off[r], sizes[r], &val, &li);
                g = (li >= 0) ? (int64_t)li + off[r] : -1;
            } else { val = -INFINITY; g = -1; }
            if (val > max_val) max_val = val;
            if (better(val, g, best_val, best_idx)) { best_val = val; best_idx = g; }
        }
        if (step == points_left) { /* tail check */
            if (sep > max_val) viable = 1;
            *steps_used = points_left;
            result = viable;
            break;
        }
        if (best_idx == INT64_MAX) best_idx = -1;
        if (sep > best_val || best_val <= 0.0f || best_idx < 0) viable = 1;
        if (best_val > 0.0f && best_val < sep) sep = best_val;
        if (best_idx >= 0) {
            norms_sel[n_sel] = norms[best_idx];
            h[best_idx] = -1.0f; v[best_idx] = n_sel;
            memcpy(X_sel + n_sel * (int64_t)D, X + best_idx * (int64_t)D, sizeof(float) * (size_t)D);
        }
        if (n_sel > 0) oracle_dsl_quarter(X_sel, norms_sel, dSL, n_sel, D);
        for (int r = 0; r < W; ++r) {
            if (sizes[r] == 0) continue;
            const float* Xr = X + off[r] * (int64_t)D;
            if (n_sel > 0)
                oracle_voronoi_update(Xr, norms + off[r], X_sel + n_sel * (int64_t)D, norms_sel[n_sel],
                                      dSL, h + off[r], v + off[r], n_sel, sizes[r], D);
            else
                oracle_fps_update(Xr, norms + off[r], X_sel, norms_sel[0], h + off[r], v + off[r], 0,
                                  sizes[r], D);
        }
        ++n_sel;
        if ((step + 1) % 16 == 0 && viable) { *steps_used = step + 1; result = 1; break; }
    }
    if (sep_out) *sep_out = sep;
    free(off); free(X_sel); free(norms_sel); free(dSL);
    return result;
}
