/*
 * coresets_b200 -- C ABI of the B200 (sm_100a) farthest-point-sampling engine.
 *
 * This is the boundary a host language binds (Python/ctypes in this package).  It replaces
 * the reference's pybind11 module `coreset_kernels`
 * (src/coresets/cuda/kernels/bindings.cu:3-152), whose functions take torch::Tensor
 * arguments, have no return code and no stream parameter.
 *
 * Conventions
 *   - every function returns 0 (CS_OK) or a negative CS_E_* code; nothing throws or traps;
 *   - all pointers are DEVICE pointers owned by the caller unless a comment says "host";
 *     no entry point declared before the "self-contained" section allocates or frees memory;
 *   - work is enqueued on the given stream and is capturable into a CUDA graph (no implicit
 *     synchronisation, no host round trip);
 *   - rows are addressed with 64-bit arithmetic; GLOBAL row indices must stay below 2^31
 *     (the reference rejects more, src/coresets/cuda/multi/fps_sharded.py:68-73).
 *
 * One FPS pick is two launches on every rank (plus one all-gather when world_size > 1):
 *   cs_commit_bound  resolve the winner, append it as centre n_sel, mark its row selected,
 *                    compute the triangle bounds dSL_quarter[0..n_sel)
 *   cs_fps_step      distance of every live row to centre n_sel, in-place min-update of h and
 *                    voronoi, fused (value, smallest global index) arg-max for the NEXT pick,
 *                    n_sel += 1, and (world_size > 1) the rank's candidate pack
 */
#ifndef CORESETS_B200_H
#define CORESETS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CS_ABI_VERSION 9

#if defined(__GNUC__)
#define CS_API __attribute__((visibility("default")))
#else
#define CS_API
#endif

/* error codes */
#define CS_OK 0
#define CS_E_ARG (-1)      /* null pointer, negative size, bad flag */
#define CS_E_ALIGN (-2)    /* X / X_sel / pack not 16-byte aligned while D % 4 == 0 */
#define CS_E_RANGE (-3)    /* global index space >= 2^31, or a size above a stated maximum */
#define CS_E_LAUNCH (-4)   /* the CUDA runtime refused the launch (see cs_last_cuda_error) */
#define CS_E_DEVICE (-5)   /* no usable sm_100 device / wrong architecture */
#define CS_E_SCRATCH (-6)  /* D exceeds CS_NOALLOC_MAX_D, the fixed scratch of cs_fps_step_noalloc */

/* cs_fps_step flags */
#define CS_MODE_PRUNE 0u   /* rows excluded by the triangle bound are not loaded (default); the rows
                              that remain are queued and evaluated in batches */
#define CS_MODE_PRUNE_INLINE 2u /* prune mode evaluating each remaining row where the scan meets it */
#define CS_MODE_DENSE 1u   /* every live row's distance is computed; the bound only masks the
                              update, so results are identical to CS_MODE_PRUNE; X is streamed by
                              bulk asynchronous (TMA) copies when D % 4 == 0 and 32 <= D <= 1024
                              (half rows, CS_F_X_HALF: D % 8 == 0 and D <= 1024), X / h / voronoi /
                              norms 16-byte aligned */
#define CS_MODE_DENSE_LDG 3u /* dense mode with plain 128-bit loads (the path other row widths take) */
/* cs_state.flags */
#define CS_F_ELEMENT_ORDER 1u /* every dot product sums element-wise (lane l takes elements l, l+32,
                              ... with one fma each) even when D % 4 == 0: the order the reference uses
                              for float16 / float64 inputs (_shared.cuh:55-58), whose rows the caller
                              passes converted to float32 */
#define CS_F_X_HALF 4u       /* X holds IEEE half rows (2 bytes per element, row-major, no alignment rule);
                              every element is widened to float where it is read, which is what the
                              reference's half instantiation does (_shared.cuh:55-58).  Requires
                              CS_F_ELEMENT_ORDER.  X_sel, the packs and every other array stay float32 */
#define CS_F_PDL 2u          /* launch the kernels of a pick (commit, cell selection, scan, evaluation, the
                              prune-mode step) as programmatic dependents of the kernel before them on the
                              stream: their start overlaps the predecessor's tail, they read nothing
                              before it has completed */
#define CS_F_TEST_STALL_PIPE 0x100u /* test hook: the dense kernel's producer starts no copy, so that the
                              consumers' bounded wait runs out (status 4) without any fault */
/* cs_commit_bound flags */
#define CS_RULE_NONE 0u    /* plain FPS: no separation bookkeeping */
#define CS_RULE_SIM_SINGLE 1u   /* commit_center_with_sep_kernel rules (commit.cu:41-51) */
#define CS_RULE_SIM_SHARDED 2u  /* reduce_and_commit_multi_sharded_kernel rules (multi.cu:331-340) */
#define CS_RULE_STOP_NONPOS 3u  /* restricted forward walk of accretion: a winner whose value is not
                                   positive (or no winner) is NOT committed; the control block's halt
                                   word is set instead (block_forward.py:45-47, _base.py:419-421) */

/* how the per-pick candidates travel between ranks (cs_state.xchg) */
#define CS_XCHG_GATHER 0   /* cs_fps_step writes pack_local; the caller all-gathers into pack_all */
#define CS_XCHG_PEER 1     /* cs_fps_step stores the candidate into every rank's exchange window
                              over NVLink and raises a flag; cs_commit_bound waits on the flags   */
#define CS_MAX_PEERS 8     /* ranks addressable with CS_XCHG_PEER (one NVSwitch box)              */
#define CS_MAX_LANES 8     /* states one cs_fps_step_lanes call can serve                         */

/* Size in bytes of the per-run device control block (n_sel counter, the two arg-max key
 * slots, ticket, status, separation / viability words).  Zero it with cs_reset_ctl. */
#define CS_CTL_BYTES 256

/* Host-visible mirror of the control block (read it back with one 256-byte copy). */
typedef struct cs_ctl_view {
    uint64_t key[2];     /* arg-max key for pick i lives in key[i & 1]                      */
    int32_t n_sel;       /* centres committed so far                                          */
    uint32_t ticket;     /* blocks of the running step kernel that have finished              */
    int32_t status;      /* sticky device-side error (0 = none)                               */
    int32_t viable;      /* simulation: 1 once separation beat coverage                       */
    float sep;           /* simulation: running min of the pick values                        */
    int32_t steps;       /* simulation: picks committed since cs_sim_begin                    */
    uint64_t live_rows;  /* rows whose distance the last cs_fps_step evaluated (dense mode over
                            half rows: rows the pruned scan would have evaluated)             */
    float last_val;      /* value (max h) of the last committed pick                          */
    int32_t last_idx;    /* global index of the last committed pick (-1: nothing left)       */
    uint32_t xseq;       /* peer exchange: sequence number of the last published candidate   */
    int32_t halt;        /* 1 once a CS_RULE_STOP_NONPOS commit met a best value <= 0: commits and
                            steps launched after it do nothing until cs_reset_ctl                  */
    uint8_t reserved[CS_CTL_BYTES - 64];
} cs_ctl_view;

/*
 * One rank's view of a run.  Filled by the host once; the library only reads it.
 * A candidate pack is (4 + D) 32-bit words: key low, key high, norm bits, 0, row bits[D].
 */
typedef struct cs_state {
    const float* X;        /* [N_local, D] row-major fp32 (IEEE half with CS_F_X_HALF)            */
    const float* norms;    /* [N_local] squared row norms                                     */
    float* h;              /* [N_local] squared distance to nearest centre; -1 = selected     */
    int32_t* voronoi;      /* [N_local] slot of the nearest centre (reference: int64)         */
    int64_t N_local;       /* rows on this rank (0 is legal)                                  */
    int64_t shard_offset;  /* global index of local row 0                                     */
    int32_t D;             /* row length                                                      */
    int32_t world_size;    /* ranks taking part (1 = no exchange)                             */
    float* X_sel;          /* [cap, D] committed centres (replicated on every rank)           */
    float* norms_sel;      /* [cap]                                                           */
    float* dSL_quarter;    /* [cap] triangle bounds of the pick in flight                     */
    int64_t cap;           /* capacity of the three arrays above and of selected / eps        */
    int64_t* selected;     /* [cap] global index per slot, or NULL                            */
    float* eps;            /* [cap] max h before each pick, or NULL                           */
    void* ctl;             /* CS_CTL_BYTES control block                                      */
    uint32_t* pack_local;  /* [4 + D] this rank's candidate (world_size > 1), else NULL       */
    const uint32_t* pack_all; /* [world_size, 4 + D] all-gathered candidates, else NULL       */
    int32_t rank;          /* this rank (CS_XCHG_PEER)                                        */
    int32_t xchg;          /* CS_XCHG_GATHER or CS_XCHG_PEER                                  */
    uint32_t* peer_win[CS_MAX_PEERS]; /* CS_XCHG_PEER: every rank's exchange window as mapped
                              into THIS process (peer_win[rank] is the local one); each holds
                              cs_xchg_window_words() zero-initialised 32-bit words             */
    int32_t xchg_timeout_ms; /* bound of every device-side wait (0 = 10 s): the exchange flag wait
                              (status 3 on expiry) and the bulk-copy pipe of dense mode (status 4) */
    int32_t flags;         /* CS_F_* bits                                                     */
} cs_state;

typedef void* cs_stream; /* cudaStream_t */

/* ABI version of the loaded library (CS_ABI_VERSION). */
CS_API int cs_version(void);

/* Static description of an error code. */
CS_API const char* cs_error_string(int code);

/* Last CUDA runtime error string seen by a failing launch on the calling thread. */
CS_API const char* cs_last_cuda_error(void);

/* Number of SMs of the current device, or a negative code.  Also verifies that the device
 * is compute capability 10.x, which the embedded sm_100a code requires. */
CS_API int cs_device_check(void);

/*
 * h[i] = +inf, voronoi[i] = 0 for every local row, and a zeroed control block.
 * Replaces the torch.full / torch.zeros state set-up of src/coresets/cuda/fps.py:37-43 and
 * src/coresets/cuda/multi/fps_sharded.py:113-119.
 */
CS_API int cs_init_state(const cs_state* s, cs_stream stream);

/* Zero the control block only, then set n_sel (used when a run continues from a state that
 * already holds n_sel centres, e.g. a bisect probe). */
CS_API int cs_reset_ctl(const cs_state* s, int32_t n_sel, cs_stream stream);

/*
 * Force the next pick to be global row `global_idx` with value `val` (+inf for a seed).
 * The owner rank publishes the candidate, every other rank publishes "nothing".  Replaces
 * `d_out_idx.fill_(new_idx)` of cuda/_internal/voronoi_step.py:25 and `pack_row_by_owner`
 * of cuda/multi/fps_sharded.py:131-146.  Follow with the all-gather (world_size > 1),
 * cs_commit_bound and cs_fps_step exactly like a normal pick.
 */
CS_API int cs_force_pick(const cs_state* s, int64_t global_idx, float val, cs_stream stream);

/*
 * Make the next pick the arg-max of h over a list of global rows (value first, then the smaller
 * index): pool[0 .. *n_pool) are global row indices, both in device memory; rows of other shards are
 * ignored, the owner ranks publish their best, the others "nothing".  Follow with the all-gather
 * (world_size > 1), cs_commit_bound(CS_RULE_STOP_NONPOS) and cs_fps_step like a normal pick; nothing
 * goes through the host, so a run of restricted picks replays from a CUDA graph and stops by itself
 * (halt) when the pool has nothing positive left.  Replaces the per-pick mask / gather / max /
 * all-gather / .item() sequence of the accretion forward loop (cuda/_internal/block_forward.py:38-53,
 * cuda/multi/sharded.py:174-215).
 */
CS_API int cs_pool_pick(const cs_state* s, const int64_t* pool, const int64_t* n_pool, cs_stream stream);

/*
 * cs_force_pick with the row read on the device: the next pick becomes list[n_sel] (a device array
 * of at least cap global row indices, each in [0, N_global)) with value vals[n_sel], or `val` when
 * vals is NULL.  Nothing depends on the host, so a run
 * of prescribed picks replays from a CUDA graph; used to rebuild the state of a resumed checkpoint
 * (replaces the chunked distance rebuild of cuda/multi/_shared.py:243-312 with the picks themselves,
 * which reproduces h and voronoi bit for bit).
 */
CS_API int cs_force_pick_list(const cs_state* s, const int64_t* list, const float* vals, float val, cs_stream stream);

/*
 * Resolve and commit pick number i = n_sel.  The winner is the largest key among the
 * world_size candidates (value first, then smallest global index: argmax_better,
 * kernels/_shared.cuh:24-27).  Writes selected[i], eps[i], X_sel[i], norms_sel[i]; the
 * owner sets h = -1 and voronoi = i on the row; then dSL_quarter[v] for every v < i.
 * `rules` selects the separation / viability bookkeeping of the simulation loops.
 * Replaces commit_center_cuda, commit_center_with_sep_cuda, compute_dSL_quarter_cuda
 * (kernels/commit.cu:162-210), reduce_and_commit_multi_sharded_cuda (kernels/multi.cu:407-422)
 * and the host-side torch.argmax + .item() of cuda/multi/fps_sharded.py:173-176.
 */
CS_API int cs_commit_bound(const cs_state* s, uint32_t rules, cs_stream stream);

/*
 * The fused hot kernel.  For centre i = n_sel (slot written by cs_commit_bound):
 *   rows with h < 0 are skipped; for i > 0 rows with dSL_quarter[voronoi] >= h are not
 *   updated; d = norms[row] + norm_new - 2*dot(row, centre) with the reference's summation
 *   order; if d < h then h = d, voronoi = i; every row then feeds (h, global index) into a
 *   block -> grid arg-max whose result is the key of pick i + 1; n_sel becomes i + 1.
 * Replaces fps_update_cuda, voronoi_update_cuda (kernels/warp.cu:159-191), argmax_cuda
 * (kernels/argmax.cu:179-193) and pack_argmax_with_row_cuda / fill_pack_with_row_neg_inf_cuda
 * (kernels/multi.cu:387-405).
 */
CS_API int cs_fps_step(const cs_state* s, uint32_t mode, cs_stream stream);

/* Start a simulation (bisect probe): zero viable / steps, set the running separation.
 * Replaces the two blocking cudaMemcpy of kernels/simulate.cu:27-29, multi.cu:448-451. */
CS_API int cs_sim_begin(const cs_state* s, float sep, cs_stream stream);

/* Tail check of a simulation: viable |= sep > (max h after the last update); the max is the
 * best candidate value over all ranks.  Replaces final_viable_check_kernel
 * (kernels/argmax.cu:152-159) and final_viable_check_multi_sharded_kernel (multi.cu:369-384). */
CS_API int cs_sim_final_check(const cs_state* s, cs_stream stream);

/* Words (32-bit) of one rank's exchange window for CS_XCHG_PEER: 64 flag words followed by two
 * buffers of world_size candidates (4 + D words each, rounded up to a multiple of 4). */
CS_API int64_t cs_xchg_window_words(int32_t world_size, int32_t D);

/*
 * CS_XCHG_PEER only: wait (bounded) until every rank's current candidate has arrived, without
 * consuming it in a commit.  Needed before publishing again when the last published candidate was
 * not consumed by cs_commit_bound / cs_sim_final_check (e.g. a forced pick right after a step):
 * a rank may publish sequence s+1 only after it has seen every peer's sequence s.  No counterpart
 * in the reference (its exchange is a host-driven all-gather, cuda/multi/fps_sharded.py:171).
 */
CS_API int cs_xchg_wait(const cs_state* s, cs_stream stream);

/*
 * Recompute the arg-max key of the NEXT pick (and, for world_size > 1, the candidate pack) from
 * the current h without touching h, voronoi or n_sel.  Call it after h was changed outside
 * cs_fps_step (roll-back to a snapshot, a reconstructed bisect state) and for "global max h"
 * queries.  Replaces the stand-alone uses of argmax_cuda (kernels/argmax.cu:179-193) in
 * cuda/multi/sharded.py:112-131, 470-490 and kernels/simulate.cu:84, multi.cu:511-517.
 */
CS_API int cs_scan_argmax(const cs_state* s, cs_stream stream);

/*
 * Exact k-th largest (k = 1 is the maximum) of the entries of h[0..n) that are >= 0, and how
 * many such entries there are.  Selected rows carry h = -1 and do not count.  Replaces the
 * `(h_mid >= 0).sum()` + `torch.kthvalue(h_mid[h_mid >= 0], rank)` pair of the bisect early exit
 * (cuda/_internal/bisect.py:64-71; rank = n_alive - k + 1 there): a selection returns one of
 * the inputs, so the value is the same float whatever algorithm finds it.  Four radix passes over
 * h, no host synchronisation.  `scratch` is CS_SELECT_SCRATCH_BYTES of device memory owned by
 * the caller; when the stream has run, its first bytes hold a cs_select_result.
 */
#define CS_SELECT_SCRATCH_BYTES 8192
typedef struct cs_select_result {
    float value;       /* the k-th largest live entry; undefined when valid == 0            */
    int32_t valid;     /* 1 when 1 <= k <= n_alive                                           */
    int64_t n_alive;   /* entries of h that are >= 0                                         */
} cs_select_result;
CS_API int cs_select_kth_largest(const float* h, int64_t n, int64_t k, void* scratch, cs_stream stream);

/*
 * Arg-max of h restricted to a list of global row indices: *out_key (device, 8 bytes) becomes the
 * largest key(h[p - shard_offset], p) over the entries p of `pool` that this shard owns, 0 when it
 * owns none.  A key orders by value, then by SMALLER index, and decodes as
 *   value = bits(key >> 32) mapped back (sign-magnitude to two's-complement order),
 *   index = 0xFFFFFFFF - (key & 0xFFFFFFFF);
 * the maximum over the ranks' keys is the global winner.  Replaces the masked gather / max /
 * min-index sequence of the accretion forward loop (cuda/_internal/block_forward.py:38-53,
 * cuda/multi/sharded.py:174-210).
 */
CS_API int cs_pool_argmax(const float* h, const int64_t* pool, int64_t n_pool, int64_t shard_offset,
                          int64_t n_local, uint64_t* out_key, cs_stream stream);

/*
 * Several probes at once: `n_lanes` (1..8) independent states that share X / norms /
 * N_local / D / shard_offset / world_size but own their h, voronoi, centres and control
 * block.  Each lane's arithmetic is that of cs_fps_step.  CS_MODE_DENSE and
 * CS_MODE_PRUNE_INLINE serve every lane from ONE pass over X; CS_MODE_PRUNE runs one
 * deferred-row step per lane, which is faster when few rows pass the triangle test.
 * Replaces voronoi_update_lanes_kernel (kernels/multi.cu:569-708).  The control block's
 * live_rows statistic is maintained by the per-lane steps only; the fused pass leaves it at 0.
 */
CS_API int cs_fps_step_lanes(const cs_state* lanes, int32_t n_lanes, uint32_t mode, cs_stream stream);

/*
 * Cell index: the rows of a shard grouped by the centre that owned them when the index was built.
 * No counterpart in the reference, whose per-pick kernel reads h and voronoi of EVERY row
 * (kernels/warp.cu:54-100).  With the index a pick reads only the cells whose rows can possibly
 * change: cell A is left alone when the triangle inequality through its centre, widened by a bound
 * on the rounding error of the distance formula, proves that every row in it keeps its h.  Rows of
 * the cells that remain are tested one by one with the reference's own predicate
 * (dSL_quarter[voronoi] >= h) and evaluated with the reference's arithmetic, so h, voronoi and the
 * picks are bit-identical to cs_fps_step.  h / voronoi stay authoritative in row order (every
 * update is written to both copies); the index goes stale whenever something else changes h.
 *
 * Memory, all owned by the caller: slots = N_local + cap * CS_CELL_TILE entries of perm / hp / vp,
 * N_local of cell0, cap (+1) of the per-cell arrays, CS_CELLS_META_BYTES of meta, q_cap pairs of queue.
 */
#define CS_CELL_TILE 256         /* segments are padded to whole tiles of this many slots */
#define CS_CELLS_META_BYTES 128
typedef struct cs_cells {
    int32_t* perm;        /* [slots] local row held by each slot, -1 = padding                */
    float* hp;            /* [slots] copy of h in slot order (-inf on padding)                */
    int32_t* vp;          /* [slots] copy of voronoi in slot order                            */
    int32_t* cell0;       /* [N_local] cell of each row when the index was built              */
    int64_t slots;        /* capacity of perm / hp / vp (< 2^31)                               */
    int32_t* seg_start;   /* [cap + 1] first slot of each cell                                 */
    int32_t* seg_count;   /* [cap] rows of each cell when the index was built                  */
    uint64_t* seg_key;    /* [cap] arg-max key over the cell's slots                           */
    float* seg_h0;        /* [cap] largest h of the cell when the index was built              */
    int32_t* cursor;      /* [cap] scratch of the build                                        */
    int32_t* work_cell;   /* [cap] cells the pick in flight visits                             */
    int32_t* work_cum;    /* [cap] running number of chunks over work_cell                     */
    void* meta;           /* CS_CELLS_META_BYTES, see cs_cells_meta_view                       */
    void* queue;          /* [q_cap] pairs of int32 (slot, cell): rows waiting for a distance  */
    float row_norm_max;   /* an upper bound of norms[0..N_local) (error bound of the skip test) */
    int32_t q_cap;        /* entries of queue (>= CS_CELL_TILE); rows beyond it are evaluated
                             by the scanning kernel itself, slower but with the same result    */
} cs_cells;

/* Host-visible mirror of cs_cells.meta. */
typedef struct cs_cells_meta_view {
    int32_t n_cells;         /* cells (= centres) when the index was built                      */
    int32_t n_work;          /* cells visited by the last pick                                  */
    int32_t n_chunks;        /* tiles of CS_CELL_TILE slots visited by the last pick             */
    int32_t total_slots;     /* slots in use                                                    */
    uint64_t visited_slots;  /* slots visited, summed over the picks since the build            */
    uint64_t picks;          /* picks since the build                                           */
    uint32_t q_count;        /* rows the last pick queued for evaluation                        */
    uint32_t q_inline;       /* rows the last pick evaluated outside the queue (queue full)     */
    uint8_t reserved[CS_CELLS_META_BYTES - 40];
} cs_cells_meta_view;

/* Build the index from the current h / voronoi with one cell per committed centre (n_sel of them).
 * Requires n_sel >= 1.  Several launches, no host synchronisation. */
CS_API int cs_cells_build(const cs_state* s, const cs_cells* c, cs_stream stream);

/* One pick with the index, after cs_commit_bound: choose the cells to visit ... */
CS_API int cs_cells_select(const cs_state* s, const cs_cells* c, cs_stream stream);

/* ... and run the update over them (two launches: scan the visited cells, then evaluate the rows
 * that need a distance); same effect on h, voronoi, the control block and the candidate pack as
 * cs_fps_step(CS_MODE_PRUNE).  Row widths: D % 4 == 0, D <= 1024. */
CS_API int cs_fps_step_cells(const cs_state* s, const cs_cells* c, cs_stream stream);

/*
 * cs_fps_step without any caller-provided scratch and without any allocation.  No counterpart
 * in the reference.
 *
 * For hosts that cannot allocate device memory while they run -- a process that gave the whole
 * HBM to its own arena at start-up, or a plug-in inside a service that forbids driver
 * allocations (and the device-wide stall they cause) on its request path.  The control block
 * and the centre slot that cs_fps_step normally finds in caller buffers live in a fixed
 * per-device array inside the library (256 + 256 + 4 * CS_NOALLOC_MAX_D bytes, held by every GPU
 * that loads the library until the process exits).  The call makes no cudaMalloc / cudaFree and
 * uses no allocating library routine.
 *
 * Inputs: X, norms, h, voronoi as in cs_state; `centre` = the D floats of the new centre,
 * `norm_new` its squared norm, `sel_pos` its position in the selection (written into voronoi;
 * 0 selects the dense first-centre update), `dSL_quarter` = sel_pos triangle bounds (may be NULL
 * when sel_pos == 0).  Precondition: the centre's own row already carries h = -1 (what
 * cs_commit_bound does for the row it commits); the step never selects, it only updates.
 * Outputs: h / voronoi updated in place; *out_key = the arg-max key of the
 * next pick (value-orderable bits << 32 | 0xFFFFFFFF - global index, 0 = no candidate);
 * *out_live_rows (optional) = rows whose distance was evaluated.  All pointers are device
 * pointers.  D above CS_NOALLOC_MAX_D returns CS_E_SCRATCH.
 *
 * The first call on a device looks up the array's device address (a synchronous runtime query):
 * make that call before starting any stream capture.  Every call on a device shares the one
 * array, which keeps the previous call's contents; each call clears what must start at zero, but
 * two calls that overlap on the GPU (different streams, no ordering) race on it.
 */
#define CS_NOALLOC_MAX_D 4096
CS_API int cs_fps_step_noalloc(const float* X, const float* norms, float* h, int32_t* voronoi,
                               int64_t N_local, int32_t D, int64_t shard_offset, const float* centre,
                               float norm_new, const float* dSL_quarter, int32_t sel_pos, uint32_t mode,
                               uint64_t* out_key, uint64_t* out_live_rows, cs_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* CORESETS_B200_H */
