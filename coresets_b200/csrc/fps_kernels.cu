// sm_100a kernels and C entry points of the farthest-point-sampling engine.
//
// Data layout in HBM (per rank): X [N_local, D] fp32 row-major (streamed once per pick),
// norms / h fp32 [N_local], voronoi int32 [N_local]; the committed centres X_sel [cap, D],
// norms_sel, dSL_quarter are small and L2-resident.  One pick = commit_bound_kernel (tiny) + one
// step kernel (the bandwidth-bound pass with the arg-max fused in).
//
// ONE translation unit: the kernels live in the .cuh files included below, this file holds the
// host-side launchers and the extern "C" entry points.
//   fps_common.cuh     constants, control block, arg-max key, the reference's dot product
//   exchange.cuh       candidate exchange between ranks, winner resolution
//   commit_bound.cuh   resolve + commit + triangle bounds
//   step_plain.cuh     step kernel with plain loads (inline prune walk, dense LDG, any row width)
//   step_queue.cuh     default prune mode: streamed scan + deferred rows in batches
//   step_tma.cuh       dense mode through a cp.async.bulk + mbarrier ring
//   step_lanes.cuh     several states sharing one pass over X
//   small_kernels.cuh  state set-up kernels, stand-alone arg-max scan
//   select.cuh         exact k-th largest, arg-max over a list of rows
//   cells.cuh          cell index: rows grouped by centre, picks that read only the cells that can change
//
// Arithmetic is spelled with __fmul_rn/__fmaf_rn/__fadd_rn so that no compiler contraction or
// reassociation can change a bit; the file is compiled with -ftz=true because the reference
// builds with --use_fast_math (src/coresets/cuda/extension.py:63).
#include "coresets_b200.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "fps_common.cuh"
#include "exchange.cuh"
#include "commit_bound.cuh"
#include "step_plain.cuh"
#include "step_queue.cuh"
#include "step_tma.cuh"
#include "step_tma_half.cuh"
#include "step_lanes.cuh"
#include "small_kernels.cuh"
#include "select.cuh"
#include "cells.cuh"

namespace {

// ---- host side ---------------------------------------------------------------------------------
struct DevInfo {
    int dev = 0;
    int sms = 0;
    int cc_major = 0;
    bool ok = false;
};
constexpr int kMaxDevices = 64;
DevInfo device_info() {
    static thread_local int cached_dev = -1;
    static thread_local DevInfo info;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return DevInfo();
    if (dev != cached_dev) {
        DevInfo d;
        d.dev = dev;
        if (dev < 0 || dev >= kMaxDevices) return DevInfo();
        if (cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return DevInfo();
        if (cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return DevInfo();
        d.ok = true;
        info = d;
        cached_dev = dev;
    }
    return info;
}

int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        g_last_cuda = e;
        return CS_E_LAUNCH;
    }
    return CS_OK;
}

// Per kernel, per device: the dynamic shared-memory size opted into and the resident blocks per SM
// found for the last shared-memory size.  cudaFuncSetAttribute applies to the device that is
// current, so a thread that moves to another device must opt in there again.
struct KernelTune {
    size_t attr_set[kMaxDevices];
    size_t occ_smem[kMaxDevices];
    int occ_blocks[kMaxDevices];
};
template <typename K>
int tune_kernel(K kernel, KernelTune& t, const int dev, const size_t smem, const int threads, int* blocks_per_sm) {
    // (opt in whenever the dynamic part grows: with the kernel's static part the total may pass 48 KB sooner)
    if (smem > t.attr_set[dev]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            g_last_cuda = cudaGetLastError();
            return CS_E_LAUNCH;
        }
        t.attr_set[dev] = smem;
    }
    if (blocks_per_sm) {
        if (t.occ_blocks[dev] == 0 || t.occ_smem[dev] != smem) {
            int per_sm = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm < 1) {
                g_last_cuda = cudaGetLastError();
                return CS_E_LAUNCH;
            }
            t.occ_blocks[dev] = per_sm;
            t.occ_smem[dev] = smem;
        }
        *blocks_per_sm = t.occ_blocks[dev];
    }
    return CS_OK;
}

// Launch that may overlap its start with the tail of the kernel before it on the stream
// (programmatic dependent launch): the grid is made resident early and its first instruction,
// griddepcontrol.wait, holds it until the predecessor has completed and flushed its memory.  Taken
// when the state carries CS_F_PDL; a plain launch otherwise (the wait is then a no-op).
template <typename... KArgs, typename... Args>
int launch_chain(const bool pdl, void (*kernel)(KArgs...), const int grid, const int block, const size_t smem,
                 cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...) != cudaSuccess) {
        g_last_cuda = cudaGetLastError();
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
    if ((s->flags & CS_F_X_HALF) && !(s->flags & CS_F_ELEMENT_ORDER)) return CS_E_ARG;
    if (s->shard_offset + s->N_local >= (int64_t)1 << 31) return CS_E_RANGE;
    if (s->cap >= (int64_t)1 << 31) return CS_E_RANGE;
    if ((s->D & 3) == 0) {
        if ((((s->flags & CS_F_X_HALF) ? 0 : (uintptr_t)s->X) | (uintptr_t)s->X_sel) & 15u) return CS_E_ALIGN;
        if (s->world_size > 1 && s->xchg == CS_XCHG_GATHER &&
            (((uintptr_t)s->pack_local | (uintptr_t)s->pack_all) & 15u)) return CS_E_ALIGN;
    }
    return CS_OK;
}

template <int CPL, bool HALF, int S, int B, int T, int W>
int launch_step_tma(const cs_state* s, cudaStream_t st, const DevInfo& dv) {
    const int sms = dv.sms;
    static_assert(W <= kTmaMaxWarps && (W % 8) == 0, "consumer warps");
    const int D = s->D;
    int tile_rows = T / (D * 4);
    tile_rows = tile_rows > 32 * W ? 32 * W : tile_rows;   // a lane owns one row of its warp's share
    tile_rows -= tile_rows % W;                             // W is a multiple of 8: 16-byte multiples of h / voronoi / norms
    if (tile_rows < W) tile_rows = W;
    const size_t smem = (size_t)S * tile_rows * (D * 4 + 12);   // rows of X, then h / voronoi / norm words
    static thread_local KernelTune tune;
    const int rc = tune_kernel(fps_step_tma_kernel<CPL, S, HALF, W, B>, tune, dv.dev, smem, (W + 1) * 32, nullptr);
    if (rc) return rc;
    const int64_t ntiles = (s->N_local + tile_rows - 1) / tile_rows;
    int64_t cap = (int64_t)sms * B;                         // resident blocks, each with its own ring
    int grid = (int)(ntiles < 1 ? 1 : (ntiles < cap ? ntiles : cap));
    fps_step_tma_kernel<CPL, S, HALF, W, B><<<grid, (W + 1) * 32, smem, st>>>(*s, tile_rows);
    return check_launch();
}

// dense mode over half rows: J elements per lane, RB rows reduced together
template <int J, int RB, int S, int B, int T, int W>
int launch_step_tma_half(const cs_state* s, cudaStream_t st, const DevInfo& dv) {
    static_assert(W <= kTmaMaxWarps && (W % 8) == 0 && 32 % RB == 0, "consumer warps / batch");
    const int D = s->D;
    int tile_rows = T / (D * 2);
    tile_rows = tile_rows > 32 * W ? 32 * W : tile_rows;
    tile_rows -= tile_rows % (W * RB);                     // a warp's share of a tile is whole batches
    if (tile_rows < W * RB) tile_rows = W * RB;
    const size_t smem = (size_t)S * tile_rows * (D * 2 + 12);
    static thread_local KernelTune tune;
    const int rc = tune_kernel(fps_step_tma_half_kernel<J, RB, S, W, B>, tune, dv.dev, smem, (W + 1) * 32, nullptr);
    if (rc) return rc;
    const int64_t ntiles = (s->N_local + tile_rows - 1) / tile_rows;
    const int64_t cap = (int64_t)dv.sms * B;
    const int grid = (int)(ntiles < 1 ? 1 : (ntiles < cap ? ntiles : cap));
    fps_step_tma_half_kernel<J, RB, S, W, B><<<grid, (W + 1) * 32, smem, st>>>(*s, tile_rows);
    return check_launch();
}

constexpr int kBoundSmemMax = 16384;     // triangle bounds staged in shared memory (64 KB)

template <int CPL, bool FULL, bool HALF = false>
int launch_step(const cs_state* s, unsigned mode, cudaStream_t st, const DevInfo& dv) {
    const int sms = dv.sms;
    static thread_local KernelTune tune;
    int occ_blocks = 0;
    const int n_bound = (int)(s->cap < kBoundSmemMax ? s->cap : kBoundSmemMax);
    const size_t smem = ((size_t)((n_bound + 3) & ~3) + (CPL ? 0 : (size_t)s->D)) * sizeof(float);
    const int rc = tune_kernel(fps_step_kernel<CPL, FULL, HALF>, tune, dv.dev, smem, kThreads, &occ_blocks);
    if (rc) return rc;
    const int64_t tiles = (s->N_local + (32 * kRowsPerLane - 1)) >> kTileShift;
    int64_t want = (tiles + kWarps - 1) / kWarps;
    int64_t cap = (int64_t)sms * occ_blocks;     // persistent grid: a multiple of the SM count
    int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    return launch_chain((s->flags & CS_F_PDL) != 0, fps_step_kernel<CPL, FULL, HALF>, grid, kThreads, smem, st, *s, mode, n_bound);
}

// prune mode with deferred rows (rows in whole 16-byte chunks, D <= 1024)
template <int CPL, bool FULL, bool HALF = false>
int launch_step_queue(const cs_state* s, cudaStream_t st, const DevInfo& dv) {
    const int sms = dv.sms;
    static thread_local KernelTune tune;
    int occ_blocks = 0;
    const int n_bound = (int)(s->cap < kBoundSmemMax ? s->cap : kBoundSmemMax);
    const size_t smem = ((size_t)kScanRingFloats + (size_t)((n_bound + 3) & ~3) + (CPL ? 0 : (size_t)s->D)) * sizeof(float);
    const int rc = tune_kernel(fps_step_queue_kernel<CPL, FULL, HALF>, tune, dv.dev, smem, kThreads, &occ_blocks);
    if (rc) return rc;
    const int64_t tiles = (s->N_local + 127) >> 7;
    int64_t want = (tiles + kWarps - 1) / kWarps;
    int64_t cap = (int64_t)sms * occ_blocks;     // persistent grid: a multiple of the SM count
    int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    return launch_chain((s->flags & CS_F_PDL) != 0, fps_step_queue_kernel<CPL, FULL, HALF>, grid, kThreads, smem, st, *s, n_bound);
}

template <int L, int CPL>
int launch_lanes_t(const LaneSet& ls, unsigned mode, cudaStream_t st, const DevInfo& dv) {
    const int sms = dv.sms;
    const size_t smem = (size_t)L * ls.s[0].D * sizeof(float);
    static thread_local KernelTune tune;
    int per_sm = 0;
    const int rc = tune_kernel(fps_step_lanes_kernel<L, CPL>, tune, dv.dev, smem, kThreads, &per_sm);
    if (rc) return rc;
    const int64_t tiles = (ls.s[0].N_local + 31) >> 5;
    int64_t want = (tiles + kWarps - 1) / kWarps;
    int64_t cap = (int64_t)sms * per_sm;
    int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    fps_step_lanes_kernel<L, CPL><<<grid, kThreads, smem, st>>>(ls, mode);
    return check_launch();
}

template <int L>
int launch_lanes_l(const LaneSet& ls, unsigned mode, cudaStream_t st, const DevInfo& sms) {
    const int D = ls.s[0].D;
    if (D <= 128) return launch_lanes_t<L, 1>(ls, mode, st, sms);
    if (D <= 256) return launch_lanes_t<L, 2>(ls, mode, st, sms);
    if (D <= 512) return launch_lanes_t<L, 4>(ls, mode, st, sms);
    return launch_lanes_t<L, 8>(ls, mode, st, sms);
}

int launch_lanes(const LaneSet& ls, int n, unsigned mode, cudaStream_t st, const DevInfo& sms) {
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

int cs_pool_pick(const cs_state* s, const int64_t* pool, const int64_t* n_pool, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    if (!pool || !n_pool) return CS_E_ARG;
    pool_pick_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(*s, pool, n_pool);
    return check_launch();
}

int cs_force_pick_list(const cs_state* s, const int64_t* list, const float* vals, float val, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    if (!list) return CS_E_ARG;
    force_pick_list_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(*s, list, vals, val);
    return check_launch();
}

int cs_commit_bound(const cs_state* s, uint32_t rules, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    if (rules > CS_RULE_STOP_NONPOS) return CS_E_ARG;
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
    return launch_chain((s->flags & CS_F_PDL) != 0, commit_bound_kernel, grid, kThreads, smem, (cudaStream_t)stream, *s, rules);
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
        if (D <= 64) return launch_step_tma<1, true, kRingNarrow.stages, kRingNarrow.blocks, kRingNarrow.tile_bytes, kRingNarrow.warps>(s, st, d);
        if (D <= 128) return launch_step_tma<1, false, kRingMid.stages, kRingMid.blocks, kRingMid.tile_bytes, kRingMid.warps>(s, st, d);
        if (D <= 256) return launch_step_tma<2, false, kRingWide.stages, kRingWide.blocks, kRingWide.tile_bytes, kRingWide.warps>(s, st, d);
        if (D <= 512) return launch_step_tma<4, false, kRingWide.stages, kRingWide.blocks, kRingWide.tile_bytes, kRingWide.warps>(s, st, d);
        return launch_step_tma<8, false, kRingWide.stages, kRingWide.blocks, kRingWide.tile_bytes, kRingWide.warps>(s, st, d);
    }
    if (mode == CS_MODE_DENSE && bulk_ok && (s->flags & CS_F_X_HALF) && (D & 7) == 0 && D <= 1024 && s->N_local > 0) {
        if (D <= 32) return launch_step_tma_half<1, 8, 5, 1, 65536, 16>(s, st, d);
        if (D <= 64) return launch_step_tma_half<2, 8, 3, 1, 65536, 16>(s, st, d);
        if (D <= 128) return launch_step_tma_half<4, 8, 3, 1, 65536, 16>(s, st, d);
        // sixteen consumer warps at every width: with eight the issue rate, not HBM, set the pace
        // (8 M x 256: 0.85 -> 0.63 ms, 4 M x 512: 1.01 -> 0.61 ms, 2 M x 1024: 0.71 -> 0.61 ms)
        if (D <= 256) return launch_step_tma_half<8, 8, 3, 1, 65536, 16>(s, st, d);
        if (D <= 512) return launch_step_tma_half<16, 4, 3, 1, 65536, 16>(s, st, d);
        return launch_step_tma_half<32, 2, 3, 1, 65536, 16>(s, st, d);
    }
    const bool generic = element_order || (D & 3) != 0 || D > 1024;
    if (generic && mode == CS_MODE_PRUNE && s->N_local > 0 && D <= 16384) return launch_step_queue<0, false>(s, st, d);
    if (generic) return launch_step<0, false>(s, mode, st, d);
    if (mode == CS_MODE_PRUNE && s->N_local > 0) {
        switch (D) {
            case 128: return launch_step_queue<1, true>(s, st, d);
            case 256: return launch_step_queue<2, true>(s, st, d);
            case 512: return launch_step_queue<4, true>(s, st, d);
            case 1024: return launch_step_queue<8, true>(s, st, d);
            default: break;
        }
        if (D <= 64) return launch_step_queue<1, false, true>(s, st, d);
        if (D < 128) return launch_step_queue<1, false>(s, st, d);
        if (D < 256) return launch_step_queue<2, false>(s, st, d);
        if (D < 512) return launch_step_queue<4, false>(s, st, d);
        return launch_step_queue<8, false>(s, st, d);
    }
    switch (D) {
        case 128: return launch_step<1, true>(s, mode, st, d);
        case 256: return launch_step<2, true>(s, mode, st, d);
        case 512: return launch_step<4, true>(s, mode, st, d);
        case 1024: return launch_step<8, true>(s, mode, st, d);
        default: break;
    }
    if (D <= 64) return launch_step<1, false, true>(s, mode, st, d);    // two rows per warp-wide load
    if (D < 128) return launch_step<1, false>(s, mode, st, d);
    if (D < 256) return launch_step<2, false>(s, mode, st, d);
    if (D < 512) return launch_step<4, false>(s, mode, st, d);
    return launch_step<8, false>(s, mode, st, d);
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
    return launch_lanes(ls, n_lanes, mode, (cudaStream_t)stream, d);
}

}  // extern "C"

namespace {

int validate_cells(const cs_state* s, const cs_cells* c) {
    if (!c || !c->perm || !c->hp || !c->vp || !c->cell0 || !c->seg_start || !c->seg_count || !c->seg_key || !c->seg_h0 ||
        !c->cursor || !c->work_cell || !c->work_cum || !c->meta || !c->queue) return CS_E_ARG;
    if (c->q_cap < kCellTile || ((uintptr_t)c->queue & 7u)) return CS_E_ARG;
    if (s->N_local <= 0) return CS_E_ARG;
    if (s->cap > 65536) return CS_E_RANGE;                      // the selection kernel takes 64 cells per thread
    if (c->slots >= (int64_t)1 << 31 || c->slots < s->N_local + s->cap * (int64_t)kCellTile) return CS_E_RANGE;
    if ((((uintptr_t)c->perm | (uintptr_t)c->hp | (uintptr_t)c->vp) & 15u) || ((uintptr_t)c->meta & 7u)) return CS_E_ALIGN;
    if (!(c->row_norm_max >= 0.0f)) return CS_E_ARG;
    return CS_OK;
}

template <int CPL, bool FULL, bool HALF = false>
int launch_step_cells(const cs_state* s, const cs_cells* c, cudaStream_t st, const DevInfo& dv) {
    static thread_local KernelTune tune_scan, tune_eval;
    int per_scan = 0, per_eval = 0;
    int rc = tune_kernel(cells_scan_kernel<CPL, FULL, HALF>, tune_scan, dv.dev, 0, kThreads, &per_scan);
    if (rc) return rc;
    rc = tune_kernel(cells_eval_kernel<CPL, FULL, HALF>, tune_eval, dv.dev, 0, kThreads, &per_eval);
    if (rc) return rc;
    // persistent grids: the numbers of tiles and of queued rows are only known on the device
    const int64_t tiles = (s->N_local + kCellTile - 1) / kCellTile + 1;
    const int64_t want_scan = (tiles + kWarps - 1) / kWarps, cap_scan = (int64_t)dv.sms * per_scan;
    const bool pdl = (s->flags & CS_F_PDL) != 0;
    rc = launch_chain(pdl, cells_scan_kernel<CPL, FULL, HALF>, (int)(want_scan < cap_scan ? want_scan : cap_scan), kThreads, 0, st, *s, *c);
    if (rc) return rc;
    const int64_t want_eval = ((int64_t)c->q_cap + kThreads - 1) / kThreads, cap_eval = (int64_t)dv.sms * per_eval;
    return launch_chain(pdl, cells_eval_kernel<CPL, FULL, HALF>, (int)(want_eval < cap_eval ? want_eval : cap_eval), kThreads, 0, st, *s, *c);
}

}  // namespace

extern "C" {

int cs_cells_build(const cs_state* s, const cs_cells* c, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    rc = validate_cells(s, c);
    if (rc) return rc;
    DevInfo d = device_info();
    if (!d.ok) return CS_E_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaMemsetAsync(c->seg_count, 0, (size_t)s->cap * sizeof(int32_t), st) != cudaSuccess) {
        g_last_cuda = cudaGetLastError();
        return CS_E_LAUNCH;
    }
    const int bins = (int)(s->cap < kCellBinsSmem ? s->cap : kCellBinsSmem);
    const size_t smem = (size_t)bins * sizeof(int);
    static thread_local KernelTune tune_hist, tune_scatter;
    int per_hist = 0, per_scatter = 0;
    rc = tune_kernel(cells_hist_kernel, tune_hist, d.dev, smem, kThreads, &per_hist);
    if (rc) return rc;
    rc = tune_kernel(cells_scatter_kernel, tune_scatter, d.dev, smem, kThreads, &per_scatter);
    if (rc) return rc;
    const int64_t row_blocks = (s->N_local + 4 * kThreads - 1) / (4 * kThreads);
    const int64_t lim_hist = (int64_t)d.sms * per_hist;
    cells_hist_kernel<<<(int)(row_blocks < lim_hist ? row_blocks : lim_hist), kThreads, smem, st>>>(*s, *c);
    cells_offsets_kernel<<<1, 1024, 0, st>>>(*s, *c);
    int rows_per_block = 4 * bins;
    rows_per_block = rows_per_block < 16384 ? 16384 : (rows_per_block > (1 << 18) ? (1 << 18) : rows_per_block);
    const int64_t chunks = (s->N_local + rows_per_block - 1) / rows_per_block;
    const int64_t lim_scatter = (int64_t)d.sms * per_scatter;
    cells_scatter_kernel<<<(int)(chunks < lim_scatter ? chunks : lim_scatter), kThreads, smem, st>>>(*s, *c, rows_per_block);
    const int64_t cell_blocks = (s->cap + kWarps - 1) / kWarps;
    const int64_t lim = (int64_t)d.sms * 8;
    cells_pad_kernel<<<(int)(cell_blocks < lim ? cell_blocks : lim), kThreads, 0, st>>>(*s, *c);
    const int64_t tile_blocks = (c->slots / kCellTile + kWarps - 1) / kWarps;
    cells_keys_kernel<<<(int)(tile_blocks < lim ? tile_blocks : lim), kThreads, 0, st>>>(*s, *c);
    const int64_t h0_blocks = (s->cap + kThreads - 1) / kThreads;
    cells_h0_kernel<<<(int)(h0_blocks < lim ? h0_blocks : lim), kThreads, 0, st>>>(*s, *c);
    return check_launch();
}

int cs_cells_select(const cs_state* s, const cs_cells* c, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    rc = validate_cells(s, c);
    if (rc) return rc;
    // rounding-error bound of one computed squared distance, relative to the sum of the two squared
    // norms: D products and sums in the dot product, D in each norm, a few more in the final formula;
    // the factor 4 is slack
    const double g = 4.0 * ((double)s->D + 32.0) * 5.9604644775390625e-8;
    return launch_chain((s->flags & CS_F_PDL) != 0, cells_select_kernel, 1, 1024, 0, (cudaStream_t)stream, *s, *c, g);
}

int cs_fps_step_cells(const cs_state* s, const cs_cells* c, cs_stream stream) {
    int rc = validate(s);
    if (rc) return rc;
    rc = validate_cells(s, c);
    if (rc) return rc;
    const int D = s->D;
    if ((D & 3) != 0 || D > 1024 || (s->flags & CS_F_ELEMENT_ORDER)) return CS_E_ARG;
    if (((uintptr_t)s->h | (uintptr_t)s->voronoi) & 3u) return CS_E_ALIGN;
    DevInfo d = device_info();
    if (!d.ok) return CS_E_DEVICE;
    cudaStream_t st = (cudaStream_t)stream;
    switch (D) {
        case 128: return launch_step_cells<1, true>(s, c, st, d);
        case 256: return launch_step_cells<2, true>(s, c, st, d);
        case 512: return launch_step_cells<4, true>(s, c, st, d);
        case 1024: return launch_step_cells<8, true>(s, c, st, d);
        default: break;
    }
    if (D <= 64) return launch_step_cells<1, false, true>(s, c, st, d);
    if (D < 128) return launch_step_cells<1, false>(s, c, st, d);
    if (D < 256) return launch_step_cells<2, false>(s, c, st, d);
    if (D < 512) return launch_step_cells<4, false>(s, c, st, d);
    return launch_step_cells<8, false>(s, c, st, d);
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
    // (the two bases below are formed by integer arithmetic on DEVICE addresses and point outside the
    // scratch object; the kernel only ever dereferences slot sel_pos, which lies inside it)
    const uintptr_t row_slot = (uintptr_t)(scratch + CS_CTL_BYTES + 256);
    const uintptr_t norm_slot = (uintptr_t)(scratch + CS_CTL_BYTES);
    s.X_sel = reinterpret_cast<float*>(row_slot - (uintptr_t)sel_pos * (uintptr_t)D * sizeof(float));
    s.norms_sel = reinterpret_cast<float*>(norm_slot - (uintptr_t)sel_pos * sizeof(float));
    s.dSL_quarter = const_cast<float*>(dSL_quarter ? dSL_quarter : reinterpret_cast<const float*>(norm_slot));
    // capacity = the next power of two above the pick position: the step kernel sizes its staged
    // bound table (and with it its shared memory and grid) from the capacity, so the launch shape
    // changes O(log k) times over a run instead of with every pick (it reads only sel_pos bounds)
    int64_t cap_q = 1;
    while (cap_q < (int64_t)sel_pos + 1) cap_q <<= 1;
    s.cap = cap_q;
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
