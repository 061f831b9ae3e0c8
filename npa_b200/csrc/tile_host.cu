// Host side of the cell-tile streaming engine (tile_stream.cuh): the shared-memory plan of a launch,
// the tuning switches and the device status word of the bounded waits.
#include <mutex>

#include "feature_tile.cuh"

namespace npa {

void set_scalar_shared_span(int span);  // scalar_ops.cu

static int align_up(int v, int a) { return (v + a - 1) / a * a; }

// Largest dynamic shared memory a CTA may ask for on this architecture (227 KB on sm_100) minus
// what the kernels hold statically.
constexpr int kTileSmemLimit = 227 * 1024 - 1024;

bool tile_make_layout(int P, bool with_mass, int floats_s, int floats_gb, int floats_gg, int consumer_warps,
                      int list_bytes, int acc_bytes, int want_rmax, int want_tp, int want_stages, int want_span,
                      bool backward, TileLayout *out) {
    TileLayout L = {};
    L.warps = consumer_warps;
    L.span = want_span > 0 ? want_span : 2;
    L.stages = want_stages > 0 ? want_stages : (backward ? 2 : 3);
    if (L.stages < 1 || L.stages > kTileMaxStages) return false;
    L.tp = want_tp > 0 ? want_tp : 32;
    // accumulator slots belong to consumer warps (slot = warp + warps * k): round up to whole rounds
    const int acc_slots = (L.tp + consumer_warps - 1) / consumer_warps * consumer_warps;
    L.acc_bytes = align_up(acc_bytes, 16);
    L.list_bytes = align_up(list_bytes, 16);
    const int fixed = align_up((int)sizeof(TileChunk) * L.stages, 128) + align_up(L.list_bytes * consumer_warps, 128) +
                      align_up(L.acc_bytes * acc_slots, 128) + align_up(16 * L.stages, 128);
    const int row_bytes = P * 4 + 4 + (with_mass ? 4 : 0) + 4 * (floats_s + floats_gb + floats_gg);
    // every array of a stage starts on a 128-byte boundary: six arrays of slack per stage
    auto fit = [&](int budget) { return ((budget - fixed - L.stages * 6 * 128) / (L.stages * row_bytes)) & ~3; };
    int rmax;
    if (want_rmax > 0) {
        if ((want_rmax & 3) || want_rmax > fit(kTileSmemLimit)) return false;
        rmax = want_rmax;
    } else {
        // automatic: two CTAs per SM (half of the shared memory each, 1 KB reserved per CTA)
        rmax = fit(kTileSmemLimit / 2 - 1024);
        if (rmax > 512) rmax = 512;
        if (rmax < 48) rmax = fit(kTileSmemLimit);  // wide rows: one CTA per SM
    }
    if (rmax < 32) return false;
    L.rmax = rmax;
    int off = 0;
    L.off_x = off;     off = align_up(off + rmax * P * 4, 128);
    L.off_rho = off;   off = align_up(off + rmax * 4, 128);
    L.off_mass = off;  off = align_up(off + (with_mass ? rmax * 4 : 0), 128);
    L.off_s = off;     off = align_up(off + rmax * floats_s * 4, 128);
    L.off_gb = off;    off = align_up(off + rmax * floats_gb * 4, 128);
    L.off_gg = off;    off = align_up(off + rmax * floats_gg * 4, 128);
    L.stage_bytes = off;
    off = L.stage_bytes * L.stages;
    L.off_chunks = off;  off = align_up(off + (int)sizeof(TileChunk) * L.stages, 128);
    L.off_lists = off;   off = align_up(off + L.list_bytes * consumer_warps, 128);
    L.off_acc = off;     off = align_up(off + L.acc_bytes * acc_slots, 128);
    L.off_bars = off;    off = align_up(off + 16 * L.stages, 128);
    L.total_bytes = off;
    if (L.total_bytes > kTileSmemLimit) return false;
    *out = L;
    return true;
}

// ---- tuning (process-wide; npa_tile_tuning) ---------------------------------------------------
// Off by default: on the measured workloads the gather kernels are as fast or faster (the sweeps are
// bound by instruction issue, not by the L2 -> SM traffic the staging saves).
static TileTuning g_tuning[2] = {{0, 0, 0, 0, kTileWarpsDefault, 0}, {0, 0, 0, 0, kTileWarpsDefault, 0}};
bool tile_forward_enabled() { return tile_tuning(false).enabled != 0; }

TileTuning tile_tuning(bool backward) { return g_tuning[backward ? 1 : 0]; }

// ---- status word ------------------------------------------------------------------------------
static __device__ unsigned int g_tile_status;  // zero at load; a timed-out wait stores its code here

int tile_status_word(unsigned int **out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static unsigned int *addr[kMaxDevices] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(NPA_ERR_UNSUPPORTED, "device ordinal %d is out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_tile_status);
        if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaGetSymbolAddress(tile status): %s", cudaGetErrorString(e));
        addr[dev] = static_cast<unsigned int *>(p);
    }
    *out = addr[dev];
    return NPA_OK;
}

// One CTA waits on an mbarrier that nothing will ever complete, with a short limit, and reports how
// the wait ended: the self-test of the bounded waits (the context stays usable).
__global__ void tile_wait_selftest_kernel(unsigned long long limit_ns, int *result) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const bool completed = mbar_wait(&bar, 0u, limit_ns);  // phase 0 never completes: no arrival is made
    if (threadIdx.x == 0) *result = completed ? 0 : TILE_STATUS_FULL_TIMEOUT;
}

}  // namespace npa

using namespace npa;

extern "C" {

int npa_tile_tuning(int32_t backward, int32_t enabled, int32_t rows_per_stage, int32_t particles_per_tile,
                    int32_t stages, int32_t consumer_warps, int32_t cells_per_tile) {
    if (rows_per_stage < 0 || (rows_per_stage & 3) || particles_per_tile < 0 || stages < 0 ||
        stages > kTileMaxStages || (consumer_warps != 0 && consumer_warps != 8 && consumer_warps != 16 && consumer_warps != 24) ||
        cells_per_tile < 0 || cells_per_tile > kTileBatch)
        return fail(NPA_ERR_INVALID_ARGUMENT,
                    "tile_tuning: rows_per_stage must be a non-negative multiple of 4, particles_per_tile >= 0, "
                    "stages in [0, %d], consumer_warps 0, 8, 16 or 24 (24: forward only), cells_per_tile in [0, %d]", kTileMaxStages,
                    kTileBatch);
    g_tuning[backward ? 1 : 0] = TileTuning{rows_per_stage, particles_per_tile, stages, enabled ? 1 : 0,
                                            consumer_warps ? consumer_warps : kTileWarpsDefault, cells_per_tile};
    return NPA_OK;
}

int npa_scalar_sweep_tuning(int32_t cells_per_tile) {
    if (cells_per_tile < 0 || (cells_per_tile > 8 && (cells_per_tile < 101 || cells_per_tile > 108)))
        return fail(NPA_ERR_INVALID_ARGUMENT, "scalar_sweep_tuning: cells_per_tile must be in [0, 8] (+100: also on 3D periodic grids)");
    set_scalar_shared_span(cells_per_tile);
    return NPA_OK;
}

int npa_tile_wait_selftest(int32_t limit_us, int32_t *device_result, void *stream) {
    if (!device_result) return fail(NPA_ERR_INVALID_ARGUMENT, "tile_wait_selftest: device_result is NULL");
    if (limit_us <= 0 || limit_us > 1000000)
        return fail(NPA_ERR_INVALID_ARGUMENT, "tile_wait_selftest: limit_us must be in (0, 1000000]");
    tile_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>((unsigned long long)limit_us * 1000ull, device_result);
    return check_launch("tile_wait_selftest_kernel");
}

int npa_tile_status(int32_t *host_status, int32_t reset) {
    if (!host_status) return fail(NPA_ERR_INVALID_ARGUMENT, "tile_status: host_status is NULL");
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_tile_status, sizeof(v));
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "tile_status: %s", cudaGetErrorString(e));
    *host_status = (int32_t)v;
    if (reset && v != 0) {
        const unsigned int zero = 0;
        e = cudaMemcpyToSymbol(g_tile_status, &zero, sizeof(zero));
        if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "tile_status: %s", cudaGetErrorString(e));
    }
    return NPA_OK;
}

}  // extern "C"
