// Uniform-grid binning for B200: cell hash -> histogram -> scan -> stable
// counting sort -> work list, and the permutation kernels.
//
// Replaces HashGrid::initialize / bin_particles / backward_bin_particles of the
// reference (sphops/sph_cuda.cu:32-206,1926-2056).  Differences by design:
//  * the slot order inside a cell is the original particle order (stable), so
//    the permutation is deterministic; the reference orders by atomic arrival;
//  * histograms use warp-aggregated atomics, held in shared memory when the
//    per-system cell table fits, so a cell-coherent input (every step after the
//    first of a rollout) does not serialise on one address;
//  * cell counts and work-item counts are scanned together in one three-phase
//    scan, and the work list is written by the scan's last phase.
// All kernels are HBM-bound integer work; nothing here is GEMM shaped.
#include <mutex>

#include "common.cuh"

namespace npa {

constexpr int kBinThreads = 256;
constexpr int kBinPerThread = 8;                       // particles per thread in the hash pass
constexpr int kBinChunk = kBinThreads * kBinPerThread;  // particles per CTA
constexpr int kSmemHistCells = 8192;                   // 32 KB of shared histogram at most
constexpr int kScanThreads = 256;
constexpr int kScanPerThread = 8;
constexpr int kScanTile = kScanThreads * kScanPerThread;
// Cells with more particles than this are ranked by rank_crowded_kernel (linear in the population)
// instead of the per-particle scan of rank_kernel (quadratic in it).
constexpr int kCrowdedCell = 256;
constexpr int kRankWindow = 1 << 17;  // particle indices per bitmap window of rank_crowded_kernel (32 KB of shared memory)
constexpr int kRankCtas = 64;

struct BinScratch {
    uint32_t *counts;   // [B*cells + 1], then one word: number of crowded cells (zeroed with the counts)
    uint32_t *crowded;  // [B*N / kCrowdedCell + 1] global cell index of each crowded cell
    uint32_t *arrive;   // [B*N]  arrival number of the particle inside its cell (any order)
    uint32_t *cellid;   // [B*N]
    uint32_t *order;    // [B*N]  slot -> particle, unsorted inside a cell
    unsigned long long *partials;  // [tiles + 1] packed (blocks << 32 | particles)
    size_t zero_bytes;  // the counts are zeroed per call
    int tiles;
};

static size_t align_up(size_t v) { return (v + 255) & ~(size_t)255; }

static size_t layout_scratch(const Geom &g, void *base, BinScratch *s) {
    const size_t nc = (size_t)g.B * g.cells;
    const size_t np = (size_t)g.B * g.N;
    const int tiles = (int)((nc + kScanTile - 1) / kScanTile);
    size_t off = 0;
    char *p = (char *)base;
    size_t counts_off = off;
    off += align_up((nc + 2) * 4);
    size_t zero_end = off;
    size_t crowded_off = off;
    off += align_up((np / kCrowdedCell + 1) * 4);
    size_t arrive_off = off;
    off += align_up(np * 4);
    size_t cellid_off = off;
    off += align_up(np * 4);
    size_t order_off = off;
    off += align_up(np * 4);
    size_t part_off = off;
    off += align_up((size_t)(tiles + 1) * 8);
    if (s) {
        s->counts = (uint32_t *)(p + counts_off);
        s->crowded = (uint32_t *)(p + crowded_off);
        s->arrive = (uint32_t *)(p + arrive_off);
        s->cellid = (uint32_t *)(p + cellid_off);
        s->order = (uint32_t *)(p + order_off);
        s->partials = (unsigned long long *)(p + part_off);
        s->zero_bytes = zero_end;
        s->tiles = tiles;
    }
    return off;
}

// ---------------------------------------------------------------------------
// Pass 1: cell id per particle + per-cell histogram.
// ---------------------------------------------------------------------------
template <int D>
__device__ inline uint32_t particle_cell(const float *__restrict__ x, size_t idx, const Geom &g) {
    int cx, cy, cz = 0;
    if (D == 2) {
        float2 p = __ldg(reinterpret_cast<const float2 *>(x) + idx);
        cx = axis_cell(p.x, g, 0);
        cy = axis_cell(p.y, g, 1);
    } else {
        float4 p = __ldg(reinterpret_cast<const float4 *>(x) + idx);
        cx = axis_cell(p.x, g, 0);
        cy = axis_cell(p.y, g, 1);
        cz = axis_cell(p.z, g, 2);
    }
    return cell_hash<D>(g, cx, cy, cz);
}

// One atomic per distinct cell per warp: lanes holding the same key elect their lowest lane, which
// adds the group's population; every lane gets its arrival number in the cell (the counter's old
// value plus its rank in the group), which later serves as its unsorted slot inside the cell.
__device__ inline uint32_t warp_aggregated_take(uint32_t *hist, uint32_t key, bool valid) {
    const unsigned mask = __ballot_sync(kFull, valid);
    if (!valid) return 0;
    const unsigned peers = __match_any_sync(mask, key);
    const int lane = threadIdx.x & 31;
    const int leader = __ffs(peers) - 1;
    uint32_t base = 0;
    if (lane == leader) base = atomicAdd(&hist[key], (uint32_t)__popc(peers));
    base = __shfl_sync(peers, base, leader);
    return base + (uint32_t)__popc(peers & ((1u << lane) - 1));
}

template <int D, bool SMEM>
__global__ void __launch_bounds__(kBinThreads)
hash_count_kernel(const float *__restrict__ x, uint32_t *__restrict__ cellid, uint32_t *__restrict__ arrive,
                  uint32_t *__restrict__ counts, Geom g) {
    extern __shared__ uint32_t hist[];
    const int b = blockIdx.y;
    const int base = blockIdx.x * kBinChunk;
    if (SMEM) {
        for (int c = threadIdx.x; c < g.cells; c += kBinThreads) hist[c] = 0;
        __syncthreads();
    }
    uint32_t *gl = counts + (size_t)b * g.cells;
    uint32_t keys[kBinPerThread], arr[kBinPerThread];
#pragma unroll
    for (int k = 0; k < kBinPerThread; ++k) {
        const int i = base + k * kBinThreads + threadIdx.x;
        const bool valid = i < g.N;
        uint32_t key = 0;
        if (valid) {
            const size_t idx = (size_t)b * g.N + i;
            key = particle_cell<D>(x, idx, g);
            cellid[idx] = key;
        }
        keys[k] = key;
        arr[k] = warp_aggregated_take(SMEM ? hist : gl, key, valid);
    }
    if (SMEM) {
        // the CTA's populations go to the global counters in one atomic per cell; the old values
        // (where this CTA's particles start in the cell) replace the local counts
        __syncthreads();
        for (int c = threadIdx.x; c < g.cells; c += kBinThreads) {
            const uint32_t v = hist[c];
            hist[c] = v ? atomicAdd(&gl[c], v) : 0u;
        }
        __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < kBinPerThread; ++k) {
        const int i = base + k * kBinThreads + threadIdx.x;
        if (i < g.N) arrive[(size_t)b * g.N + i] = arr[k] + (SMEM ? hist[keys[k]] : 0u);
    }
}

// ---------------------------------------------------------------------------
// Three-phase exclusive scan of (particles per cell, work items per cell),
// packed as one 64-bit word so both prefix sums ride the same shuffles.
// ---------------------------------------------------------------------------
__device__ inline unsigned long long pack_cell(uint32_t count, int mpb) {
    uint32_t blocks = (count + (uint32_t)mpb - 1) / (uint32_t)mpb;
    return ((unsigned long long)blocks << 32) | count;
}

__device__ inline unsigned long long warp_inclusive(unsigned long long v) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        unsigned long long t = __shfl_up_sync(kFull, v, o);
        if (lane >= o) v += t;
    }
    return v;
}

// Exclusive scan of one value per thread across the CTA; returns the prefix of
// this thread and the CTA total through `total`.
template <int THREADS>
__device__ inline unsigned long long block_exclusive(unsigned long long v, unsigned long long &total) {
    __shared__ unsigned long long warp_tot[THREADS / 32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    unsigned long long inc = warp_inclusive(v);
    if (lane == 31) warp_tot[w] = inc;
    __syncthreads();
    if (w == 0) {
        unsigned long long t = lane < THREADS / 32 ? warp_tot[lane] : 0ull;
        unsigned long long ti = warp_inclusive(t);
        if (lane < THREADS / 32) warp_tot[lane] = ti - t;
        if (lane == THREADS / 32 - 1) total = ti;
    }
    __syncthreads();
    unsigned long long r = warp_tot[w] + inc - v;
    return r;
}

__global__ void __launch_bounds__(kScanThreads)
scan_tile_sums_kernel(const uint32_t *__restrict__ counts, unsigned long long *__restrict__ partials,
                      int n, int mpb) {
    __shared__ unsigned long long tot;
    const int base = blockIdx.x * kScanTile + threadIdx.x * kScanPerThread;
    unsigned long long v = 0;
#pragma unroll
    for (int k = 0; k < kScanPerThread; ++k)
        if (base + k < n) v += pack_cell(counts[base + k], mpb);
    block_exclusive<kScanThreads>(v, tot);
    __syncthreads();
    if (threadIdx.x == 0) partials[blockIdx.x] = tot;
}

__global__ void __launch_bounds__(1024)
scan_partials_kernel(unsigned long long *partials, int tiles) {
    __shared__ unsigned long long tot;
    __shared__ unsigned long long carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < tiles; base += 1024) {
        const int i = base + threadIdx.x;
        unsigned long long v = i < tiles ? partials[i] : 0ull;
        unsigned long long ex = block_exclusive<1024>(v, tot);
        unsigned long long carry = carry_s;
        if (i < tiles) partials[i] = carry + ex;
        __syncthreads();
        if (threadIdx.x == 0) carry_s = carry + tot;
        __syncthreads();
    }
    if (threadIdx.x == 0) partials[tiles] = carry_s;
}

// Writes bin_offsets, the work list rows of every non-empty cell, and zeroes
// the unused tail of the work list (rows [total_items, max_blocks)).
__global__ void __launch_bounds__(kScanThreads)
scan_apply_kernel(const uint32_t *__restrict__ counts, const unsigned long long *__restrict__ partials,
                  int32_t *__restrict__ bin_offsets, int4 *__restrict__ block_info, uint32_t *__restrict__ crowded,
                  uint32_t *__restrict__ crowded_count, int n, Geom g) {
    __shared__ unsigned long long tot;
    const int base = blockIdx.x * kScanTile + threadIdx.x * kScanPerThread;
    uint32_t c[kScanPerThread];
    unsigned long long v = 0;
#pragma unroll
    for (int k = 0; k < kScanPerThread; ++k) {
        c[k] = base + k < n ? counts[base + k] : 0u;
        v += pack_cell(c[k], g.mpb);
    }
    unsigned long long run = partials[blockIdx.x] + block_exclusive<kScanThreads>(v, tot);
#pragma unroll
    for (int k = 0; k < kScanPerThread; ++k) {
        const int cell = base + k;
        if (cell < n) {
            const uint32_t start = (uint32_t)run;
            uint32_t row = (uint32_t)(run >> 32);
            bin_offsets[cell] = (int32_t)start;
            if (c[k] > (uint32_t)kCrowdedCell) crowded[atomicAdd(crowded_count, 1u)] = (uint32_t)cell;
            const int sys = cell / g.cells;
            for (uint32_t off = 0; off < c[k]; off += (uint32_t)g.mpb, ++row)
                block_info[row] = make_int4(cell, (int)off, (int)min((uint32_t)g.mpb, c[k] - off), sys);
        }
        run += pack_cell(c[k], g.mpb);
    }
    const unsigned long long grand = partials[gridDim.x];
    if (blockIdx.x == 0 && threadIdx.x == 0) bin_offsets[n] = (int32_t)(uint32_t)grand;
    const int total_items = (int)(grand >> 32);
    for (int r = total_items + blockIdx.x * kScanThreads + threadIdx.x; r < g.max_blocks;
         r += gridDim.x * kScanThreads)
        block_info[r] = make_int4(0, 0, 0, 0);
}

// ---------------------------------------------------------------------------
// Pass 2: scatter particle indices to their cell's slots (any order inside the
// cell), then rank each slot by original index -> stable permutation.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kBinThreads)
scatter_kernel(const uint32_t *__restrict__ cellid, const uint32_t *__restrict__ arrive,
               const int32_t *__restrict__ bin_offsets, uint32_t *__restrict__ order, Geom g) {
    const int b = blockIdx.y;
    const int i = blockIdx.x * kBinThreads + threadIdx.x;
    if (i >= g.N) return;
    const size_t idx = (size_t)b * g.N + i;
    const size_t cell = (size_t)b * g.cells + cellid[idx];
    order[(uint32_t)bin_offsets[cell] + arrive[idx]] = (uint32_t)i;  // no atomics: the slot was drawn in pass 1
}

__global__ void __launch_bounds__(kBinThreads)
rank_kernel(const uint32_t *__restrict__ cellid, const int32_t *__restrict__ bin_offsets,
            const uint32_t *__restrict__ order, int32_t *__restrict__ permutation, Geom g) {
    const int b = blockIdx.y;
    const int p = blockIdx.x * kBinThreads + threadIdx.x;
    if (p >= g.N) return;
    const size_t sys = (size_t)b * g.N;
    const uint32_t i = order[sys + p];
    const uint32_t key = cellid[sys + i];
    const size_t cell = (size_t)b * g.cells + key;
    const uint32_t s = (uint32_t)bin_offsets[cell], e = (uint32_t)bin_offsets[cell + 1];
    if (e - s > (uint32_t)kCrowdedCell) return;  // ranked by rank_crowded_kernel
    uint32_t rank = 0;
    for (uint32_t q = s; q < e; ++q) rank += order[q] < i ? 1u : 0u;
    permutation[sys + i] = (int32_t)(s - (uint32_t)sys + rank);
}

// Stable ranks inside crowded cells (a collapsed system, or particles clamped into an edge cell): a
// CTA takes one crowded cell at a time, marks the original indices of its particles in a bitmap over
// the system's particle indices (in windows of kRankWindow indices), turns the bitmap into prefix
// popcounts, and a particle's rank is the number of marked indices below its own.  Linear in the
// population plus N / 32 words per window; no sort, no atomics in global memory.
__global__ void __launch_bounds__(256)
rank_crowded_kernel(const int32_t *__restrict__ bin_offsets, const uint32_t *__restrict__ order,
                    int32_t *__restrict__ permutation, const uint32_t *__restrict__ crowded,
                    const uint32_t *__restrict__ crowded_count, Geom g) {
    extern __shared__ uint32_t rank_smem[];
    __shared__ uint32_t warp_tot[8];
    __shared__ uint32_t carry;
    const int win = g.N < kRankWindow ? g.N : kRankWindow;
    const int words = (win + 31) / 32;
    uint32_t *bits = rank_smem, *pre = rank_smem + words;
    const uint32_t n = *crowded_count;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (uint32_t entry = blockIdx.x; entry < n; entry += gridDim.x) {
        const uint32_t cell = crowded[entry];
        const uint32_t sys = (cell / (uint32_t)g.cells) * (uint32_t)g.N;
        const uint32_t s = (uint32_t)bin_offsets[cell], e = (uint32_t)bin_offsets[cell + 1];
        uint32_t below = 0;  // particles of the cell with an index below the current window
        for (uint32_t w0 = 0; w0 < (uint32_t)g.N; w0 += (uint32_t)win) {
            for (int k = threadIdx.x; k < words; k += 256) bits[k] = 0u;
            if (threadIdx.x == 0) carry = 0u;
            __syncthreads();
            for (uint32_t q = s + threadIdx.x; q < e; q += 256) {
                const uint32_t i = order[q] - w0;
                if (i < (uint32_t)win) atomicOr(&bits[i >> 5], 1u << (i & 31));
            }
            __syncthreads();
            // exclusive prefix of the word popcounts, 256 words per round
            for (int base = 0; base < words; base += 256) {
                const int k = base + threadIdx.x;
                const uint32_t v = k < words ? (uint32_t)__popc(bits[k]) : 0u;
                uint32_t inc = v;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t t = __shfl_up_sync(kFull, inc, o);
                    if (lane >= o) inc += t;
                }
                if (lane == 31) warp_tot[w] = inc;
                __syncthreads();
                uint32_t before = carry;
                for (int ww = 0; ww < w; ++ww) before += warp_tot[ww];
                if (k < words) pre[k] = before + inc - v;
                __syncthreads();
                if (threadIdx.x == 255) carry = before + inc;
                __syncthreads();
            }
            for (uint32_t q = s + threadIdx.x; q < e; q += 256) {
                const uint32_t idx = order[q];
                const uint32_t i = idx - w0;
                if (i < (uint32_t)win) {
                    const uint32_t rank = below + pre[i >> 5] + (uint32_t)__popc(bits[i >> 5] & ((1u << (i & 31)) - 1u));
                    permutation[sys + idx] = (int32_t)(s - sys + rank);
                }
            }
            below += carry;
            __syncthreads();
        }
    }
}

// ---------------------------------------------------------------------------
// Permutation kernels.  One thread moves one 16-byte piece of a feature row
// (or one float when C % 4 != 0); the thread that owns piece 0 also moves the
// position and the mass.  FORWARD: out[perm[i]] = in[i]; else out[i] = in[perm[i]].
// ---------------------------------------------------------------------------
template <int D, bool FORWARD, typename VEC>
__global__ void __launch_bounds__(256)
permute_kernel(const float *__restrict__ x, const float *__restrict__ s, const float *__restrict__ m,
               const int32_t *__restrict__ perm, float *__restrict__ xo, float *__restrict__ so,
               float *__restrict__ mo, int pieces, long long total, int N) {
    const long long t = (long long)blockIdx.x * 256 + threadIdx.x;
    if (t >= total) return;
    const long long particle = t / pieces;
    const int piece = (int)(t - particle * pieces);
    const long long sys0 = (particle / N) * N;
    const long long other = sys0 + __ldg(perm + particle);
    const long long src = FORWARD ? particle : other;
    const long long dst = FORWARD ? other : particle;
    if (s) {
        const VEC *in = reinterpret_cast<const VEC *>(s);
        VEC *out = reinterpret_cast<VEC *>(so);
        out[dst * pieces + piece] = __ldg(in + src * pieces + piece);
    }
    if (piece == 0) {
        if (x) {
            if (D == 2)
                reinterpret_cast<float2 *>(xo)[dst] = __ldg(reinterpret_cast<const float2 *>(x) + src);
            else
                reinterpret_cast<float4 *>(xo)[dst] = __ldg(reinterpret_cast<const float4 *>(x) + src);
        }
        if (m) mo[dst] = __ldg(m + src);
    }
}

template <bool FORWARD>
static int launch_permute(const Geom &g, int C, const float *x, const float *s, const float *m,
                          const int32_t *perm, float *xo, float *so, float *mo, cudaStream_t st) {
    if (!perm) return fail(NPA_ERR_INVALID_ARGUMENT, "permutation is NULL");
    if ((x == nullptr) != (xo == nullptr) || (s == nullptr) != (so == nullptr) || (m == nullptr) != (mo == nullptr))
        return fail(NPA_ERR_INVALID_ARGUMENT, "each input of a permutation needs its output (and vice versa)");
    if (s && C <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "channels must be positive, got %d", C);
    const bool vec = s && (C % 4 == 0) && ((((uintptr_t)s) | ((uintptr_t)so)) % 16 == 0);
    const int pieces = s ? (vec ? C / 4 : C) : 1;
    const long long total = (long long)g.B * g.N * pieces;
    const unsigned blocks = (unsigned)((total + 255) / 256);
#define NPA_PERMUTE(DD, VEC) \
    permute_kernel<DD, FORWARD, VEC><<<blocks, 256, 0, st>>>(x, s, m, perm, xo, so, mo, pieces, total, g.N)
    if (g.dim == 2) {
        if (vec) NPA_PERMUTE(2, float4); else NPA_PERMUTE(2, float);
    } else {
        if (vec) NPA_PERMUTE(3, float4); else NPA_PERMUTE(3, float);
    }
#undef NPA_PERMUTE
    return check_launch(FORWARD ? "permute_kernel(forward)" : "permute_kernel(inverse)");
}

// ---------------------------------------------------------------------------
// safe inverse of symmetric 2x2 / 3x3 matrices (sphops/sph_cuda.cu:3095-3179):
// only the upper triangle is read; |det| < tol gives the identity.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
safe_inv2_kernel(const float4 *__restrict__ in, float4 *__restrict__ out, long long n, float tol) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const float4 a = __ldg(in + i);
    const float det = a.x * a.w - a.y * a.y;
    if (fabsf(det) < tol) {
        out[i] = make_float4(1.f, 0.f, 0.f, 1.f);
    } else {
        const float r = 1.0f / det;
        out[i] = make_float4(a.w * r, -a.y * r, -a.y * r, a.x * r);
    }
}

__global__ void __launch_bounds__(256)
safe_inv3_kernel(const float *__restrict__ in, float *__restrict__ out, long long n, float tol) {
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    const float *p = in + i * 9;
    const float a = p[0], b = p[1], c = p[2], d = p[4], e = p[5], f = p[8];
    const float t1 = d * f - e * e, t2 = c * e - b * f, t3 = b * e - c * d;
    const float det = a * t1 + b * t2 + c * t3;
    float *o = out + i * 9;
    if (fabsf(det) < tol) {
        o[0] = 1.f; o[1] = 0.f; o[2] = 0.f;
        o[3] = 0.f; o[4] = 1.f; o[5] = 0.f;
        o[6] = 0.f; o[7] = 0.f; o[8] = 1.f;
    } else {
        const float r = 1.0f / det;
        const float m01 = t2 * r, m02 = t3 * r, m12 = (b * c - a * e) * r;
        o[0] = t1 * r;  o[1] = m01;                o[2] = m02;
        o[3] = m01;     o[4] = (a * f - c * c) * r; o[5] = m12;
        o[6] = m02;     o[7] = m12;                o[8] = (a * d - b * b) * r;
    }
}

}  // namespace npa

using namespace npa;

extern "C" {

int64_t npa_grid_scratch_bytes(const npa_grid *gd) {
    Geom g;
    int rc = make_geom(gd, &g);
    if (rc != NPA_OK) return rc;
    return (int64_t)layout_scratch(g, nullptr, nullptr);
}

int npa_grid_build(const npa_grid *gd, const float *x, int32_t *permutation, int32_t *bin_offsets,
                   int32_t *block_info, void *scratch, int64_t scratch_bytes, void *stream) {
    Geom g;
    int rc = make_geom(gd, &g);
    if (rc != NPA_OK) return rc;
    if (!x || !permutation || !bin_offsets || !block_info || !scratch)
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_grid_build: x, permutation, bin_offsets, block_info and scratch must be non-NULL");
    if (((uintptr_t)x % (g.dim == 2 ? 8 : 16)) || ((uintptr_t)block_info % 16) || ((uintptr_t)scratch % 16))
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_grid_build: x / block_info / scratch are not aligned to their vector width");
    BinScratch s;
    const size_t need = layout_scratch(g, scratch, &s);
    if (scratch_bytes < (int64_t)need)
        return fail(NPA_ERR_SCRATCH_TOO_SMALL, "npa_grid_build: scratch has %lld bytes, %zu needed", (long long)scratch_bytes, need);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(s.counts, 0, s.zero_bytes, st);
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaMemsetAsync(scratch): %s", cudaGetErrorString(e));

    const dim3 pgrid((g.N + kBinChunk - 1) / kBinChunk, g.B);
    const bool smem = g.cells <= kSmemHistCells;
    const size_t smem_bytes = smem ? (size_t)g.cells * 4 : 0;
    if (g.dim == 2) {
        if (smem) hash_count_kernel<2, true><<<pgrid, kBinThreads, smem_bytes, st>>>(x, s.cellid, s.arrive, s.counts, g);
        else hash_count_kernel<2, false><<<pgrid, kBinThreads, 0, st>>>(x, s.cellid, s.arrive, s.counts, g);
    } else {
        if (smem) hash_count_kernel<3, true><<<pgrid, kBinThreads, smem_bytes, st>>>(x, s.cellid, s.arrive, s.counts, g);
        else hash_count_kernel<3, false><<<pgrid, kBinThreads, 0, st>>>(x, s.cellid, s.arrive, s.counts, g);
    }
    if ((rc = check_launch("hash_count_kernel")) != NPA_OK) return rc;

    const int n = g.B * g.cells;
    scan_tile_sums_kernel<<<s.tiles, kScanThreads, 0, st>>>(s.counts, s.partials, n, g.mpb);
    if ((rc = check_launch("scan_tile_sums_kernel")) != NPA_OK) return rc;
    scan_partials_kernel<<<1, 1024, 0, st>>>(s.partials, s.tiles);
    if ((rc = check_launch("scan_partials_kernel")) != NPA_OK) return rc;
    uint32_t *crowded_count = s.counts + (size_t)n + 1;
    scan_apply_kernel<<<s.tiles, kScanThreads, 0, st>>>(s.counts, s.partials, bin_offsets,
                                                        reinterpret_cast<int4 *>(block_info), s.crowded, crowded_count, n, g);
    if ((rc = check_launch("scan_apply_kernel")) != NPA_OK) return rc;

    const dim3 tgrid((g.N + kBinThreads - 1) / kBinThreads, g.B);
    scatter_kernel<<<tgrid, kBinThreads, 0, st>>>(s.cellid, s.arrive, bin_offsets, s.order, g);
    if ((rc = check_launch("scatter_kernel")) != NPA_OK) return rc;
    rank_kernel<<<tgrid, kBinThreads, 0, st>>>(s.cellid, bin_offsets, s.order, permutation, g);
    if ((rc = check_launch("rank_kernel")) != NPA_OK) return rc;
    const int win = g.N < kRankWindow ? g.N : kRankWindow;
    rank_crowded_kernel<<<kRankCtas, 256, (size_t)((win + 31) / 32) * 8, st>>>(bin_offsets, s.order, permutation, s.crowded,
                                                                             crowded_count, g);
    return check_launch("rank_crowded_kernel");
}

}  // extern "C"

// Work arrays of npa_grid_build_static(): a fixed device array owned by the library, so that the
// call needs no scratch from the caller and allocates nothing.  In host code the symbol is only a
// handle; its device address is looked up once per device and cached below.
static __device__ __align__(256) unsigned char g_static_scratch[NPA_STATIC_SCRATCH_BYTES];

namespace npa {
constexpr int kMaxDevices = 64;
static std::mutex g_static_mutex;
static void *g_static_ptr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the current device (queried once per device).
static int static_scratch_address(void **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(NPA_ERR_UNSUPPORTED, "device ordinal %d is out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return fail(NPA_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", dev, cudaGetErrorString(e));
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return NPA_OK;
}
}  // namespace npa

extern "C" {

int npa_grid_build_static(const npa_grid *gd, const float *x, int32_t *permutation, int32_t *bin_offsets,
                          int32_t *block_info, void *stream) {
    const int64_t need = npa_grid_scratch_bytes(gd);
    if (need < 0) return (int)need;
    if (need > (int64_t)NPA_STATIC_SCRATCH_BYTES)
        return fail(NPA_ERR_SCRATCH_TOO_SMALL,
                    "npa_grid_build_static: this grid needs %lld bytes of work arrays, the built-in array holds %u; "
                    "use npa_grid_build with caller scratch", (long long)need, (unsigned)NPA_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != NPA_OK) return rc;
    return npa_grid_build(gd, x, permutation, bin_offsets, block_info, scratch, (int64_t)NPA_STATIC_SCRATCH_BYTES, stream);
}

int npa_bin_particles(const npa_grid *gd, int32_t channels, const float *x, const float *s,
                      const float *mass, const int32_t *permutation, float *x_out, float *s_out,
                      float *mass_out, void *stream) {
    Geom g;
    int rc = make_geom(gd, &g);
    if (rc != NPA_OK) return rc;
    return launch_permute<true>(g, channels, x, s, mass, permutation, x_out, s_out, mass_out, (cudaStream_t)stream);
}

int npa_unbin_particles(const npa_grid *gd, int32_t channels, const float *x_bin, const float *s_bin,
                        const float *mass_bin, const int32_t *permutation, float *x_out, float *s_out,
                        float *mass_out, void *stream) {
    Geom g;
    int rc = make_geom(gd, &g);
    if (rc != NPA_OK) return rc;
    return launch_permute<false>(g, channels, x_bin, s_bin, mass_bin, permutation, x_out, s_out, mass_out, (cudaStream_t)stream);
}

int npa_safe_inv_sym_mat(int32_t dim, int64_t n, const float *m, float *m_inv, float tol, void *stream) {
    if (dim != 2 && dim != 3) return fail(NPA_ERR_INVALID_ARGUMENT, "safe_inverse only supports 2x2 or 3x3 matrices.");
    if (n < 0 || !m || !m_inv) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_safe_inv_sym_mat: bad arguments");
    if (n == 0) return NPA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dim == 2) {
        if (((uintptr_t)m | (uintptr_t)m_inv) % 16)
            return fail(NPA_ERR_INVALID_ARGUMENT, "npa_safe_inv_sym_mat: 2x2 matrices must be 16-byte aligned");
        safe_inv2_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const float4 *>(m), reinterpret_cast<float4 *>(m_inv), n, tol);
    } else {
        safe_inv3_kernel<<<blocks, 256, 0, st>>>(m, m_inv, n, tol);
    }
    return check_launch("safe_inv_kernel");
}

}  // extern "C"
