// Cell-tile streaming engine of the feature sweeps.
//
// A CTA owns one work item at a time (<= MPB particles of one cell, the "tile").  The rows of the
// tile's 3^D neighbour cells -- positions, densities, masses and the feature rows the sweep reads --
// are contiguous per x-row of cells (sphops/sph_cuda.cu:1561-1660 stages the same ranges), so a
// producer warp copies them into shared memory with bulk asynchronous copies (cp.async.bulk,
// completion counted by an mbarrier) in chunks of at most `rmax` rows, several chunks in flight,
// and the consumer warps read every neighbour row from shared memory: a row crosses L2 -> SM once
// per tile instead of once per pair, and the copies use neither instruction slots nor the
// load/store pipe of the consumers.
//
// Flow control is two mbarriers per stage: `full` (producer arrives with the byte count, the copies
// complete it) and `empty` (one arrival per consumer warp).  Every copy lands in the issuing CTA's own shared memory
// only, and every tensor is memory of this GPU.  Every wait is bounded: after kTileWaitNs of unsuccessful polling a
// thread records a code in the status word, stops waiting and the CTA drains to its exit.
//
// Alignment: bulk copies need 16-byte aligned addresses and sizes.  Feature rows are C floats with
// C % 4 == 0, so any row range qualifies; positions, densities and masses are copied for the range
// rounded outwards to multiples of four particles ([lo4, hi4)), and slot = piece.slot + (j - lo4)
// addresses every staged array.  The launcher refuses shapes that break these rules (B*N % 4 != 0,
// C % 4 != 0, misaligned base pointers) and the gather kernels run instead.
#pragma once
#include "neighbors.cuh"
#include "ops.cuh"

namespace npa {

constexpr int kTilePieces = 32;        // ranges per chunk (a tile has at most kMaxRanges = 28)
constexpr int kTileList = 64;          // accepted-pair slots per consumer warp
constexpr unsigned long long kTileWaitNs = 2000000000ull;  // a wait gives up after two seconds
constexpr int kTileMaxStages = 4;

enum { TILE_FIRST = 1, TILE_LAST = 2, TILE_END = 4 };
// Status codes written to the device status word when a bounded wait runs out.
enum { TILE_STATUS_OK = 0, TILE_STATUS_FULL_TIMEOUT = 1, TILE_STATUS_EMPTY_TIMEOUT = 2 };

struct __align__(16) TilePiece {
    int lo, hi;   // global particle rows [lo, hi) of this piece
    int lo4;      // lo rounded down to a multiple of four: row j sits in slot `slot + (j - lo4)`
    int slot;     // first slot of the piece in the stage (multiple of four)
    int code;     // periodic image shift of the piece (shift_code)
    int pad[3];
};

struct __align__(16) TileChunk {
    int npieces;
    int first;   // global index of the first particle of the (sub-)tile
    int count;   // particles of the (sub-)tile, <= tp
    int flags;   // TILE_FIRST: first chunk of the tile, TILE_LAST: last one, TILE_END: no more work
    int rot;     // particle p of the tile belongs to consumer warp (p + rot) % consumer warps
    int pad[3];
    TilePiece piece[kTilePieces];
};

// Shared-memory plan of one launch, computed on the host (byte offsets into dynamic shared memory).
struct TileLayout {
    int rmax;         // rows (slots) per stage, multiple of four
    int tp;           // particles per sub-tile (accumulator slots)
    int stages;       // stage buffers in flight
    int span;         // a tile merges work items of up to `span` x-adjacent cells
    int warps;        // consumer warps
    int off_x, off_rho, off_mass, off_s, off_gb, off_gg;  // arrays inside one stage
    int stage_bytes;
    int off_chunks;   // TileChunk[stages]
    int off_lists;    // per consumer warp pair lists
    int list_bytes;   // bytes per consumer warp
    int off_acc;      // accumulator slots, tp x acc_bytes
    int acc_bytes;
    int off_bars;     // uint64 full[stages], empty[stages]
    int total_bytes;
};

// ---- mbarrier / bulk-copy primitives (shared::cta addresses) ---------------------------------
__device__ inline unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ inline void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ inline void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ inline void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline void mbar_arrive_expect(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One try_wait: the hardware suspends the thread until the phase completes or `hint_ns` have passed,
// so a waiting warp issues next to nothing while it waits.
__device__ inline bool mbar_try_wait(uint64_t *bar, unsigned parity, unsigned hint_ns) {
    unsigned ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ inline unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait for the phase with the given parity; false when it gave up after `limit_ns`.
__device__ inline bool mbar_wait(uint64_t *bar, unsigned parity, unsigned long long limit_ns = kTileWaitNs) {
    if (mbar_try_wait(bar, parity, 20000u)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        if (mbar_try_wait(bar, parity, 1000000u)) return true;
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
}
// Global -> shared bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned); completion
// is counted on `bar`.  The destination is this CTA's own shared memory and nothing else.
__device__ inline void bulk_copy_g2s(void *dst, const void *src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ inline int warp_inclusive_scan(int v) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(kFull, v, o);
        if (lane >= o) v += t;
    }
    return v;
}
__device__ inline int warp_sum_int(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

// What the producer needs to know about the arrays of one sweep.
struct TileSources {
    const float *x;     // [B*N, P]
    const float *rho;   // [B*N]
    const float *mass;  // [B*N] or NULL
    const float *s;     // [B*N, C] or NULL
    const float *gb;    // [B*N, C] or NULL
    const float *gg;    // [B*N, C*D] or NULL
    int P, C, CD;
};

constexpr int kTileBatch = 8;  // work-list rows a producer draws per ticket

// Producer warp: draws work-list rows by ticket (kTileBatch consecutive rows per draw, their records
// loaded by as many lanes at once) and merges consecutive rows into one tile while they lie in the
// same x-row of cells, at most L.span cells apart, and hold at most L.tp particles together (their
// particles are then contiguous).  It cuts the candidate ranges of each tile into chunks of at most
// L.rmax slots, describes each chunk in shared memory and issues its copies.  Everything that needs
// global memory (ticket, item records, cell offsets of the ranges) is fetched before the wait for a
// free stage, so that latency overlaps the consumers' work on the stages already in flight.  Ends by
// publishing a TILE_END chunk.  All 32 lanes call it.
template <int D>
__device__ inline void tile_producer(const Geom &g, const TileLayout &L, const TileSources &src,
                                     const int32_t *__restrict__ bin_offsets, const int32_t *__restrict__ block_info,
                                     unsigned int *tickets, unsigned int *status, unsigned char *smem, int4 *rng) {
    const int lane = threadIdx.x & 31;
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.off_bars);
    uint64_t *empty = full + L.stages;
    TileChunk *chunks = reinterpret_cast<TileChunk *>(smem + L.off_chunks);
    bool have = false, first_chunk = true, end = false;
    WorkItem mine = {0, 0, 0, 0};  // lane k < kTileBatch holds row (draw + k); count 0 past the work list
    int mcx = 0, mcy = 0, mcz = 0;  // its cell coordinates
    int batch_next = kTileBatch;    // next row of the draw to hand out; kTileBatch = draw again
    int tile_first = 0, tile_count = 0, rot = 0;
    int sub_first = 0, sub_left = 0;  // a single row with more than L.tp particles is streamed in sub-tiles
    int nr = 0, r0 = 0, pos = 0;
    for (unsigned c = 0;; ++c) {
        const int st = (int)(c % (unsigned)L.stages);
        const unsigned use = c / (unsigned)L.stages;
        TileChunk *ch = chunks + st;
        if (!have && !end) {
            if (batch_next >= kTileBatch) {
                int row = 0;
                if (lane == 0) row = (int)atomicAdd(tickets, (unsigned)kTileBatch);
                row = __shfl_sync(kFull, row, 0) + lane;
                mine.count = 0;
                if (lane < kTileBatch && row < g.max_blocks) mine = load_item(block_info, bin_offsets, row);
                if (mine.count > 0) hash_to_cell<D>(g, (uint32_t)(mine.cell - mine.sys * g.cells), mcx, mcy, mcz);
                batch_next = 0;
            }
            // head of the tile = row batch_next of the draw; lanes after it join while the rules hold
            const int h = batch_next;
            const int hcount = __shfl_sync(kFull, mine.count, h);
            if (hcount <= 0) {  // rows after the last work item are zero
                end = true;
            } else {
                const int hfirst = __shfl_sync(kFull, mine.first, h);
                const int hsys = __shfl_sync(kFull, mine.sys, h);
                const int hcx = __shfl_sync(kFull, mcx, h), hcy = __shfl_sync(kFull, mcy, h), hcz = __shfl_sync(kFull, mcz, h);
                // particles up to and including this lane's row, counted from the head (rows are contiguous
                // only while every row in between qualifies, checked with the ballot below)
                const bool in_batch = lane >= h && lane < kTileBatch && mine.count > 0;
                const int upto = in_batch ? mine.first + mine.count - hfirst : 0;
                const bool wide = g.periodic && (mcx - hcx + 3 >= g.g[0]);  // window would wrap onto itself
                const bool okrow = in_batch && mine.sys == hsys && mcy == hcy && mcz == hcz && mcx >= hcx &&
                                   mcx - hcx < L.span && upto <= L.tp && upto > 0 && (lane == h || !wide);
                const unsigned okm = __ballot_sync(kFull, okrow || lane == h);
                // rows h, h+1, ... while consecutive lanes qualify
                const unsigned run = ~okm & ~((1u << h) - 1u);
                const int stop = run ? __ffs(run) - 1 : 32;  // first lane >= h that does not qualify
                const int last = stop - 1;                   // >= h
                const int lcx = __shfl_sync(kFull, mcx, last);
                const int lend = __shfl_sync(kFull, mine.first + mine.count, last);
                tile_first = hfirst;
                tile_count = lend - hfirst;
                batch_next = stop;
                sub_left = 0;
                if (tile_count > L.tp) {  // only a lone head row can exceed the accumulator slots
                    sub_first = hfirst + L.tp;
                    sub_left = tile_count - L.tp;
                    tile_count = L.tp;
                }
                __syncwarp();
                nr = build_ranges_span<D>(g, bin_offsets, hsys, hcx, lcx, hcy, hcz, rng);
                have = true;
                first_chunk = true;
                r0 = 0;
                pos = rng[0].x;
            }
        }
        // the stage is free once every consumer warp has released its previous contents
        if (!mbar_wait(empty + st, (use & 1u) ^ 1u)) {
            if (lane == 0) atomicExch(status, (unsigned)TILE_STATUS_EMPTY_TIMEOUT);
            return;  // the consumers run into their own bounded waits and leave
        }
        if (end) {
            if (lane == 0) ch->flags = TILE_END;
            __syncwarp();
            if (lane == 0) mbar_arrive(full + st);
            return;
        }
        // lanes 0.. take the ranges r0, r0+1, ... until the stage is full
        const int r = r0 + lane;
        const bool valid = r < nr;
        const int4 rg = valid ? rng[r] : make_int4(0, 0, 0, 0);
        const int lo = lane == 0 ? pos : rg.x;
        const int hi = rg.y;
        const int lo4 = lo & ~3;
        const int len4 = valid ? ((hi + 3) & ~3) - lo4 : 0;
        const int incl = warp_inclusive_scan(len4);
        const int excl = incl - len4;
        const bool take = valid && excl < L.rmax;
        const int room = L.rmax - excl;
        const bool trunc = take && len4 > room;
        const int hi_t = trunc ? lo4 + room : hi;  // a cut falls on a multiple of four rows
        const unsigned take_m = __ballot_sync(kFull, take);
        const unsigned trunc_m = __ballot_sync(kFull, trunc);
        const int ntake = __popc(take_m);
        int r0n, posn;
        if (trunc_m) {
            const int l = __ffs(trunc_m) - 1;
            r0n = r0 + l;
            posn = __shfl_sync(kFull, hi_t, l);
        } else {
            r0n = r0 + ntake;
            posn = r0n < nr ? rng[r0n].x : 0;
        }
        const bool done = r0n >= nr;
        unsigned bytes = 0;
        const int hi4 = (hi_t + 3) & ~3;
        if (take) {
            TilePiece pc;
            pc.lo = lo; pc.hi = hi_t; pc.lo4 = lo4; pc.slot = excl; pc.code = rg.z;
            pc.pad[0] = pc.pad[1] = pc.pad[2] = 0;
            ch->piece[lane] = pc;
            const unsigned n4 = (unsigned)(hi4 - lo4), n = (unsigned)(hi_t - lo);
            bytes = n4 * (unsigned)(src.P * 4) + n4 * 4u + (src.mass ? n4 * 4u : 0u);
            if (src.s) bytes += n * (unsigned)(src.C * 4);
            if (src.gb) bytes += n * (unsigned)(src.C * 4);
            if (src.gg) bytes += n * (unsigned)(src.CD * 4);
        }
        if (lane == 0) {
            ch->npieces = ntake;
            ch->first = tile_first;
            ch->count = tile_count;
            ch->flags = (first_chunk ? TILE_FIRST : 0) | (done ? TILE_LAST : 0);
            ch->rot = rot;
        }
        const unsigned total = (unsigned)warp_sum_int((int)bytes);
        __syncwarp();
        if (lane == 0) mbar_arrive_expect(full + st, total);
        __syncwarp();
        if (take) {
            unsigned char *stage = smem + (size_t)st * L.stage_bytes;
            const size_t n4 = (size_t)(hi4 - lo4), n = (size_t)(hi_t - lo);
            const size_t fslot = (size_t)excl + (size_t)(lo - lo4);
            bulk_copy_g2s(stage + L.off_x + (size_t)excl * src.P * 4, src.x + (size_t)lo4 * src.P,
                          (unsigned)(n4 * src.P * 4), full + st);
            bulk_copy_g2s(stage + L.off_rho + (size_t)excl * 4, src.rho + lo4, (unsigned)(n4 * 4), full + st);
            if (src.mass)
                bulk_copy_g2s(stage + L.off_mass + (size_t)excl * 4, src.mass + lo4, (unsigned)(n4 * 4), full + st);
            if (src.s)
                bulk_copy_g2s(stage + L.off_s + fslot * src.C * 4, src.s + (size_t)lo * src.C,
                              (unsigned)(n * src.C * 4), full + st);
            if (src.gb)
                bulk_copy_g2s(stage + L.off_gb + fslot * src.C * 4, src.gb + (size_t)lo * src.C,
                              (unsigned)(n * src.C * 4), full + st);
            if (src.gg)
                bulk_copy_g2s(stage + L.off_gg + fslot * src.CD * 4, src.gg + (size_t)lo * src.CD,
                              (unsigned)(n * src.CD * 4), full + st);
        }
        first_chunk = false;
        r0 = r0n;
        pos = posn;
        if (done) {
            rot = (rot + tile_count) % L.warps;  // the next tile starts at the next warp
            if (sub_left > 0) {  // crowded cell: the next sub-tile streams the same ranges again
                tile_first = sub_first;
                tile_count = min(L.tp, sub_left);
                sub_first += tile_count;
                sub_left -= tile_count;
                first_chunk = true;
                r0 = 0;
                pos = rng[0].x;
            } else {
                have = false;
            }
        }
    }
}

// Host: lay out the shared memory of a tile sweep.  `feature_floats` = floats per staged particle
// beyond position, density and mass, split as s / g_blur / g_grad (0 = array not staged);
// `list_bytes` = pair-list bytes per consumer warp; `acc_bytes` = accumulator bytes per particle of a
// sub-tile.  want_* = 0 chooses automatically.  Returns false when not even a minimal plan fits.
bool tile_make_layout(int P, bool with_mass, int floats_s, int floats_gb, int floats_gg, int consumer_warps,
                      int list_bytes, int acc_bytes, int want_rmax, int want_tp, int want_stages, int want_span,
                      bool backward, TileLayout *out);

// Device status word of the tile sweeps (zero unless a bounded wait ran out).  Defined in capi.cu.
int tile_status_word(unsigned int **out);

}  // namespace npa
