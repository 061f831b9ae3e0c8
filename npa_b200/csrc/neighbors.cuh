// Neighbour enumeration shared by every perception kernel.
//
// One warp owns one work item (a row of block_info: <= MPB particles of one
// cell).  The warp first turns the 3^D neighbour cells into a short list of
// contiguous particle ranges: with the linear hash the three x-adjacent cells
// of a (y, z) row are contiguous in cell order (the observation the reference's
// block-per-cell kernel is built on, sphops/sph_cuda.cu:1561-1660), so a row is
// one range, or two when a periodic row wraps; with the Morton hash each cell is
// its own range.  The warp is split into sub-groups of LPP lanes; each sub-group
// owns one particle i of the item and its lanes test LPP candidates j per round.
#pragma once
#include "common.cuh"

namespace npa {

constexpr int kWarpsPerCta = 8;
constexpr int kMaxRanges = 28;

struct WorkItem {
    int first;  // global index of the item's first particle (cell order)
    int count;  // particles in the item, 0 = unused row
    int cell;   // global cell index (system * cells + hash)
    int sys;    // system (batch) index
};

__device__ inline WorkItem load_item(const int32_t *__restrict__ block_info,
                                     const int32_t *__restrict__ bin_offsets, int row) {
    const int4 rec = __ldg(reinterpret_cast<const int4 *>(block_info) + row);
    WorkItem it;
    it.cell = rec.x;
    it.count = rec.z;
    it.sys = rec.w;
    it.first = rec.z > 0 ? __ldg(bin_offsets + rec.x) + rec.y : 0;
    return it;
}

// Dynamic distribution of work-list rows over the resident warps of a persistent launch.
// `tickets` points at two words that are zero when the launch starts: [0] the next row to hand
// out, [1] the number of CTAs that have finished.  A warp draws rows until they run out; rows
// come out in cell order, so warps running at the same time work on neighbouring cells.  The
// last CTA to finish puts both words back to zero for the next launch that uses them.
__device__ inline int next_row(unsigned int *tickets) {
    int row = 0;
    if ((threadIdx.x & 31) == 0) row = (int)atomicAdd(tickets, 1u);
    return __shfl_sync(kFull, row, 0);
}

// Called by every thread of the CTA once its warps will draw no more rows.
__device__ inline void release_rows(unsigned int *tickets) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int done = atomicAdd(tickets + 1, 1u);
        if (done == gridDim.x - 1) {  // every other CTA has drawn its last row before it counted itself
            tickets[0] = 0u;
            tickets[1] = 0u;
        }
    }
}

// Neighbour coordinate along one axis; false when the clamped grid ends there
// or when a small periodic axis would visit the same cell twice.  `shift` is
// the periodic image the neighbour cell lies in relative to cell c: -1 when the
// walk left the grid below 0 (its particles sit one box length higher, so the
// displacement needs -L), +1 above, 0 otherwise or when the axis is too short
// to tell (then the half-box test in periodic_delta decides per pair).
__device__ inline bool neighbor_axis(int c, int o, int n, int periodic, int &out, int &shift) {
    shift = 0;
    if (!periodic) {
        out = c + o;
        return out >= 0 && out < n;
    }
    if (n == 1) {
        out = c;
        return o == 0;
    }
    if (n == 2) {
        out = (c + o) & 1;
        return o >= 0;
    }
    out = c + o;
    if (out < 0) { out += n; shift = -1; }
    else if (out >= n) { out -= n; shift = 1; }
    return true;
}

// Candidate range [x, y) of global particle indices plus the image shift code
// (sx+1) | (sy+1) << 2 | (sz+1) << 4 in z.
__device__ inline int shift_code(int sx, int sy, int sz) { return (sx + 1) | ((sy + 1) << 2) | ((sz + 1) << 4); }

// Position of particle i as seen from one candidate range.  For a periodic grid
// the range carries the image shift S = k * L (k in {-1, 0, 1} per axis) of the
// neighbour cell, and the displacement is r = x_j - x_i + S.  Evaluating
// (x_j + S) - x_i in fp32 would round at the magnitude of the box; instead the
// shifted origin x_i - S is formed once per (particle, range) as an unevaluated
// sum  x + e  (error-free two-sum, with S itself split in a high and a low fp32
// part because g * eps is not representable), so that per pair
// r = (x_j - x) + c  with c = S_lo - e is as accurate as a clamped displacement.
template <int D, bool PER>
struct Origin {
    float x[3];
    float c[3];
};

template <int D, bool PER>
__device__ inline Origin<D, PER> make_origin(const Geom &g, float px, float py, float pz, int code) {
    Origin<D, PER> o;
    const float p[3] = {px, py, pz};
#pragma unroll
    for (int d = 0; d < 3; ++d) {
        o.x[d] = p[d];
        o.c[d] = 0.f;
        if (PER && d < D) {
            const float k = (float)(((code >> (2 * d)) & 3) - 1);
            const float b = -k * g.L[d];
            const float sum = __fadd_rn(p[d], b);
            const float bb = __fsub_rn(sum, p[d]);
            const float err = __fadd_rn(__fsub_rn(p[d], __fsub_rn(sum, bb)), __fsub_rn(b, bb));
            o.x[d] = sum;
            o.c[d] = __fsub_rn(k * g.Llo[d], err);
        }
    }
    return o;
}

// Fills rng[0..n) with the non-empty candidate ranges [start, end) of global
// particle indices for the cell of `it`; returns n.  Must be called by all 32
// lanes; rng is per-warp shared memory of kMaxRanges entries.
template <int D>
__device__ inline int build_ranges(const Geom &g, const int32_t *__restrict__ bin_offsets,
                                   const WorkItem &it, int4 *rng) {
    const int lane = threadIdx.x & 31;
    int cx, cy, cz;
    hash_to_cell<D>(g, (uint32_t)(it.cell - it.sys * g.cells), cx, cy, cz);
    const int32_t *off = bin_offsets + (size_t)it.sys * g.cells;
    int start = 0, end = 0, sx = 0, sy = 0, sz = 0;
    if (!g.morton) {
        const int row = lane >> 1, piece = lane & 1;
        if (row < (D == 2 ? 3 : 9)) {
            int ny = 0, nz = 0;
            bool ok = neighbor_axis(cy, row % 3 - 1, g.g[1], g.periodic, ny, sy);
            if (D == 3) ok = neighbor_axis(cz, row / 3 - 1, g.g[2], g.periodic, nz, sz) && ok;
            const int gx = g.g[0];
            int xlo = 0, xhi = -1;
            if (!g.periodic) {
                if (piece == 0) { xlo = max(cx - 1, 0); xhi = min(cx + 1, gx - 1); }
            } else if (gx <= 3) {
                if (piece == 0) { xlo = 0; xhi = gx - 1; }
            } else if (cx == 0) {
                if (piece == 0) { xlo = 0; xhi = 1; } else { xlo = xhi = gx - 1; sx = -1; }
            } else if (cx == gx - 1) {
                if (piece == 0) { xlo = gx - 2; xhi = gx - 1; } else { xlo = xhi = 0; sx = 1; }
            } else if (piece == 0) {
                xlo = cx - 1; xhi = cx + 1;
            }
            if (ok && xhi >= xlo) {
                start = __ldg(off + cell_hash<D>(g, xlo, ny, nz));
                end = __ldg(off + cell_hash<D>(g, xhi, ny, nz) + 1);
            }
        }
    } else {
        if (lane < (D == 2 ? 9 : 27)) {
            int nx = 0, ny = 0, nz = 0;
            bool ok = neighbor_axis(cx, lane % 3 - 1, g.g[0], g.periodic, nx, sx);
            ok = neighbor_axis(cy, (lane / 3) % 3 - 1, g.g[1], g.periodic, ny, sy) && ok;
            if (D == 3) ok = neighbor_axis(cz, lane / 9 - 1, g.g[2], g.periodic, nz, sz) && ok;
            if (ok) {
                const uint32_t hsh = cell_hash<D>(g, nx, ny, nz);
                start = __ldg(off + hsh);
                end = __ldg(off + hsh + 1);
            }
        }
    }
    const bool nonempty = end > start;
    const unsigned m = __ballot_sync(kFull, nonempty);
    if (nonempty) rng[__popc(m & ((1u << lane) - 1))] = make_int4(start, end, shift_code(sx, sy, sz), 0);
    __syncwarp();
    return __popc(m);
}

// Candidate ranges of a tile that covers the cells [cx0, cx1] of one x-row (cy, cz) of system `sys`:
// per neighbour row (3 in 2D, 9 in 3D) the cells [cx0 - 1, cx1 + 1], which are contiguous in cell
// order, plus on a periodic grid the wrapped cell beyond either end with its image shift.  The caller
// guarantees cx1 - cx0 + 3 < g.g[0] unless the window is the whole row (then one range per row with
// no shift; displacement() falls back to the general minimum image per pair).  Fills rng[0..n) with
// (start, end, shift code, 0) of the non-empty ranges and returns n.  All 32 lanes call it.
template <int D>
__device__ inline int build_ranges_span(const Geom &g, const int32_t *__restrict__ bin_offsets, int sys, int cx0,
                                        int cx1, int cy, int cz, int4 *rng) {
    const int lane = threadIdx.x & 31;
    const int32_t *off = bin_offsets + (size_t)sys * g.cells;
    int start = 0, end = 0, sx = 0, sy = 0, sz = 0;
    const int row = lane / 3, piece = lane % 3;  // piece 0: main window, 1: wrapped below, 2: wrapped above
    if (row < (D == 2 ? 3 : 9)) {
        int ny = 0, nz = 0;
        bool ok = neighbor_axis(cy, row % 3 - 1, g.g[1], g.periodic, ny, sy);
        if (D == 3) ok = neighbor_axis(cz, row / 3 - 1, g.g[2], g.periodic, nz, sz) && ok;
        const int gx = g.g[0];
        int xlo = 0, xhi = -1;
        if (!g.periodic) {
            if (piece == 0) { xlo = max(cx0 - 1, 0); xhi = min(cx1 + 1, gx - 1); }
        } else if (cx1 - cx0 + 3 >= gx) {
            if (piece == 0) { xlo = 0; xhi = gx - 1; }
        } else if (piece == 0) {
            xlo = max(cx0 - 1, 0); xhi = min(cx1 + 1, gx - 1);
        } else if (piece == 1) {
            if (cx0 == 0) { xlo = xhi = gx - 1; sx = -1; }
        } else {
            if (cx1 == gx - 1) { xlo = xhi = 0; sx = 1; }
        }
        if (ok && xhi >= xlo) {
            start = __ldg(off + cell_hash<D>(g, xlo, ny, nz));
            end = __ldg(off + cell_hash<D>(g, xhi, ny, nz) + 1);
        }
    }
    const bool nonempty = end > start;
    const unsigned m = __ballot_sync(kFull, nonempty);
    if (nonempty) rng[__popc(m & ((1u << lane) - 1))] = make_int4(start, end, shift_code(sx, sy, sz), 0);
    __syncwarp();
    return __popc(m);
}

template <int D>
struct Pos {
    float x, y, z;
};

template <int D>
__device__ inline Pos<D> load_pos(const float *__restrict__ x, long long idx) {
    Pos<D> p;
    if (D == 2) {
        const float2 v = __ldg(reinterpret_cast<const float2 *>(x) + idx);
        p.x = v.x; p.y = v.y; p.z = 0.f;
    } else {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(x) + idx);
        p.x = v.x; p.y = v.y; p.z = v.z;
    }
    return p;
}

// r = x_j - x_i (minimum image when PER) and q = |r|^2.
template <int D, bool PER, bool EXACT = true>
__device__ inline float displacement(const Geom &g, const Origin<D, PER> &o, float jx, float jy, float jz,
                                     float &rx, float &ry, float &rz) {
    rx = jx - o.x[0];
    ry = jy - o.x[1];
    rz = D == 3 ? jz - o.x[2] : 0.f;
    if (PER) {
        rx += o.c[0];
        ry += o.c[1];
        if (D == 3) rz += o.c[2];
        if (fabsf(rx) > g.halfL[0]) rx = wrap_general(rx, g.L[0], g.Llo[0], g.invL[0]);
        if (fabsf(ry) > g.halfL[1]) ry = wrap_general(ry, g.L[1], g.Llo[1], g.invL[1]);
        if (D == 3 && fabsf(rz) > g.halfL[2]) rz = wrap_general(rz, g.L[2], g.Llo[2], g.invL[2]);
    }
    return EXACT ? sq_norm<D>(rx, ry, rz) : sq_norm_fast<D>(rx, ry, rz);
}

// Visits every candidate of every range of one particle, 32 per round: body(acc, j, rx, ry, rz, q)
// is called by all lanes once per round (acc = this lane's candidate exists and is within the
// cut-off).  The position of the next round's candidate is loaded before the current round is
// tested, so the load latency overlaps the test.  EXACT selects the contraction-free r^2.
template <int D, bool PER, bool EXACT, typename Body>
__device__ inline void scan_candidates(const Geom &g, const float *__restrict__ x, const Pos<D> &pi,
                                       const int4 *rng, int nr, Body &&body) {
    if (nr <= 0) return;
    const int lane = threadIdx.x & 31;
    int r = 0;
    int4 rg = rng[0];
    int j0 = rg.x;
    Pos<D> pj = {0.f, 0.f, 0.f};
    if (j0 + lane < rg.y) pj = load_pos<D>(x, j0 + lane);
    Origin<D, PER> org = make_origin<D, PER>(g, pi.x, pi.y, pi.z, rg.z);
    while (true) {
        int nxt_r = r, nxt_j0 = j0 + 32;
        int4 nxt_rg = rg;
        if (nxt_j0 >= rg.y) {
            nxt_r = r + 1;
            if (nxt_r < nr) {
                nxt_rg = rng[nxt_r];
                nxt_j0 = nxt_rg.x;
            }
        }
        Pos<D> pn = {0.f, 0.f, 0.f};
        if (nxt_r < nr && nxt_j0 + lane < nxt_rg.y) pn = load_pos<D>(x, nxt_j0 + lane);
        const int j = j0 + lane;
        float rx = 0.f, ry = 0.f, rz = 0.f, q = 0.f;
        bool acc = false;
        if (j < rg.y) {
            q = displacement<D, PER, EXACT>(g, org, pj.x, pj.y, pj.z, rx, ry, rz);
            acc = q < g.h2;
        }
        body(acc, j, rx, ry, rz, q);
        if (nxt_r >= nr) break;
        if (PER && nxt_r != r) org = make_origin<D, PER>(g, pi.x, pi.y, pi.z, nxt_rg.z);
        r = nxt_r; rg = nxt_rg; j0 = nxt_j0; pj = pn;
    }
}

// Displacement x_j - x_i of a pair taken from a neighbour list (no cell walk, so no known image
// shift): on a periodic grid the image is recovered from the raw difference, which lies within
// half a box of a multiple of the box length, and applied through the same error-free shifted
// origin the cell walk uses.
template <int D, bool PER>
__device__ inline void listed_displacement(const Geom &g, const Pos<D> &pi, const Pos<D> &pj, float &rx, float &ry,
                                           float &rz) {
    if (PER) {
        const float pv[3] = {pi.x, pi.y, pi.z}, jv[3] = {pj.x, pj.y, pj.z};
        float r[3] = {0.f, 0.f, 0.f};
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const float k = -rintf((jv[d] - pv[d]) * g.invL[d]);  // image shift in box lengths
            const float b = -k * g.L[d];
            const float sum = __fadd_rn(pv[d], b);
            const float bb = __fsub_rn(sum, pv[d]);
            const float err = __fadd_rn(__fsub_rn(pv[d], __fsub_rn(sum, bb)), __fsub_rn(b, bb));
            r[d] = (jv[d] - sum) + __fsub_rn(k * g.Llo[d], err);
        }
        rx = r[0]; ry = r[1]; rz = r[2];
    } else {
        rx = pj.x - pi.x;
        ry = pj.y - pi.y;
        rz = D == 3 ? pj.z - pi.z : 0.f;
    }
}

// Sum over the LPP lanes of a sub-group (LPP a power of two <= 32).
template <int LPP>
__device__ inline float subgroup_sum(float v) {
#pragma unroll
    for (int o = LPP >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

}  // namespace npa
