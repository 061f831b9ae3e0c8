// Per-particle scalar SPH operators: count, density, density gradient and
// moment matrix, forward and backward, on the warp-per-work-item neighbour
// walk of neighbors.cuh.  Any subset of the four runs fused in one sweep.
//
// Replaces forward_kernel / backward_kernel of the reference for the
// Count, Density, DensityGradient and MomentMatrix computation types
// (sphops/sph_cuda.cu:1418-1812 and 723-1416; pair math at :1160-1184,
// :1236-1264, :1328-1375).  The backward is a gather: particle i accumulates
// the terms of both roles it plays in a pair, so no global atomics are needed.
// The forward sweep can also record each particle's accepted neighbours (the
// neighbour-list cache) so that later sweeps of the same snapshot skip the search.
#include "neighbors.cuh"
#include "ops.cuh"

namespace npa {

// dK/dr applied to u:  J u = phi u - psi (r.u) r.
template <int D>
__device__ inline void apply_jacobian(float phi, float psi, float rx, float ry, float rz,
                                      float ux, float uy, float uz, float &ox, float &oy, float &oz) {
    float ru = rx * ux + ry * uy;
    if (D == 3) ru = fmaf(rz, uz, ru);
    const float s = psi * ru;
    ox = phi * ux - s * rx;
    oy = phi * uy - s * ry;
    oz = D == 3 ? phi * uz - s * rz : 0.f;
}

constexpr int kScalarLpp = 4;                // lanes per particle
constexpr int kScalarPpw = 32 / kScalarLpp;  // particles per warp pass
constexpr unsigned kScalarSubMask = (1u << kScalarLpp) - 1u;

// One warp per work item (several warps share an item when items are scarce).  The warp handles 8
// particles of the item per pass: each particle has a sub-group of 4 lanes that split its
// candidates, every lane adds the contribution of its own accepted pair, and a sub-group shuffle
// reduction yields the sums.  Eight independent particles per warp keep many loads in flight.
// The sweep can record the accepted pairs of each particle (in candidate order) in the
// neighbour-list cache for the sweeps that follow.
template <int D, bool PER, int MASK>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
scalar_forward_kernel(ScalarFwdArgs a, Geom g) {
    __shared__ int4 s_ranges[kWarpsPerCta][kMaxRanges];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int4 *rng = s_ranges[warp];
    const int sub = lane / kScalarLpp, sl = lane % kScalarLpp;
    constexpr bool kSpiky = (MASK & (S_DGRAD | S_MOMENT)) != 0;
    constexpr bool kPoly = (MASK & S_DENSITY) != 0;
    constexpr int kSym = D * (D + 1) / 2;
    const int K = a.pair_stride;

    const int vrows = g.max_blocks * g.split;
    for (int vrow = next_row(a.tickets); vrow < vrows; vrow = next_row(a.tickets)) {
        const int row = vrow / g.split, part = vrow - row * g.split;
        const WorkItem it = load_item(a.block_info, a.bin_offsets, row);
        if (it.count <= 0) break;  // rows after the last work item are zero
        if (part * kScalarPpw >= it.count) continue;
        __syncwarp();
        const int nr = build_ranges<D>(g, a.bin_offsets, it, rng);

        for (int k0 = part * kScalarPpw; k0 < it.count; k0 += g.split * kScalarPpw) {
            const int k = k0 + sub;
            const bool ivalid = k < it.count;
            const long long i = it.first + (ivalid ? k : 0);
            const Pos<D> pi = load_pos<D>(a.x, i);
            int32_t *list = a.pair_cache ? a.pair_cache + i * K + 1 : nullptr;
            float cnt = 0.f, rho = 0.f, dg[3] = {0.f, 0.f, 0.f}, mom[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            int listed = 0;
            for (int r = 0; r < nr; ++r) {
                const int4 rg = rng[r];
                const Origin<D, PER> org = make_origin<D, PER>(g, pi.x, pi.y, pi.z, rg.z);
                for (int j0 = rg.x; j0 < rg.y; j0 += kScalarLpp) {
                    const int j = j0 + sl;
                    float rx = 0.f, ry = 0.f, rz = 0.f, q = 0.f;
                    bool acc = false;
                    if (ivalid && j < rg.y) {
                        const Pos<D> pj = load_pos<D>(a.x, j);
                        q = displacement<D, PER>(g, org, pj.x, pj.y, pj.z, rx, ry, rz);
                        acc = q < g.h2;
                    }
                    if (list) {  // warp-uniform
                        const unsigned bits = (__ballot_sync(kFull, acc) >> (sub * kScalarLpp)) & kScalarSubMask;
                        const int pos = listed + __popc(bits & ((1u << sl) - 1u));
                        if (acc && pos < K - 1) list[pos] = j;
                        listed += __popc(bits);
                    }
                    if (!acc) continue;
                    if (MASK & S_COUNT) cnt += 1.0f;
                    const float mj = (kPoly || kSpiky) ? (a.mass ? __ldg(a.mass + j) : 1.0f) : 0.f;
                    if (kPoly) {
                        const float t = fmaxf(g.h2 - q, 0.f);
                        rho = fmaf(mj, t * t * t, rho);
                    }
                    if (kSpiky && q > 0.f) {
                        float d;
                        const float phi = spiky_phi(q, g.h, d);
                        if (MASK & S_DGRAD) {
                            const float w = mj * phi;
                            dg[0] = fmaf(w, rx, dg[0]);
                            dg[1] = fmaf(w, ry, dg[1]);
                            if (D == 3) dg[2] = fmaf(w, rz, dg[2]);
                        }
                        if (MASK & S_MOMENT) {
                            const float w = phi * mj / __ldg(a.rho_in + j);
                            mom[0] = fmaf(w * rx, rx, mom[0]);
                            mom[1] = fmaf(w * rx, ry, mom[1]);
                            if (D == 2) {
                                mom[2] = fmaf(w * ry, ry, mom[2]);
                            } else {
                                mom[2] = fmaf(w * rx, rz, mom[2]);
                                mom[3] = fmaf(w * ry, ry, mom[3]);
                                mom[4] = fmaf(w * ry, rz, mom[4]);
                                mom[5] = fmaf(w * rz, rz, mom[5]);
                            }
                        }
                    }
                }
            }
            if (MASK & S_COUNT) cnt = subgroup_sum<kScalarLpp>(cnt);
            if (kPoly) rho = subgroup_sum<kScalarLpp>(rho);
            if (MASK & S_DGRAD) {
#pragma unroll
                for (int d = 0; d < D; ++d) dg[d] = subgroup_sum<kScalarLpp>(dg[d]);
            }
            if (MASK & S_MOMENT) {
#pragma unroll
                for (int d = 0; d < kSym; ++d) mom[d] = subgroup_sum<kScalarLpp>(mom[d]);
            }
            if (ivalid && sl == 0) {
                if (list) list[-1] = listed <= K - 1 ? listed : -1;
                if ((MASK & S_COUNT) && a.count) a.count[i] = cnt;
                if (kPoly && a.rho_out) a.rho_out[i] = g.c_s * rho;
                if ((MASK & S_DGRAD) && a.rho_grad) {
#pragma unroll
                    for (int d = 0; d < D; ++d) a.rho_grad[i * D + d] = g.c_g * dg[d];
                }
                if ((MASK & S_MOMENT) && a.moment) {
                    float *o = a.moment + i * (D * D);
                    if (D == 2) {
                        reinterpret_cast<float4 *>(o)[0] =
                            make_float4(g.c_g * mom[0], g.c_g * mom[1], g.c_g * mom[1], g.c_g * mom[2]);
                    } else {
                        o[0] = g.c_g * mom[0]; o[1] = g.c_g * mom[1]; o[2] = g.c_g * mom[2];
                        o[3] = g.c_g * mom[1]; o[4] = g.c_g * mom[3]; o[5] = g.c_g * mom[4];
                        o[6] = g.c_g * mom[2]; o[7] = g.c_g * mom[4]; o[8] = g.c_g * mom[5];
                    }
                }
            }
        }
    }
    release_rows(a.tickets);
}

// ---------------------------------------------------------------------------
// Forward sweep with the candidates shared by the particles of a tile.
//
// The particles of one cell (and of its x-neighbours) test the same candidates, so a warp takes a
// tile of up to 32 particles -- consecutive work-list rows of one x-row of cells, at most `span`
// cells apart (sphops/sph_cuda.cu:1664-1690 shares a staged cell among the threads of a block in the
// same way) -- gives every particle one lane, loads 32 candidates at a time into shared memory and
// lets every lane test each of them against its own particle: a candidate position is loaded once
// per tile instead of once per particle, every lane accumulates its own sums (no reductions), and
// the test costs ~a dozen instructions per candidate for all particles of the tile together.
// Linear hash only (the cells of an x-row must be contiguous); same outputs, same neighbour lists
// (candidate order) as scalar_forward_kernel.
// ---------------------------------------------------------------------------
constexpr int kSharedBatch = 8;  // most work-list rows a warp draws per ticket

template <int D, bool PER, int MASK>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
scalar_forward_shared_kernel(ScalarFwdArgs a, Geom g, int span, int batch) {
    __shared__ int4 s_ranges[kWarpsPerCta][kMaxRanges];
    __shared__ float4 s_cand[kWarpsPerCta][2][32];  // x, y, z, mass of the staged candidates (two batches)
    __shared__ float s_vol[kWarpsPerCta][2][32];    // m / rho of the staged candidates (moment matrix only)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int4 *rng = s_ranges[warp];
    constexpr bool kSpiky = (MASK & (S_DGRAD | S_MOMENT)) != 0;
    constexpr bool kPoly = (MASK & S_DENSITY) != 0;
    // the neighbour count must agree bit for bit with the fp32 oracle on borderline pairs (r^2 without
    // fused multiply-adds); every other output is continuous at the cut-off
    constexpr bool kExact = (MASK & S_COUNT) != 0;
    // density alone on a clamped grid: two candidates per step in packed fp32x2 arithmetic (the staged
    // candidates are kept as four arrays x[32] y[32] z[32] m[32], so that a pair is one 8-byte broadcast)
    constexpr bool kPacked = !PER && MASK == S_DENSITY;
    const int K = a.pair_stride;

    bool finished = false;
    while (!finished) {
        int row = 0;
        if (lane == 0) row = (int)atomicAdd(a.tickets, (unsigned)batch);
        row = __shfl_sync(kFull, row, 0) + lane;
        WorkItem mine = {0, 0, 0, 0};
        int mcx = 0, mcy = 0, mcz = 0;
        if (lane < batch && row < g.max_blocks) mine = load_item(a.block_info, a.bin_offsets, row);
        if (mine.count > 0) hash_to_cell<D>(g, (uint32_t)(mine.cell - mine.sys * g.cells), mcx, mcy, mcz);
        int next = 0;
        while (next < batch) {
            const int h = next;
            const int hcount = __shfl_sync(kFull, mine.count, h);
            if (hcount <= 0) {  // rows after the last work item are zero
                finished = true;
                break;
            }
            const int hfirst = __shfl_sync(kFull, mine.first, h);
            const int hsys = __shfl_sync(kFull, mine.sys, h);
            const int hcx = __shfl_sync(kFull, mcx, h), hcy = __shfl_sync(kFull, mcy, h), hcz = __shfl_sync(kFull, mcz, h);
            // rows h, h+1, ... join the tile while they lie in the same x-row, within `span` cells, and the
            // tile holds at most 32 particles (rows of one x-row are contiguous in memory)
            const bool in_batch = lane >= h && lane < batch && mine.count > 0;
            const int upto = in_batch ? mine.first + mine.count - hfirst : 0;
            const bool wide = g.periodic && (mcx - hcx + 3 >= g.g[0]);
            const bool okrow = in_batch && mine.sys == hsys && mcy == hcy && mcz == hcz && mcx >= hcx &&
                               mcx - hcx < span && upto <= 32 && upto > 0 && (lane == h || !wide);
            const unsigned okm = __ballot_sync(kFull, okrow || lane == h);
            const unsigned run = ~okm & ~((1u << h) - 1u);
            const int stop = run ? __ffs(run) - 1 : 32;
            const int last = stop - 1;
            const int lcx = __shfl_sync(kFull, mcx, last);
            const int tile_count = __shfl_sync(kFull, mine.first + mine.count, last) - hfirst;
            next = stop;
            __syncwarp();
            const int nr = build_ranges_span<D>(g, a.bin_offsets, hsys, hcx, lcx, hcy, hcz, rng);

            for (int p0 = 0; p0 < tile_count; p0 += 32) {  // a lone row of more than 32 particles: passes of 32
                const bool ivalid = p0 + lane < tile_count;
                const long long i = hfirst + p0 + (ivalid ? lane : 0);
                const Pos<D> pi = load_pos<D>(a.x, i);
                int32_t *list = a.pair_cache ? a.pair_cache + i * K + 1 : nullptr;
                float cnt = 0.f, rho = 0.f, dg[3] = {0.f, 0.f, 0.f}, mom[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                unsigned long long rho2 = 0ull;  // kPacked: sums over the even and the odd candidates of the batches
                int listed = 0;

                // candidates are staged 32 at a time; the next batch is fetched from global memory while the
                // current one is tested.  A batch is (range r, first candidate j0); this walks them in order.
                auto fetch = [&](int r, int j0, float4 &c, float &v) {
                    c = make_float4(0.f, 0.f, 0.f, 0.f);
                    v = 0.f;
                    if (r < nr) {
                        const int j = j0 + lane;
                        if (j < rng[r].y) {
                            const Pos<D> pj = load_pos<D>(a.x, j);
                            const float mj = a.mass ? __ldg(a.mass + j) : 1.0f;
                            c = make_float4(pj.x, pj.y, pj.z, mj);
                            if (MASK & S_MOMENT) v = mj / __ldg(a.rho_in + j);
                        }
                    }
                };
                int r = 0, j0 = nr > 0 ? rng[0].x : 0, buf = 0;
                float4 c_next;
                float v_next;
                fetch(r, j0, c_next, v_next);
                while (r < nr) {
                    const int4 rg = rng[r];
                    float4 *cand = s_cand[warp][buf];
                    float *cvol = s_vol[warp][buf];
                    if (kPacked) {
                        float *cs = reinterpret_cast<float *>(cand);
                        cs[lane] = c_next.x; cs[32 + lane] = c_next.y; cs[64 + lane] = c_next.z; cs[96 + lane] = c_next.w;
                    } else {
                        cand[lane] = c_next;
                    }
                    if (MASK & S_MOMENT) cvol[lane] = v_next;
                    __syncwarp();
                    // the batch after this one
                    int rn = r, jn0 = j0 + 32;
                    if (jn0 >= rg.y) {
                        rn = r + 1;
                        jn0 = rn < nr ? rng[rn].x : 0;
                    }
                    fetch(rn, jn0, c_next, v_next);
                    if (kPacked && ivalid) {
                        const unsigned long long *cs = reinterpret_cast<const unsigned long long *>(cand);
                        const unsigned long long nox = pack2(-pi.x, -pi.x), noy = pack2(-pi.y, -pi.y), noz = pack2(-pi.z, -pi.z);
                        const int jn = min(32, rg.y - j0);
#pragma unroll 2
                        for (int k = 0; k < jn; k += 2) {
                            // candidates k and k + 1 (a batch that ends on an odd count is followed by a zero-mass entry)
                            const unsigned long long rx = add2(cs[k >> 1], nox), ry = add2(cs[16 + (k >> 1)], noy);
                            unsigned long long q = fma2(ry, ry, mul2(rx, rx));
                            if (D == 3) {
                                const unsigned long long rz = add2(cs[32 + (k >> 1)], noz);
                                q = fma2(rz, rz, q);
                            }
                            float q0, q1;
                            unpack2(q, q0, q1);
                            const bool acc0 = q0 < g.h2, acc1 = q1 < g.h2 && k + 1 < jn;
                            if (list) {
                                if (acc0 && listed < K - 1) list[listed] = j0 + k;
                                listed += acc0 ? 1 : 0;
                                if (acc1 && listed < K - 1) list[listed] = j0 + k + 1;
                                listed += acc1 ? 1 : 0;
                            }
                            const unsigned long long t = pack2(fmaxf(g.h2 - q0, 0.f), fmaxf(g.h2 - q1, 0.f));
                            rho2 = fma2(cs[48 + (k >> 1)], mul2(mul2(t, t), t), rho2);
                        }
                    } else if (ivalid) {
                        const Origin<D, PER> org = make_origin<D, PER>(g, pi.x, pi.y, pi.z, rg.z);
                        const int jn = min(32, rg.y - j0);
#pragma unroll 4
                        for (int k = 0; k < jn; ++k) {
                            const float4 c = cand[k];  // same address in every lane: one broadcast
                            float rx, ry, rz;
                            const float q = displacement<D, PER, kExact>(g, org, c.x, c.y, c.z, rx, ry, rz);
                            const bool acc = q < g.h2;
                            if (list) {
                                if (acc && listed < K - 1) list[listed] = j0 + k;
                                listed += acc ? 1 : 0;
                            }
                            if (MASK & S_COUNT) cnt += acc ? 1.0f : 0.f;
                            // both kernels vanish at the cut-off: no branch on `acc` is needed
                            if (kPoly) {
                                const float t = fmaxf(g.h2 - q, 0.f);
                                rho = fmaf(c.w, t * t * t, rho);
                            }
                            if (kSpiky) {
                                float d;
                                const float phi = acc ? spiky_phi(q, g.h, d) : 0.f;  // phi r = 0 for the self pair
                                if (MASK & S_DGRAD) {
                                    const float w = c.w * phi;
                                    dg[0] = fmaf(w, rx, dg[0]);
                                    dg[1] = fmaf(w, ry, dg[1]);
                                    if (D == 3) dg[2] = fmaf(w, rz, dg[2]);
                                }
                                if (MASK & S_MOMENT) {
                                    const float w = phi * cvol[k];
                                    mom[0] = fmaf(w * rx, rx, mom[0]);
                                    mom[1] = fmaf(w * rx, ry, mom[1]);
                                    if (D == 2) {
                                        mom[2] = fmaf(w * ry, ry, mom[2]);
                                    } else {
                                        mom[2] = fmaf(w * rx, rz, mom[2]);
                                        mom[3] = fmaf(w * ry, ry, mom[3]);
                                        mom[4] = fmaf(w * ry, rz, mom[4]);
                                        mom[5] = fmaf(w * rz, rz, mom[5]);
                                    }
                                }
                            }
                        }
                    }
                    r = rn;
                    j0 = jn0;
                    buf ^= 1;
                }
                __syncwarp();
                if (kPacked) {
                    float lo, hi;
                    unpack2(rho2, lo, hi);
                    rho = lo + hi;
                }
                if (ivalid) {
                    if (list) list[-1] = listed <= K - 1 ? listed : -1;
                    if ((MASK & S_COUNT) && a.count) a.count[i] = cnt;
                    if (kPoly && a.rho_out) a.rho_out[i] = g.c_s * rho;
                    if ((MASK & S_DGRAD) && a.rho_grad) {
#pragma unroll
                        for (int d = 0; d < D; ++d) a.rho_grad[i * D + d] = g.c_g * dg[d];
                    }
                    if ((MASK & S_MOMENT) && a.moment) {
                        float *o = a.moment + i * (D * D);
                        if (D == 2) {
                            reinterpret_cast<float4 *>(o)[0] =
                                make_float4(g.c_g * mom[0], g.c_g * mom[1], g.c_g * mom[1], g.c_g * mom[2]);
                        } else {
                            o[0] = g.c_g * mom[0]; o[1] = g.c_g * mom[1]; o[2] = g.c_g * mom[2];
                            o[3] = g.c_g * mom[1]; o[4] = g.c_g * mom[3]; o[5] = g.c_g * mom[4];
                            o[6] = g.c_g * mom[2]; o[7] = g.c_g * mom[4]; o[8] = g.c_g * mom[5];
                        }
                    }
                }
            }
        }
    }
    release_rows(a.tickets);
}

// Gather backward of density / density gradient / moment matrix, same layout (8 particles per warp
// pass, 4 lanes each).  With a neighbour-list cache of the snapshot the lanes of a sub-group walk
// the list of their particle; particles without a list (cache off, or more neighbours than the
// list holds) test the candidates of the cells.
template <int D, bool PER, int MASK>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
scalar_backward_kernel(ScalarBwdArgs a, Geom g) {
    __shared__ int4 s_ranges[kWarpsPerCta][kMaxRanges];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int4 *rng = s_ranges[warp];
    const int sub = lane / kScalarLpp, sl = lane % kScalarLpp;
    constexpr bool kSpiky = (MASK & (S_DGRAD | S_MOMENT)) != 0;
    constexpr int DD = D * D;
    const int K = a.pair_stride;

    const int vrows = g.max_blocks * g.split;
    for (int vrow = next_row(a.tickets); vrow < vrows; vrow = next_row(a.tickets)) {
        const int row = vrow / g.split, part = vrow - row * g.split;
        const WorkItem it = load_item(a.block_info, a.bin_offsets, row);
        if (it.count <= 0) break;
        if (part * kScalarPpw >= it.count) continue;
        __syncwarp();
        const int nr = build_ranges<D>(g, a.bin_offsets, it, rng);

        for (int k0 = part * kScalarPpw; k0 < it.count; k0 += g.split * kScalarPpw) {
            const int k = k0 + sub;
            const bool ivalid = k < it.count;
            const long long i = it.first + (ivalid ? k : 0);
            const Pos<D> pi = load_pos<D>(a.x, i);
            const float mi = a.mass ? __ldg(a.mass + i) : 1.0f;
            float gri = 0.f, gdi[3] = {0.f, 0.f, 0.f}, gmi[DD], vi = 0.f;
            if (MASK & S_DENSITY) {
                if (a.g_rho_a) gri += __ldg(a.g_rho_a + i);
                if (a.g_rho_b) gri += __ldg(a.g_rho_b + i);
            }
            if (MASK & S_DGRAD) {
#pragma unroll
                for (int d = 0; d < D; ++d) gdi[d] = __ldg(a.g_rho_grad + i * D + d);
            }
            if (MASK & S_MOMENT) {
#pragma unroll
                for (int d = 0; d < DD; ++d) gmi[d] = __ldg(a.g_moment + i * DD + d);
                vi = mi / __ldg(a.rho_in + i);
            }
            float dxs[3] = {0.f, 0.f, 0.f};  // poly6 part, scaled by c_s at the end
            float dxg[3] = {0.f, 0.f, 0.f};  // spiky part, scaled by c_g at the end
            float drho = 0.f;

            // contribution of one pair (the self / coincident pair has zero gradient)
            auto visit = [&](long long j, float rx, float ry, float rz, float q) {
                if (!(q > 0.f)) return;
                const float rv[3] = {rx, ry, rz};
                const float mj = a.mass ? __ldg(a.mass + j) : 1.0f;
                if (MASK & S_DENSITY) {
                    float grj = 0.f;
                    if (a.g_rho_a) grj += __ldg(a.g_rho_a + j);
                    if (a.g_rho_b) grj += __ldg(a.g_rho_b + j);
                    const float t = fmaxf(g.h2 - q, 0.f);
                    const float w = 6.0f * t * t * (gri * mj + grj * mi);
#pragma unroll
                    for (int d = 0; d < D; ++d) dxs[d] = fmaf(w, rv[d], dxs[d]);
                }
                if (kSpiky) {
                    float dist;
                    const float phi = spiky_phi(q, g.h, dist);
                    const float psi = spiky_psi(dist, g.h);
                    if (MASK & S_DGRAD) {
                        float u[3] = {0.f, 0.f, 0.f}, o[3];
#pragma unroll
                        for (int d = 0; d < D; ++d) u[d] = mi * __ldg(a.g_rho_grad + j * D + d) - mj * gdi[d];
                        apply_jacobian<D>(phi, psi, rv[0], rv[1], rv[2], u[0], u[1], u[2], o[0], o[1], o[2]);
#pragma unroll
                        for (int d = 0; d < D; ++d) dxg[d] += o[d];
                    }
                    if (MASK & S_MOMENT) {
                        const float vj = mj / __ldg(a.rho_in + j);
                        float w[3] = {0.f, 0.f, 0.f}, o[3];
                        float rr = 0.f;  // sum_ab gM_j[a,b] r_a r_b
#pragma unroll
                        for (int p = 0; p < D; ++p) {
                            float kc = 0.f;  // sum_b Cm[p,b] K_b
#pragma unroll
                            for (int b = 0; b < D; ++b) {
                                const float gj = __ldg(a.g_moment + j * DD + p * D + b);
                                const float cm = vj * gmi[p * D + b] + vi * gj;
                                kc = fmaf(cm, phi * rv[b], kc);
                                w[b] = fmaf(rv[p], cm, w[b]);
                                rr = fmaf(gj * rv[p], rv[b], rr);
                            }
                            dxg[p] -= kc;
                        }
                        apply_jacobian<D>(phi, psi, rv[0], rv[1], rv[2], w[0], w[1], w[2], o[0], o[1], o[2]);
#pragma unroll
                        for (int d = 0; d < D; ++d) dxg[d] -= o[d];
                        drho = fmaf(rr, phi, drho);
                    }
                }
            };

            int listed = -1;  // the same in the four lanes of a sub-group
            if (a.pair_cache && ivalid) listed = __ldg(a.pair_cache + i * K);
            if (listed >= 0) {
                const int32_t *list = a.pair_cache + i * K + 1;
                for (int e = sl; e < listed; e += kScalarLpp) {
                    const int j = __ldg(list + e);
                    const Pos<D> pj = load_pos<D>(a.x, j);
                    float rx, ry, rz;
                    listed_displacement<D, PER>(g, pi, pj, rx, ry, rz);
                    visit(j, rx, ry, rz, sq_norm_fast<D>(rx, ry, rz));
                }
            }
            if (__any_sync(kFull, ivalid && listed < 0)) {
                for (int r = 0; r < nr; ++r) {
                    const int4 rg = rng[r];
                    const Origin<D, PER> org = make_origin<D, PER>(g, pi.x, pi.y, pi.z, rg.z);
                    for (int j0 = rg.x; j0 < rg.y; j0 += kScalarLpp) {
                        const int j = j0 + sl;
                        if (!(ivalid && listed < 0 && j < rg.y)) continue;
                        const Pos<D> pj = load_pos<D>(a.x, j);
                        float rx, ry, rz;
                        const float q = displacement<D, PER, false>(g, org, pj.x, pj.y, pj.z, rx, ry, rz);
                        if (q < g.h2) visit(j, rx, ry, rz, q);
                    }
                }
            }

            float out[3];
#pragma unroll
            for (int d = 0; d < D; ++d) out[d] = subgroup_sum<kScalarLpp>(g.c_s * dxs[d] + g.c_g * dxg[d]);
            if (MASK & S_MOMENT) drho = subgroup_sum<kScalarLpp>(drho);
            if (ivalid && sl == 0) {
                if (a.grad_x) {
                    if (D == 2) {
                        float2 *o = reinterpret_cast<float2 *>(a.grad_x) + i;
                        float2 v = make_float2(out[0], out[1]);
                        if (a.accumulate_x) { const float2 p = *o; v.x += p.x; v.y += p.y; }
                        *o = v;
                    } else {
                        float4 *o = reinterpret_cast<float4 *>(a.grad_x) + i;
                        float4 v = make_float4(out[0], out[1], out[2], 0.f);
                        if (a.accumulate_x) { const float4 p = *o; v.x += p.x; v.y += p.y; v.z += p.z; }
                        *o = v;
                    }
                }
                if ((MASK & S_MOMENT) && a.grad_rho) a.grad_rho[i] = -g.c_g * (vi * vi / mi) * drho;
            }
        }
    }
    release_rows(a.tickets);
}

// ---------------------------------------------------------------------------
// dispatch: persistent launches (every SM filled to the kernel's occupancy)
// ---------------------------------------------------------------------------
template <typename Kernel, typename Args>
static int launch_persistent(const Geom &g, Kernel kernel, const Args &a, cudaStream_t st, const char *what) {
    const int threads = kWarpsPerCta * 32;
    int ctas = 0;
    int rc = persistent_ctas(kernel, threads, 0, &ctas);
    if (rc != NPA_OK) return rc;
    const int needed = (g.max_blocks * g.split + kWarpsPerCta - 1) / kWarpsPerCta;
    Args b = a;
    if ((rc = acquire_row_tickets(st, &b.tickets)) != NPA_OK) return rc;
    kernel<<<needed < ctas ? needed : ctas, threads, 0, st>>>(b, g);
    return check_launch(what);
}

// Cells per tile of the shared-candidate forward sweep (0 = keep the per-particle kernel).
static int g_shared_span = 3;
void set_scalar_shared_span(int span) { g_shared_span = span; }

template <typename Kernel>
static int launch_shared(const Geom &g, Kernel kernel, const ScalarFwdArgs &a, cudaStream_t st) {
    const int threads = kWarpsPerCta * 32;
    int ctas = 0;
    int rc = persistent_ctas(kernel, threads, 0, &ctas);
    if (rc != NPA_OK) return rc;
    // rows a warp draws per ticket: enough tickets for two rounds over the resident warps, at most kSharedBatch
    // (consecutive rows of one ticket can merge into a tile; a single row cannot)
    int batch = g.max_blocks / (2 * ctas * kWarpsPerCta);
    batch = batch < 1 ? 1 : (batch > kSharedBatch ? kSharedBatch : batch);
    const int needed = (g.max_blocks + batch * kWarpsPerCta - 1) / (batch * kWarpsPerCta);
    ScalarFwdArgs b = a;
    if ((rc = acquire_row_tickets(st, &b.tickets)) != NPA_OK) return rc;
    kernel<<<needed < ctas ? (needed > 0 ? needed : 1) : ctas, threads, 0, st>>>(b, g, g_shared_span % 100, batch);
    return check_launch("scalar_forward_shared_kernel");
}

template <int MASK>
static int launch_scalar_fwd_mask(const Geom &g, const ScalarFwdArgs &a, cudaStream_t st) {
    // Shared candidates need the cells of an x-row contiguous (linear hash).  Measured: the sweep of the
    // poly6 operators (count, density) gains 30-40 % on clamped grids in 2D and 3D; with the spiky operators
    // in the mask, and on 3D periodic grids, the per-particle walk is as fast or faster and stays.
    constexpr bool kSpikyMask = (MASK & (S_DGRAD | S_MOMENT)) != 0;
    if (!g.morton && g_shared_span > 0 && !kSpikyMask && (!g.periodic || g.dim == 2 || g_shared_span >= 100)) {
        if (g.dim == 2) {
            if (g.periodic) return launch_shared(g, scalar_forward_shared_kernel<2, true, MASK>, a, st);
            return launch_shared(g, scalar_forward_shared_kernel<2, false, MASK>, a, st);
        }
        if (g.periodic) return launch_shared(g, scalar_forward_shared_kernel<3, true, MASK>, a, st);
        return launch_shared(g, scalar_forward_shared_kernel<3, false, MASK>, a, st);
    }
    const char *what = "scalar_forward_kernel";
    if (g.dim == 2) {
        if (g.periodic) return launch_persistent(g, scalar_forward_kernel<2, true, MASK>, a, st, what);
        return launch_persistent(g, scalar_forward_kernel<2, false, MASK>, a, st, what);
    }
    if (g.periodic) return launch_persistent(g, scalar_forward_kernel<3, true, MASK>, a, st, what);
    return launch_persistent(g, scalar_forward_kernel<3, false, MASK>, a, st, what);
}

int launch_scalar_forward(const Geom &g, int mask, const ScalarFwdArgs &a, cudaStream_t st) {
    switch (mask) {
        case S_COUNT: return launch_scalar_fwd_mask<S_COUNT>(g, a, st);
        case S_DENSITY: return launch_scalar_fwd_mask<S_DENSITY>(g, a, st);
        case S_DGRAD: return launch_scalar_fwd_mask<S_DGRAD>(g, a, st);
        case S_MOMENT: return launch_scalar_fwd_mask<S_MOMENT>(g, a, st);
        case S_DENSITY | S_DGRAD: return launch_scalar_fwd_mask<S_DENSITY | S_DGRAD>(g, a, st);
        default:
            if ((mask & ~(S_COUNT | S_DENSITY | S_DGRAD)) == 0)
                return launch_scalar_fwd_mask<S_COUNT | S_DENSITY | S_DGRAD>(g, a, st);
            return fail(NPA_ERR_INVALID_ARGUMENT, "unsupported scalar forward mask %d", mask);
    }
}

template <int MASK>
static int launch_scalar_bwd_mask(const Geom &g, const ScalarBwdArgs &a, cudaStream_t st) {
    const char *what = "scalar_backward_kernel";
    if (g.dim == 2) {
        if (g.periodic) return launch_persistent(g, scalar_backward_kernel<2, true, MASK>, a, st, what);
        return launch_persistent(g, scalar_backward_kernel<2, false, MASK>, a, st, what);
    }
    if (g.periodic) return launch_persistent(g, scalar_backward_kernel<3, true, MASK>, a, st, what);
    return launch_persistent(g, scalar_backward_kernel<3, false, MASK>, a, st, what);
}

int launch_scalar_backward(const Geom &g, int mask, const ScalarBwdArgs &a, cudaStream_t st) {
    switch (mask) {
        case S_DENSITY: return launch_scalar_bwd_mask<S_DENSITY>(g, a, st);
        case S_DGRAD: return launch_scalar_bwd_mask<S_DGRAD>(g, a, st);
        case S_MOMENT: return launch_scalar_bwd_mask<S_MOMENT>(g, a, st);
        case S_DENSITY | S_DGRAD: return launch_scalar_bwd_mask<S_DENSITY | S_DGRAD>(g, a, st);
        default: return fail(NPA_ERR_INVALID_ARGUMENT, "unsupported scalar backward mask %d", mask);
    }
}

}  // namespace npa
