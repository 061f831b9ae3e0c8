// Feature-carrying SPH operators: blur (kernel-weighted feature average) and
// the SPH feature gradient, forward and backward, fused in one sweep when both
// are asked for.
//
// Replaces forward_kernel / backward_kernel of the reference for the Blur and
// Gradient computation types (sphops/sph_cuda.cu:1699-1716, 1185-1235,
// 1265-1327).  The reference maps a thread to (particle, feature) and redoes the
// distance test and the kernel weight once per feature.  Here one warp owns one
// work item and walks its particles one at a time in three stages:
//   1. test: the 32 lanes test 32 candidates per round and ballot-compact the
//      accepted displacements into a per-warp shared-memory list;
//   2. weights: the lanes turn list entries into pair scalars (kernel weight,
//      spiky factors, m_j / rho_j), one entry per lane, all lanes busy;
//   3. drain: the warp is split into 32 / LPP sub-groups of LPP lanes; each
//      sub-group takes every (32 / LPP)-th pair and its lanes cover the features
//      (VW = 4 per lane, 128-bit loads when C % 4 == 0).  Sub-group partial sums
//      are combined by shuffles once per particle.
// Every pair is tested once and its scalars are computed once; the work of a
// particle is spread evenly over the warp whatever its neighbour count.
//
// Backward is a gather (no global atomics): particle i collects the terms of
// both roles it plays in each pair.  Sums over features (the position and
// density gradients) stay lane-local until the final reduction.
#pragma once
#include "neighbors.cuh"
#include "ops.cuh"

namespace npa {

constexpr int kListPerWarp = 128;  // accepted-pair slots per warp
constexpr int kBwdStages = 2;       // same, backward (five pieces per pair)
// Full backward: smaller CTAs give the register allocator a finer occupancy grid (5 x 4 warps)
constexpr int kBwdFullWarps = 4;
constexpr int kBwdFullCtas = 5;
constexpr int bwd_warps(bool full) { return full ? kBwdFullWarps : kWarpsPerCta; }
constexpr bool kBwdRing = true;     // backward: cp.async ring (true) or register double buffer (false)

template <int VW>
__device__ inline void load_feat(const float *__restrict__ p, float (&v)[VW]) {
    if (VW == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
#pragma unroll
        for (int k = 0; k < VW; ++k) v[k] = __ldg(p + k);
    }
}

// n contiguous floats, n = VW * D; 16-byte aligned when VW == 4.
template <int VW, int NF>
__device__ inline void load_run(const float *__restrict__ p, float (&v)[NF]) {
    if (VW == 4) {
#pragma unroll
        for (int k = 0; k < NF / 4; ++k) {
            const float4 t = __ldg(reinterpret_cast<const float4 *>(p) + k);
            v[4 * k] = t.x; v[4 * k + 1] = t.y; v[4 * k + 2] = t.z; v[4 * k + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int k = 0; k < NF; ++k) v[k] = __ldg(p + k);
    }
}

template <int VW, int NF>
__device__ inline void store_run(float *__restrict__ p, const float (&v)[NF]) {
    if (VW == 4) {
#pragma unroll
        for (int k = 0; k < NF / 4; ++k)
            reinterpret_cast<float4 *>(p)[k] = make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
    } else {
#pragma unroll
        for (int k = 0; k < NF; ++k) p[k] = v[k];
    }
}

// 4-, 8- or 16-byte asynchronous global -> shared copy (cp.async, L1-allocating).  Each lane
// copies only what it will read back itself, so completion is tracked per thread with
// cp.async.wait_group and no barrier or cross-lane flag is involved.
template <int BYTES>
__device__ inline void async_copy(void *smem_dst, const void *gmem_src) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(dst), "l"(gmem_src), "n"(BYTES) : "memory");
}
__device__ inline void async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int PENDING>
__device__ inline void async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(PENDING) : "memory"); }

// VW floats per lane: the element type of a lane's staging slot.
template <int VW> struct Piece { float v[VW]; };
template <> struct __align__(16) Piece<4> { float v[4]; };

// Sum over the sub-groups of a warp: lanes with equal (lane % LPP) are combined.
template <int LPP>
__device__ inline float across_subgroups(float v) {
#pragma unroll
    for (int o = LPP; o < 32; o <<= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
}

// Stage 1 for one particle: test every candidate of every range, append the
// accepted displacements (r, index of j) to `geo`; calls flush(n) whenever the
// list could overflow and once at the end.
template <int D, bool PER, typename Flush>
__device__ inline void collect_pairs(const Geom &g, const float *__restrict__ x, const Pos<D> &pi,
                                     const int4 *rng, int nr, float4 *geo, Flush &&flush) {
    const int lane = threadIdx.x & 31;
    int n = 0;
    scan_candidates<D, PER, false>(g, x, pi, rng, nr, [&](bool acc, int j, float rx, float ry, float rz, float) {
        const unsigned bal = __ballot_sync(kFull, acc);
        if (acc) geo[n + __popc(bal & ((1u << lane) - 1u))] = make_float4(rx, ry, rz, __int_as_float(j));
        n += __popc(bal);
        if (n + 32 > kListPerWarp) {
            flush(n);
            n = 0;
        }
    });
    flush(n);
}

// Stage 1 from a cached neighbour list (written by the forward sweep of the same snapshot): the
// lanes fetch the listed positions and rebuild the displacements; no candidate is tested.  On a
// periodic grid the image of each pair is recovered from the raw difference (x_j - x_i is within half
// a box of a multiple of the box length) and applied with the same error-free shifted origin as the
// cell walk uses.
// Starts `width` floats at `row` on their way into L1 (one or two lines; rows are read in pieces of at
// most 128 bytes).
__device__ inline void prefetch_row(const float *row, int width) {
    asm volatile("prefetch.global.L1 [%0];" ::"l"(row));
    if ((reinterpret_cast<uintptr_t>(row) & 127) != 0 && width > 4) asm volatile("prefetch.global.L1 [%0];" ::"l"(row + width - 1));
}

// `rows` (optional): feature rows of `pitch` floats of which stage 3 will read `width` floats per neighbour;
// they are prefetched as soon as the index is known.
template <int D, bool PER>
__device__ inline void expand_pairs(const Geom &g, const float *__restrict__ x, const Pos<D> &pi,
                                    const int32_t *__restrict__ list, int count, float4 *geo,
                                    const float *__restrict__ rows = nullptr, int pitch = 0, int width = 0) {
    const int lane = threadIdx.x & 31;
    for (int e = lane; e < count; e += 32) {
        const int j = __ldg(list + e);
        if (rows) prefetch_row(rows + (long long)j * pitch, width);
        const Pos<D> pj = load_pos<D>(x, j);
        float rx, ry, rz;
        listed_displacement<D, PER>(g, pi, pj, rx, ry, rz);
        geo[e] = make_float4(rx, ry, rz, __int_as_float(j));
    }
}

template <int D, bool PER, int LPP, int VW, int MASK>
__global__ void __launch_bounds__(kWarpsPerCta * 32, (MASK & (F_MOMENT | F_PACK)) ? 3 : 4)
feature_forward_kernel(FeatureFwdArgs a, Geom g) {
    constexpr int PP = 32 / LPP;  // pairs drained in parallel
    __shared__ int4 s_ranges[kWarpsPerCta][kMaxRanges];
    __shared__ float4 s_geo[kWarpsPerCta][kListPerWarp];  // r.x r.y r.z, index of j
    __shared__ float4 s_ent[kWarpsPerCta][kListPerWarp];  // v_j K.x, v_j K.y, v_j K.z, v_j W

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sg = lane / LPP, sl = lane % LPP;
    int4 *rng = s_ranges[warp];
    float4 *geo = s_geo[warp];
    float4 *ent = s_ent[warp];
    const int C = a.C;

    // persistent warps: consecutive rows go to the warps of one CTA, then to the next CTA
    // g.split warps share one row (its particles are dealt round-robin) when rows are scarce
    const int vrows = g.max_blocks * g.split;
    for (int vrow = next_row(a.tickets); vrow < vrows; vrow = next_row(a.tickets)) {
    const int row = vrow / g.split, part = vrow - row * g.split;
    const WorkItem it = load_item(a.block_info, a.bin_offsets, row);
    if (it.count <= 0) break;  // rows after the last work item are zero
    if (part >= it.count) continue;
    __syncwarp();
    const int nr = build_ranges<D>(g, a.bin_offsets, it, rng);

    for (int k = part; k < it.count; k += g.split) {
        const long long i = it.first + k;
        const Pos<D> pi = load_pos<D>(a.x, i);
        if (a.pair_cache && a.pair_cache_valid && k + g.split < it.count && lane * 32 < a.pair_stride && lane < 4) {
            // the head of the next particle's neighbour list (the first 512 bytes) on its way into L1
            asm volatile("prefetch.global.L1 [%0];" ::"l"(a.pair_cache + (i + g.split) * a.pair_stride + lane * 32));
        }
        float mom[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};  // F_MOMENT: upper triangle, lane-partial over pairs
        float dgs[3] = {0.f, 0.f, 0.f};                   // F_PACK with rho_grad_out: density gradient, lane-partial over pairs
        for (int fbase = 0; fbase < C; fbase += LPP * VW) {
            const int f0 = fbase + sl * VW;
            const bool fvalid = f0 < C;
            float si[VW], blur[VW], gr[VW * D];
#pragma unroll
            for (int q = 0; q < VW; ++q) { si[q] = 0.f; blur[q] = 0.f; }
#pragma unroll
            for (int q = 0; q < VW * D; ++q) gr[q] = 0.f;
            if (fvalid && (MASK & F_GRAD)) load_feat<VW>(a.s + i * C + f0, si);
            // VW == 4: the sums live in packed pairs while the pairs are drained -- blur of features (0, 1) and (2, 3),
            // then per axis the gradient of (0, 1) and (2, 3) -- and are unpacked into blur[] / gr[] afterwards
            unsigned long long pacc[2 + 2 * D];
#pragma unroll
            for (int q = 0; q < 2 + 2 * D; ++q) pacc[q] = 0ull;
            const unsigned long long nsi01 = pack2(-si[0], -si[VW == 4 ? 1 : 0]), nsi23 = pack2(-si[VW == 4 ? 2 : 0], -si[VW == 4 ? 3 : 0]);

            int cached = 0;  // pairs of this particle already written to the neighbour list cache
            bool from_list = false;
            const int chunk_w = C - fbase < LPP * VW ? C - fbase : LPP * VW;  // floats of a row read in this chunk
            auto flush = [&](int n) {
                __syncwarp();
                for (int e = lane; e < n; e += 32) {  // stage 2: pair scalars, one entry per lane
                    const float4 ge = geo[e];
                    const int j = __float_as_int(ge.w);
                    if (a.pair_cache && !a.pair_cache_valid && fbase == 0 && cached + e < a.pair_stride - 1)
                        a.pair_cache[i * a.pair_stride + 1 + cached + e] = j;
                    // the neighbour's feature row is wanted in stage 3: start it on its way into L1 (the list path
                    // has done so already, in expand_pairs)
                    if (!from_list) prefetch_row(a.s + ((long long)j * C + fbase), chunk_w);
                    const float q = sq_norm_fast<D>(ge.x, ge.y, ge.z);
                    const float mj = a.mass ? __ldg(a.mass + j) : 1.0f;
                    const float vj = mj / __ldg(a.rho + j);
                    float wv = 0.f, kv = 0.f;
                    if (MASK & F_BLUR) {
                        const float t = fmaxf(g.h2 - q, 0.f);
                        wv = vj * (t * t * t);
                    }
                    if ((MASK & (F_GRAD | F_MOMENT)) && q > 0.f) {
                        float dist;
                        const float phi = spiky_phi(q, g.h, dist);
                        kv = vj * phi;
                        if ((MASK & F_PACK) && a.rho_grad_out && fbase == 0) {  // the density gradient's pair term: m_j phi r
                            const float w = mj * phi;
                            dgs[0] = fmaf(w, ge.x, dgs[0]);
                            dgs[1] = fmaf(w, ge.y, dgs[1]);
                            if (D == 3) dgs[2] = fmaf(w, ge.z, dgs[2]);
                        }
                    }
                    if ((MASK & F_MOMENT) && fbase == 0) {  // every pair is seen once per feature chunk
                        mom[0] = fmaf(kv * ge.x, ge.x, mom[0]);
                        mom[1] = fmaf(kv * ge.x, ge.y, mom[1]);
                        if (D == 2) {
                            mom[2] = fmaf(kv * ge.y, ge.y, mom[2]);
                        } else {
                            mom[2] = fmaf(kv * ge.x, ge.z, mom[2]);
                            mom[3] = fmaf(kv * ge.y, ge.y, mom[3]);
                            mom[4] = fmaf(kv * ge.y, ge.z, mom[4]);
                            mom[5] = fmaf(kv * ge.z, ge.z, mom[5]);
                        }
                    }
                    ent[e] = make_float4(kv * ge.x, kv * ge.y, kv * ge.z, wv);
                }
                // zero weights fill the last pass of stage 3 (n <= kListPerWarp, a multiple of PP: the slots exist)
                if (n + lane < (n + PP - 1) / PP * PP) ent[n + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
                __syncwarp();
                if (fvalid) {
                    // stage 3: each sub-group drains every PP-th pair; the neighbour's feature rows pass
                    // through three rotating register sets, the rows of the next two pairs in flight
                    auto consume = [&](int e, const float (&sj)[VW]) {
                        const float4 en = ent[e];
                        if (VW == 4) {
                            const unsigned long long s01 = pack2(sj[0], sj[VW == 4 ? 1 : 0]), s23 = pack2(sj[VW == 4 ? 2 : 0], sj[VW == 4 ? 3 : 0]);
                            if (MASK & F_BLUR) {
                                const unsigned long long ww = pack2(en.w, en.w);
                                pacc[0] = fma2(ww, s01, pacc[0]);
                                pacc[1] = fma2(ww, s23, pacc[1]);
                            }
                            if (MASK & F_GRAD) {
                                const unsigned long long d01 = add2(s01, nsi01), d23 = add2(s23, nsi23);  // s_j - s_i
                                const float kd[3] = {en.x, en.y, en.z};
#pragma unroll
                                for (int d = 0; d < D; ++d) {
                                    const unsigned long long kk = pack2(kd[d], kd[d]);
                                    pacc[2 + 2 * d] = fma2(d01, kk, pacc[2 + 2 * d]);
                                    pacc[3 + 2 * d] = fma2(d23, kk, pacc[3 + 2 * d]);
                                }
                            }
                        } else {
#pragma unroll
                            for (int q = 0; q < VW; ++q) {
                                if (MASK & F_BLUR) blur[q] = fmaf(en.w, sj[q], blur[q]);
                                if (MASK & F_GRAD) {
                                    const float df = sj[q] - si[q];
                                    gr[q * D + 0] = fmaf(df, en.x, gr[q * D + 0]);
                                    gr[q * D + 1] = fmaf(df, en.y, gr[q * D + 1]);
                                    if (D == 3) gr[q * D + 2] = fmaf(df, en.z, gr[q * D + 2]);
                                }
                            }
                        }
                    };
                    {
                        // row address = lane base + index x row pitch: one wide multiply-add per load
                        const char *srow = reinterpret_cast<const char *>(a.s + f0);
                        const unsigned pitch = (unsigned)C * 4u;
                        auto load = [&](int e, float (&sj)[VW]) {
                            if (e < n)
                                load_feat<VW>(reinterpret_cast<const float *>(
                                                  srow + (unsigned long long)(unsigned)__float_as_int(geo[e].w) * pitch), sj);
                        };
                        // every sub-group makes the same number of passes (the entries that fill the last pass
                        // have zero weights), so the loop has no divergent exit
                        float r0[VW] = {}, r1[VW] = {}, r2[VW] = {};
                        int e = sg, left = (n + PP - 1) / PP;
                        load(e, r0);
                        load(e + PP, r1);
                        for (; left >= 3; left -= 3, e += 3 * PP) {
                            load(e + 2 * PP, r2);
                            consume(e, r0);
                            load(e + 3 * PP, r0);
                            consume(e + PP, r1);
                            load(e + 4 * PP, r1);
                            consume(e + 2 * PP, r2);
                        }
                        if (left >= 1) consume(e, r0);
                        if (left == 2) consume(e + PP, r1);
                    }
                }
                cached += n;
                __syncwarp();
            };
            int listed = -1;
            if (a.pair_cache && a.pair_cache_valid) listed = __ldg(a.pair_cache + i * a.pair_stride);
            from_list = listed >= 0;
            if (listed >= 0 && listed <= kListPerWarp) {
                expand_pairs<D, PER>(g, a.x, pi, a.pair_cache + i * a.pair_stride + 1, listed, geo, a.s + fbase, C, chunk_w);
                flush(listed);
            } else if (listed > kListPerWarp) {
                // a list longer than the warp's pair slots goes through in pieces (the sums carry over); kept apart
                // from the common case above, which a loop around it was measured to slow down by 4 %
                const int32_t *list = a.pair_cache + i * a.pair_stride + 1;
#pragma unroll 1
                for (int off = 0; off < listed; off += kListPerWarp) {
                    const int n = listed - off < kListPerWarp ? listed - off : kListPerWarp;
                    expand_pairs<D, PER>(g, a.x, pi, list + off, n, geo, a.s + fbase, C, chunk_w);
                    flush(n);
                }
            } else {
                collect_pairs<D, PER>(g, a.x, pi, rng, nr, geo, flush);
                if (a.pair_cache && !a.pair_cache_valid && fbase == 0 && lane == 0)
                    a.pair_cache[i * a.pair_stride] = cached <= a.pair_stride - 1 ? cached : -1;
            }

            if (VW == 4) {
                unpack2(pacc[0], blur[0], blur[VW == 4 ? 1 : 0]);
                unpack2(pacc[1], blur[VW == 4 ? 2 : 0], blur[VW == 4 ? 3 : 0]);
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    unpack2(pacc[2 + 2 * d], gr[0 * D + d], gr[(VW == 4 ? 1 : 0) * D + d]);
                    unpack2(pacc[3 + 2 * d], gr[(VW == 4 ? 2 : 0) * D + d], gr[(VW == 4 ? 3 : 0) * D + d]);
                }
            }
            if (MASK & F_BLUR) {
#pragma unroll
                for (int q = 0; q < VW; ++q) blur[q] = g.c_s * across_subgroups<LPP>(blur[q]);
            }
            if (MASK & F_GRAD) {
#pragma unroll
                for (int q = 0; q < VW * D; ++q) gr[q] = g.c_g * across_subgroups<LPP>(gr[q]);
            }
            if (sg == 0 && fvalid) {
                if ((MASK & F_BLUR) && a.blur) store_run<VW, VW>(a.blur + i * C + f0, blur);
                if ((MASK & F_GRAD) && a.grad) store_run<VW, VW * D>(a.grad + (i * C + f0) * D, gr);
            }
            if (MASK & F_PACK) {
                // perception epilogue (the launcher guarantees a single feature chunk): moment matrix ->
                // safe inverse -> corrected gradient -> scaling and log-normalisation -> packed row
#pragma unroll
                for (int q = 0; q < D * (D + 1) / 2; ++q) mom[q] = g.c_g * subgroup_sum<32>(mom[q]);
                float L[D * D];
                safe_inverse_sym<D>(mom, a.inv_tol, L);
                // the row is assembled in the (now idle) pair list of this warp and written coalesced
                float *zr = a.z + i * a.zstride;
                const bool staged = a.zstride <= kListPerWarp * 4;
                float *zs = staged ? reinterpret_cast<float *>(ent) : zr;
                __syncwarp();
                // after the butterfly every sub-group holds the full sums: sub-group sg finishes the
                // features q = sg, sg + PP, ... of its lanes, so the epilogue arithmetic is spread over the warp
#pragma unroll
                for (int t = 0; t < (VW + PP - 1) / PP; ++t) {
                    const int qsel = t * PP + sg;
                    float gsel[D], ssel = 0.f, bsel = 0.f;
#pragma unroll
                    for (int d = 0; d < D; ++d) gsel[d] = 0.f;
#pragma unroll
                    for (int q = 0; q < VW; ++q) {
                        if (q == qsel) {
                            ssel = si[q];
                            bsel = blur[q];
#pragma unroll
                            for (int d = 0; d < D; ++d) gsel[d] = gr[q * D + d];
                        }
                    }
                    float v[D];
#pragma unroll
                    for (int d = 0; d < D; ++d) {
                        float acc = 0.f;
#pragma unroll
                        for (int kk = 0; kk < D; ++kk) acc = fmaf(gsel[kk], L[kk * D + d], acc);
                        v[d] = acc;
                    }
                    const int f = f0 + qsel;
                    if (fvalid && qsel < VW && f < C) {
                        zs[f] = ssel;
                        zs[C + f] = bsel;
                        if (a.vgrad) {
#pragma unroll
                            for (int d = 0; d < D; ++d) a.vgrad[(i * C + f) * D + d] = v[d];
                        }
#pragma unroll
                        for (int d = 0; d < D; ++d) v[d] *= a.coef;
                        if (a.log_norm_grad) log_normalize<D>(v);
#pragma unroll
                        for (int d = 0; d < D; ++d) zs[2 * C + f * D + d] = v[d];
                    }
                }
                if (a.rho_grad_out) {
#pragma unroll
                    for (int d = 0; d < D; ++d) dgs[d] = g.c_g * subgroup_sum<32>(dgs[d]);
                }
                if (lane == 0) {
                    float w[D];
#pragma unroll
                    for (int d = 0; d < D; ++d) {
                        float dgd;
                        if (a.rho_grad_out) {
                            dgd = dgs[d];
                            a.rho_grad_out[i * D + d] = dgd;  // the backward pass reads it
                        } else {
                            dgd = __ldg(a.rho_grad + i * D + d);
                        }
                        w[d] = dgd * a.dg_scale;
                    }
                    if (a.log_norm_dg) log_normalize<D>(w);
#pragma unroll
                    for (int d = 0; d < D; ++d) zs[2 * C + C * D + d] = w[d];
                }
                if (staged) {
                    __syncwarp();
                    for (int c = lane; c < a.zstride; c += 32) zr[c] = zs[c];
                    __syncwarp();
                }
            }
        }
        if ((MASK & F_MOMENT) && !(MASK & F_PACK)) {
#pragma unroll
            for (int q = 0; q < D * (D + 1) / 2; ++q) mom[q] = g.c_g * subgroup_sum<32>(mom[q]);
            if (lane == 0 && a.moment) {
                float *o = a.moment + i * (D * D);
                if (D == 2) {
                    o[0] = mom[0]; o[1] = mom[1]; o[2] = mom[1]; o[3] = mom[2];
                } else {
                    o[0] = mom[0]; o[1] = mom[1]; o[2] = mom[2];
                    o[3] = mom[1]; o[4] = mom[3]; o[5] = mom[4];
                    o[6] = mom[2]; o[7] = mom[4]; o[8] = mom[5];
                }
            }
        }
    }
    }  // rows
    release_rows(a.tickets);
}

template <int D, bool PER, int LPP, int VW, int MASK, bool FULL>
__global__ void __launch_bounds__(bwd_warps(FULL) * 32, FULL ? kBwdFullCtas : 3)
feature_backward_kernel(FeatureBwdArgs a, Geom g) {
    constexpr int PP = 32 / LPP;
    constexpr int WB = bwd_warps(FULL);  // warps per CTA
    __shared__ int4 s_ranges[WB][kMaxRanges];
    __shared__ float4 s_geo[WB][kListPerWarp];  // r.x r.y r.z, index of j
    __shared__ float4 s_ker[WB][kListPerWarp];  // W, 6(h^2-q)^2, phi, psi
    __shared__ float s_vol[WB][kListPerWarp];   // v_j = m_j / rho_j
    extern __shared__ __align__(16) unsigned char s_dyn[];
    constexpr int S = kBwdStages;
    constexpr int NP = 2 + D;  // pieces per pair and lane: s_j, dL/dblur_j, D pieces of dL/dgrad_j

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sg = lane / LPP, sl = lane % LPP;
    int4 *rng = s_ranges[warp];
    float4 *geo = s_geo[warp];
    float4 *ker = s_ker[warp];
    float *vol = s_vol[warp];
    // lane-private staging ring: [stage][piece][lane]
    Piece<VW> *ring = reinterpret_cast<Piece<VW> *>(s_dyn) + (size_t)warp * S * NP * 32 + lane;
    const int C = a.C;

    // g.split warps share one row (its particles are dealt round-robin) when rows are scarce
    const int vrows = g.max_blocks * g.split;
    for (int vrow = next_row(a.tickets); vrow < vrows; vrow = next_row(a.tickets)) {
    const int row = vrow / g.split, part = vrow - row * g.split;
    const WorkItem it = load_item(a.block_info, a.bin_offsets, row);
    if (it.count <= 0) break;  // rows after the last work item are zero
    if (part >= it.count) continue;
    __syncwarp();
    const int nr = build_ranges<D>(g, a.bin_offsets, it, rng);

    for (int k = part; k < it.count; k += g.split) {
        const long long i = it.first + k;
        const Pos<D> pi = load_pos<D>(a.x, i);
        const float mi = a.mass ? __ldg(a.mass + i) : 1.0f;
        const float vi = mi / __ldg(a.rho + i);
        // lane-partial sums over this lane's features and pairs, reduced over the whole warp at the end
        float dxs[3] = {0.f, 0.f, 0.f}, dxg[3] = {0.f, 0.f, 0.f}, drs = 0.f, drg = 0.f;

        for (int fbase = 0; fbase < C; fbase += LPP * VW) {
            const int f0 = fbase + sl * VW;
            const bool fvalid = f0 < C;
            float si[VW], gbi[VW], ggi[VW * D], ds[VW], dsg[VW];
            float tsum[3] = {0.f, 0.f, 0.f};  // features-only pass: sum_j v_j K_j (identical in every lane)
#pragma unroll
            for (int q = 0; q < VW; ++q) { si[q] = 0.f; gbi[q] = 0.f; ds[q] = 0.f; dsg[q] = 0.f; }
#pragma unroll
            for (int q = 0; q < VW * D; ++q) ggi[q] = 0.f;
            if (fvalid) {
                if (FULL) load_feat<VW>(a.s + i * C + f0, si);
                if (FULL && (MASK & F_BLUR)) load_feat<VW>(a.g_blur + i * C + f0, gbi);
                if (FULL && (MASK & F_GRAD)) load_run<VW, VW * D>(a.g_grad + (i * C + f0) * D, ggi);
            }

            auto flush = [&](int n) {
                __syncwarp();
                auto fetch = [&](int e, int slot) {
                    if (e < n) {
                        const long long row = (long long)__float_as_int(geo[e].w) * C + f0;
                        Piece<VW> *dst = ring + slot * NP * 32;
                        if (FULL) async_copy<VW * 4>(dst, a.s + row);
                        if (MASK & F_BLUR) async_copy<VW * 4>(dst + 32, a.g_blur + row);
                        if (MASK & F_GRAD) {
#pragma unroll
                            for (int d = 0; d < D; ++d)
                                async_copy<VW * 4>(dst + (2 + d) * 32, a.g_grad + (row * D + d * VW));
                        }
                    }
                    async_commit();
                };
                if (kBwdRing && FULL && fvalid) {  // the rows of the first S pairs travel while stage 2 computes
#pragma unroll
                    for (int p = 0; p < S; ++p) fetch(sg + p * PP, p);
                }
                for (int e = lane; e < n; e += 32) {  // stage 2: pair scalars, one entry per lane
                    const float4 ge = geo[e];
                    const int j = __float_as_int(ge.w);
                    const float q = sq_norm_fast<D>(ge.x, ge.y, ge.z);
                    const float mj = a.mass ? __ldg(a.mass + j) : 1.0f;
                    const float t = fmaxf(g.h2 - q, 0.f);
                    float phi = 0.f, psi = 0.f;
                    if ((MASK & F_GRAD) && q > 0.f) {
                        float dist;
                        phi = spiky_phi(q, g.h, dist);
                        if (FULL) psi = spiky_psi(dist, g.h);
                    }
                    ker[e] = make_float4(t * t * t, 6.0f * t * t, phi, psi);
                    vol[e] = mj / __ldg(a.rho + j);
                }
                __syncwarp();
                if (fvalid) {
                    // stage 3: each sub-group drains every PP-th pair.  The neighbour's rows (s_j, dL/dblur_j,
                    // dL/dgrad_j) are loaded one pair ahead into a second register set (kBwdRing == false)
                    // or S pairs ahead with cp.async into this lane's shared-memory ring.
                    auto compute = [&](int e, const float (&sj)[VW], const float (&gbj)[VW], const float (&ggj)[VW * D]) {
                        const float4 e0 = geo[e];
                        const float4 e1 = ker[e];
                        const float vj = vol[e];
                        const float rv[3] = {e0.x, e0.y, e0.z};
                        if (MASK & F_BLUR) {
                            float A = 0.f, Bp = 0.f;
#pragma unroll
                            for (int q = 0; q < VW; ++q) {
                                ds[q] = fmaf(e1.x, gbj[q], ds[q]);
                                if (FULL) {
                                    A = fmaf(gbi[q], sj[q], A);
                                    Bp = fmaf(gbj[q], si[q], Bp);
                                }
                            }
                            if (FULL) {
                                const float t = e1.y * (vj * A + vi * Bp);
#pragma unroll
                                for (int d = 0; d < D; ++d) dxs[d] = fmaf(t, rv[d], dxs[d]);
                                drs = fmaf(e1.x, Bp, drs);
                            }
                        }
                        if ((MASK & F_GRAD) && !FULL) {
                            // ds_i[f] = -cg ( gG_i[f] . T + v_i sum_j K_j . gG_j[f] ),  T = sum_j v_j K_j
#pragma unroll
                            for (int d = 0; d < D; ++d) {
                                const float kd = e1.z * rv[d];
                                tsum[d] = fmaf(vj, kd, tsum[d]);
#pragma unroll
                                for (int q = 0; q < VW; ++q) dsg[q] = fmaf(kd, ggj[q * D + d], dsg[q]);
                            }
                        }
                        if ((MASK & F_GRAD) && FULL) {
                            float kvec[3];
#pragma unroll
                            for (int d = 0; d < D; ++d) kvec[d] = e1.z * rv[d];
                            float u[3] = {0.f, 0.f, 0.f};
#pragma unroll
                            for (int q = 0; q < VW; ++q) {
                                float hk = 0.f, gk = 0.f;
                                const float df = FULL ? si[q] - sj[q] : 0.f;
#pragma unroll
                                for (int d = 0; d < D; ++d) {
                                    const float hd = fmaf(vj, ggi[q * D + d], vi * ggj[q * D + d]);
                                    hk = fmaf(kvec[d], hd, hk);
                                    if (FULL) {
                                        u[d] = fmaf(df, hd, u[d]);
                                        gk = fmaf(ggj[q * D + d], kvec[d], gk);
                                    }
                                }
                                dsg[q] += hk;
                                if (FULL) drg = fmaf(df, gk, drg);
                            }
                            if (FULL) {
                                float ru = rv[0] * u[0] + rv[1] * u[1];
                                if (D == 3) ru = fmaf(rv[2], u[2], ru);
                                const float sc = e1.w * ru;
#pragma unroll
                                for (int d = 0; d < D; ++d) dxg[d] += e1.z * u[d] - sc * rv[d];
                            }
                        }
                    };
                    if (!(kBwdRing && FULL)) {  // the features-only pass has registers to spare

                        auto load = [&](int e, float (&sj)[VW], float (&gbj)[VW], float (&ggj)[VW * D]) {
                            const long long row = (long long)__float_as_int(geo[e].w) * C + f0;
                            if (FULL) load_feat<VW>(a.s + row, sj);
                            if (MASK & F_BLUR) load_feat<VW>(a.g_blur + row, gbj);
                            if (MASK & F_GRAD) load_run<VW, VW * D>(a.g_grad + row * D, ggj);
                        };
                        float sA[VW] = {}, bA[VW] = {}, gA[VW * D] = {}, sB[VW] = {}, bB[VW] = {}, gB[VW * D] = {};
                        int e = sg;
                        if (e < n) load(e, sA, bA, gA);
                        while (e < n) {
                            if (e + PP < n) load(e + PP, sB, bB, gB);
                            compute(e, sA, bA, gA);
                            e += PP;
                            if (e >= n) break;
                            if (e + PP < n) load(e + PP, sA, bA, gA);
                            compute(e, sB, bB, gB);
                            e += PP;
                        }
                    } else {
                        int slot = 0;
                        for (int e = sg; e < n; e += PP) {
                            async_wait<S - 1>();
                            const Piece<VW> *src = ring + slot * NP * 32;
                            float sj[VW] = {}, gbj[VW] = {}, ggj[VW * D] = {};
                            if (FULL) {
                                const Piece<VW> t = src[0];
#pragma unroll
                                for (int q = 0; q < VW; ++q) sj[q] = t.v[q];
                            }
                            if (MASK & F_BLUR) {
                                const Piece<VW> t = src[32];
#pragma unroll
                                for (int q = 0; q < VW; ++q) gbj[q] = t.v[q];
                            }
                            if (MASK & F_GRAD) {
#pragma unroll
                                for (int d = 0; d < D; ++d) {
                                    const Piece<VW> t = src[(2 + d) * 32];
#pragma unroll
                                    for (int q = 0; q < VW; ++q) ggj[d * VW + q] = t.v[q];
                                }
                            }
                            compute(e, sj, gbj, ggj);
                            // refill the slot only after its values were consumed by the arithmetic above
                            fetch(e + S * PP, slot);
                            slot = slot + 1 == S ? 0 : slot + 1;
                        }
                        async_wait<0>();
                    }
                }
                __syncwarp();
            };
            int listed = -1;
            if (a.pair_cache) listed = __ldg(a.pair_cache + i * a.pair_stride);
            if (listed >= 0 && listed <= kListPerWarp) {
                expand_pairs<D, PER>(g, a.x, pi, a.pair_cache + i * a.pair_stride + 1, listed, geo);
                flush(listed);
            } else if (listed > kListPerWarp) {
                // a list longer than the warp's pair slots goes through in pieces (the sums carry over); kept apart
                // from the common case above (a loop around it slows the sweeps that have few registers to spare)
                const int32_t *list = a.pair_cache + i * a.pair_stride + 1;
#pragma unroll 1
                for (int off = 0; off < listed; off += kListPerWarp) {
                    const int n = listed - off < kListPerWarp ? listed - off : kListPerWarp;
                    expand_pairs<D, PER>(g, a.x, pi, list + off, n, geo);
                    flush(n);
                }
            } else {
                collect_pairs<D, PER>(g, a.x, pi, rng, nr, geo, flush);
            }

            if (a.grad_s) {
                float out[VW];
                if (FULL) {
#pragma unroll
                    for (int q = 0; q < VW; ++q)
                        out[q] = across_subgroups<LPP>(g.c_s * vi * ds[q] - g.c_g * dsg[q]);
                } else {
                    // each sub-group saw every PP-th pair: combine, then add the i-side term once
#pragma unroll
                    for (int d = 0; d < D; ++d) tsum[d] = across_subgroups<LPP>(tsum[d]);
                    if (fvalid && (MASK & F_GRAD)) load_run<VW, VW * D>(a.g_grad + (i * C + f0) * D, ggi);
#pragma unroll
                    for (int q = 0; q < VW; ++q) {
                        float own = 0.f;
#pragma unroll
                        for (int d = 0; d < D; ++d) own = fmaf(ggi[q * D + d], tsum[d], own);
                        out[q] = across_subgroups<LPP>(vi * (g.c_s * ds[q] - g.c_g * dsg[q])) - g.c_g * own;
                    }
                }
                if (sg == 0 && fvalid) store_run<VW, VW>(a.grad_s + i * C + f0, out);
            }
        }

        if (FULL) {
            float out[3];
#pragma unroll
            for (int d = 0; d < D; ++d) out[d] = subgroup_sum<32>(g.c_s * dxs[d] + g.c_g * dxg[d]);
            const float dr = subgroup_sum<32>(g.c_g * drg - g.c_s * drs);
            if (lane == 0) {
                if (a.grad_x) {
                    if (D == 2) reinterpret_cast<float2 *>(a.grad_x)[i] = make_float2(out[0], out[1]);
                    else reinterpret_cast<float4 *>(a.grad_x)[i] = make_float4(out[0], out[1], out[2], 0.f);
                }
                if (a.grad_rho) a.grad_rho[i] = (vi * vi / mi) * dr;
            }
        }
    }
    }  // rows
    release_rows(a.tickets);
}

// ---------------------------------------------------------------------------
// Dispatch on the feature count: VW = 4 floats per lane when rows are 16-byte
// addressable, LPP lanes per particle = the smallest supported power of two
// that covers C / VW; wider rows loop over feature chunks.
// ---------------------------------------------------------------------------
inline bool feature_rows_vectorisable(int C, const void *p0, const void *p1, const void *p2, const void *p3,
                                      const void *p4) {
    uintptr_t bits = (uintptr_t)p0 | (uintptr_t)p1 | (uintptr_t)p2 | (uintptr_t)p3 | (uintptr_t)p4;
    return C % 4 == 0 && bits % 16 == 0;
}

template <int VW, typename Kernel>
int launch_feature_forward_mask(const Geom &g, Kernel kernel, const FeatureFwdArgs &a, cudaStream_t st) {
    const int threads = kWarpsPerCta * 32;
    const size_t dyn = 0;
    int ctas = 0;
    int rc = persistent_ctas(kernel, threads, dyn, &ctas);
    if (rc != NPA_OK) return rc;
    const int needed = (g.max_blocks * g.split + kWarpsPerCta - 1) / kWarpsPerCta;
    FeatureFwdArgs b = a;
    if ((rc = acquire_row_tickets(st, &b.tickets)) != NPA_OK) return rc;
    kernel<<<needed < ctas ? needed : ctas, threads, dyn, st>>>(b, g);
    return check_launch("feature_forward_kernel");
}

template <int D, bool PER, int LPP, int VW>
int launch_feature_forward_shape(const Geom &g, int mask, const FeatureFwdArgs &a, cudaStream_t st) {
    switch (mask) {
        case F_BLUR:
            return launch_feature_forward_mask<VW>(g, feature_forward_kernel<D, PER, LPP, VW, F_BLUR>, a, st);
        case F_GRAD:
            return launch_feature_forward_mask<VW>(g, feature_forward_kernel<D, PER, LPP, VW, F_GRAD>, a, st);
        case F_BLUR | F_GRAD:
            return launch_feature_forward_mask<VW>(g, feature_forward_kernel<D, PER, LPP, VW, F_BLUR | F_GRAD>, a, st);
        case F_BLUR | F_GRAD | F_MOMENT:
            return launch_feature_forward_mask<VW>(
                g, feature_forward_kernel<D, PER, LPP, VW, F_BLUR | F_GRAD | F_MOMENT>, a, st);
        case F_BLUR | F_GRAD | F_MOMENT | F_PACK:
            if (a.C > LPP * VW)
                return fail(NPA_ERR_UNSUPPORTED, "the packed perception sweep supports up to %d features here", LPP * VW);
            return launch_feature_forward_mask<VW>(
                g, feature_forward_kernel<D, PER, LPP, VW, F_BLUR | F_GRAD | F_MOMENT | F_PACK>, a, st);
        default: return fail(NPA_ERR_INVALID_ARGUMENT, "unsupported feature forward mask %d", mask);
    }
}

template <int D, bool PER>
int launch_feature_forward_geom(const Geom &g, int mask, const FeatureFwdArgs &a, cudaStream_t st) {
    {
        bool taken = false;  // the cell-tile streaming engine takes the shapes it covers
        const int rc = launch_feature_tile_forward<D, PER>(g, mask, a, st, &taken);
        if (rc != NPA_OK || taken) return rc;
    }
    if (feature_rows_vectorisable(a.C, a.s, a.blur, a.grad, nullptr, nullptr)) {
        const int need = a.C / 4;
        if (need <= 4) return launch_feature_forward_shape<D, PER, 4, 4>(g, mask, a, st);
        if (need <= 8) return launch_feature_forward_shape<D, PER, 8, 4>(g, mask, a, st);
        if (need <= 16) return launch_feature_forward_shape<D, PER, 16, 4>(g, mask, a, st);
        return launch_feature_forward_shape<D, PER, 32, 4>(g, mask, a, st);
    }
    if (a.C <= 8) return launch_feature_forward_shape<D, PER, 8, 1>(g, mask, a, st);
    return launch_feature_forward_shape<D, PER, 32, 1>(g, mask, a, st);
}

template <int D, int VW, bool FULL, typename Kernel>
int launch_feature_backward_mask(const Geom &g, Kernel kernel, const FeatureBwdArgs &a, cudaStream_t st) {
    constexpr int WB = bwd_warps(FULL);
    const int threads = WB * 32;
    const size_t dyn = (kBwdRing && FULL) ? (size_t)WB * kBwdStages * (2 + D) * 32 * sizeof(Piece<VW>) : 0;
    int ctas = 0;
    int rc = persistent_ctas(kernel, threads, dyn, &ctas);
    if (rc != NPA_OK) return rc;
    const int needed = (g.max_blocks * g.split + WB - 1) / WB;
    FeatureBwdArgs b = a;
    if ((rc = acquire_row_tickets(st, &b.tickets)) != NPA_OK) return rc;
    kernel<<<needed < ctas ? needed : ctas, threads, dyn, st>>>(b, g);
    return check_launch("feature_backward_kernel");
}

template <int D, bool PER, int LPP, int VW, bool FULL>
int launch_feature_backward_shape(const Geom &g, int mask, const FeatureBwdArgs &a, cudaStream_t st) {
    switch (mask) {
        case F_BLUR:
            return launch_feature_backward_mask<D, VW, FULL>(g, feature_backward_kernel<D, PER, LPP, VW, F_BLUR, FULL>, a, st);
        case F_GRAD:
            return launch_feature_backward_mask<D, VW, FULL>(g, feature_backward_kernel<D, PER, LPP, VW, F_GRAD, FULL>, a, st);
        case F_BLUR | F_GRAD:
            return launch_feature_backward_mask<D, VW, FULL>(g, feature_backward_kernel<D, PER, LPP, VW, F_BLUR | F_GRAD, FULL>, a, st);
        default: return fail(NPA_ERR_INVALID_ARGUMENT, "unsupported feature backward mask %d", mask);
    }
}

template <int D, bool PER, bool FULL>
int launch_feature_backward_geom(const Geom &g, int mask, const FeatureBwdArgs &a, cudaStream_t st) {
    {
        bool taken = false;  // the cell-tile streaming engine takes the shapes it covers
        const int rc = launch_feature_tile_backward<D, PER, FULL>(g, mask, a, st, &taken);
        if (rc != NPA_OK || taken) return rc;
    }
    if (feature_rows_vectorisable(a.C, a.s, a.g_blur, a.g_grad, a.grad_s, nullptr)) {
        const int need = a.C / 4;
        if (need <= 4) return launch_feature_backward_shape<D, PER, 4, 4, FULL>(g, mask, a, st);
        if (need <= 8) return launch_feature_backward_shape<D, PER, 8, 4, FULL>(g, mask, a, st);
        if (need <= 16) return launch_feature_backward_shape<D, PER, 16, 4, FULL>(g, mask, a, st);
        return launch_feature_backward_shape<D, PER, 32, 4, FULL>(g, mask, a, st);
    }
    if (a.C <= 8) return launch_feature_backward_shape<D, PER, 8, 1, FULL>(g, mask, a, st);
    return launch_feature_backward_shape<D, PER, 32, 1, FULL>(g, mask, a, st);
}

}  // namespace npa
