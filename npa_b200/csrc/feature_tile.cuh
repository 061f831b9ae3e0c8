// Blur + feature-gradient sweeps on the cell-tile streaming engine (tile_stream.cuh): the rows of a
// tile's neighbour cells are staged in shared memory by bulk copies and every consumer warp reads
// positions, densities and feature rows of the neighbours from there.
//
// Same operators, masks and formulas as the gather kernels of feature_kernels.cuh (which remain the
// path for shapes this engine does not take: Morton order, C % 4 != 0, C > 128, unaligned tensors):
// forward blur / gradient (+ moment matrix, + packed perception epilogue) replacing
// sphops/sph_cuda.cu:1561-1716, and their gather backward replacing :1185-1327.
//
// Work split: one consumer warp owns one particle of the tile at a time and keeps it for every chunk
// of the tile.  Per (particle, chunk) it (1) tests the staged positions 32 at a time and
// ballot-compacts the accepted displacements into its pair list, (2) turns list entries into pair
// scalars, one entry per lane, (3) drains the pairs with 32 / LPP sub-groups of LPP lanes (4 features
// per lane, 128-bit shared-memory loads).  A tile that fits one chunk finishes in registers; a longer
// one parks its partial sums in a per-particle accumulator slot of shared memory between chunks.
#pragma once
#include "feature_kernels.cuh"
#include "tile_stream.cuh"

namespace npa {

struct TileViews {
    const float *xs, *rho, *mass, *s, *gb, *gg;
};

__device__ inline TileViews tile_views(const unsigned char *stage, const TileLayout &L) {
    TileViews v;
    v.xs = reinterpret_cast<const float *>(stage + L.off_x);
    v.rho = reinterpret_cast<const float *>(stage + L.off_rho);
    v.mass = reinterpret_cast<const float *>(stage + L.off_mass);
    v.s = reinterpret_cast<const float *>(stage + L.off_s);
    v.gb = reinterpret_cast<const float *>(stage + L.off_gb);
    v.gg = reinterpret_cast<const float *>(stage + L.off_gg);
    return v;
}

template <int D>
__device__ inline Pos<D> staged_pos(const float *xs, int slot) {
    Pos<D> p;
    if (D == 2) {
        const float2 v = reinterpret_cast<const float2 *>(xs)[slot];
        p.x = v.x; p.y = v.y; p.z = 0.f;
    } else {
        const float4 v = reinterpret_cast<const float4 *>(xs)[slot];
        p.x = v.x; p.y = v.y; p.z = v.z;
    }
    return p;
}

__device__ inline void lds4(const float *p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <int NF>
__device__ inline void lds_run(const float *p, float (&v)[NF]) {
#pragma unroll
    for (int k = 0; k < NF / 4; ++k) {
        const float4 t = reinterpret_cast<const float4 *>(p)[k];
        v[4 * k] = t.x; v[4 * k + 1] = t.y; v[4 * k + 2] = t.z; v[4 * k + 3] = t.w;
    }
}

// Stage 1 of one (particle, chunk): every staged candidate of every piece is tested, the accepted
// displacements and their slots are appended to `geo`; flush(n) drains the list when it could overflow
// and once at the end.
template <int D, bool PER, typename Flush>
__device__ inline void tile_collect_pairs(const Geom &g, const TileChunk *ch, const float *xs, const Pos<D> &pi,
                                          float4 *geo, Flush &&flush) {
    const int lane = threadIdx.x & 31;
    const int np = ch->npieces;
    int n = 0;
    for (int k = 0; k < np; ++k) {
        const int4 pa = *reinterpret_cast<const int4 *>(&ch->piece[k]);  // lo, hi, lo4, slot
        const int code = ch->piece[k].code;
        const Origin<D, PER> org = make_origin<D, PER>(g, pi.x, pi.y, pi.z, code);
        for (int base = pa.x; base < pa.y; base += 32) {
            const int j = base + lane;
            const int slot = pa.w + (j - pa.z);
            float rx = 0.f, ry = 0.f, rz = 0.f;
            bool acc = false;
            if (j < pa.y) {
                const Pos<D> pj = staged_pos<D>(xs, slot);
                const float q = displacement<D, PER, false>(g, org, pj.x, pj.y, pj.z, rx, ry, rz);
                acc = q < g.h2;
            }
            const unsigned bal = __ballot_sync(kFull, acc);
            if (acc) geo[n + __popc(bal & ((1u << lane) - 1u))] = make_float4(rx, ry, rz, __int_as_float(slot));
            n += __popc(bal);
            if (n + 32 > kTileList) {
                flush(n);
                n = 0;
            }
        }
    }
    flush(n);
}

__device__ inline void tile_setup_barriers(const TileLayout &L, unsigned char *smem, int consumer_warps) {
    if (threadIdx.x == 0) {
        uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.off_bars);
        uint64_t *empty = full + L.stages;
        for (int s = 0; s < L.stages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, consumer_warps);
        }
        mbar_fence_init();
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------
// Forward: blur and gradient (+ moment matrix, + packed perception epilogue)
// ---------------------------------------------------------------------------------------------
template <int D, bool PER, int LPP, int MASK, int W>
__global__ void __launch_bounds__((W + 1) * 32, 1)
feature_tile_forward_kernel(FeatureFwdArgs a, Geom g, TileLayout L, unsigned int *status) {
    constexpr int VW = 4;
    constexpr int PP = 32 / LPP;
    constexpr int NM = D * (D + 1) / 2;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int4 s_rng[kMaxRanges];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    tile_setup_barriers(L, smem, W);

    if (warp == W) {
        TileSources src = {a.x, a.rho, a.mass, a.s, nullptr, nullptr, D == 2 ? 2 : 4, a.C, a.C * D};
        tile_producer<D>(g, L, src, a.bin_offsets, a.block_info, a.tickets, status, smem, s_rng);
    } else {
        uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.off_bars);
        uint64_t *empty = full + L.stages;
        const TileChunk *chunks = reinterpret_cast<const TileChunk *>(smem + L.off_chunks);
        float4 *geo = reinterpret_cast<float4 *>(smem + L.off_lists + (size_t)warp * L.list_bytes);
        float4 *ent = geo + kTileList;  // v_j K.x, v_j K.y, v_j K.z, v_j W
        const int C = a.C;
        const int sg = lane / LPP, sl = lane % LPP;
        const int f0 = sl * VW;
        const bool fvalid = f0 < C;

        for (unsigned c = 0;; ++c) {
            const int st = (int)(c % (unsigned)L.stages);
            if (!mbar_wait(full + st, (c / (unsigned)L.stages) & 1u)) {
                if (lane == 0) atomicExch(status, (unsigned)TILE_STATUS_FULL_TIMEOUT);
                break;
            }
            const TileChunk *ch = chunks + st;
            const int flags = ch->flags;
            if (flags & TILE_END) break;
            const TileViews v = tile_views(smem + (size_t)st * L.stage_bytes, L);
            const int first = ch->first, count = ch->count;
            const bool whole = (flags & (TILE_FIRST | TILE_LAST)) == (TILE_FIRST | TILE_LAST);
            int pfirst = warp - ch->rot;  // particles p = pfirst, pfirst + W, ... are this warp's
            if (pfirst < 0) pfirst += W;

            for (int p = pfirst, aslot = warp; p < count; p += W, aslot += W) {  // aslot: this warp's accumulator slot
                const long long i = first + p;
                const Pos<D> pi = load_pos<D>(a.x, i);
                float si[VW], blur[VW], gr[VW * D], mom[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int q = 0; q < VW; ++q) { si[q] = 0.f; blur[q] = 0.f; }
#pragma unroll
                for (int q = 0; q < VW * D; ++q) gr[q] = 0.f;
                if (fvalid && (MASK & F_GRAD)) load_feat<VW>(a.s + i * C + f0, si);

                auto flush = [&](int n) {
                    __syncwarp();
                    for (int e = lane; e < n; e += 32) {  // stage 2: pair scalars, one entry per lane
                        const float4 ge = geo[e];
                        const int slot = __float_as_int(ge.w);
                        const float q = sq_norm_fast<D>(ge.x, ge.y, ge.z);
                        const float mj = a.mass ? v.mass[slot] : 1.0f;
                        const float vj = mj / v.rho[slot];
                        float wv = 0.f, kv = 0.f;
                        if (MASK & F_BLUR) {
                            const float t = fmaxf(g.h2 - q, 0.f);
                            wv = vj * (t * t * t);
                        }
                        if ((MASK & (F_GRAD | F_MOMENT)) && q > 0.f) {
                            float dist;
                            kv = vj * spiky_phi(q, g.h, dist);
                        }
                        if (MASK & F_MOMENT) {
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
                    __syncwarp();
                    if (fvalid) {
                        // stage 3: each sub-group drains every PP-th pair from shared memory; the scalars and the
                        // feature row of the next pair are loaded before the current pair is accumulated
                        int e = sg;
                        float4 en = make_float4(0.f, 0.f, 0.f, 0.f);
                        float sj[VW] = {0.f, 0.f, 0.f, 0.f};
                        if (e < n) {
                            en = ent[e];
                            lds4(v.s + (size_t)__float_as_int(geo[e].w) * C + f0, sj);
                        }
                        while (e < n) {
                            const int e2 = e + PP;
                            float4 en2 = en;
                            float sj2[VW] = {0.f, 0.f, 0.f, 0.f};
                            if (e2 < n) {
                                en2 = ent[e2];
                                lds4(v.s + (size_t)__float_as_int(geo[e2].w) * C + f0, sj2);
                            }
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
                            en = en2;
#pragma unroll
                            for (int q = 0; q < VW; ++q) sj[q] = sj2[q];
                            e = e2;
                        }
                    }
                    __syncwarp();
                };
                tile_collect_pairs<D, PER>(g, ch, v.xs, pi, geo, flush);

                // sums of this chunk: over the sub-groups (features) and over the lanes (moment)
                if (MASK & F_BLUR) {
#pragma unroll
                    for (int q = 0; q < VW; ++q) blur[q] = across_subgroups<LPP>(blur[q]);
                }
                if (MASK & F_GRAD) {
#pragma unroll
                    for (int q = 0; q < VW * D; ++q) gr[q] = across_subgroups<LPP>(gr[q]);
                }
                if (MASK & F_MOMENT) {
#pragma unroll
                    for (int q = 0; q < NM; ++q) mom[q] = subgroup_sum<32>(mom[q]);
                }
                if (!whole) {
                    // the tile spans several chunks: running sums live in this particle's accumulator slot
                    float *acc = reinterpret_cast<float *>(smem + L.off_acc + (size_t)aslot * L.acc_bytes);
                    float *acc_b = acc, *acc_g = acc + C, *acc_m = acc + C + C * D;
                    if (!(flags & TILE_FIRST)) {
                        if (fvalid) {
                            float t[VW], u[VW * D];
                            if (MASK & F_BLUR) {
                                lds4(acc_b + f0, t);
#pragma unroll
                                for (int q = 0; q < VW; ++q) blur[q] += t[q];
                            }
                            if (MASK & F_GRAD) {
                                lds_run<VW * D>(acc_g + f0 * D, u);
#pragma unroll
                                for (int q = 0; q < VW * D; ++q) gr[q] += u[q];
                            }
                        }
                        if (MASK & F_MOMENT) {
#pragma unroll
                            for (int q = 0; q < NM; ++q) mom[q] += acc_m[q];
                        }
                    }
                    __syncwarp();
                    if (!(flags & TILE_LAST)) {
                        if (sg == 0 && fvalid) {
                            if (MASK & F_BLUR) store_run<VW, VW>(acc_b + f0, blur);
                            if (MASK & F_GRAD) store_run<VW, VW * D>(acc_g + f0 * D, gr);
                        }
                        if ((MASK & F_MOMENT) && lane == 0) {
#pragma unroll
                            for (int q = 0; q < NM; ++q) acc_m[q] = mom[q];
                        }
                        __syncwarp();
                    }
                }
                if (!(flags & TILE_LAST)) continue;

                // ---- the particle is complete: scale and write ------------------------------
                if (MASK & F_BLUR) {
#pragma unroll
                    for (int q = 0; q < VW; ++q) blur[q] *= g.c_s;
                }
                if (MASK & F_GRAD) {
#pragma unroll
                    for (int q = 0; q < VW * D; ++q) gr[q] *= g.c_g;
                }
                if (MASK & F_MOMENT) {
#pragma unroll
                    for (int q = 0; q < NM; ++q) mom[q] *= g.c_g;
                }
                if (sg == 0 && fvalid) {
                    if ((MASK & F_BLUR) && a.blur) store_run<VW, VW>(a.blur + i * C + f0, blur);
                    if ((MASK & F_GRAD) && a.grad) store_run<VW, VW * D>(a.grad + (i * C + f0) * D, gr);
                }
                if ((MASK & F_MOMENT) && !(MASK & F_PACK) && lane == 0 && a.moment) {
                    float *o = a.moment + i * (D * D);
                    if (D == 2) {
                        o[0] = mom[0]; o[1] = mom[1]; o[2] = mom[1]; o[3] = mom[2];
                    } else {
                        o[0] = mom[0]; o[1] = mom[1]; o[2] = mom[2];
                        o[3] = mom[1]; o[4] = mom[3]; o[5] = mom[4];
                        o[6] = mom[2]; o[7] = mom[4]; o[8] = mom[5];
                    }
                }
                if (MASK & F_PACK) {
                    // perception epilogue: moment matrix -> safe inverse -> corrected gradient -> scaling and
                    // log-normalisation -> packed row, assembled in the (idle) pair lists and written coalesced
                    float Linv[D * D];
                    safe_inverse_sym<D>(mom, a.inv_tol, Linv);
                    float *zr = a.z + i * a.zstride;
                    const bool staged = a.zstride <= 2 * kTileList * 4;
                    float *zs = staged ? reinterpret_cast<float *>(geo) : zr;
                    __syncwarp();
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
                        float w[D];
#pragma unroll
                        for (int d = 0; d < D; ++d) {
                            float acc = 0.f;
#pragma unroll
                            for (int kk = 0; kk < D; ++kk) acc = fmaf(gsel[kk], Linv[kk * D + d], acc);
                            w[d] = acc;
                        }
                        const int f = f0 + qsel;
                        if (fvalid && qsel < VW && f < C) {
                            zs[f] = ssel;
                            zs[C + f] = bsel;
                            if (a.vgrad) {
#pragma unroll
                                for (int d = 0; d < D; ++d) a.vgrad[(i * C + f) * D + d] = w[d];
                            }
#pragma unroll
                            for (int d = 0; d < D; ++d) w[d] *= a.coef;
                            if (a.log_norm_grad) log_normalize<D>(w);
#pragma unroll
                            for (int d = 0; d < D; ++d) zs[2 * C + f * D + d] = w[d];
                        }
                    }
                    if (lane == 0) {
                        float w[D];
#pragma unroll
                        for (int d = 0; d < D; ++d) w[d] = __ldg(a.rho_grad + i * D + d) * a.dg_scale;
                        if (a.log_norm_dg) log_normalize<D>(w);
#pragma unroll
                        for (int d = 0; d < D; ++d) zs[2 * C + C * D + d] = w[d];
                    }
                    if (staged) {
                        __syncwarp();
                        for (int cc = lane; cc < a.zstride; cc += 32) zr[cc] = zs[cc];
                        __syncwarp();
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + st);  // this warp is done with the stage
        }
    }
    release_rows(a.tickets);
}

// ---------------------------------------------------------------------------------------------
// Backward of blur + gradient as a gather: full (dx, ds, drho) or with respect to the features only.
//
// With r = x_j - x_i, W' = (c_s / c_g) (h^2 - q)^3, E' = (c_s / c_g) 6 (h^2 - q)^2, K = phi r,
// J = phi I - psi r r^T, v = m / rho, df = s_i - s_j, and per pair the feature sums
//   A = gB_i . s_j,  B = gB_j . s_i,  pu_d = sum_f df gG_i[f,d],  qu_d = sum_f df gG_j[f,d]:
//   ds_i[f]  = c_g ( v_i sum_j (W' gB_j[f] - K . gG_j[f,:])  -  gG_i[f,:] . T ),  T = sum_j v_j K
//   dx_i     = c_g sum_j ( E' (v_j A + v_i B) r + J (v_j pu + v_i qu) )
//   drho_i   = c_g v_i^2 / m_i sum_j ( K . qu - W' B )
// (the formulas of the gather kernels with the i-side terms factored out of the pair loop; every
// feature sum stays a lane-partial over this lane's four features until the particle is complete).
// ---------------------------------------------------------------------------------------------
template <int D, bool PER, int LPP, int MASK, bool FULL, int W>
__global__ void __launch_bounds__((W + 1) * 32, 1)
feature_tile_backward_kernel(FeatureBwdArgs a, Geom g, TileLayout L, unsigned int *status) {
    constexpr int VW = 4;
    constexpr int PP = 32 / LPP;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int4 s_rng[kMaxRanges];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    tile_setup_barriers(L, smem, W);

    if (warp == W) {
        TileSources src = {a.x, a.rho, a.mass, FULL ? a.s : nullptr, (MASK & F_BLUR) ? a.g_blur : nullptr,
                           (MASK & F_GRAD) ? a.g_grad : nullptr, D == 2 ? 2 : 4, a.C, a.C * D};
        tile_producer<D>(g, L, src, a.bin_offsets, a.block_info, a.tickets, status, smem, s_rng);
    } else {
        uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.off_bars);
        uint64_t *empty = full + L.stages;
        const TileChunk *chunks = reinterpret_cast<const TileChunk *>(smem + L.off_chunks);
        float4 *geo = reinterpret_cast<float4 *>(smem + L.off_lists + (size_t)warp * L.list_bytes);  // r, slot
        float4 *ker = geo + kTileList;                          // W', E', phi, psi
        float *vol = reinterpret_cast<float *>(ker + kTileList);  // v_j
        const int C = a.C;
        const int sg = lane / LPP, sl = lane % LPP;
        const int f0 = sl * VW;
        const bool fvalid = f0 < C;
        const float ratio = g.c_s / g.c_g;

        for (unsigned c = 0;; ++c) {
            const int st = (int)(c % (unsigned)L.stages);
            if (!mbar_wait(full + st, (c / (unsigned)L.stages) & 1u)) {
                if (lane == 0) atomicExch(status, (unsigned)TILE_STATUS_FULL_TIMEOUT);
                break;
            }
            const TileChunk *ch = chunks + st;
            const int flags = ch->flags;
            if (flags & TILE_END) break;
            const TileViews v = tile_views(smem + (size_t)st * L.stage_bytes, L);
            const int first = ch->first, count = ch->count;
            const bool whole = (flags & (TILE_FIRST | TILE_LAST)) == (TILE_FIRST | TILE_LAST);
            int pfirst = warp - ch->rot;  // particles p = pfirst, pfirst + W, ... are this warp's
            if (pfirst < 0) pfirst += W;

            for (int p = pfirst, aslot = warp; p < count; p += W, aslot += W) {  // aslot: this warp's accumulator slot
                const long long i = first + p;
                const Pos<D> pi = load_pos<D>(a.x, i);
                const float mi = a.mass ? __ldg(a.mass + i) : 1.0f;
                const float vi = mi / __ldg(a.rho + i);
                float si[VW], gbi[VW], ggi[VW * D], ds[VW];
                float dx[3] = {0.f, 0.f, 0.f}, dr = 0.f, tsum[3] = {0.f, 0.f, 0.f};
#pragma unroll
                for (int q = 0; q < VW; ++q) { si[q] = 0.f; gbi[q] = 0.f; ds[q] = 0.f; }
#pragma unroll
                for (int q = 0; q < VW * D; ++q) ggi[q] = 0.f;
                if (FULL && fvalid) {
                    load_feat<VW>(a.s + i * C + f0, si);
                    if (MASK & F_BLUR) load_feat<VW>(a.g_blur + i * C + f0, gbi);
                    if (MASK & F_GRAD) load_run<VW, VW * D>(a.g_grad + (i * C + f0) * D, ggi);
                }

                auto flush = [&](int n) {
                    __syncwarp();
                    for (int e = lane; e < n; e += 32) {  // stage 2: pair scalars, one entry per lane
                        const float4 ge = geo[e];
                        const int slot = __float_as_int(ge.w);
                        const float q = sq_norm_fast<D>(ge.x, ge.y, ge.z);
                        const float mj = a.mass ? v.mass[slot] : 1.0f;
                        const float t = fmaxf(g.h2 - q, 0.f);
                        float phi = 0.f, psi = 0.f;
                        if ((MASK & F_GRAD) && q > 0.f) {
                            float dist;
                            phi = spiky_phi(q, g.h, dist);
                            if (FULL) psi = spiky_psi(dist, g.h);
                        }
                        const float t2 = ratio * t * t;
                        ker[e] = make_float4(t2 * t, 6.0f * t2, phi, psi);
                        vol[e] = mj / v.rho[slot];
                    }
                    __syncwarp();
                    if (fvalid) {
                        // stage 3: each sub-group drains every PP-th pair from shared memory; the scalars and the
                        // rows of the next pair are loaded before the current pair is accumulated
                        auto fetch = [&](int e, float4 &e0, float4 &e1, float &vj, float (&sj)[VW], float (&gbj)[VW],
                                         float (&ggj)[VW * D]) {
                            e0 = geo[e];
                            e1 = ker[e];
                            vj = vol[e];
                            const size_t row = (size_t)__float_as_int(e0.w) * C + f0;
                            if (FULL) lds4(v.s + row, sj);
                            if (MASK & F_BLUR) lds4(v.gb + row, gbj);
                            if (MASK & F_GRAD) lds_run<VW * D>(v.gg + row * D, ggj);
                        };
                        int e = sg;
                        float4 e0 = make_float4(0.f, 0.f, 0.f, 0.f), e1 = e0;
                        float vj = 0.f, sj[VW] = {0.f, 0.f, 0.f, 0.f}, gbj[VW] = {0.f, 0.f, 0.f, 0.f}, ggj[VW * D];
#pragma unroll
                        for (int q = 0; q < VW * D; ++q) ggj[q] = 0.f;
                        if (e < n) fetch(e, e0, e1, vj, sj, gbj, ggj);
                        while (e < n) {
                            const int e2 = e + PP;
                            float4 n0 = e0, n1 = e1;
                            float nvj = vj, nsj[VW] = {0.f, 0.f, 0.f, 0.f}, ngbj[VW] = {0.f, 0.f, 0.f, 0.f}, nggj[VW * D];
#pragma unroll
                            for (int q = 0; q < VW * D; ++q) nggj[q] = 0.f;
                            if (e2 < n) fetch(e2, n0, n1, nvj, nsj, ngbj, nggj);

                            const float rv[3] = {e0.x, e0.y, e0.z};
                            float kv[3];
#pragma unroll
                            for (int d = 0; d < 3; ++d) kv[d] = e1.z * rv[d];
                            float A = 0.f, Bp = 0.f, pu[3] = {0.f, 0.f, 0.f}, qu[3] = {0.f, 0.f, 0.f};
#pragma unroll
                            for (int q = 0; q < VW; ++q) {
                                if (MASK & F_BLUR) {
                                    ds[q] = fmaf(e1.x, gbj[q], ds[q]);
                                    if (FULL) {
                                        A = fmaf(gbi[q], sj[q], A);
                                        Bp = fmaf(gbj[q], si[q], Bp);
                                    }
                                }
                                if (MASK & F_GRAD) {
                                    const float df = FULL ? si[q] - sj[q] : 0.f;
#pragma unroll
                                    for (int d = 0; d < D; ++d) {
                                        ds[q] = fmaf(-kv[d], ggj[q * D + d], ds[q]);
                                        if (FULL) {
                                            pu[d] = fmaf(df, ggi[q * D + d], pu[d]);
                                            qu[d] = fmaf(df, ggj[q * D + d], qu[d]);
                                        }
                                    }
                                }
                            }
                            if (MASK & F_GRAD) {
#pragma unroll
                                for (int d = 0; d < D; ++d) tsum[d] = fmaf(vj, kv[d], tsum[d]);
                            }
                            if (FULL) {
                                float w = 0.f;
                                if (MASK & F_BLUR) {
                                    w = e1.y * fmaf(vj, A, vi * Bp);
                                    dr = fmaf(-e1.x, Bp, dr);
                                }
                                if (MASK & F_GRAD) {
                                    float u[3] = {0.f, 0.f, 0.f};
#pragma unroll
                                    for (int d = 0; d < D; ++d) u[d] = fmaf(vj, pu[d], vi * qu[d]);
                                    float ru = rv[0] * u[0];
                                    ru = fmaf(rv[1], u[1], ru);
                                    if (D == 3) ru = fmaf(rv[2], u[2], ru);
                                    w = fmaf(-e1.w, ru, w);
#pragma unroll
                                    for (int d = 0; d < D; ++d) {
                                        dx[d] = fmaf(e1.z, u[d], dx[d]);
                                        dr = fmaf(kv[d], qu[d], dr);
                                    }
                                }
#pragma unroll
                                for (int d = 0; d < D; ++d) dx[d] = fmaf(w, rv[d], dx[d]);
                            }
                            e0 = n0; e1 = n1; vj = nvj;
#pragma unroll
                            for (int q = 0; q < VW; ++q) { sj[q] = nsj[q]; gbj[q] = ngbj[q]; }
#pragma unroll
                            for (int q = 0; q < VW * D; ++q) ggj[q] = nggj[q];
                            e = e2;
                        }
                    }
                    __syncwarp();
                };
                tile_collect_pairs<D, PER>(g, ch, v.xs, pi, geo, flush);

                if (!whole) {
                    // lane-partial sums of this chunk join the particle's accumulator slot (no reduction
                    // until the particle is complete): [32 lanes x (dx, dr)] [PP x C of ds] [PP x 4 of T]
                    unsigned char *acc = smem + L.off_acc + (size_t)aslot * L.acc_bytes;
                    float4 *acc_x = reinterpret_cast<float4 *>(acc);
                    float *acc_s = reinterpret_cast<float *>(acc + (FULL ? 512 : 0));
                    float4 *acc_t = reinterpret_cast<float4 *>(acc_s + PP * C);
                    if (!(flags & TILE_FIRST)) {
                        if (FULL) {
                            const float4 t = acc_x[lane];
                            dx[0] += t.x; dx[1] += t.y; dx[2] += t.z; dr += t.w;
                        }
                        if (fvalid) {
                            float t[VW];
                            lds4(acc_s + sg * C + f0, t);
#pragma unroll
                            for (int q = 0; q < VW; ++q) ds[q] += t[q];
                        }
                        if (MASK & F_GRAD) {
                            const float4 t = acc_t[sg];
                            tsum[0] += t.x; tsum[1] += t.y; tsum[2] += t.z;
                        }
                    }
                    if (!(flags & TILE_LAST)) {
                        __syncwarp();
                        if (FULL) acc_x[lane] = make_float4(dx[0], dx[1], dx[2], dr);
                        if (fvalid) store_run<VW, VW>(acc_s + sg * C + f0, ds);
                        if ((MASK & F_GRAD) && sl == 0) acc_t[sg] = make_float4(tsum[0], tsum[1], tsum[2], 0.f);
                        __syncwarp();
                    }
                }
                if (!(flags & TILE_LAST)) continue;

                // ---- the particle is complete: reduce and write -----------------------------
                if (a.grad_s) {
                    float out[VW];
                    if (MASK & F_GRAD) {
#pragma unroll
                        for (int d = 0; d < D; ++d) tsum[d] = across_subgroups<LPP>(tsum[d]);
                        if (!FULL && fvalid) load_run<VW, VW * D>(a.g_grad + (i * C + f0) * D, ggi);
                    }
#pragma unroll
                    for (int q = 0; q < VW; ++q) {
                        float own = 0.f;
                        if (MASK & F_GRAD) {
#pragma unroll
                            for (int d = 0; d < D; ++d) own = fmaf(ggi[q * D + d], tsum[d], own);
                        }
                        out[q] = g.c_g * (vi * across_subgroups<LPP>(ds[q]) - own);
                    }
                    if (sg == 0 && fvalid) store_run<VW, VW>(a.grad_s + i * C + f0, out);
                }
                if (FULL) {
                    float o[3];
#pragma unroll
                    for (int d = 0; d < 3; ++d) o[d] = d < D ? g.c_g * subgroup_sum<32>(dx[d]) : 0.f;
                    const float drt = subgroup_sum<32>(dr);
                    if (lane == 0) {
                        if (a.grad_x) {
                            if (D == 2) reinterpret_cast<float2 *>(a.grad_x)[i] = make_float2(o[0], o[1]);
                            else reinterpret_cast<float4 *>(a.grad_x)[i] = make_float4(o[0], o[1], o[2], 0.f);
                        }
                        if (a.grad_rho) a.grad_rho[i] = g.c_g * (vi * vi / mi) * drt;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + st);  // this warp is done with the stage
        }
    }
    release_rows(a.tickets);
}

// ---------------------------------------------------------------------------------------------
// Launch: eligibility, shared-memory plan, dispatch on lanes per particle
// ---------------------------------------------------------------------------------------------

// Tuning of the tile sweeps (npa_tile_tuning in the C ABI); zero = choose automatically.
struct TileTuning {
    int rmax, tp, stages, enabled, warps, span;
};
constexpr int kTileWarpsDefault = 8;  // consumer warps per CTA (8 or 16); one more warp produces
TileTuning tile_tuning(bool backward);

inline bool tile_aligned16(const void *p) { return ((uintptr_t)p % 16) == 0; }

// True when the streaming engine can take this sweep.
inline bool tile_eligible(const Geom &g, int C, const void *x, const void *rho, const void *mass, const void *s,
                          const void *gb, const void *gg) {
    if (g.morton) return false;                       // cells of an x-row are not contiguous in Morton order
    if (C % 4 != 0 || C > 128) return false;          // feature rows must be 16-byte multiples, one chunk of lanes
    if (((long long)g.B * g.N) % 4 != 0) return false;  // rounded position / density ranges must stay inside the arrays
    return tile_aligned16(x) && tile_aligned16(rho) && tile_aligned16(mass) && tile_aligned16(s) &&
           tile_aligned16(gb) && tile_aligned16(gg);
}

template <int W, typename Kernel, typename Args>
int launch_tile_kernel(const Geom &g, Kernel kernel, const Args &a, const TileLayout &L, const char *what,
                       cudaStream_t st) {
    const int threads = (W + 1) * 32;
    int ctas = 0;
    int rc = persistent_ctas(kernel, threads, (size_t)L.total_bytes, &ctas);
    if (rc != NPA_OK) return rc;
    Args b = a;
    if ((rc = acquire_row_tickets(st, &b.tickets)) != NPA_OK) return rc;
    unsigned int *status = nullptr;
    if ((rc = tile_status_word(&status)) != NPA_OK) return rc;
    const int grid = g.max_blocks < ctas ? g.max_blocks : ctas;
    kernel<<<grid > 0 ? grid : 1, threads, (size_t)L.total_bytes, st>>>(b, g, L, status);
    return check_launch(what);
}

inline int tile_lanes_per_particle(int C) {
    const int need = C / 4;
    return need <= 4 ? 4 : need <= 8 ? 8 : need <= 16 ? 16 : 32;
}

template <int D, bool PER, int LPP, int W>
int launch_tile_forward_lpp(const Geom &g, int mask, const FeatureFwdArgs &a, const TileLayout &L, cudaStream_t st) {
    const char *what = "feature_tile_forward_kernel";
    switch (mask) {
        case F_BLUR | F_GRAD:
            return launch_tile_kernel<W>(g, feature_tile_forward_kernel<D, PER, LPP, F_BLUR | F_GRAD, W>, a, L, what, st);
        case F_BLUR | F_GRAD | F_MOMENT:
            return launch_tile_kernel<W>(g, feature_tile_forward_kernel<D, PER, LPP, F_BLUR | F_GRAD | F_MOMENT, W>, a,
                                         L, what, st);
        case F_BLUR | F_GRAD | F_MOMENT | F_PACK:
            return launch_tile_kernel<W>(
                g, feature_tile_forward_kernel<D, PER, LPP, F_BLUR | F_GRAD | F_MOMENT | F_PACK, W>, a, L, what, st);
        default: return fail(NPA_ERR_INVALID_ARGUMENT, "unsupported tile forward mask %d", mask);
    }
}

template <int D, bool PER, int W>
int launch_tile_forward_warps(const Geom &g, int mask, const FeatureFwdArgs &a, const TileLayout &L, cudaStream_t st) {
    switch (tile_lanes_per_particle(a.C)) {
        case 4: return launch_tile_forward_lpp<D, PER, 4, W>(g, mask, a, L, st);
        case 8: return launch_tile_forward_lpp<D, PER, 8, W>(g, mask, a, L, st);
        case 16: return launch_tile_forward_lpp<D, PER, 16, W>(g, mask, a, L, st);
        default: return launch_tile_forward_lpp<D, PER, 32, W>(g, mask, a, L, st);
    }
}

// Runs the sweep on the streaming engine when it can (*taken = true); otherwise launches nothing
// and the caller falls back to the gather kernel.
template <int D, bool PER>
int launch_feature_tile_forward(const Geom &g, int mask, const FeatureFwdArgs &a, cudaStream_t st, bool *taken) {
    *taken = false;
    const TileTuning t = tile_tuning(false);
    if (!t.enabled) return NPA_OK;
    if ((mask & (F_BLUR | F_GRAD)) != (F_BLUR | F_GRAD)) return NPA_OK;  // single operators stay on the gather path
    if (a.pair_cache && !a.pair_cache_valid) return NPA_OK;              // asked to record the neighbour lists
    if (!tile_eligible(g, a.C, a.x, a.rho, a.mass, a.s, nullptr, nullptr)) return NPA_OK;
    const int C = a.C;
    const int warps = t.warps == 24 ? 24 : t.warps == 16 ? 16 : 8;
    TileLayout L;
    const int acc_bytes = ((C + C * D + 8) * 4 + 15) & ~15;
    if (!tile_make_layout(D == 2 ? 2 : 4, a.mass != nullptr, C, 0, 0, warps, 2 * kTileList * 16, acc_bytes,
                          t.rmax, t.tp, t.stages, t.span, false, &L))
        return NPA_OK;
    *taken = true;
    return warps == 24   ? launch_tile_forward_warps<D, PER, 24>(g, mask, a, L, st)
           : warps == 16 ? launch_tile_forward_warps<D, PER, 16>(g, mask, a, L, st)
                         : launch_tile_forward_warps<D, PER, 8>(g, mask, a, L, st);
}

template <int D, bool PER, bool FULL, int W>
int launch_tile_backward_warps(const Geom &g, const FeatureBwdArgs &a, const TileLayout &L, cudaStream_t st) {
    const char *what = "feature_tile_backward_kernel";
    constexpr int M = F_BLUR | F_GRAD;
    switch (tile_lanes_per_particle(a.C)) {
        case 4: return launch_tile_kernel<W>(g, feature_tile_backward_kernel<D, PER, 4, M, FULL, W>, a, L, what, st);
        case 8: return launch_tile_kernel<W>(g, feature_tile_backward_kernel<D, PER, 8, M, FULL, W>, a, L, what, st);
        case 16: return launch_tile_kernel<W>(g, feature_tile_backward_kernel<D, PER, 16, M, FULL, W>, a, L, what, st);
        default: return launch_tile_kernel<W>(g, feature_tile_backward_kernel<D, PER, 32, M, FULL, W>, a, L, what, st);
    }
}

template <int D, bool PER, bool FULL>
int launch_feature_tile_backward(const Geom &g, int mask, const FeatureBwdArgs &a, cudaStream_t st, bool *taken) {
    *taken = false;
    const TileTuning t = tile_tuning(true);
    if (!t.enabled) return NPA_OK;
    if (mask != (F_BLUR | F_GRAD)) return NPA_OK;  // single operators stay on the gather path
    if (!tile_eligible(g, a.C, a.x, a.rho, a.mass, a.s, a.g_blur, a.g_grad)) return NPA_OK;
    if (!tile_aligned16(a.grad_s) || (D == 3 && !tile_aligned16(a.grad_x))) return NPA_OK;
    const int C = a.C;
    const int pp = 32 / tile_lanes_per_particle(C);
    const int warps = t.warps == 16 ? 16 : 8;
    TileLayout L;
    const int acc_bytes = (FULL ? 512 : 0) + pp * C * 4 + pp * 16;
    if (!tile_make_layout(D == 2 ? 2 : 4, a.mass != nullptr, FULL ? C : 0, C, C * D, warps,
                          2 * kTileList * 16 + kTileList * 4, acc_bytes, t.rmax, t.tp, t.stages, t.span, true, &L))
        return NPA_OK;
    *taken = true;
    return warps == 16 ? launch_tile_backward_warps<D, PER, FULL, 16>(g, a, L, st)
                       : launch_tile_backward_warps<D, PER, FULL, 8>(g, a, L, st);
}

}  // namespace npa
