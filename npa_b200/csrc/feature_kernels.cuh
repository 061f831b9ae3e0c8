// Feature-carrying SPH operators: blur (kernel-weighted feature average) and
// the SPH feature gradient, forward and backward, fused in one sweep when both
// are asked for.
//
// Replaces forward_kernel / backward_kernel of the reference for the Blur and
// Gradient computation types (sphops/sph_cuda.cu:1699-1716, 1185-1235,
// 1265-1327).  The reference maps a thread to (particle, feature) and redoes the
// distance test and the kernel weight once per feature; here a pair is tested
// once, by one lane, and the accepted pairs of a particle go through a small
// per-warp shared-memory list that the particle's LPP lanes then walk with VW
// features each (128-bit feature loads when C % 4 == 0).
//
// Backward is a gather (no global atomics): particle i collects the terms of
// both roles it plays in each pair.  Sums over features (the position and
// density gradients) stay lane-local until one sub-group reduction at the end.
#pragma once
#include "neighbors.cuh"
#include "ops.cuh"

namespace npa {

constexpr int kListPerWarp = 128;  // accepted-pair slots per warp, split evenly between its sub-groups

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

template <int D, bool PER, int LPP, int VW, int MASK>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
feature_forward_kernel(FeatureFwdArgs a, Geom g) {
    constexpr int PPW = 32 / LPP;
    constexpr int CAP = kListPerWarp / PPW;
    constexpr unsigned SUBMASK = LPP == 32 ? 0xffffffffu : ((1u << LPP) - 1u);
    __shared__ int4 s_ranges[kWarpsPerCta][kMaxRanges];
    __shared__ float4 s_ent[kWarpsPerCta][kListPerWarp];
    __shared__ int s_idx[kWarpsPerCta][kListPerWarp];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarpsPerCta + warp;
    if (row >= g.max_blocks) return;
    const WorkItem it = load_item(a.block_info, a.bin_offsets, row);
    if (it.count <= 0) return;
    int4 *rng = s_ranges[warp];
    const int nr = build_ranges<D>(g, a.bin_offsets, it, rng);
    const int sub = lane / LPP, sl = lane % LPP;
    float4 *ent = s_ent[warp] + sub * CAP;
    int *idx = s_idx[warp] + sub * CAP;
    const int C = a.C;

    for (int k0 = 0; k0 < it.count; k0 += PPW) {
        const int k = k0 + sub;
        const bool ivalid = k < it.count;
        const long long i = it.first + (ivalid ? k : 0);
        const Pos<D> pi = load_pos<D>(a.x, i);
        for (int fbase = 0; fbase < C; fbase += LPP * VW) {
            const int f0 = fbase + sl * VW;
            const bool fvalid = f0 < C;
            float si[VW], blur[VW], gr[VW * D];
#pragma unroll
            for (int q = 0; q < VW; ++q) { si[q] = 0.f; blur[q] = 0.f; }
#pragma unroll
            for (int q = 0; q < VW * D; ++q) gr[q] = 0.f;
            if (ivalid && fvalid && (MASK & F_GRAD)) load_feat<VW>(a.s + i * C + f0, si);
            int n_sub = 0;

            auto drain = [&]() {
                __syncwarp();
                const int nmax = __reduce_max_sync(kFull, n_sub);
                for (int e = 0; e < nmax; ++e) {
                    if (e < n_sub && fvalid) {
                        const float4 en = ent[e];
                        const long long j = idx[e];
                        float sj[VW];
                        load_feat<VW>(a.s + j * C + f0, sj);
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
                }
                n_sub = 0;
                __syncwarp();
            };

            for (int r = 0; r < nr; ++r) {
                const int4 rg = rng[r];
                const Origin<D, PER> org = make_origin<D, PER>(g, pi.x, pi.y, pi.z, rg.z);
                for (int j0 = rg.x; j0 < rg.y; j0 += LPP) {
                    const int j = j0 + sl;
                    float rx = 0.f, ry = 0.f, rz = 0.f, q = 0.f;
                    bool acc = false;
                    if (ivalid && j < rg.y) {
                        const Pos<D> pj = load_pos<D>(a.x, j);
                        q = displacement<D, PER>(g, org, pj.x, pj.y, pj.z, rx, ry, rz);
                        acc = q < g.h2;
                    }
                    const unsigned bal = __ballot_sync(kFull, acc);
                    const unsigned sb = (bal >> (sub * LPP)) & SUBMASK;
                    if (acc) {
                        const int pos = n_sub + __popc(sb & ((1u << sl) - 1u));
                        const float mj = a.mass ? __ldg(a.mass + j) : 1.0f;
                        const float vj = mj / __ldg(a.rho + j);
                        float wv = 0.f, kv = 0.f;
                        if (MASK & F_BLUR) {
                            const float t = fmaxf(g.h2 - q, 0.f);
                            wv = vj * (t * t * t);
                        }
                        if ((MASK & F_GRAD) && q > 0.f) {
                            float dist;
                            kv = vj * spiky_phi(q, g.h, dist);
                        }
                        ent[pos] = make_float4(kv * rx, kv * ry, kv * rz, wv);
                        idx[pos] = j;
                    }
                    n_sub += __popc(sb);
                    if (__any_sync(kFull, n_sub + LPP > CAP)) drain();
                }
            }
            drain();

            if (ivalid && fvalid) {
                if ((MASK & F_BLUR) && a.blur) {
#pragma unroll
                    for (int q = 0; q < VW; ++q) blur[q] *= g.c_s;
                    store_run<VW, VW>(a.blur + i * C + f0, blur);
                }
                if ((MASK & F_GRAD) && a.grad) {
#pragma unroll
                    for (int q = 0; q < VW * D; ++q) gr[q] *= g.c_g;
                    store_run<VW, VW * D>(a.grad + (i * C + f0) * D, gr);
                }
            }
        }
    }
}

template <int D, bool PER, int LPP, int VW, int MASK, bool FULL>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
feature_backward_kernel(FeatureBwdArgs a, Geom g) {
    constexpr int PPW = 32 / LPP;
    constexpr int CAP = kListPerWarp / PPW;
    constexpr unsigned SUBMASK = LPP == 32 ? 0xffffffffu : ((1u << LPP) - 1u);
    __shared__ int4 s_ranges[kWarpsPerCta][kMaxRanges];
    __shared__ float4 s_geo[kWarpsPerCta][kListPerWarp];  // r.x r.y r.z v_j
    __shared__ float4 s_ker[kWarpsPerCta][kListPerWarp];  // W, 6(h^2-q)^2, phi, psi
    __shared__ int s_idx[kWarpsPerCta][kListPerWarp];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarpsPerCta + warp;
    if (row >= g.max_blocks) return;
    const WorkItem it = load_item(a.block_info, a.bin_offsets, row);
    if (it.count <= 0) return;
    int4 *rng = s_ranges[warp];
    const int nr = build_ranges<D>(g, a.bin_offsets, it, rng);
    const int sub = lane / LPP, sl = lane % LPP;
    float4 *geo = s_geo[warp] + sub * CAP;
    float4 *ker = s_ker[warp] + sub * CAP;
    int *idx = s_idx[warp] + sub * CAP;
    const int C = a.C;

    for (int k0 = 0; k0 < it.count; k0 += PPW) {
        const int k = k0 + sub;
        const bool ivalid = k < it.count;
        const long long i = it.first + (ivalid ? k : 0);
        const Pos<D> pi = load_pos<D>(a.x, i);
        const float mi = a.mass ? __ldg(a.mass + i) : 1.0f;
        const float vi = mi / __ldg(a.rho + i);
        // lane-partial sums over this lane's features, reduced across the sub-group at the end
        float dxs[3] = {0.f, 0.f, 0.f}, dxg[3] = {0.f, 0.f, 0.f}, drs = 0.f, drg = 0.f;

        for (int fbase = 0; fbase < C; fbase += LPP * VW) {
            const int f0 = fbase + sl * VW;
            const bool fvalid = f0 < C;
            float si[VW], gbi[VW], ggi[VW * D], ds[VW], dsg[VW];
#pragma unroll
            for (int q = 0; q < VW; ++q) { si[q] = 0.f; gbi[q] = 0.f; ds[q] = 0.f; dsg[q] = 0.f; }
#pragma unroll
            for (int q = 0; q < VW * D; ++q) ggi[q] = 0.f;
            if (ivalid && fvalid) {
                if (FULL) load_feat<VW>(a.s + i * C + f0, si);
                if (FULL && (MASK & F_BLUR)) load_feat<VW>(a.g_blur + i * C + f0, gbi);
                if (MASK & F_GRAD) load_run<VW, VW * D>(a.g_grad + (i * C + f0) * D, ggi);
            }
            int n_sub = 0;

            auto drain = [&]() {
                __syncwarp();
                const int nmax = __reduce_max_sync(kFull, n_sub);
                for (int e = 0; e < nmax; ++e) {
                    if (e < n_sub && fvalid) {
                        const float4 e0 = geo[e];
                        const float4 e1 = ker[e];
                        const long long j = idx[e];
                        const float rv[3] = {e0.x, e0.y, e0.z};
                        const float vj = e0.w;
                        float sj[VW];
                        if (FULL) load_feat<VW>(a.s + j * C + f0, sj);
                        if (MASK & F_BLUR) {
                            float gbj[VW];
                            load_feat<VW>(a.g_blur + j * C + f0, gbj);
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
                        if (MASK & F_GRAD) {
                            float ggj[VW * D];
                            load_run<VW, VW * D>(a.g_grad + (j * C + f0) * D, ggj);
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
                    }
                }
                n_sub = 0;
                __syncwarp();
            };

            for (int r = 0; r < nr; ++r) {
                const int4 rg = rng[r];
                const Origin<D, PER> org = make_origin<D, PER>(g, pi.x, pi.y, pi.z, rg.z);
                for (int j0 = rg.x; j0 < rg.y; j0 += LPP) {
                    const int j = j0 + sl;
                    float rx = 0.f, ry = 0.f, rz = 0.f, q = 0.f;
                    bool acc = false;
                    if (ivalid && j < rg.y) {
                        const Pos<D> pj = load_pos<D>(a.x, j);
                        q = displacement<D, PER>(g, org, pj.x, pj.y, pj.z, rx, ry, rz);
                        acc = q < g.h2;
                    }
                    const unsigned bal = __ballot_sync(kFull, acc);
                    const unsigned sb = (bal >> (sub * LPP)) & SUBMASK;
                    if (acc) {
                        const int pos = n_sub + __popc(sb & ((1u << sl) - 1u));
                        const float mj = a.mass ? __ldg(a.mass + j) : 1.0f;
                        const float vj = mj / __ldg(a.rho + j);
                        const float t = fmaxf(g.h2 - q, 0.f);
                        float phi = 0.f, psi = 0.f;
                        if ((MASK & F_GRAD) && q > 0.f) {
                            float dist;
                            phi = spiky_phi(q, g.h, dist);
                            if (FULL) psi = spiky_psi(dist, g.h);
                        }
                        geo[pos] = make_float4(rx, ry, rz, vj);
                        ker[pos] = make_float4(t * t * t, 6.0f * t * t, phi, psi);
                        idx[pos] = j;
                    }
                    n_sub += __popc(sb);
                    if (__any_sync(kFull, n_sub + LPP > CAP)) drain();
                }
            }
            drain();

            if (ivalid && fvalid && a.grad_s) {
                float out[VW];
#pragma unroll
                for (int q = 0; q < VW; ++q) out[q] = g.c_s * vi * ds[q] - g.c_g * dsg[q];
                store_run<VW, VW>(a.grad_s + i * C + f0, out);
            }
        }

        if (FULL) {
            float out[3];
#pragma unroll
            for (int d = 0; d < D; ++d) out[d] = subgroup_sum<LPP>(g.c_s * dxs[d] + g.c_g * dxg[d]);
            const float dr = subgroup_sum<LPP>(g.c_g * drg - g.c_s * drs);
            if (ivalid && sl == 0) {
                if (a.grad_x) {
                    if (D == 2) reinterpret_cast<float2 *>(a.grad_x)[i] = make_float2(out[0], out[1]);
                    else reinterpret_cast<float4 *>(a.grad_x)[i] = make_float4(out[0], out[1], out[2], 0.f);
                }
                if (a.grad_rho) a.grad_rho[i] = (vi * vi / mi) * dr;
            }
        }
    }
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

template <int D, bool PER, int LPP, int VW>
int launch_feature_forward_shape(const Geom &g, int mask, const FeatureFwdArgs &a, cudaStream_t st) {
    const unsigned blocks = (unsigned)((g.max_blocks + kWarpsPerCta - 1) / kWarpsPerCta);
    const unsigned threads = kWarpsPerCta * 32;
    switch (mask) {
        case F_BLUR: feature_forward_kernel<D, PER, LPP, VW, F_BLUR><<<blocks, threads, 0, st>>>(a, g); break;
        case F_GRAD: feature_forward_kernel<D, PER, LPP, VW, F_GRAD><<<blocks, threads, 0, st>>>(a, g); break;
        case F_BLUR | F_GRAD:
            feature_forward_kernel<D, PER, LPP, VW, F_BLUR | F_GRAD><<<blocks, threads, 0, st>>>(a, g);
            break;
        default: return fail(NPA_ERR_INVALID_ARGUMENT, "unsupported feature forward mask %d", mask);
    }
    return check_launch("feature_forward_kernel");
}

template <int D, bool PER>
int launch_feature_forward_geom(const Geom &g, int mask, const FeatureFwdArgs &a, cudaStream_t st) {
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

template <int D, bool PER, int LPP, int VW, bool FULL>
int launch_feature_backward_shape(const Geom &g, int mask, const FeatureBwdArgs &a, cudaStream_t st) {
    const unsigned blocks = (unsigned)((g.max_blocks + kWarpsPerCta - 1) / kWarpsPerCta);
    const unsigned threads = kWarpsPerCta * 32;
    switch (mask) {
        case F_BLUR:
            feature_backward_kernel<D, PER, LPP, VW, F_BLUR, FULL><<<blocks, threads, 0, st>>>(a, g);
            break;
        case F_GRAD:
            feature_backward_kernel<D, PER, LPP, VW, F_GRAD, FULL><<<blocks, threads, 0, st>>>(a, g);
            break;
        case F_BLUR | F_GRAD:
            feature_backward_kernel<D, PER, LPP, VW, F_BLUR | F_GRAD, FULL><<<blocks, threads, 0, st>>>(a, g);
            break;
        default: return fail(NPA_ERR_INVALID_ARGUMENT, "unsupported feature backward mask %d", mask);
    }
    return check_launch("feature_backward_kernel");
}

template <int D, bool PER, bool FULL>
int launch_feature_backward_geom(const Geom &g, int mask, const FeatureBwdArgs &a, cudaStream_t st) {
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
