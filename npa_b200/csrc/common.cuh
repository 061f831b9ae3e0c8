// Shared device/host definitions of the npa_b200 kernels: grid geometry, cell
// hashing, SPH pair kernels and the error plumbing of the C ABI.
//
// Math follows the reference operators as restated by its pure-torch oracle
// (sphops/torch_sph.py:96-162: poly6 (h^2-r^2)^3 with cut-off r^2 < h^2, spiky
// 3(h-d)^2/d * r with d = sqrt(r^2 + 1e-12) inside 0 < r < h) and the cell
// geometry of sphops/utils.cuh:303-524.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/npa_b200.h"

namespace npa {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

// Device-side copy of npa_grid plus everything derived from it, passed by
// value to every kernel (the role of GridConfig, sphops/utils.cuh:303-318).
struct Geom {
    int dim, periodic, morton;
    int g[3];       // cells per axis (1 on unused axes)
    int half[3];    // g / 2: the grid is centred on the origin
    int cells;      // per system
    int B, N, mpb;
    int max_blocks;
    int split;      // warps sharing one work item in the feature kernels (small problems only)
    float inv_eps;  // 1.0f / float(eps): the multiplier pos2cell uses
    float h;        // float(eps)
    float h2;       // float(eps * eps) rounded once from double, as torch does
    float L[3];     // box length per axis = g * eps (rounded from double)
    float Llo[3];   // double(g * eps) - L: the part of the box length fp32 cannot hold
    float invL[3];
    float halfL[3];
    float c_s;      // poly6 normalisation
    float c_g;      // spiky normalisation
};

// Host: validate an npa_grid and derive Geom.  Returns an npa_status.
int make_geom(const npa_grid *in, Geom *out);
// Host: record an error message for npa_last_error() and return `code`.
int fail(int code, const char *fmt, ...);
// Host: convert the last CUDA launch error into a status.
int check_launch(const char *what);

// ---- cell hashing (sphops/utils.cuh:394-524) -------------------------------

__host__ __device__ inline uint32_t dilate2(uint32_t x) {
    x &= 0x3FFu;
    x = (x | (x << 16)) & 0x0000FFFFu;
    x = (x | (x << 8)) & 0x00FF00FFu;
    x = (x | (x << 4)) & 0x0F0F0F0Fu;
    x = (x | (x << 2)) & 0x33333333u;
    x = (x | (x << 1)) & 0x55555555u;
    return x;
}
__host__ __device__ inline uint32_t dilate3(uint32_t x) {
    x &= 0x3FFu;
    x = (x | (x << 16)) & 0x030000FFu;
    x = (x | (x << 8)) & 0x0300F00Fu;
    x = (x | (x << 4)) & 0x030C30C3u;
    x = (x | (x << 2)) & 0x09249249u;
    return x;
}
__host__ __device__ inline uint32_t undilate2(uint32_t x) {
    x &= 0x55555555u;
    x = (x | (x >> 1)) & 0x33333333u;
    x = (x | (x >> 2)) & 0x0F0F0F0Fu;
    x = (x | (x >> 4)) & 0x00FF00FFu;
    x = (x | (x >> 8)) & 0x0000FFFFu;
    return x & 0x3FFu;
}
__host__ __device__ inline uint32_t undilate3(uint32_t x) {
    x &= 0x09249249u;
    x = (x | (x >> 2)) & 0x030C30C3u;
    x = (x | (x >> 4)) & 0x0300F00Fu;
    x = (x | (x >> 8)) & 0x030000FFu;
    x = (x | (x >> 16)) & 0x000003FFu;
    return x;
}

template <int D>
__host__ __device__ inline uint32_t cell_hash(const Geom &g, int cx, int cy, int cz) {
    if (g.morton) {
        if (D == 2) return dilate2((uint32_t)cx) | (dilate2((uint32_t)cy) << 1);
        return dilate3((uint32_t)cx) | (dilate3((uint32_t)cy) << 1) | (dilate3((uint32_t)cz) << 2);
    }
    if (D == 2) return (uint32_t)(cy * g.g[0] + cx);
    return (uint32_t)((cz * g.g[1] + cy) * g.g[0] + cx);
}

template <int D>
__device__ inline void hash_to_cell(const Geom &g, uint32_t hsh, int &cx, int &cy, int &cz) {
    cz = 0;
    if (g.morton) {
        if (D == 2) {
            cx = (int)undilate2(hsh);
            cy = (int)undilate2(hsh >> 1);
        } else {
            cx = (int)undilate3(hsh);
            cy = (int)undilate3(hsh >> 1);
            cz = (int)undilate3(hsh >> 2);
        }
        return;
    }
    cx = (int)(hsh % (uint32_t)g.g[0]);
    if (D == 2) {
        cy = (int)(hsh / (uint32_t)g.g[0]);
    } else {
        cy = (int)((hsh / (uint32_t)g.g[0]) % (uint32_t)g.g[1]);
        cz = (int)(hsh / (uint32_t)(g.g[0] * g.g[1]));
    }
}

__device__ inline int wrap_or_clamp(int c, int n, int periodic) {
    if (periodic) {
        c %= n;
        return c < 0 ? c + n : c;
    }
    return min(max(c, 0), n - 1);
}

// Cell coordinate of one position component: floor(x * (1/eps)) + g/2, then
// the boundary rule (sphops/utils.cuh:426-440).
__device__ inline int axis_cell(float x, const Geom &g, int axis) {
    int c = __float2int_rd(__fmul_rn(x, g.inv_eps)) + g.half[axis];
    return wrap_or_clamp(c, g.g[axis], g.periodic);
}

// ---- pair geometry -----------------------------------------------------------

// General minimum image of one displacement component: used only when the
// image shift could not be known in advance (a particle outside the primary
// box, or an axis with fewer than three cells).
__device__ inline float wrap_general(float r, float L, float Llo, float invL) {
    const float n = rintf(r * invL);
    r = __fmaf_rn(-n, L, r);
    return __fmaf_rn(-n, Llo, r);
}

// r^2 accumulated in the order torch.sum uses on a length-D vector, without
// fused multiply-adds, so that the strict cut-off test r^2 < h^2 agrees with
// the fp32 oracle on borderline pairs.
template <int D>
__device__ inline float sq_norm(float rx, float ry, float rz) {
    float q = __fadd_rn(__fmul_rn(rx, rx), __fmul_rn(ry, ry));
    if (D == 3) q = __fadd_rn(q, __fmul_rn(rz, rz));
    return q;
}

// Same quantity with fused multiply-adds, for kernels whose outputs are continuous in r^2
// (everything except the neighbour count).
template <int D>
__device__ inline float sq_norm_fast(float rx, float ry, float rz) {
    float q = fmaf(ry, ry, rx * rx);
    if (D == 3) q = fmaf(rz, rz, q);
    return q;
}

// Two fp32 lanes in one 64-bit register pair and the packed arithmetic of sm_100 on them: one issue slot per
// two multiply-adds, each lane rounded exactly like the scalar instruction.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// Spiky pair factors for 0 < q < h2: phi = 3 (h - d)^2 / d with
// d = sqrt(q + 1e-12), so that K(r) = phi * r; psi = 3 (h^2 - d^2) / d^3 so that
// dK/dr = phi * I - psi * r r^T.
__device__ inline float spiky_phi(float q, float h, float &d_out) {
    float d = sqrtf(q + 1e-12f);
    float t = fmaxf(h - d, 0.0f);
    d_out = d;
    return 3.0f * t * t / d;
}
__device__ inline float spiky_psi(float d, float h) {
    // d(phi)/dd / d with phi = 3 max(h-d,0)^2 / d  ==  -3 (h - d)(h + d) / d^3
    float t = fmaxf(h - d, 0.0f);
    return 3.0f * t * (h + d) / (d * d * d);
}


// Inverse of a symmetric DxD matrix given by its upper triangle m (row-major order of the
// triangle), identity when |det| < tol: the rule of the reference's safe_inv_sym_mat
// (sphops/sph_cuda.cu:3095-3179).  L is the full DxD inverse, row-major.
template <int D>
__device__ inline void safe_inverse_sym(const float *m, float tol, float *L) {
    if (D == 2) {
        const float det = m[0] * m[2] - m[1] * m[1];
        if (fabsf(det) < tol) {
            L[0] = 1.f; L[1] = 0.f; L[2] = 0.f; L[3] = 1.f;
        } else {
            const float r = 1.0f / det;
            L[0] = m[2] * r; L[1] = -m[1] * r; L[2] = -m[1] * r; L[3] = m[0] * r;
        }
    } else {
        const float a = m[0], b = m[1], c = m[2], d = m[3], e = m[4], f = m[5];
        const float t1 = d * f - e * e, t2 = c * e - b * f, t3 = b * e - c * d;
        const float det = a * t1 + b * t2 + c * t3;
        if (fabsf(det) < tol) {
            L[0] = 1.f; L[1] = 0.f; L[2] = 0.f; L[3] = 0.f; L[4] = 1.f; L[5] = 0.f; L[6] = 0.f; L[7] = 0.f; L[8] = 1.f;
        } else {
            const float r = 1.0f / det;
            const float m01 = t2 * r, m02 = t3 * r, m12 = (b * c - a * e) * r;
            L[0] = t1 * r; L[1] = m01; L[2] = m02;
            L[3] = m01; L[4] = (a * f - c * c) * r; L[5] = m12;
            L[6] = m02; L[7] = m12; L[8] = (a * d - b * b) * r;
        }
    }
}

// w <- log(1 + |w|) * w / max(|w|, 1e-12): the log-normalisation NPA applies to its gradient
// features (models/npa.py:83-85, torch.nn.functional.normalize's epsilon).
template <int D>
__device__ inline void log_normalize(float *w) {
    float n2 = w[0] * w[0] + w[1] * w[1];
    if (D == 3) n2 += w[2] * w[2];
    const float n = sqrtf(n2);
    const float sc = logf(1.0f + n) / fmaxf(n, 1e-12f);
#pragma unroll
    for (int d = 0; d < D; ++d) w[d] *= sc;
}

}  // namespace npa
