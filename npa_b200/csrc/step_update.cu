// The Euler update that follows perception and the per-particle MLP in one elementwise pass.
//
// Replaces the torch glue of NPA.forward (models/npa.py:145-153: the displacement limiter
// dx = alpha * dx * eps / (1 + |dx|)) and of step_euler (models/npa.py:183-203: zero padding of the
// 3D displacement, x = x_bin + dt * dx * mask, s = s_bin + dt * ds * mask) -- about ten elementwise
// torch kernels over [B,N,D+C] -- and optionally HashGrid.wrap_positions (sphops/sph.py:107-123).
// `y` is the MLP output in cell order, [B*N, D + C]: the first D columns are the raw displacement,
// the rest the state update.  One thread per four elements of y; HBM bound (every tensor is read or
// written once: 4(D+C) + 8P + 8C + 4 bytes per particle).
#include "ops.cuh"

namespace npa {

struct StepArgs {
    const float *y;       // [BN, D + C]
    const float *x_bin;   // [BN, P]
    const float *s_bin;   // [BN, C]
    const float *mask;    // [BN] (0 / 1) or NULL = every particle updates
    float *x_out;         // [BN, P]
    float *s_out;         // [BN, C]
    const float *g_x_out; // backward: upstream of x_out [BN, P]
    const float *g_s_out; // backward: upstream of s_out [BN, C]
    float *g_y;           // backward: [BN, D + C]
    long long particles;
    int C;
    float alpha, eps, dt;
    int wrap;
};

// remainder(x + L/2, L) - L/2 with torch's sign convention (result of remainder in [0, L)).
__device__ inline float wrap_axis(float x, float L) {
    const float half = 0.5f * L;
    float r = fmodf(x + half, L);
    if (r < 0.f) r += L;
    return r - half;
}

// One element of y: column c of particle i.
template <int D>
__device__ inline void step_forward_element(const StepArgs &a, const Geom &g, long long i, int c, float v) {
    constexpr int P = D == 2 ? 2 : 4;
    const float m = a.mask ? __ldg(a.mask + i) : 1.0f;
    if (c >= D) {
        const long long o = i * a.C + (c - D);
        a.s_out[o] = __ldg(a.s_bin + o) + (a.dt * v) * m;
    } else {
        const float *row = a.y + i * (D + a.C);
        float n2 = 0.f;
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const float t = __ldg(row + d);
            n2 = fmaf(t, t, n2);
        }
        // the reference's order: ((alpha * dx) * eps) / (1 + |dx|), then (dt * dx) * mask
        const float lim = ((a.alpha * v) * a.eps) / (1.0f + sqrtf(n2));
        float xo = __ldg(a.x_bin + i * P + c) + (a.dt * lim) * m;
        if (a.wrap && g.periodic) xo = wrap_axis(xo, g.L[c]);
        a.x_out[i * P + c] = xo;
        if (D == 3 && c == 0) a.x_out[i * P + 3] = __ldg(a.x_bin + i * P + 3);  // padding column
    }
}

// dL/dy of one element.  The limiter f(u) = k u / (1 + |u|), k = alpha * eps, has the Jacobian
//   df_a/du_b = k [ delta_ab / (1 + n) - u_a u_b / (n (1 + n)^2) ],  n = |u|  (second term 0 at n = 0,
// as torch's norm backward); the wrap and the additions are the identity for gradients.
template <int D>
__device__ inline float step_backward_element(const StepArgs &a, long long i, int c) {
    constexpr int P = D == 2 ? 2 : 4;
    const float m = a.mask ? __ldg(a.mask + i) : 1.0f;
    if (c >= D) return a.g_s_out ? (a.dt * m) * __ldg(a.g_s_out + i * a.C + (c - D)) : 0.f;
    if (!a.g_x_out) return 0.f;
    const float *row = a.y + i * (D + a.C);
    float n2 = 0.f, gu = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        const float t = __ldg(row + d);
        n2 = fmaf(t, t, n2);
        gu = fmaf(t, __ldg(a.g_x_out + i * P + d), gu);
    }
    const float n = sqrtf(n2);
    const float k = a.alpha * a.eps * a.dt * m;
    const float inv = 1.0f / (1.0f + n);
    float out = __ldg(a.g_x_out + i * P + c) * inv;
    if (n > 0.f) out -= __ldg(row + c) * gu * inv * inv / n;
    return k * out;
}

// A thread takes four consecutive elements of the flat y (a 16-byte load / store whatever the row
// length) and finds its particle and column with one division; Index is 32-bit when the tensor
// has fewer than 2^31 elements.
template <int D, typename Index, bool BACKWARD>
__global__ void __launch_bounds__(256) step_update_kernel(StepArgs a, Geom g) {
    const Index W = (Index)(D + a.C);
    const Index total = (Index)a.particles * W;
    const Index quads = (total + 3) / 4;
    for (Index q = blockIdx.x * (Index)blockDim.x + threadIdx.x; q < quads; q += (Index)gridDim.x * blockDim.x) {
        const Index e0 = q * 4;
        Index i = e0 / W;
        int c = (int)(e0 - i * W);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        const bool whole = e0 + 4 <= total;
        if (!BACKWARD) {
            if (whole) {
                const float4 t = __ldg(reinterpret_cast<const float4 *>(a.y) + q);
                v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
            } else {
                for (int k = 0; e0 + k < total; ++k) v[k] = __ldg(a.y + e0 + k);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (e0 + k < total) {
                if (BACKWARD) v[k] = step_backward_element<D>(a, (long long)i, c);
                else step_forward_element<D>(a, g, (long long)i, c, v[k]);
            }
            if (++c == (int)W) { c = 0; ++i; }
        }
        if (BACKWARD) {
            if (whole) reinterpret_cast<float4 *>(a.g_y)[q] = make_float4(v[0], v[1], v[2], v[3]);
            else for (int k = 0; e0 + k < total; ++k) a.g_y[e0 + k] = v[k];
        }
    }
}

// Tiled variant for feature counts that are a multiple of 4: a CTA stages the y rows of 64
// particles in shared memory with 16-byte loads (rows of D + C floats are not 16-byte aligned, the
// tile as a whole is), so that the state columns move as float4 and the position as one vector per
// particle.  Backward assembles the dL/dy tile in shared memory the same way.
constexpr int kStepRows = 64;

__device__ inline void tile_copy_async(float *smem_dst, const float *gmem_src, int floats) {
    // 16-byte pieces; the caller guarantees floats % 4 == 0 and 16-byte aligned addresses
    for (int q = threadIdx.x; q < floats / 4; q += blockDim.x) {
        const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst + 4 * q);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src + 4 * q) : "memory");
    }
}

template <int D, bool BACKWARD>
__global__ void __launch_bounds__(256) step_update_tiled_kernel(StepArgs a, Geom g) {
    extern __shared__ __align__(16) float tile_mem[];  // forward: two tiles [kStepRows][D + C]; backward: one
    const int W = D + a.C, C4 = a.C / 4;
    const long long tiles = (a.particles + kStepRows - 1) / kStepRows;
    auto rows_of = [&](long long t) {
        const long long left = a.particles - t * kStepRows;
        return (int)(left < kStepRows ? left : kStepRows);
    };
    if (!BACKWARD) {
        // The y tile of the next iteration is copied (cp.async) while the current one is processed.
        // A tile whose float count is not a multiple of 4 (only the last one can be) is loaded directly.
        long long t = blockIdx.x;
        int buf = 0;
        if (t < tiles && (rows_of(t) * W) % 4 == 0) tile_copy_async(tile_mem, a.y + t * kStepRows * W, rows_of(t) * W);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        for (; t < tiles; t += gridDim.x, buf ^= 1) {
            float *tile = tile_mem + (size_t)buf * kStepRows * W;
            const long long r0 = t * kStepRows;
            const int rows = rows_of(t), n = rows * W;
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
            if (n % 4 != 0)
                for (int e = threadIdx.x; e < n; e += blockDim.x) tile[e] = __ldg(a.y + r0 * W + e);
            __syncthreads();  // tile t is complete, and every thread has finished with the other buffer
            const long long tn = t + gridDim.x;
            if (tn < tiles && (rows_of(tn) * W) % 4 == 0)
                tile_copy_async(tile_mem + (size_t)(buf ^ 1) * kStepRows * W, a.y + tn * kStepRows * W, rows_of(tn) * W);
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            for (int f = threadIdx.x; f < rows * C4; f += blockDim.x) {
                const int row = f / C4, c4 = f - row * C4;
                const long long i = r0 + row;
                const float m = a.mask ? __ldg(a.mask + i) : 1.0f;
                const float4 sv = __ldg(reinterpret_cast<const float4 *>(a.s_bin) + i * C4 + c4);
                const float *yr = tile + row * W + D + 4 * c4;
                reinterpret_cast<float4 *>(a.s_out)[i * C4 + c4] =
                    make_float4(sv.x + (a.dt * yr[0]) * m, sv.y + (a.dt * yr[1]) * m, sv.z + (a.dt * yr[2]) * m,
                                sv.w + (a.dt * yr[3]) * m);
            }
            for (int row = threadIdx.x; row < rows; row += blockDim.x) {
                const long long i = r0 + row;
                const float m = a.mask ? __ldg(a.mask + i) : 1.0f;
                const float *yr = tile + row * W;
                float n2 = 0.f;
#pragma unroll
                for (int d = 0; d < D; ++d) n2 = fmaf(yr[d], yr[d], n2);
                const float den = 1.0f + sqrtf(n2);
                float xi[4] = {0.f, 0.f, 0.f, 0.f};
                if (D == 2) {
                    const float2 v = __ldg(reinterpret_cast<const float2 *>(a.x_bin) + i);
                    xi[0] = v.x; xi[1] = v.y;
                } else {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(a.x_bin) + i);
                    xi[0] = v.x; xi[1] = v.y; xi[2] = v.z; xi[3] = v.w;
                }
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const float lim = ((a.alpha * yr[d]) * a.eps) / den;
                    xi[d] = xi[d] + (a.dt * lim) * m;
                    if (a.wrap && g.periodic) xi[d] = wrap_axis(xi[d], g.L[d]);
                }
                if (D == 2) reinterpret_cast<float2 *>(a.x_out)[i] = make_float2(xi[0], xi[1]);
                else reinterpret_cast<float4 *>(a.x_out)[i] = make_float4(xi[0], xi[1], xi[2], xi[3]);
            }
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        return;
    }
    float *tile = tile_mem;
    for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
        const long long r0 = t * kStepRows;
        const int rows = rows_of(t);
        const int n = rows * W;
        {
            for (int f = threadIdx.x; f < rows * C4; f += blockDim.x) {
                const int row = f / C4, c4 = f - row * C4;
                const long long i = r0 + row;
                const float k = a.dt * (a.mask ? __ldg(a.mask + i) : 1.0f);
                float4 gs = make_float4(0.f, 0.f, 0.f, 0.f);
                if (a.g_s_out) gs = __ldg(reinterpret_cast<const float4 *>(a.g_s_out) + i * C4 + c4);
                float *o = tile + row * W + D + 4 * c4;
                o[0] = k * gs.x; o[1] = k * gs.y; o[2] = k * gs.z; o[3] = k * gs.w;
            }
            for (int row = threadIdx.x; row < rows; row += blockDim.x) {
                const long long i = r0 + row;
#pragma unroll
                for (int d = 0; d < D; ++d) tile[row * W + d] = step_backward_element<D>(a, i, d);
            }
            __syncthreads();
            float *dst = a.g_y + r0 * W;
            if (n % 4 == 0) {
                for (int q = threadIdx.x; q < n / 4; q += blockDim.x)
                    reinterpret_cast<float4 *>(dst)[q] = reinterpret_cast<const float4 *>(tile)[q];
            } else {
                for (int e = threadIdx.x; e < n; e += blockDim.x) dst[e] = tile[e];
            }
            __syncthreads();
        }
    }
}

static bool aligned16(const void *p) { return ((uintptr_t)p % 16) == 0; }

template <bool BACKWARD>
static int launch_step(const Geom &g, const StepArgs &a, cudaStream_t st) {
    // forward keeps two tiles (the next one is copied while the current one is processed)
    const size_t tile_bytes = (size_t)(BACKWARD ? 1 : 2) * kStepRows * (g.dim + a.C) * sizeof(float);
    const bool vec = a.C % 4 == 0 && tile_bytes <= 48 * 1024 &&
                     (BACKWARD ? aligned16(a.g_y) && aligned16(a.g_s_out) && aligned16(a.g_x_out)
                               : aligned16(a.y) && aligned16(a.s_bin) && aligned16(a.s_out) && aligned16(a.x_bin) &&
                                     aligned16(a.x_out));
    if (vec) {
        const long long tiles = (a.particles + kStepRows - 1) / kStepRows;
        const long long cap = 148ll * 8;
        const int ctas = (int)(tiles < cap ? (tiles > 0 ? tiles : 1) : cap);
        if (g.dim == 2) step_update_tiled_kernel<2, BACKWARD><<<ctas, 256, tile_bytes, st>>>(a, g);
        else step_update_tiled_kernel<3, BACKWARD><<<ctas, 256, tile_bytes, st>>>(a, g);
        return check_launch(BACKWARD ? "step_update_tiled_kernel (backward)" : "step_update_tiled_kernel (forward)");
    }
    const long long total = a.particles * (g.dim + a.C);
    const long long quads = (total + 3) / 4;
    const long long want = (quads + 255) / 256;
    const long long cap = 148ll * 8 * 8;  // a few waves of 8 CTAs per SM, grid-stride beyond
    const int ctas = (int)(want < cap ? (want > 0 ? want : 1) : cap);
    const bool small = total < (1ll << 31) - 4;
    if (g.dim == 2) {
        if (small) step_update_kernel<2, unsigned, BACKWARD><<<ctas, 256, 0, st>>>(a, g);
        else step_update_kernel<2, long long, BACKWARD><<<ctas, 256, 0, st>>>(a, g);
    } else {
        if (small) step_update_kernel<3, unsigned, BACKWARD><<<ctas, 256, 0, st>>>(a, g);
        else step_update_kernel<3, long long, BACKWARD><<<ctas, 256, 0, st>>>(a, g);
    }
    return check_launch(BACKWARD ? "step_update_kernel (backward)" : "step_update_kernel (forward)");
}

}  // namespace npa

using namespace npa;

extern "C" {

int npa_step_update_forward(const npa_grid *gd, const float *y, const float *x_bin, const float *s_bin,
                            const float *mask, int32_t channels, float alpha, float dt, int32_t wrap, float *x_out,
                            float *s_out, void *stream) {
    Geom g;
    int rc = make_geom(gd, &g);
    if (rc != NPA_OK) return rc;
    if (channels <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_step_update_forward: channels must be positive, got %d", channels);
    if (!y || !x_bin || !s_bin || !x_out || !s_out)
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_step_update_forward: y, x_bin, s_bin, x_out and s_out must be non-NULL");
    StepArgs a = {};
    a.y = y; a.x_bin = x_bin; a.s_bin = s_bin; a.mask = mask; a.x_out = x_out; a.s_out = s_out;
    a.particles = (long long)g.B * g.N; a.C = channels; a.alpha = alpha; a.eps = g.h; a.dt = dt; a.wrap = wrap;
    if (((uintptr_t)y % 16)) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_step_update_forward: y must be 16-byte aligned");
    return launch_step<false>(g, a, (cudaStream_t)stream);
}

int npa_step_update_backward(const npa_grid *gd, const float *y, const float *mask, int32_t channels, float alpha,
                             float dt, const float *g_x_out, const float *g_s_out, float *g_y, void *stream) {
    Geom g;
    int rc = make_geom(gd, &g);
    if (rc != NPA_OK) return rc;
    if (channels <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_step_update_backward: channels must be positive, got %d", channels);
    if (!y || !g_y) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_step_update_backward: y and g_y must be non-NULL");
    StepArgs a = {};
    a.y = y; a.mask = mask; a.g_x_out = g_x_out; a.g_s_out = g_s_out; a.g_y = g_y;
    a.particles = (long long)g.B * g.N; a.C = channels; a.alpha = alpha; a.eps = g.h; a.dt = dt;
    if (((uintptr_t)g_y % 16)) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_step_update_backward: g_y must be 16-byte aligned");
    return launch_step<true>(g, a, (cudaStream_t)stream);
}

}  // extern "C"
