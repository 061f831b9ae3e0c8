// Packed perception: the whole per-step perception of an NPA model as two neighbour sweeps that
// write the MLP input row directly, and its backward.
//
// NPA.perceive (models/npa.py:87-137) computes density, blur, the moment-corrected feature
// gradient (gradient_hybrid, sphops/sph.py:474-484: raw @ safe_inv(M) with the gradient of the
// raw operator), the density gradient, then scales by eps/eps0, log-normalises the two gradient
// features and concatenates everything into z[B,N,2C+C*D+D] with a dozen torch kernels that each
// re-read the [B,N,C,D] gradient tensor.  Here sweep 2 applies that per-particle epilogue while
// the sums are still in registers (feature_kernels.cuh, F_PACK) and writes z once; backward turns
// dL/dz into the upstream gradients of blur / gradient / density gradient with one elementwise
// kernel and then runs the ordinary fused backward sweeps.
#include "ops.cuh"

namespace npa {

// Gradient of  f(w) = log(1 + |w|) w / |w|  (symmetric Jacobian) applied to g, times `scale`;
// without log-normalisation f is the identity.
template <int D>
__device__ inline void log_normalize_backward(const float *w, const float *gin, int log_norm, float scale, float *gout) {
    if (!log_norm) {
#pragma unroll
        for (int d = 0; d < D; ++d) gout[d] = scale * gin[d];
        return;
    }
    float n2 = w[0] * w[0] + w[1] * w[1];
    float wg = w[0] * gin[0] + w[1] * gin[1];
    if (D == 3) { n2 += w[2] * w[2]; wg += w[2] * gin[2]; }
    const float n = sqrtf(n2);
    const float l = logf(1.0f + n);
    const float a = l / fmaxf(n, 1e-12f);
    const float b = n > 1e-12f ? (1.0f / ((1.0f + n) * n2) - l / (n2 * n)) : 0.0f;
#pragma unroll
    for (int d = 0; d < D; ++d) gout[d] = scale * (a * gin[d] + b * wg * w[d]);
}

// One thread per (particle, feature): dL/dz -> dL/dblur, dL/dgrad; the thread of feature 0 also
// handles the density-gradient part.
template <int D>
__global__ void __launch_bounds__(256)
pack_backward_kernel(const float *__restrict__ gz, const float *__restrict__ vgrad, const float *__restrict__ rho_grad,
                     float *__restrict__ g_blur, float *__restrict__ g_grad, float *__restrict__ g_rho_grad,
                     long long particles, int C, float coef, float dg_scale, int log_norm_grad, int log_norm_dg) {
    const long long t = (long long)blockIdx.x * 256 + threadIdx.x;
    if (t >= particles * C) return;
    const long long i = t / C;
    const int f = (int)(t - i * C);
    const int Z = 2 * C + C * D + D;
    const float *gr = gz + i * Z;
    g_blur[t] = gr[C + f];
    float w[D], gin[D], gout[D];
#pragma unroll
    for (int d = 0; d < D; ++d) {
        w[d] = vgrad[t * D + d] * coef;
        gin[d] = gr[2 * C + f * D + d];
    }
    log_normalize_backward<D>(w, gin, log_norm_grad, coef, gout);
#pragma unroll
    for (int d = 0; d < D; ++d) g_grad[t * D + d] = gout[d];
    if (f == 0 && g_rho_grad) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
            w[d] = rho_grad[i * D + d] * dg_scale;
            gin[d] = gr[2 * C + C * D + d];
        }
        log_normalize_backward<D>(w, gin, log_norm_dg, dg_scale, gout);
#pragma unroll
        for (int d = 0; d < D; ++d) g_rho_grad[i * D + d] = gout[d];
    }
}

// grad_s[i][f] += dL/dz[i][f]: the features enter z unchanged as its first C columns.
__global__ void __launch_bounds__(256)
add_direct_kernel(const float *__restrict__ gz, float *__restrict__ grad_s, long long particles, int C, int Z) {
    const long long t = (long long)blockIdx.x * 256 + threadIdx.x;
    if (t >= particles * C) return;
    const long long i = t / C;
    grad_s[t] += gz[i * Z + (t - i * C)];
}

}  // namespace npa

using namespace npa;

extern "C" {

int npa_perceive_features_forward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *mass,
                                  const float *s_bin, float coef, float dg_scale, float inv_tol,
                                  int32_t log_norm_grad, int32_t log_norm_dg, float *rho, float *rho_grad,
                                  float *z, float *vgrad, const int32_t *bin_offsets, const int32_t *block_info,
                                  int32_t *pair_cache, int32_t pair_stride, void *stream) {
    Geom g;
    int rc = make_geom(gd, &g);
    if (rc != NPA_OK) return rc;
    if (!x_bin || !s_bin || !rho || !rho_grad || !z || !bin_offsets || !block_info)
        return fail(NPA_ERR_INVALID_ARGUMENT, "perceive_features_forward: a required pointer is NULL");
    if (channels <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "perceive_features_forward: channels must be positive");
    if (((uintptr_t)x_bin % (g.dim == 2 ? 8 : 16)) || ((uintptr_t)block_info % 16))
        return fail(NPA_ERR_INVALID_ARGUMENT, "perceive_features_forward: positions / block_info are misaligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (pair_cache && (pair_stride < 2 || pair_stride > 513))
        return fail(NPA_ERR_INVALID_ARGUMENT, "perceive_features_forward: pair_stride must be in [2, 513]");
    // The packed sweep meets every pair with its spiky kernel value in hand, so it also sums the density
    // gradient; the first sweep is then the density alone (and the neighbour lists), which the shared-
    // candidate kernel runs in about half the time of the density + density-gradient sweep.  With the
    // cell-tile engine switched on (it has no such sum) the first sweep computes both as before.
    const bool in_sweep = !tile_forward_enabled();
    ScalarFwdArgs sa = {x_bin, mass, nullptr, nullptr, rho, in_sweep ? nullptr : rho_grad, nullptr, bin_offsets, block_info, pair_cache, pair_stride};
    if ((rc = launch_scalar_forward(g, in_sweep ? S_DENSITY : (S_DENSITY | S_DGRAD), sa, st)) != NPA_OK) return rc;
    FeatureFwdArgs fa = {x_bin, mass, rho, s_bin, nullptr, nullptr, channels, bin_offsets, block_info, nullptr};
    fa.z = z;
    fa.zstride = 2 * channels + channels * g.dim + g.dim;
    fa.vgrad = vgrad;
    fa.rho_grad = in_sweep ? nullptr : rho_grad;
    fa.rho_grad_out = in_sweep ? rho_grad : nullptr;
    fa.coef = coef;
    fa.dg_scale = dg_scale;
    fa.inv_tol = inv_tol;
    fa.log_norm_grad = log_norm_grad;
    fa.log_norm_dg = log_norm_dg;
    if (pair_cache && (pair_stride < 2 || pair_stride > 513))
        return fail(NPA_ERR_INVALID_ARGUMENT, "perceive_features_forward: pair_stride must be in [2, 513]");
    fa.pair_cache = pair_cache;
    fa.pair_stride = pair_stride;
    fa.pair_cache_valid = pair_cache != nullptr;  // written by the density sweep above
    return launch_feature_forward(g, F_BLUR | F_GRAD | F_MOMENT | F_PACK, fa, st);
}

int npa_perceive_features_backward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *mass,
                                   const float *s_bin, const float *rho, const float *rho_grad,
                                   const float *vgrad, const float *dL_dz, float coef, float dg_scale,
                                   int32_t log_norm_grad, int32_t log_norm_dg, float *g_blur_scratch,
                                   float *g_grad_scratch, float *g_rho_grad_scratch, float *grad_rho_scratch,
                                   float *grad_x, float *grad_s, const int32_t *bin_offsets,
                                   const int32_t *block_info, const int32_t *pair_cache, int32_t pair_stride,
                                   void *stream) {
    Geom g;
    int rc = make_geom(gd, &g);
    if (rc != NPA_OK) return rc;
    if (!x_bin || !s_bin || !rho || !rho_grad || !vgrad || !dL_dz || !g_blur_scratch || !g_grad_scratch)
        return fail(NPA_ERR_INVALID_ARGUMENT, "perceive_features_backward: a required pointer is NULL");
    if (grad_x && (!g_rho_grad_scratch || !grad_rho_scratch))
        return fail(NPA_ERR_INVALID_ARGUMENT, "perceive_features_backward: grad_x needs g_rho_grad_scratch and grad_rho_scratch");
    if (channels <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "perceive_features_backward: channels must be positive");
    if (!grad_x && !grad_s) return NPA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const long long particles = (long long)g.B * g.N;
    const unsigned blocks = (unsigned)((particles * channels + 255) / 256);
    float *grg = grad_x ? g_rho_grad_scratch : nullptr;
    if (g.dim == 2)
        pack_backward_kernel<2><<<blocks, 256, 0, st>>>(dL_dz, vgrad, rho_grad, g_blur_scratch, g_grad_scratch, grg,
                                                        particles, channels, coef, dg_scale, log_norm_grad, log_norm_dg);
    else
        pack_backward_kernel<3><<<blocks, 256, 0, st>>>(dL_dz, vgrad, rho_grad, g_blur_scratch, g_grad_scratch, grg,
                                                        particles, channels, coef, dg_scale, log_norm_grad, log_norm_dg);
    if ((rc = check_launch("pack_backward_kernel")) != NPA_OK) return rc;
    rc = npa_perception_backward(gd, channels, x_bin, mass, s_bin, rho, nullptr, g_blur_scratch, g_grad_scratch, grg,
                                 grad_x, grad_s, grad_rho_scratch, bin_offsets, block_info, pair_cache, pair_stride, stream);
    if (rc != NPA_OK) return rc;
    if (grad_s) {
        add_direct_kernel<<<blocks, 256, 0, st>>>(dL_dz, grad_s, particles, channels,
                                                  2 * channels + channels * g.dim + g.dim);
        rc = check_launch("add_direct_kernel");
    }
    return rc;
}

}  // extern "C"
