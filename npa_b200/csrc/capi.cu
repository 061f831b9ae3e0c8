// Operator entry points of the C ABI (include/npa_b200.h): argument checks and
// dispatch into the kernel translation units.  One function per method of the
// reference's HashGrid class (sphops/sph_cuda.cu:2058-3046) plus the two fused
// perception calls.
#include <map>
#include <mutex>
#include <tuple>
#include <utility>

#include "ops.cuh"

namespace npa {

template <int D, bool PER>
int launch_feature_forward_geom(const Geom &, int, const FeatureFwdArgs &, cudaStream_t);
template <int D, bool PER, bool FULL>
int launch_feature_backward_geom(const Geom &, int, const FeatureBwdArgs &, cudaStream_t);

int launch_feature_forward(const Geom &g, int mask, const FeatureFwdArgs &a, cudaStream_t st) {
    if (g.dim == 2)
        return g.periodic ? launch_feature_forward_geom<2, true>(g, mask, a, st)
                          : launch_feature_forward_geom<2, false>(g, mask, a, st);
    return g.periodic ? launch_feature_forward_geom<3, true>(g, mask, a, st)
                      : launch_feature_forward_geom<3, false>(g, mask, a, st);
}

int launch_feature_backward(const Geom &g, int mask, bool full, const FeatureBwdArgs &a, cudaStream_t st) {
#define NPA_FB(DD, PP) \
    (full ? launch_feature_backward_geom<DD, PP, true>(g, mask, a, st) \
          : launch_feature_backward_geom<DD, PP, false>(g, mask, a, st))
    if (g.dim == 2) return g.periodic ? NPA_FB(2, true) : NPA_FB(2, false);
    return g.periodic ? NPA_FB(3, true) : NPA_FB(3, false);
#undef NPA_FB
}

int persistent_ctas_impl(const void *kernel, int threads, size_t dyn_smem, int *out) {
    static std::mutex mu;
    static std::map<std::tuple<int, const void *, int, size_t>, int> cache;
    static std::map<std::pair<int, const void *>, size_t> smem_limit;  // largest dynamic size enabled so far
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_tuple(dev, kernel, threads, dyn_smem);
    auto it = cache.find(key);
    if (it == cache.end()) {
        int sms = 0, per_sm = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        size_t &enabled = smem_limit[std::make_pair(dev, kernel)];
        if (e == cudaSuccess && dyn_smem > enabled) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_smem);
            if (e == cudaSuccess) enabled = dyn_smem;
        }
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, dyn_smem);
        if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "sizing a persistent launch: %s", cudaGetErrorString(e));
        it = cache.emplace(key, sms * (per_sm > 0 ? per_sm : 1)).first;
    }
    *out = it->second;
    return NPA_OK;
}

constexpr int kTicketSlots = 8192;  // first half: eager launches; second half: launches under stream capture
static __device__ unsigned int g_row_tickets[kTicketSlots * 2];  // zero at load; every launch leaves its words zero

int acquire_row_tickets(cudaStream_t st, unsigned int **out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static unsigned int *base[kMaxDevices] = {nullptr};
    static unsigned int next[2] = {0u, 0u};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(NPA_ERR_UNSUPPORTED, "device ordinal %d is out of range", dev);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    e = cudaStreamIsCapturing(st, &cap);
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaStreamIsCapturing: %s", cudaGetErrorString(e));
    const int half = cap == cudaStreamCaptureStatusNone ? 0 : 1;
    std::lock_guard<std::mutex> lock(mu);
    if (!base[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_row_tickets);
        if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaGetSymbolAddress(row tickets): %s", cudaGetErrorString(e));
        base[dev] = static_cast<unsigned int *>(p);
    }
    if (half == 1 && next[1] >= (unsigned)(kTicketSlots / 2))
        // a replaying graph owns its words for as long as it exists: never hand one out twice
        return fail(NPA_ERR_UNSUPPORTED, "more than %d sweeps have been recorded under stream capture in this process",
                    kTicketSlots / 2);
    const unsigned int slot = half * (kTicketSlots / 2) + next[half]++ % (kTicketSlots / 2);
    *out = base[dev] + 2 * slot;
    return NPA_OK;
}

// Host-side check of the ticket words (synchronises): every sweep leaves its two words zero, so a
// non-zero word with no sweep in flight means a launch was cut short (e.g. a sticky CUDA error) and
// later sweeps drawing that slot would skip rows.
static int row_tickets_status(int *nonzero, bool reset) {
    static unsigned int host[kTicketSlots * 2];
    cudaError_t e = cudaMemcpyFromSymbol(host, g_row_tickets, sizeof(host));
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "row_tickets_status: %s", cudaGetErrorString(e));
    int n = 0;
    for (unsigned int v : host) n += v != 0u;
    *nonzero = n;
    if (reset && n) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_row_tickets);
        if (e == cudaSuccess) e = cudaMemset(p, 0, sizeof(host));
        if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "row_tickets_status: %s", cudaGetErrorString(e));
    }
    return NPA_OK;
}

// Common checks of an operator call: geometry, the two snapshot arrays, the
// positions and their vector alignment.
static int begin_op(const char *name, const npa_grid *gd, Geom *g, const float *x,
                    const int32_t *bin_offsets, const int32_t *block_info) {
    int rc = make_geom(gd, g);
    if (rc != NPA_OK) return rc;
    if (!x) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: binned_positions is NULL", name);
    if (!bin_offsets || !block_info) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: bin_offsets / block_info is NULL", name);
    if ((uintptr_t)x % (g->dim == 2 ? 8 : 16))
        return fail(NPA_ERR_INVALID_ARGUMENT, "%s: binned_positions must be aligned to one position (%d bytes)", name,
                    g->dim == 2 ? 8 : 16);
    if ((uintptr_t)block_info % 16) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: block_info must be 16-byte aligned", name);
    return NPA_OK;
}

static int check_channels(const char *name, int C) {
    if (C <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: channels must be positive, got %d", name, C);
    return NPA_OK;
}

static int check_pair_cache(const char *name, const void *cache, int stride) {
    if (cache && (stride < 2 || stride > 513))
        return fail(NPA_ERR_INVALID_ARGUMENT, "%s: pair_stride must be in [2, 513], got %d", name, stride);
    return NPA_OK;
}

static int check_grad_x(const char *name, const Geom &g, const float *grad_x) {
    if (grad_x && (uintptr_t)grad_x % (g.dim == 2 ? 8 : 16))
        return fail(NPA_ERR_INVALID_ARGUMENT, "%s: grad_x must be aligned to one position", name);
    return NPA_OK;
}

}  // namespace npa

using namespace npa;

#define NPA_REQUIRE(ptr, name, what) \
    if (!(ptr)) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: %s is NULL", name, what)

extern "C" {

int npa_count_forward(const npa_grid *gd, const float *x_bin, float *count, const int32_t *bin_offsets,
                      const int32_t *block_info, void *stream) {
    Geom g;
    int rc = begin_op("count_forward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    NPA_REQUIRE(count, "count_forward", "count");
    ScalarFwdArgs a = {x_bin, nullptr, nullptr, count, nullptr, nullptr, nullptr, bin_offsets, block_info};
    return launch_scalar_forward(g, S_COUNT, a, (cudaStream_t)stream);
}

int npa_density_forward(const npa_grid *gd, const float *x_bin, const float *mass, float *rho,
                        const int32_t *bin_offsets, const int32_t *block_info, void *stream) {
    Geom g;
    int rc = begin_op("density_forward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    NPA_REQUIRE(rho, "density_forward", "rho");
    ScalarFwdArgs a = {x_bin, mass, nullptr, nullptr, rho, nullptr, nullptr, bin_offsets, block_info};
    return launch_scalar_forward(g, S_DENSITY, a, (cudaStream_t)stream);
}

int npa_density_gradient_forward(const npa_grid *gd, const float *x_bin, const float *mass, float *rho_grad,
                                 const int32_t *bin_offsets, const int32_t *block_info, void *stream) {
    Geom g;
    int rc = begin_op("density_gradient_forward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    NPA_REQUIRE(rho_grad, "density_gradient_forward", "density_gradient_out");
    ScalarFwdArgs a = {x_bin, mass, nullptr, nullptr, nullptr, rho_grad, nullptr, bin_offsets, block_info};
    return launch_scalar_forward(g, S_DGRAD, a, (cudaStream_t)stream);
}

int npa_moment_matrix_forward(const npa_grid *gd, const float *x_bin, const float *rho, const float *mass,
                              float *moment, const int32_t *bin_offsets, const int32_t *block_info,
                              void *stream) {
    Geom g;
    int rc = begin_op("moment_matrix_forward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    NPA_REQUIRE(rho, "moment_matrix_forward", "rho");
    NPA_REQUIRE(moment, "moment_matrix_forward", "moment_matrix_out");
    if (g.dim == 2 && (uintptr_t)moment % 16)
        return fail(NPA_ERR_INVALID_ARGUMENT, "moment_matrix_forward: moment_matrix_out must be 16-byte aligned");
    ScalarFwdArgs a = {x_bin, mass, rho, nullptr, nullptr, nullptr, moment, bin_offsets, block_info};
    return launch_scalar_forward(g, S_MOMENT, a, (cudaStream_t)stream);
}

int npa_blur_forward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *rho,
                     const float *mass, const float *s_bin, float *s_blur, const int32_t *bin_offsets,
                     const int32_t *block_info, void *stream) {
    Geom g;
    int rc = begin_op("blur_forward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if ((rc = check_channels("blur_forward", channels)) != NPA_OK) return rc;
    NPA_REQUIRE(rho, "blur_forward", "rho");
    NPA_REQUIRE(s_bin, "blur_forward", "state_in");
    NPA_REQUIRE(s_blur, "blur_forward", "state_out");
    FeatureFwdArgs a = {x_bin, mass, rho, s_bin, s_blur, nullptr, channels, bin_offsets, block_info, nullptr};
    return launch_feature_forward(g, F_BLUR, a, (cudaStream_t)stream);
}

int npa_gradient_forward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *rho,
                         const float *mass, const float *s_bin, float *s_grad, const int32_t *bin_offsets,
                         const int32_t *block_info, void *stream) {
    Geom g;
    int rc = begin_op("gradient_forward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if ((rc = check_channels("gradient_forward", channels)) != NPA_OK) return rc;
    NPA_REQUIRE(rho, "gradient_forward", "rho");
    NPA_REQUIRE(s_bin, "gradient_forward", "state_in");
    NPA_REQUIRE(s_grad, "gradient_forward", "state_gradient_out");
    FeatureFwdArgs a = {x_bin, mass, rho, s_bin, nullptr, s_grad, channels, bin_offsets, block_info, nullptr};
    return launch_feature_forward(g, F_GRAD, a, (cudaStream_t)stream);
}

int npa_density_backward(const npa_grid *gd, const float *x_bin, const float *mass, const float *dL_drho,
                         float *grad_x, const int32_t *bin_offsets, const int32_t *block_info, void *stream) {
    Geom g;
    int rc = begin_op("density_backward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if (!grad_x) return NPA_OK;  // dLdx == false: nothing to compute (sph_cuda.cu:2519-2520)
    NPA_REQUIRE(dL_drho, "density_backward", "dL_rho_out");
    if ((rc = check_grad_x("density_backward", g, grad_x)) != NPA_OK) return rc;
    ScalarBwdArgs a = {x_bin, mass, nullptr, dL_drho, nullptr, nullptr, nullptr, grad_x, nullptr, 0, bin_offsets, block_info};
    return launch_scalar_backward(g, S_DENSITY, a, (cudaStream_t)stream);
}

int npa_density_gradient_backward(const npa_grid *gd, const float *x_bin, const float *mass,
                                  const float *dL_drho_grad, float *grad_x, const int32_t *bin_offsets,
                                  const int32_t *block_info, void *stream) {
    Geom g;
    int rc = begin_op("density_gradient_backward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if (!grad_x) return NPA_OK;
    NPA_REQUIRE(dL_drho_grad, "density_gradient_backward", "dL_density_gradient_out");
    if ((rc = check_grad_x("density_gradient_backward", g, grad_x)) != NPA_OK) return rc;
    ScalarBwdArgs a = {x_bin, mass, nullptr, nullptr, nullptr, dL_drho_grad, nullptr, grad_x, nullptr, 0, bin_offsets, block_info};
    return launch_scalar_backward(g, S_DGRAD, a, (cudaStream_t)stream);
}

int npa_moment_matrix_backward(const npa_grid *gd, const float *x_bin, const float *rho, const float *mass,
                               const float *dL_dmoment, float *grad_x, float *grad_rho,
                               const int32_t *bin_offsets, const int32_t *block_info, void *stream) {
    Geom g;
    int rc = begin_op("moment_matrix_backward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if (!grad_x && !grad_rho) return NPA_OK;
    NPA_REQUIRE(rho, "moment_matrix_backward", "rho");
    NPA_REQUIRE(dL_dmoment, "moment_matrix_backward", "dL_moment_matrix_out");
    if ((rc = check_grad_x("moment_matrix_backward", g, grad_x)) != NPA_OK) return rc;
    ScalarBwdArgs a = {x_bin, mass, rho, nullptr, nullptr, nullptr, dL_dmoment, grad_x, grad_rho, 0, bin_offsets, block_info};
    return launch_scalar_backward(g, S_MOMENT, a, (cudaStream_t)stream);
}

int npa_blur_backward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *rho,
                      const float *mass, const float *s_bin, const float *dL_dblur, float *grad_x,
                      float *grad_s, float *grad_rho, const int32_t *bin_offsets, const int32_t *block_info,
                      void *stream) {
    Geom g;
    int rc = begin_op("blur_backward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if ((rc = check_channels("blur_backward", channels)) != NPA_OK) return rc;
    if (!grad_x && !grad_s && !grad_rho) return NPA_OK;
    NPA_REQUIRE(rho, "blur_backward", "rho");
    NPA_REQUIRE(s_bin, "blur_backward", "state_in");
    NPA_REQUIRE(dL_dblur, "blur_backward", "dL_blur_state_out");
    if ((rc = check_grad_x("blur_backward", g, grad_x)) != NPA_OK) return rc;
    FeatureBwdArgs a = {x_bin, mass, rho, s_bin, dL_dblur, nullptr, grad_x, grad_s, grad_rho, channels, bin_offsets, block_info};
    return launch_feature_backward(g, F_BLUR, grad_x || grad_rho, a, (cudaStream_t)stream);
}

int npa_gradient_backward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *rho,
                          const float *mass, const float *s_bin, const float *dL_dgrad, float *grad_x,
                          float *grad_s, float *grad_rho, const int32_t *bin_offsets,
                          const int32_t *block_info, void *stream) {
    Geom g;
    int rc = begin_op("gradient_backward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if ((rc = check_channels("gradient_backward", channels)) != NPA_OK) return rc;
    if (!grad_x && !grad_s && !grad_rho) return NPA_OK;
    NPA_REQUIRE(rho, "gradient_backward", "rho");
    NPA_REQUIRE(s_bin, "gradient_backward", "state_in");
    NPA_REQUIRE(dL_dgrad, "gradient_backward", "dL_grad_state_out");
    if ((rc = check_grad_x("gradient_backward", g, grad_x)) != NPA_OK) return rc;
    FeatureBwdArgs a = {x_bin, mass, rho, s_bin, nullptr, dL_dgrad, grad_x, grad_s, grad_rho, channels, bin_offsets, block_info};
    return launch_feature_backward(g, F_GRAD, grad_x || grad_rho, a, (cudaStream_t)stream);
}

int npa_blur_gradient_forward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *rho,
                              const float *mass, const float *s_bin, float *s_blur, float *s_grad, float *moment,
                              const int32_t *bin_offsets, const int32_t *block_info, int32_t *pair_cache, int32_t pair_stride, int32_t pair_cache_valid, void *stream) {
    Geom g;
    int rc = begin_op("blur_gradient_forward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if ((rc = check_channels("blur_gradient_forward", channels)) != NPA_OK) return rc;
    NPA_REQUIRE(rho, "blur_gradient_forward", "rho");
    NPA_REQUIRE(s_bin, "blur_gradient_forward", "state_in");
    int mask = (s_blur ? F_BLUR : 0) | (s_grad ? F_GRAD : 0);
    if (moment) {
        if (mask != (F_BLUR | F_GRAD))
            return fail(NPA_ERR_INVALID_ARGUMENT, "blur_gradient_forward: moment needs both state_out and state_gradient_out");
        mask |= F_MOMENT;
    }
    if (!mask) return NPA_OK;
    if ((rc = check_pair_cache("blur_gradient_forward", pair_cache, pair_stride)) != NPA_OK) return rc;
    FeatureFwdArgs a = {x_bin, mass, rho, s_bin, s_blur, s_grad, channels, bin_offsets, block_info, moment};
    a.pair_cache = pair_cache;
    a.pair_stride = pair_stride;
    a.pair_cache_valid = pair_cache && pair_cache_valid;
    return launch_feature_forward(g, mask, a, (cudaStream_t)stream);
}

int npa_blur_gradient_backward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *rho,
                               const float *mass, const float *s_bin, const float *dL_dblur,
                               const float *dL_dgrad, float *grad_x, float *grad_s, float *grad_rho,
                               const int32_t *bin_offsets, const int32_t *block_info, const int32_t *pair_cache, int32_t pair_stride, void *stream) {
    Geom g;
    int rc = begin_op("blur_gradient_backward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if ((rc = check_channels("blur_gradient_backward", channels)) != NPA_OK) return rc;
    if (!grad_x && !grad_s && !grad_rho) return NPA_OK;
    NPA_REQUIRE(rho, "blur_gradient_backward", "rho");
    NPA_REQUIRE(s_bin, "blur_gradient_backward", "state_in");
    if ((rc = check_grad_x("blur_gradient_backward", g, grad_x)) != NPA_OK) return rc;
    const int mask = (dL_dblur ? F_BLUR : 0) | (dL_dgrad ? F_GRAD : 0);
    if (!mask) return fail(NPA_ERR_INVALID_ARGUMENT, "blur_gradient_backward: both upstream gradients are NULL");
    if ((rc = check_pair_cache("blur_gradient_backward", pair_cache, pair_stride)) != NPA_OK) return rc;
    FeatureBwdArgs a = {x_bin, mass, rho, s_bin, dL_dblur, dL_dgrad, grad_x, grad_s, grad_rho, channels, bin_offsets, block_info,
                        pair_cache, pair_stride};
    return launch_feature_backward(g, mask, grad_x || grad_rho, a, (cudaStream_t)stream);
}

int npa_density_chain_backward(const npa_grid *gd, const float *x_bin, const float *mass, const float *dL_drho_a,
                               const float *dL_drho_b, const float *dL_drho_grad, float *grad_x,
                               int32_t accumulate, const int32_t *bin_offsets, const int32_t *block_info,
                               const int32_t *pair_cache, int32_t pair_stride, void *stream) {
    Geom g;
    int rc = begin_op("density_chain_backward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    NPA_REQUIRE(grad_x, "density_chain_backward", "grad_x");
    if ((rc = check_grad_x("density_chain_backward", g, grad_x)) != NPA_OK) return rc;
    const int mask = ((dL_drho_a || dL_drho_b) ? S_DENSITY : 0) | (dL_drho_grad ? S_DGRAD : 0);
    if (!mask) return fail(NPA_ERR_INVALID_ARGUMENT, "density_chain_backward: every upstream gradient is NULL");
    if ((rc = check_pair_cache("density_chain_backward", pair_cache, pair_stride)) != NPA_OK) return rc;
    ScalarBwdArgs a = {x_bin, mass, nullptr, dL_drho_a, dL_drho_b, dL_drho_grad, nullptr, grad_x, nullptr,
                       accumulate ? 1 : 0, bin_offsets, block_info, pair_cache, pair_stride};
    return launch_scalar_backward(g, mask, a, (cudaStream_t)stream);
}

int npa_perception_forward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *mass,
                           const float *s_bin, float *rho, float *count, float *rho_grad, float *s_blur,
                           float *s_grad, float *moment, const int32_t *bin_offsets,
                           const int32_t *block_info, int32_t *pair_cache, int32_t pair_stride, void *stream) {
    Geom g;
    int rc = begin_op("perception_forward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    NPA_REQUIRE(rho, "perception_forward", "rho");
    cudaStream_t st = (cudaStream_t)stream;
    int smask = S_DENSITY | (count ? S_COUNT : 0) | (rho_grad ? S_DGRAD : 0);
    if ((rc = check_pair_cache("perception_forward", pair_cache, pair_stride)) != NPA_OK) return rc;
    // every argument is checked before the first sweep is enqueued
    if (s_blur || s_grad) {
        if ((rc = check_channels("perception_forward", channels)) != NPA_OK) return rc;
        NPA_REQUIRE(s_bin, "perception_forward", "state_in");
    }
    if (moment && g.dim == 2 && (uintptr_t)moment % 16)
        return fail(NPA_ERR_INVALID_ARGUMENT, "perception_forward: moment must be 16-byte aligned");
    ScalarFwdArgs sa = {x_bin, mass, nullptr, count, rho, rho_grad, nullptr, bin_offsets, block_info, pair_cache, pair_stride};
    if ((rc = launch_scalar_forward(g, smask, sa, st)) != NPA_OK) return rc;
    const int fmask = (s_blur ? F_BLUR : 0) | (s_grad ? F_GRAD : 0);
    if (fmask) {
        if ((rc = check_channels("perception_forward", channels)) != NPA_OK) return rc;
        NPA_REQUIRE(s_bin, "perception_forward", "state_in");
        // the moment matrix shares every pair scalar with the gradient: fold it into the same sweep
        const bool fold = moment && fmask == (F_BLUR | F_GRAD);
        if ((rc = check_pair_cache("perception_forward", pair_cache, pair_stride)) != NPA_OK) return rc;
        FeatureFwdArgs fa = {x_bin, mass, rho, s_bin, s_blur, s_grad, channels, bin_offsets, block_info,
                             fold ? moment : nullptr};
        fa.pair_cache = pair_cache;
        fa.pair_stride = pair_stride;
        fa.pair_cache_valid = pair_cache != nullptr;  // written by the density sweep above
        if ((rc = launch_feature_forward(g, fold ? (fmask | F_MOMENT) : fmask, fa, st)) != NPA_OK) return rc;
        if (fold) moment = nullptr;
    }
    if (moment) {
        if (g.dim == 2 && (uintptr_t)moment % 16)
            return fail(NPA_ERR_INVALID_ARGUMENT, "perception_forward: moment must be 16-byte aligned");
        ScalarFwdArgs ma = {x_bin, mass, rho, nullptr, nullptr, nullptr, moment, bin_offsets, block_info};
        if ((rc = launch_scalar_forward(g, S_MOMENT, ma, st)) != NPA_OK) return rc;
    }
    return NPA_OK;
}

int npa_perception_backward(const npa_grid *gd, int32_t channels, const float *x_bin, const float *mass,
                            const float *s_bin, const float *rho, const float *dL_drho_out,
                            const float *dL_dblur, const float *dL_dgrad, const float *dL_drho_grad,
                            float *grad_x, float *grad_s, float *grad_rho_scratch,
                            const int32_t *bin_offsets, const int32_t *block_info, const int32_t *pair_cache, int32_t pair_stride, void *stream) {
    Geom g;
    int rc = begin_op("perception_backward", gd, &g, x_bin, bin_offsets, block_info);
    if (rc != NPA_OK) return rc;
    if ((rc = check_grad_x("perception_backward", g, grad_x)) != NPA_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int fmask = (dL_dblur ? F_BLUR : 0) | (dL_dgrad ? F_GRAD : 0);
    const bool full = grad_x != nullptr;
    if (full && fmask && !grad_rho_scratch)
        return fail(NPA_ERR_INVALID_ARGUMENT, "perception_backward: grad_rho_scratch is required when grad_x is requested");
    bool x_written = false;
    if (fmask && (grad_s || full)) {
        if ((rc = check_channels("perception_backward", channels)) != NPA_OK) return rc;
        NPA_REQUIRE(s_bin, "perception_backward", "state_in");
        NPA_REQUIRE(rho, "perception_backward", "rho");
        if ((rc = check_pair_cache("perception_backward", pair_cache, pair_stride)) != NPA_OK) return rc;
        FeatureBwdArgs fa = {x_bin, mass, rho, s_bin, dL_dblur, dL_dgrad, grad_x, grad_s,
                             full ? grad_rho_scratch : nullptr, channels, bin_offsets, block_info, pair_cache, pair_stride};
        if ((rc = launch_feature_backward(g, fmask, full, fa, st)) != NPA_OK) return rc;
        x_written = full;
    } else if (grad_s) {
        cudaError_t e = cudaMemsetAsync(grad_s, 0, sizeof(float) * (size_t)g.B * g.N * (channels > 0 ? channels : 0), st);
        if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaMemsetAsync(grad_s): %s", cudaGetErrorString(e));
    }
    if (full) {
        const float *ga = dL_drho_out;
        const float *gb = x_written ? grad_rho_scratch : nullptr;
        const int smask = ((ga || gb) ? S_DENSITY : 0) | (dL_drho_grad ? S_DGRAD : 0);
        if (smask) {
            ScalarBwdArgs sa = {x_bin, mass, nullptr, ga, gb, dL_drho_grad, nullptr, grad_x, nullptr,
                                x_written ? 1 : 0, bin_offsets, block_info, pair_cache, pair_stride};
            if ((rc = launch_scalar_backward(g, smask, sa, st)) != NPA_OK) return rc;
        } else if (!x_written) {
            cudaError_t e = cudaMemsetAsync(grad_x, 0, sizeof(float) * (size_t)g.B * g.N * (g.dim == 2 ? 2 : 4), st);
            if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "cudaMemsetAsync(grad_x): %s", cudaGetErrorString(e));
        }
    }
    return NPA_OK;
}

int npa_row_tickets_status(int32_t *host_nonzero_words, int32_t reset) {
    if (!host_nonzero_words) return fail(NPA_ERR_INVALID_ARGUMENT, "row_tickets_status: host_nonzero_words is NULL");
    int n = 0;
    const int rc = row_tickets_status(&n, reset != 0);
    if (rc == NPA_OK) *host_nonzero_words = n;
    return rc;
}

}  // extern "C"
