// Argument blocks and launch functions of the perception kernels; the glue
// between the C ABI (capi.cu) and the kernel translation units.
#pragma once
#include "common.cuh"

namespace npa {

// Which per-particle scalar operators a sweep computes.
enum { S_COUNT = 1, S_DENSITY = 2, S_DGRAD = 4, S_MOMENT = 8 };
// Which feature operators a sweep computes.
// F_MOMENT (forward only) adds the moment matrix to a blur + gradient sweep.
// F_PACK (forward only, with all three others) applies the perception epilogue per particle and
// writes the packed perception vector instead of the separate tensors.
enum { F_BLUR = 1, F_GRAD = 2, F_MOMENT = 4, F_PACK = 8 };
bool tile_forward_enabled();  // tile_host.cu: the cell-tile streaming engine is switched on for forward sweeps

struct ScalarFwdArgs {
    const float *x;       // [B,N,P] cell order
    const float *mass;    // [B,N] or NULL (all ones)
    const float *rho_in;  // [B,N], only for S_MOMENT
    float *count;         // [B,N]
    float *rho_out;       // [B,N]
    float *rho_grad;      // [B,N,D]
    float *moment;        // [B,N,D,D]
    const int32_t *bin_offsets;
    const int32_t *block_info;
    int32_t *pair_cache;  // neighbour lists to write ([B*N, pair_stride]) or NULL
    int pair_stride;
    unsigned int *tickets;  // row tickets of this launch (set by the launcher)
};

struct ScalarBwdArgs {
    const float *x;
    const float *mass;
    const float *rho_in;      // S_MOMENT
    const float *g_rho_a;     // upstream of density output; the two are summed, either may be NULL
    const float *g_rho_b;
    const float *g_rho_grad;  // upstream of density gradient [B,N,D]
    const float *g_moment;    // upstream of moment matrix [B,N,D,D]
    float *grad_x;            // [B,N,P]
    float *grad_rho;          // [B,N], S_MOMENT only
    int accumulate_x;         // add into grad_x instead of overwriting
    const int32_t *bin_offsets;
    const int32_t *block_info;
    const int32_t *pair_cache;  // neighbour lists of this snapshot to read, or NULL
    int pair_stride;
    unsigned int *tickets;  // row tickets of this launch (set by the launcher)
};

struct FeatureFwdArgs {
    const float *x;
    const float *mass;
    const float *rho;
    const float *s;      // [B,N,C]
    float *blur;         // [B,N,C]
    float *grad;         // [B,N,C,D]
    int C;
    const int32_t *bin_offsets;
    const int32_t *block_info;
    float *moment;       // [B,N,D,D], only with F_MOMENT
    // ---- F_PACK: z[i] = [ s_i | blur_i | lognorm(coef * grad_i @ safe_inv(M_i)) | lognorm(dg_scale * rho_grad_i) ]
    float *z;                // [B,N,zstride], zstride = 2C + C*D + D
    int zstride;
    float *vgrad;            // [B,N,C,D] or NULL: grad_i @ safe_inv(M_i), kept for the backward pass
    const float *rho_grad;   // [B,N,D] density gradient of the same positions, or NULL when rho_grad_out is set
    float *rho_grad_out;     // [B,N,D] or NULL: the packed sweep computes the density gradient itself and writes it here
    float coef, dg_scale, inv_tol;
    int log_norm_grad, log_norm_dg;
    // ---- neighbour list cache (optional): row i = [count | j_0 .. j_{count-1}], count = -1 when the
    // particle has more than pair_stride - 1 neighbours (the reader then searches the cells itself)
    int32_t *pair_cache;     // [B*N, pair_stride] or NULL
    int pair_stride;
    int pair_cache_valid;    // 0: this sweep writes the lists; 1: they are valid, read them instead of searching
    unsigned int *tickets;  // row tickets of this launch (set by the launcher)
};

struct FeatureBwdArgs {
    const float *x;
    const float *mass;
    const float *rho;
    const float *s;
    const float *g_blur;  // [B,N,C]
    const float *g_grad;  // [B,N,C,D]
    float *grad_x;        // [B,N,P] or NULL
    float *grad_s;        // [B,N,C] or NULL
    float *grad_rho;      // [B,N] or NULL
    int C;
    const int32_t *bin_offsets;
    const int32_t *block_info;
    const int32_t *pair_cache;  // neighbour lists written by the forward sweep of the same snapshot, or NULL
    int pair_stride;
    unsigned int *tickets;  // row tickets of this launch (set by the launcher)
};

// Number of CTAs of a persistent launch of `kernel`: every SM filled to the kernel's occupancy.
// Cached per (device, kernel); the first call also raises the kernel's dynamic shared-memory
// limit to what it needs.  Defined in capi.cu.
int persistent_ctas_impl(const void *kernel, int threads, size_t dyn_smem, int *out);
template <typename Kernel>
int persistent_ctas(Kernel kernel, int threads, size_t dyn_smem, int *out) {
    return persistent_ctas_impl(reinterpret_cast<const void *>(kernel), threads, dyn_smem, out);
}

// Two zeroed words in device memory for the row tickets of one persistent launch (next_row /
// release_rows in neighbors.cuh).  They live in a small array inside the library, handed out round
// robin: launches in one stream are ordered, and launches in different streams get different words
// unless hundreds of launches lie between them.  Launches recorded into a CUDA graph draw from a
// separate half of the array, so a replaying graph never shares words with an eager launch.
// Defined in capi.cu.
int acquire_row_tickets(cudaStream_t st, unsigned int **out);

// The same sweeps on the cell-tile streaming engine (feature_tile.cuh).  *taken = false means the
// engine does not cover this call (nothing was launched) and the gather kernel must run.
template <int D, bool PER>
int launch_feature_tile_forward(const Geom &g, int mask, const FeatureFwdArgs &a, cudaStream_t st, bool *taken);
template <int D, bool PER, bool FULL>
int launch_feature_tile_backward(const Geom &g, int mask, const FeatureBwdArgs &a, cudaStream_t st, bool *taken);

int launch_scalar_forward(const Geom &g, int mask, const ScalarFwdArgs &a, cudaStream_t st);
int launch_scalar_backward(const Geom &g, int mask, const ScalarBwdArgs &a, cudaStream_t st);
int launch_feature_forward(const Geom &g, int mask, const FeatureFwdArgs &a, cudaStream_t st);
// full = false differentiates with respect to s only.
int launch_feature_backward(const Geom &g, int mask, bool full, const FeatureBwdArgs &a, cudaStream_t st);

}  // namespace npa
