/*
 * npa_b200 -- C ABI of the B200 (sm_100a) SPH neighbour-perception library.
 *
 * Every entry point replaces one method of the reference's native module
 * `sph_cuda` (sphops/sph_cuda.cu, bound with nanobind at sph_cuda.cu:3229-3441)
 * and is what a ctypes / nanobind / pybind11 stub on the reference side binds.
 *
 * Conventions
 *  - All pointers are DEVICE pointers unless the name says "host".  Float
 *    tensors are contiguous fp32, index tensors contiguous int32.
 *  - Positions are [B, N, P] with P = 2 (dim 2) or P = 4 (dim 3, w ignored on
 *    input and written as 0 on output), as in the reference
 *    (sphops/utils.cuh:14-111, sph_cuda.cu:1898).
 *  - Inputs are const, outputs and scratch are caller-allocated; the library
 *    allocates nothing and never synchronises.  What it keeps between calls:
 *    the thread-local text returned by npa_last_error(), per-device launch
 *    sizes, and a small device array of row-ticket counters that its sweep
 *    kernels draw work from (two words per launch, zero again when the launch
 *    ends).  Slots are handed out round robin, 4096 for eager launches: sweeps
 *    issued on different streams must lie fewer than 4096 launches apart to be
 *    sure of distinct words.  Launches recorded under stream capture draw from
 *    4096 further slots that are never reused (the graph owns them); the 4097th
 *    captured sweep of a process is refused with NPA_ERR_UNSUPPORTED.  The first call of an operator on a device queries those once:
 *    make it before any stream capture.
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *  - Return value: NPA_OK (0) or a negative npa_status.  Arguments are checked
 *    before the first kernel of a call is enqueued, so an argument error means
 *    nothing has been launched; only a failing kernel launch (NPA_ERR_CUDA) can
 *    interrupt a multi-kernel call midway.  No C++ exception crosses this boundary.
 *  - `mass` may be NULL: every particle then has mass 1.0
 *    (sphops/sph.py:11-14, sph_cuda.cu:1843).
 */
#ifndef NPA_B200_H
#define NPA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NPA_B200_ABI_VERSION 1

typedef enum npa_status {
    NPA_OK = 0,
    NPA_ERR_INVALID_ARGUMENT = -1, /* bad geometry, NULL pointer, size mismatch  */
    NPA_ERR_UNSUPPORTED = -2,      /* e.g. Morton hash on a non power-of-two grid */
    NPA_ERR_CUDA = -3,             /* a CUDA runtime call / launch failed         */
    NPA_ERR_SCRATCH_TOO_SMALL = -4 /* scratch_bytes < npa_grid_scratch_bytes()    */
} npa_status;

/* Boundary condition, sphops/utils.cuh:282-286. */
enum { NPA_BOUNDARY_CLAMPED = 0, NPA_BOUNDARY_PERIODIC = 1 };
/* Cell hash order: linear ("grid" mode) or Morton ("particle" mode),
 * sphops/utils.cuh:442-453. */
enum { NPA_HASH_LINEAR = 0, NPA_HASH_MORTON = 1 };

/*
 * Geometry of one HashGrid; replaces the constructor arguments of the eight
 * `{,V}HashGrid{2D,3D}{Periodic,Box}` classes (sph_cuda.cu:3049-3093, ctor
 * `(gx, gy[, gz], eps, particle_count, batch_size, max_particles_per_block)`).
 * Plain data, passed by pointer and copied; the library keeps no reference.
 */
typedef struct npa_grid {
    int32_t dim;        /* 2 or 3                                            */
    int32_t boundary;   /* NPA_BOUNDARY_*                                    */
    int32_t hash;       /* NPA_HASH_*                                        */
    int32_t grid[3];    /* cells per axis (grid[2] ignored when dim == 2)    */
    double eps;         /* cell size == cut-off radius h                     */
    int32_t batch;      /* B, independent particle systems                   */
    int32_t particles;  /* N, particles per system                           */
    int32_t max_particles_per_block; /* MPB: a work item covers <= MPB particles of one cell */
} npa_grid;

/* Text of the last error raised on the calling thread ("" if none). */
const char *npa_last_error(void);
/* NPA_B200_ABI_VERSION the library was built with. */
int npa_abi_version(void);

/* Cells per system (product of grid[0..dim)), or a negative npa_status. */
int64_t npa_grid_num_cells(const npa_grid *g);
/* Rows of `block_info`: B * min(N, cells + ceil(N / MPB))
 * (sph_cuda.cu:1851-1853).  Unlike the reference, the same size is used with
 * the Morton hash, because the work list drives every kernel here. */
int64_t npa_grid_max_blocks(const npa_grid *g);
/* Bytes of device scratch npa_grid_build() needs (cell histogram, arrival numbers,
 * cell ids, unsorted slots, scan partials); replaces the cudaMalloc'ed members
 * of the reference's HashGrid (sph_cuda.cu:1881-1895). */
int64_t npa_grid_scratch_bytes(const npa_grid *g);

/*
 * Uniform-grid binning; replaces HashGrid::initialize (sph_cuda.cu:1926-1992:
 * grid_count_particles, two CUB scans, grid_compute_permutation,
 * assign_block_info).
 *   x            [B, N, P]            in
 *   permutation  [B, N]               out: destination slot of particle i inside its system
 *   bin_offsets  [B*cells + 1]        out: exclusive scan of the cell counts over all systems
 *                                          (entry b*cells + c includes b*N; last entry = B*N)
 *   block_info   [max_blocks, 4]      out: (global cell, offset in cell, particle count, system)
 *                                          per work item, in cell order; unused tail rows are zero
 *   scratch      scratch_bytes        scratch, contents undefined on entry and exit
 * The slot order inside a cell is the original particle order (a stable
 * counting sort), so the result is deterministic; the reference's order inside
 * a cell depends on atomic arrival order (sph_cuda.cu:81-83).
 */
int npa_grid_build(const npa_grid *g, const float *x, int32_t *permutation,
                   int32_t *bin_offsets, int32_t *block_info, void *scratch,
                   int64_t scratch_bytes, void *stream);

/*
 * Same binning as npa_grid_build(), for callers that cannot hand over scratch memory.
 * (No counterpart in the reference: its grid object cudaMallocs its work arrays.)
 *
 * Who needs this: a host program that owns all device memory itself -- a simulation or
 * inference server that partitions the GPU into fixed arenas at start-up, or a plugin host
 * that only passes in the buffers it registered -- and therefore forbids its plugins to call
 * cudaMalloc (an allocation there can fail late, fragments the arena, and synchronises the
 * whole device in the middle of a step).  Such a caller still passes x and the three outputs,
 * but has nowhere to take the work arrays from.
 *
 * The work arrays live in one fixed array inside the library (device global memory,
 * NPA_STATIC_SCRATCH_BYTES, reserved on every GPU that loads the library until the process
 * exits).  Consequences:
 *   - geometries with npa_grid_scratch_bytes(g) > NPA_STATIC_SCRATCH_BYTES are refused with
 *     NPA_ERR_SCRATCH_TOO_SMALL and nothing is launched;
 *   - the first call on each device looks up the array's device address (one host-side query,
 *     with that device current); make that first call before starting any stream capture;
 *   - all calls on one device share the array: two calls whose kernels can overlap on the GPU
 *     (different streams, no ordering between them) race on it.  Calls on one stream are safe;
 *     the parts that must start from zero are cleared at the start of every call;
 *   - nothing is allocated or freed, here or in any library routine this call uses.
 */
#define NPA_STATIC_SCRATCH_BYTES (8u << 20)
int npa_grid_build_static(const npa_grid *g, const float *x, int32_t *permutation,
                          int32_t *bin_offsets, int32_t *block_info, void *stream);

/*
 * Reorder into cell order: out[perm[i]] = in[i].  Replaces
 * HashGrid::bin_particles (sph_cuda.cu:1994-2024, kernel apply_permutation
 * :86-123).  Any of the (in, out) pairs may be NULL together to skip it.
 *   x/x_out [B,N,P]   s/s_out [B,N,C]   mass/mass_out [B,N]
 */
int npa_bin_particles(const npa_grid *g, int32_t channels, const float *x,
                      const float *s, const float *mass,
                      const int32_t *permutation, float *x_out, float *s_out,
                      float *mass_out, void *stream);

/*
 * Inverse reorder: out[i] = in[perm[i]].  Replaces
 * HashGrid::backward_bin_particles (sph_cuda.cu:2026-2056, kernel
 * backward_apply_permutation :125-167); also what unbin_particles calls
 * (sphops/sph.py:187-198).
 */
int npa_unbin_particles(const npa_grid *g, int32_t channels, const float *x_bin,
                        const float *s_bin, const float *mass_bin,
                        const int32_t *permutation, float *x_out, float *s_out,
                        float *mass_out, void *stream);

/* ---- single-operator forward passes (inputs are in cell order) ---------- */

/* count[B,N] = number of j with |x_j - x_i|^2 < h^2, self included.
 * Replaces HashGrid::count_forward (sph_cuda.cu:2127-2189). */
int npa_count_forward(const npa_grid *g, const float *x_bin, float *count,
                      const int32_t *bin_offsets, const int32_t *block_info,
                      void *stream);

/* rho[B,N] = c_s * sum_j m_j (h^2 - r^2)^3.
 * Replaces HashGrid::density_forward (sph_cuda.cu:2058-2125). */
int npa_density_forward(const npa_grid *g, const float *x_bin, const float *mass,
                        float *rho, const int32_t *bin_offsets,
                        const int32_t *block_info, void *stream);

/* out[B,N,C] = c_s * sum_j s_j (m_j / rho_j) (h^2 - r^2)^3.
 * Replaces HashGrid::blur_forward (sph_cuda.cu:2191-2277). */
int npa_blur_forward(const npa_grid *g, int32_t channels, const float *x_bin,
                     const float *rho, const float *mass, const float *s_bin,
                     float *s_blur, const int32_t *bin_offsets,
                     const int32_t *block_info, void *stream);

/* out[B,N,C,D] = c_g * sum_j (s_j - s_i) (m_j / rho_j) 3(h-r)^2/r (x_j - x_i).
 * Replaces HashGrid::gradient_forward (sph_cuda.cu:2279-2365). */
int npa_gradient_forward(const npa_grid *g, int32_t channels, const float *x_bin,
                         const float *rho, const float *mass, const float *s_bin,
                         float *s_grad, const int32_t *bin_offsets,
                         const int32_t *block_info, void *stream);

/* out[B,N,D] = c_g * sum_j m_j 3(h-r)^2/r (x_j - x_i).
 * Replaces HashGrid::density_gradient_forward (sph_cuda.cu:2367-2431). */
int npa_density_gradient_forward(const npa_grid *g, const float *x_bin,
                                 const float *mass, float *rho_grad,
                                 const int32_t *bin_offsets,
                                 const int32_t *block_info, void *stream);

/* out[B,N,D,D] = c_g * sum_j (m_j / rho_j) 3(h-r)^2/r (x_j-x_i)(x_j-x_i)^T.
 * Replaces HashGrid::moment_matrix_forward (sph_cuda.cu:2433-2499). */
int npa_moment_matrix_forward(const npa_grid *g, const float *x_bin,
                              const float *rho, const float *mass, float *moment,
                              const int32_t *bin_offsets,
                              const int32_t *block_info, void *stream);

/* ---- single-operator backward passes ------------------------------------ *
 * Each `grad_*` output may be NULL: that gradient is then not computed (the
 * reference's dLdx / dLds / dLdrho flags, sph_cuda.cu:2624,2854).           */

/* Replaces HashGrid::density_backward (sph_cuda.cu:2501-2578). */
int npa_density_backward(const npa_grid *g, const float *x_bin, const float *mass,
                         const float *dL_drho, float *grad_x,
                         const int32_t *bin_offsets, const int32_t *block_info,
                         void *stream);

/* Replaces HashGrid::blur_backward (sph_cuda.cu:2580-2728). */
int npa_blur_backward(const npa_grid *g, int32_t channels, const float *x_bin,
                      const float *rho, const float *mass, const float *s_bin,
                      const float *dL_dblur, float *grad_x, float *grad_s,
                      float *grad_rho, const int32_t *bin_offsets,
                      const int32_t *block_info, void *stream);

/* Replaces HashGrid::gradient_backward (sph_cuda.cu:2810-2958). */
int npa_gradient_backward(const npa_grid *g, int32_t channels, const float *x_bin,
                          const float *rho, const float *mass, const float *s_bin,
                          const float *dL_dgrad, float *grad_x, float *grad_s,
                          float *grad_rho, const int32_t *bin_offsets,
                          const int32_t *block_info, void *stream);

/* Replaces HashGrid::density_gradient_backward (sph_cuda.cu:2730-2808). */
int npa_density_gradient_backward(const npa_grid *g, const float *x_bin,
                                  const float *mass, const float *dL_drho_grad,
                                  float *grad_x, const int32_t *bin_offsets,
                                  const int32_t *block_info, void *stream);

/* Replaces HashGrid::moment_matrix_backward (sph_cuda.cu:2960-3046). */
int npa_moment_matrix_backward(const npa_grid *g, const float *x_bin,
                               const float *rho, const float *mass,
                               const float *dL_dmoment, float *grad_x,
                               float *grad_rho, const int32_t *bin_offsets,
                               const int32_t *block_info, void *stream);

/* out = inverse of each symmetric DxD matrix, identity when |det| < tol.
 * n = number of matrices (B*N).  Replaces the module function
 * safe_inv_sym_mat (sph_cuda.cu:3095-3226). */
int npa_safe_inv_sym_mat(int32_t dim, int64_t n, const float *m, float *m_inv,
                         float tol, void *stream);

/* ---- neighbour list cache ---------------------------------------------------- *
 * All sweeps over one snapshot visit the same pairs.  The fused entry points
 * below take an optional cache  pair_cache [B*N, pair_stride] (int32,
 * caller-allocated; NULL = off): the first sweep that searches the cells (the
 * density sweep of npa_perception_forward / npa_perceive_features_forward, or
 * npa_blur_gradient_forward with pair_cache_valid == 0) records, per particle,
 * the number of accepted neighbours and their indices (row = count, j_0, j_1,
 * ...; count = -1 when there are more than pair_stride - 1); every later sweep
 * given the same cache (pair_cache_valid != 0 for a forward sweep; all backward
 * sweeps) rebuilds the displacements from the list instead of testing the ~3^D
 * cells of candidates again (particles marked -1 are searched as usual).
 * The cache belongs to one snapshot AND one set of positions.  2 <= pair_stride
 * <= 513.  No counterpart in the reference.                                   */

/* ---- blur + gradient in one launch ------------------------------------------ *
 * The two feature operators share every pair test and every neighbour feature
 * load, so one sweep produces both.  Results equal npa_blur_* / npa_gradient_*
 * (sph_cuda.cu:2191-2365 forward, :2580-2728 and :2810-2958 backward); either
 * output (forward) or upstream gradient (backward) may be NULL.  `moment`
 * [B,N,D,D] (may be NULL) additionally returns the moment matrix
 * (npa_moment_matrix_forward), which shares every pair factor with the
 * gradient; it needs both s_blur and s_grad.                                  */
int npa_blur_gradient_forward(const npa_grid *g, int32_t channels, const float *x_bin,
                              const float *rho, const float *mass, const float *s_bin,
                              float *s_blur, float *s_grad, float *moment,
                              const int32_t *bin_offsets, const int32_t *block_info, int32_t *pair_cache, int32_t pair_stride,
                              int32_t pair_cache_valid, void *stream);

/* grad_x == NULL and grad_rho == NULL selects the variant that differentiates
 * with respect to s only. */
int npa_blur_gradient_backward(const npa_grid *g, int32_t channels, const float *x_bin,
                               const float *rho, const float *mass, const float *s_bin,
                               const float *dL_dblur, const float *dL_dgrad, float *grad_x,
                               float *grad_s, float *grad_rho, const int32_t *bin_offsets,
                               const int32_t *block_info, const int32_t *pair_cache, int32_t pair_stride, void *stream);

/* ---- density + density gradient backward in one launch ---------------------- *
 * Gradient with respect to the positions of  rho = density(x)  and
 * density_gradient(x)  in one sweep (sph_cuda.cu:2501-2578 and :2730-2808 as two
 * launches in the reference).  The upstream gradient of rho is the sum of
 * dL_drho_a and dL_drho_b (either may be NULL), which is how the gradient that
 * blur / gradient return for their rho input joins the one given for rho
 * itself; dL_drho_grad may be NULL.  With accumulate != 0 the result is added
 * to grad_x instead of overwriting it.                                        */
int npa_density_chain_backward(const npa_grid *g, const float *x_bin, const float *mass,
                               const float *dL_drho_a, const float *dL_drho_b,
                               const float *dL_drho_grad, float *grad_x, int32_t accumulate,
                               const int32_t *bin_offsets, const int32_t *block_info,
                               const int32_t *pair_cache,
                               int32_t pair_stride, void *stream);

/* ---- fused perception (one launch set for what NPA.perceive asks for) ---- *
 * The reference runs density, blur, gradient, density_gradient and
 * moment_matrix as separate launches that each re-stage the same neighbour
 * cells (models/npa.py:105-126, sphops/sph.py:474-484).  These two calls
 * produce the same tensors in two sweeps forward (rho must be complete before
 * a neighbour's m/rho can be used) and two sweeps backward.                  */

/*
 * Forward.  Sweep 1 writes rho (required) and, when non-NULL, count and
 * rho_grad; sweep 2 writes s_blur and s_grad (either may be NULL) and, when
 * non-NULL, moment.  Results equal the single-operator calls above.
 */
int npa_perception_forward(const npa_grid *g, int32_t channels,
                           const float *x_bin, const float *mass,
                           const float *s_bin, float *rho, float *count,
                           float *rho_grad, float *s_blur, float *s_grad,
                           float *moment, const int32_t *bin_offsets,
                           const int32_t *block_info, int32_t *pair_cache, int32_t pair_stride, void *stream);

/*
 * Backward of  rho = density(x); blur(x, rho, s); gradient(x, rho, s);
 * density_gradient(x)  as one autograd chain.  Upstream gradients dL_drho_out,
 * dL_dblur, dL_dgrad, dL_drho_grad may each be NULL (treated as zero).
 * Sweep 1 differentiates blur + gradient and writes grad_s, the rho gradient
 * (into grad_rho_scratch [B,N], required when grad_x is requested) and the
 * first part of grad_x; sweep 2 pushes (dL_drho_out + grad_rho_scratch) through
 * density and dL_drho_grad through density_gradient and adds into grad_x.
 * grad_x == NULL selects the cheaper variant that differentiates with respect
 * to s only (the reference's COMPUTE_DS_ONLY kernels, sph_cuda.cu:2624,2854).
 */
int npa_perception_backward(const npa_grid *g, int32_t channels,
                            const float *x_bin, const float *mass,
                            const float *s_bin, const float *rho,
                            const float *dL_drho_out, const float *dL_dblur,
                            const float *dL_dgrad, const float *dL_drho_grad,
                            float *grad_x, float *grad_s, float *grad_rho_scratch,
                            const int32_t *bin_offsets, const int32_t *block_info,
                            const int32_t *pair_cache, int32_t pair_stride, void *stream);

/* ---- packed perception: the MLP input row of NPA.perceive in two sweeps ------- *
 * No single counterpart in the reference: replaces the operator calls AND the
 * torch glue of NPA.perceive (models/npa.py:87-137) with its defaults
 * state_grad = density_grad = True:
 *   rho = density(x); blur(x, rho, s); gradient_hybrid(x, rho, s) (sphops/sph.py:474-484,
 *   value raw @ safe_inv_sym_mat(moment, inv_tol), gradient of the raw operator);
 *   density_gradient(x); then  z[i] = [ s_i | blur_i | LN(coef * grad_i) | LN(dg_scale * rho_grad_i) ],
 *   LN(w) = log(1 + |w|) w / |w| when the matching log_norm flag is set, else w.
 * NPA uses coef = eps / eps0 and dg_scale = coef^(1 + dim) / N.
 *   z [B,N,2C + C*D + D] out;  rho [B,N], rho_grad [B,N,D] out (needed by backward);
 *   vgrad [B,N,C,D] out or NULL: the corrected gradient before scaling, needed by backward.
 * Supports channels <= 128 when channels % 4 == 0 (else <= 32); NPA_ERR_UNSUPPORTED otherwise. */
int npa_perceive_features_forward(const npa_grid *g, int32_t channels, const float *x_bin,
                                  const float *mass, const float *s_bin, float coef,
                                  float dg_scale, float inv_tol, int32_t log_norm_grad,
                                  int32_t log_norm_dg, float *rho, float *rho_grad, float *z,
                                  float *vgrad, const int32_t *bin_offsets,
                                  const int32_t *block_info, int32_t *pair_cache, int32_t pair_stride, void *stream);

/* Backward of the above: dL_dz [B,N,2C+C*D+D] -> grad_s [B,N,C] and, when grad_x != NULL,
 * grad_x [B,N,P] (through blur, gradient, density and density gradient, as autograd would).
 * Scratch (caller-allocated, contents undefined): g_blur_scratch [B,N,C], g_grad_scratch
 * [B,N,C,D]; with grad_x also g_rho_grad_scratch [B,N,D] and grad_rho_scratch [B,N]. */
int npa_perceive_features_backward(const npa_grid *g, int32_t channels, const float *x_bin,
                                   const float *mass, const float *s_bin, const float *rho,
                                   const float *rho_grad, const float *vgrad, const float *dL_dz,
                                   float coef, float dg_scale, int32_t log_norm_grad,
                                   int32_t log_norm_dg, float *g_blur_scratch,
                                   float *g_grad_scratch, float *g_rho_grad_scratch,
                                   float *grad_rho_scratch, float *grad_x, float *grad_s,
                                   const int32_t *bin_offsets, const int32_t *block_info,
                                   const int32_t *pair_cache, int32_t pair_stride, void *stream);

/* ---- the Euler update after perception and the per-particle MLP ----------------- *
 * Replaces the elementwise torch code of NPA.forward (models/npa.py:145-153, the
 * displacement limiter) and of step_euler (models/npa.py:183-203) and, with
 * wrap != 0 on a periodic grid, HashGrid.wrap_positions (sphops/sph.py:107-123).
 *   y [B,N,D+C]   MLP output in cell order: D raw displacement columns, C state updates
 *   dx = alpha * y[:D] * eps / (1 + |y[:D]|)           (eps = the grid's cell size)
 *   x_out = x_bin + dt * dx * mask      (P columns; the 3D padding column is copied)
 *   s_out = s_bin + dt * y[D:] * mask
 * mask [B,N] holds 0 / 1 per particle (the reference draws rand < update_prob), NULL = all
 * ones.  The reference's optional position noise is not part of this call. */
int npa_step_update_forward(const npa_grid *g, const float *y, const float *x_bin, const float *s_bin,
                            const float *mask, int32_t channels, float alpha, float dt, int32_t wrap,
                            float *x_out, float *s_out, void *stream);

/* dL/dy [B,N,D+C] from the upstream gradients of x_out [B,N,P] and s_out [B,N,C] (either
 * may be NULL = zero).  The gradients with respect to x_bin and s_bin are the upstream
 * gradients themselves and need no kernel. */
int npa_step_update_backward(const npa_grid *g, const float *y, const float *mask, int32_t channels,
                             float alpha, float dt, const float *g_x_out, const float *g_s_out, float *g_y,
                             void *stream);

/* ---- 2D Gaussian splatting of particles into an image --------------------------- *
 * Replaces splat_particles / splat_particles_batch (utils/splatting.py:6-113), the
 * renderer of the reference's splat loss (losses/splat_loss.py:71-86).
 *   x [B,N,2] world positions, color [B,N,3]; out [B,img,img,4] = (r, g, b, density).
 *   pixel position p = (x - lo) / (hi - lo) * (img - 1), y flipped when y_up != 0;
 *   a particle adds w(dx,dy) = exp(-((dx - frac_x)^2 + (dy - frac_y)^2) / (2 sigma^2)) to the
 *   pixels floor(p) + (dx,dy), |dx|,|dy| <= radius, that lie inside the image; with
 *   normalize != 0, w is divided by (1e-8 + its sum over the whole patch) and multiplied by
 *   norm_scale.  sigma_pixels, radius and norm_scale are the values the reference derives
 *   from (sigma, img_size, pixel_size, lo, hi) at utils/splatting.py:43-46,75-77.
 * scale_scratch [B*N] floats (contents undefined) is needed when normalize != 0.
 * Every pixel of out is written; sums run in particle order (deterministic). */
int npa_splat_forward(const float *x, const float *color, int32_t batch, int32_t particles, int32_t img_size,
                      double sigma_pixels, int32_t radius, double lo, double hi, int32_t y_up,
                      int32_t normalize, double norm_scale, float *scale_scratch, float *out, void *stream);

/* Gradients of npa_splat_forward: g_x [B,N,2] and g_color [B,N,3] (either may be NULL)
 * from g_out [B,img,img,4]. */
int npa_splat_backward(const float *x, const float *color, const float *g_out, int32_t batch, int32_t particles,
                       int32_t img_size, double sigma_pixels, int32_t radius, double lo, double hi, int32_t y_up,
                       int32_t normalize, double norm_scale, float *g_x, float *g_color, void *stream);

/* ---- weight gradients of the per-particle MLP ------------------------------------ *
 * The adaptation MLP of an NPA model (models/npa.py:63-75) is Linear(in, 128) -> ReLU ->
 * Linear(128, out, bias = False), applied to every particle.  One pass over the rows gives
 *   dW1 [128, in] = dh^T z,   dW2 [out, 128] = dy^T h,   db1 [128] = sum over rows of dh
 * from z [rows, in] (the perception rows), h [rows, 128] (hidden activations after the ReLU),
 * dh [rows, 128] (gradient at the hidden layer, ReLU mask applied) and dy [rows, out]; these
 * replace three tall-skinny library kernels of torch's autograd.  hidden must be 128, in <= 176,
 * out <= 48.  scratch (contents undefined) holds the per-CTA partial sums, which are added in a
 * fixed order: the results are deterministic.  The outputs are overwritten, not accumulated. */
int64_t npa_mlp_weight_grad_scratch_floats(int64_t rows, int32_t in_dim, int32_t out_dim);
int npa_mlp_weight_grad(const float *z, const float *dh, const float *h, const float *dy, int64_t rows,
                        int32_t in_dim, int32_t hidden, int32_t out_dim, float *scratch, int64_t scratch_floats,
                        float *dW1, float *dW2, float *db1, void *stream);

/* Gradient at the hidden layer with the ReLU mask: dh [rows, 128] = (dy [rows, out] . W2 [out, 128]) where
 * h > 0, else 0 -- the backward of Linear(128, out, bias = False) and of the ReLU that produced h
 * (models/npa.py:63-75) in one pass (torch: a thin GEMM plus a masking pass).  fp32 on the CUDA cores.
 * hidden must be 128, out <= 48; W2 is addressed through its strides; h and dh 16-byte aligned. */
int npa_mlp_hidden_grad(const float *dy, const float *W2, const float *h, float *dh, int64_t rows,
                        int32_t hidden, int32_t out_dim, int64_t w_stride_out, int64_t w_stride_in, void *stream);

/* The same three reductions on the fifth-generation tensor cores (tcgen05.mma, TF32 head / tail
 * products, accumulators in tensor memory drained into fp32 partial sums every 128 rows so that no
 * accumulation chain of the tensor cores is longer than 48 MMAs).  Same arguments and results as
 * npa_mlp_weight_grad; in <= 175, out <= 48, hidden 128; inputs and scratch 16-byte aligned,
 * scratch with npa_mlp_weight_grad_tcgen05_scratch_floats() floats.  Bounded waits report through
 * npa_linear_tcgen05_status (bits 16, 32, 64: MMA lane, producers, epilogue of this kernel). */
int64_t npa_mlp_weight_grad_tcgen05_scratch_floats(int64_t rows, int32_t in_dim, int32_t out_dim);
int npa_mlp_weight_grad_tcgen05(const float *z, const float *dh, const float *h, const float *dy, int64_t rows,
                                int32_t in_dim, int32_t hidden, int32_t out_dim, float *scratch,
                                int64_t scratch_floats, float *dW1, float *dW2, float *db1, void *stream);

/* ---- linear layers of the MLP on the tensor cores, fp32 accuracy ----------------- *
 *   C [rows, out] = act( A [rows, in] . B + bias ),  B[k][n] = W[n * w_stride_out + k * w_stride_in]
 * with act = ReLU when relu != 0; bias [out] may be NULL; with gate [rows, out] != NULL the output
 * is zero where gate <= 0 (the backward of a ReLU whose output is gate).  torch's F.linear(x, W) with
 * W [out, in] is (w_stride_out, w_stride_in) = (in, 1); x @ W with W [in, out] is (1, out).
 * Each product is three TF32 tensor-core MMAs on operands split into a TF32 head and tail
 * (fp32 accumulation), accurate to ~1e-6 relative.  in, out <= 176 and the weights must fit in
 * shared memory with two 64-row tiles of A (else NPA_ERR_UNSUPPORTED).  Replaces the four SIMT
 * fp32 GEMMs of the adaptation MLP (models/npa.py:63-75,143) and its bias / ReLU passes. */
int npa_linear_tf32x3(const float *A, const float *W, const float *bias, const float *gate, float *C,
                      int64_t rows, int32_t in_dim, int32_t out_dim, int64_t w_stride_out,
                      int64_t w_stride_in, int32_t relu, void *stream);

/*
 * The same product as npa_linear_tf32x3 on the fifth-generation tensor cores: tcgen05.mma with the
 * accumulators in tensor memory, operands split into TF32 head and tail (three MMAs per product, fp32
 * accuracy), tiles of 128 rows, one persistent warp-specialised CTA per SM.  in_dim <= 1024 and
 * out_dim <= 256 (else NPA_ERR_UNSUPPORTED).  `scratch` is device memory of at least
 * npa_linear_tcgen05_scratch_bytes(in_dim, out_dim) bytes, 16-byte aligned, private to the call
 * until its kernels have run: it receives the split, swizzled image of the weights.  Two launches on
 * `stream`.  Every wait inside the kernel is bounded in time; npa_linear_tcgen05_status() copies the
 * device status word to the host (0 = no wait ever gave up; bits 1, 2, 4, 8 = the MMA warp, the
 * weight copies, the producers, the epilogue) and clears it when `reset` is non-zero; it
 * synchronises the device.  Replaces the SIMT fp32 GEMMs of the adaptation MLP
 * (models/npa.py:63-75,143) like npa_linear_tf32x3.
 */
int64_t npa_linear_tcgen05_scratch_bytes(int32_t in_dim, int32_t out_dim);
int npa_linear_tcgen05(const float *A, const float *W, const float *bias, const float *gate, float *C,
                       int64_t rows, int32_t in_dim, int32_t out_dim, int64_t w_stride_out,
                       int64_t w_stride_in, int32_t relu, void *scratch, int64_t scratch_bytes, void *stream);
int npa_linear_tcgen05_status(uint32_t *host_status, int32_t reset);
/* Both layers of the adaptation MLP's forward in the same kernel (models/npa.py:63-75,143):
 *   h [rows, 128] = relu(z [rows, in] . W1^T + b1),   y [rows, out] = h . W2^T   (no bias on the second layer)
 * with h kept in tensor memory between the layers: the epilogue activates the first layer's tile in
 * place, adds its TF32 tail next to it, and the second product reads both from tensor memory as its A
 * operand (W2 resident in shared memory).  h is also stored (the backward needs it).  Hidden width 128,
 * in <= 1024, out <= 64; W1 [128, in] and W2 [out, 128] are addressed through their strides; scratch of
 * npa_mlp_forward_tcgen05_scratch_bytes() bytes, 16-byte aligned; three launches on `stream`; bounded waits
 * and status as npa_linear_tcgen05. */
int64_t npa_mlp_forward_tcgen05_scratch_bytes(int32_t in_dim, int32_t out_dim);
int npa_mlp_forward_tcgen05(const float *z, const float *W1, const float *b1, const float *W2, float *h, float *y,
                            int64_t rows, int32_t in_dim, int32_t out_dim, int64_t w1_stride_out,
                            int64_t w1_stride_in, int64_t w2_stride_out, int64_t w2_stride_in, void *scratch,
                            int64_t scratch_bytes, void *stream);
/* Self-test of those bounded waits: a two-warp kernel in which warp 0 waits `limit_us` (1..1,000,000)
 * on an mbarrier that nothing completes, gives up and raises the kernel's leave flag, and warp 1,
 * waiting on a second such mbarrier with the full limit, leaves through the flag.  device_result[0]
 * and [1] (device memory) both read 1 afterwards; the context stays usable. */
int npa_linear_tcgen05_wait_selftest(int32_t limit_us, int32_t *device_result, void *stream);

/*
 * Cell-tile streaming engine of the blur + gradient sweeps (no counterpart in the reference's
 * binding; the reference stages neighbour cells per block inside forward_kernel / backward_kernel,
 * sphops/sph_cuda.cu:1561-1660, 903-1160, without a switch).
 *
 * When enabled, the fused blur + gradient sweeps (npa_blur_gradient_forward / _backward, the feature
 * sweeps of npa_perception_* and npa_perceive_features_*) stage the rows of a tile's neighbour cells
 * in shared memory with bulk asynchronous copies and read them from there.  The engine takes a call
 * when the hash is linear, channels % 4 == 0 and <= 128, B * N % 4 == 0 and every tensor is 16-byte
 * aligned; anything else runs on the gather kernels, with the same results to rounding.
 *
 * npa_tile_tuning: process-wide switches per direction (backward = 0 / 1): `enabled` = 0 (the
 * default: on the measured workloads the gather kernels are as fast or faster) keeps the direction
 * on the gather kernels; rows_per_stage (multiple of 4), particles_per_tile, stages
 * (<= 4), consumer_warps (8 or 16 per CTA; 24 forward only) and cells_per_tile (work items of up
 * to that many x-adjacent cells share one staged neighbourhood) size the plan, 0 = chosen
 * automatically.  A plan that does not fit in shared memory falls back to the gather kernels.
 *
 * npa_tile_status: every wait inside the engine is bounded; a wait that runs out stores a code in a
 * device word (1: a consumer gave up waiting for copies, 2: the producer gave up waiting for a free
 * stage) and the launch drains without finishing its work.  This call copies the word to
 * *host_status (0 = no wait ever ran out) and, with reset != 0, clears it.  It synchronises the
 * device: call it outside the timed path, e.g. once after a step, never during stream capture.
 */
int npa_tile_tuning(int32_t backward, int32_t enabled, int32_t rows_per_stage,
                    int32_t particles_per_tile, int32_t stages, int32_t consumer_warps,
                    int32_t cells_per_tile);
int npa_tile_status(int32_t *host_status, int32_t reset);
/* Health check of the row-ticket words the sweep kernels draw work from (no counterpart in the
 * reference).  Every sweep leaves its two words zero; with no sweep in flight a non-zero word means a
 * launch was cut short (a sticky CUDA error, a killed context) and later sweeps that draw the same
 * slot would skip rows.  Writes the number of non-zero words to *host_nonzero_words and, with reset
 * != 0, clears them.  Synchronises the device: call it after an error status, never in the timed path
 * or during stream capture. */
int npa_row_tickets_status(int32_t *host_nonzero_words, int32_t reset);
/* The forward sweeps of the scalar operators (count, density, density gradient, moment matrix) on a
 * linear-hash grid let the particles of a tile -- work items of up to cells_per_tile x-adjacent
 * cells, at most 32 particles -- share the candidates they test (the sharing of a staged cell among
 * the threads of a block in sphops/sph_cuda.cu:1664-1690).  Used for the poly6 operators (count,
 * density) on clamped grids and 2D periodic grids, where it is measured faster; adding 100 forces it
 * on 3D periodic grids too.  cells_per_tile = 0 switches back to the per-particle candidate walk;
 * default 3.  Process-wide. */
int npa_scalar_sweep_tuning(int32_t cells_per_tile);
/* Self-test of the bounded waits: one CTA waits for an mbarrier phase that is never completed and
 * writes to *device_result (int32, device memory) 1 when the wait gave up after limit_us
 * microseconds (the expected outcome) or 0 had it completed.  Faults nothing; the context stays
 * usable. */
int npa_tile_wait_selftest(int32_t limit_us, int32_t *device_result, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* NPA_B200_H */
