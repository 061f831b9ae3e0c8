// Host-side geometry validation and error plumbing shared by every entry point
// of the C ABI (include/npa_b200.h).
#include <stdlib.h>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace npa {

static thread_local char g_last_error[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(NPA_ERR_CUDA, "CUDA error launching %s: %s", what, cudaGetErrorString(e));
    return NPA_OK;
}

static bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// Mirrors HashGrid::_init (sphops/sph_cuda.cu:1836-1899) except that the
// normalisation constants are evaluated in double and rounded once, which is
// how the torch oracle obtains them (sphops/torch_sph.py:96-104,130-138).
int make_geom(const npa_grid *in, Geom *out) {
    if (!in) return fail(NPA_ERR_INVALID_ARGUMENT, "grid descriptor is NULL");
    if (in->dim != 2 && in->dim != 3)
        return fail(NPA_ERR_INVALID_ARGUMENT, "dim must be 2 or 3, got %d", in->dim);
    if (in->boundary != NPA_BOUNDARY_CLAMPED && in->boundary != NPA_BOUNDARY_PERIODIC)
        return fail(NPA_ERR_INVALID_ARGUMENT, "boundary must be 0 (clamped) or 1 (periodic), got %d", in->boundary);
    if (in->hash != NPA_HASH_LINEAR && in->hash != NPA_HASH_MORTON)
        return fail(NPA_ERR_INVALID_ARGUMENT, "hash must be 0 (linear) or 1 (morton), got %d", in->hash);
    if (!(in->eps > 0.0) || !std::isfinite(in->eps))
        return fail(NPA_ERR_INVALID_ARGUMENT, "eps must be positive and finite, got %g", in->eps);
    if (in->batch <= 0 || in->particles <= 0)
        return fail(NPA_ERR_INVALID_ARGUMENT, "batch and particles must be positive, got %d and %d", in->batch, in->particles);
    if (in->max_particles_per_block <= 0)
        return fail(NPA_ERR_INVALID_ARGUMENT, "max_particles_per_block must be positive, got %d", in->max_particles_per_block);

    Geom g;
    memset(&g, 0, sizeof(g));
    g.dim = in->dim;
    g.periodic = in->boundary == NPA_BOUNDARY_PERIODIC;
    g.morton = in->hash == NPA_HASH_MORTON;
    long long cells = 1;
    for (int d = 0; d < 3; ++d) {
        int n = d < in->dim ? in->grid[d] : 1;
        if (n <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "grid[%d] must be positive, got %d", d, n);
        g.g[d] = n;
        g.half[d] = d < in->dim ? n / 2 : 0;
        cells *= n;
    }
    if (g.morton) {
        uint32_t top;
        for (int d = 0; d < in->dim; ++d) {
            if (!is_pow2(g.g[d]))
                return fail(NPA_ERR_UNSUPPORTED, "grid_size must be a power of 2 with the Morton hash, got %d", g.g[d]);
            if (g.g[d] > 1024)
                return fail(NPA_ERR_UNSUPPORTED, "the Morton hash interleaves 10 bits per axis; grid[%d]=%d is too large", d, g.g[d]);
        }
        if (in->dim == 2)
            top = dilate2(g.g[0] - 1) | (dilate2(g.g[1] - 1) << 1);
        else
            top = dilate3(g.g[0] - 1) | (dilate3(g.g[1] - 1) << 1) | (dilate3(g.g[2] - 1) << 2);
        if ((long long)top >= cells)
            return fail(NPA_ERR_UNSUPPORTED,
                        "Morton hash of the last cell (%u) does not fit %lld cells; use equal grid sizes", top, cells);
    }
    long long total_cells = cells * in->batch;
    long long total_particles = (long long)in->batch * in->particles;
    if (total_cells + 1 >= (1ll << 31) || total_particles >= (1ll << 31))
        return fail(NPA_ERR_INVALID_ARGUMENT, "batch*cells (%lld) and batch*particles (%lld) must stay below 2^31",
                    total_cells, total_particles);
    g.cells = (int)cells;
    g.B = in->batch;
    g.N = in->particles;
    g.mpb = in->max_particles_per_block;
    long long per_system = cells + (in->particles + g.mpb - 1) / g.mpb;
    if (per_system > in->particles) per_system = in->particles;
    long long max_blocks = per_system * in->batch;
    if (max_blocks >= (1ll << 29))
        return fail(NPA_ERR_INVALID_ARGUMENT, "work list of %lld rows is too large", max_blocks);
    g.max_blocks = (int)max_blocks;
    // Warps sharing a work item (its particles are dealt round-robin).  Small problems have fewer
    // items than a B200 has warp slots (148 SMs x ~24 warps): up to 8 warps share one.  Large ones
    // still use 2 when items can be big, so that the last rows handed out are short.
    {
        long long items = (long long)in->batch * (cells < in->particles ? cells : in->particles);
        long long split = (2ll * 148 * 24) / (items > 0 ? items : 1);
        const long long least = in->max_particles_per_block > 8 ? 2 : 1;
        g.split = (int)(split < least ? least : (split > 8 ? 8 : split));
    }

    const float eps_f = (float)in->eps;
    g.h = eps_f;
    g.inv_eps = 1.0f / eps_f;
    g.h2 = (float)(in->eps * in->eps);
    for (int d = 0; d < 3; ++d) {
        const double Ld = (double)g.g[d] * in->eps;
        g.L[d] = (float)Ld;
        g.Llo[d] = (float)(Ld - (double)g.L[d]);
        g.invL[d] = 1.0f / g.L[d];
        g.halfL[d] = 0.5f * g.L[d];
    }
    const double pi = 3.14159265358979323846;
    if (in->dim == 2) {
        g.c_s = (float)(4.0 / (pi * std::pow(in->eps, 8.0)));
        g.c_g = (float)(10.0 / (pi * std::pow(in->eps, 5.0)));
    } else {
        g.c_s = (float)(315.0 / (64.0 * pi * std::pow(in->eps, 9.0)));
        g.c_g = (float)(15.0 / (pi * std::pow(in->eps, 6.0)));
    }
    *out = g;
    return NPA_OK;
}

}  // namespace npa

extern "C" {

const char *npa_last_error(void) { return npa::g_last_error; }

int npa_abi_version(void) { return NPA_B200_ABI_VERSION; }

int64_t npa_grid_num_cells(const npa_grid *g) {
    npa::Geom geo;
    int rc = npa::make_geom(g, &geo);
    return rc != NPA_OK ? rc : geo.cells;
}

int64_t npa_grid_max_blocks(const npa_grid *g) {
    npa::Geom geo;
    int rc = npa::make_geom(g, &geo);
    return rc != NPA_OK ? rc : geo.max_blocks;
}

}  // extern "C"
