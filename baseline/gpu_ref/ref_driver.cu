// extern "C" driver around the reference's own CUDA kernels (its sphops/sph_cuda.cu, compiled
// unmodified for sm_100 against the stand-in nanobind headers of this directory), so that bench.py
// can time them on the same GPU and the same inputs as the kernels of this repository.
//
// Comparator only: nothing in npa_b200/ links or loads this.  The reference's translation unit is
// found through the include path (-I <reference checkout>/sphops); it is not copied.
#include "sph_cuda.cu"

#include <cstring>
#include <string>

namespace {

thread_local std::string g_error;

struct GridBase {
    virtual ~GridBase() = default;
    virtual int max_blocks() const = 0;
    virtual void initialize(const float *x, int32_t *perm, int32_t *offs, int32_t *info) = 0;
    virtual void bin(const float *x, const float *s, const float *m, const int32_t *perm, float *xo, float *so,
                     float *mo, int C) = 0;
    virtual void density_forward(const float *x, const float *m, float *rho, const int32_t *offs, const int32_t *info) = 0;
    virtual void blur_forward(const float *x, const float *rho, const float *m, const float *s, float *out, int C,
                              const int32_t *offs, const int32_t *info) = 0;
    virtual void gradient_forward(const float *x, const float *rho, const float *m, const float *s, float *out, int C,
                                  const int32_t *offs, const int32_t *info) = 0;
    virtual void density_backward(const float *x, const float *m, const float *g, float *gx, const int32_t *offs,
                                  const int32_t *info) = 0;
    virtual void blur_backward(const float *x, const float *rho, const float *m, const float *s, const float *g,
                               float *gx, float *gs, float *gr, int C, const int32_t *offs, const int32_t *info) = 0;
    virtual void gradient_backward(const float *x, const float *rho, const float *m, const float *s, const float *g,
                                   float *gx, float *gs, float *gr, int C, const int32_t *offs, const int32_t *info) = 0;
};

template <typename Grid, int DIM>
struct GridImpl : GridBase {
    Grid grid;
    size_t B, N, P, cells;
    template <typename... A>
    GridImpl(size_t b, size_t n, size_t c, A... a) : grid(a...), B(b), N(n), P(DIM == 2 ? 2 : 4), cells(c) {}

    FloatArray3D pos(const float *p) const { return FloatArray3D(const_cast<float *>(p), {B, N, P}); }
    FloatArray2D bn(const float *p) const { return FloatArray2D(const_cast<float *>(p), {B, N}); }
    FloatArray3D feat(const float *p, int C) const { return FloatArray3D(const_cast<float *>(p), {B, N, (size_t)C}); }
    FloatArray4D feat4(const float *p, int C) const {
        return FloatArray4D(const_cast<float *>(p), {B, N, (size_t)C, (size_t)DIM});
    }
    IntArray1D offsets(const int32_t *p) const { return IntArray1D(const_cast<int32_t *>(p), {B * cells + 1}); }
    IntArray2D permutation(const int32_t *p) const { return IntArray2D(const_cast<int32_t *>(p), {B, N}); }
    BlockInfoArray blocks(const int32_t *p) const {
        return BlockInfoArray(const_cast<int32_t *>(p), {(size_t)grid.max_blocks(), 4});
    }

    int max_blocks() const override { return grid.max_blocks(); }
    void initialize(const float *x, int32_t *perm, int32_t *offs, int32_t *info) override {
        grid.initialize(pos(x), permutation(perm), offsets(offs), blocks(info));
    }
    void bin(const float *x, const float *s, const float *m, const int32_t *perm, float *xo, float *so, float *mo,
             int C) override {
        grid.bin_particles(pos(x), feat(s, C), bn(m), permutation(perm), pos(xo), feat(so, C), bn(mo));
    }
    void density_forward(const float *x, const float *m, float *rho, const int32_t *offs, const int32_t *info) override {
        grid.density_forward(pos(x), bn(m), bn(rho), offsets(offs), blocks(info));
    }
    void blur_forward(const float *x, const float *rho, const float *m, const float *s, float *out, int C,
                      const int32_t *offs, const int32_t *info) override {
        grid.blur_forward(pos(x), bn(rho), bn(m), feat(s, C), feat(out, C), offsets(offs), blocks(info));
    }
    void gradient_forward(const float *x, const float *rho, const float *m, const float *s, float *out, int C,
                          const int32_t *offs, const int32_t *info) override {
        grid.gradient_forward(pos(x), bn(rho), bn(m), feat(s, C), feat4(out, C), offsets(offs), blocks(info));
    }
    void density_backward(const float *x, const float *m, const float *g, float *gx, const int32_t *offs,
                          const int32_t *info) override {
        grid.density_backward(pos(x), bn(m), bn(g), pos(gx), offsets(offs), blocks(info), true);
    }
    void blur_backward(const float *x, const float *rho, const float *m, const float *s, const float *g, float *gx,
                       float *gs, float *gr, int C, const int32_t *offs, const int32_t *info) override {
        grid.blur_backward(pos(x), bn(rho), bn(m), feat(s, C), feat(g, C), pos(gx), feat(gs, C), bn(gr), offsets(offs),
                           blocks(info), true, true, true);
    }
    void gradient_backward(const float *x, const float *rho, const float *m, const float *s, const float *g, float *gx,
                           float *gs, float *gr, int C, const int32_t *offs, const int32_t *info) override {
        grid.gradient_backward(pos(x), bn(rho), bn(m), feat(s, C), feat4(g, C), pos(gx), feat(gs, C), bn(gr),
                               offsets(offs), blocks(info), true, true, true);
    }
};

template <typename F>
int guarded(F &&f) {
    try {
        f();
        return 0;
    } catch (const std::exception &e) {
        g_error = e.what();
        return -1;
    }
}

}  // namespace

extern "C" {

const char *ref_last_error() { return g_error.c_str(); }

void *ref_grid_create(int dim, int periodic, int gx, int gy, int gz, float eps, unsigned N, unsigned B, unsigned mpb) {
    GridBase *g = nullptr;
    const int rc = guarded([&] {
        if (dim == 2) {
            const size_t cells = (size_t)gx * gy;
            if (periodic) g = new GridImpl<HashGrid2DPeriodic, 2>(B, N, cells, gx, gy, eps, N, B, mpb);
            else g = new GridImpl<HashGrid2DBox, 2>(B, N, cells, gx, gy, eps, N, B, mpb);
        } else {
            const size_t cells = (size_t)gx * gy * gz;
            if (periodic) g = new GridImpl<HashGrid3DPeriodic, 3>(B, N, cells, gx, gy, gz, eps, N, B, mpb);
            else g = new GridImpl<HashGrid3DBox, 3>(B, N, cells, gx, gy, gz, eps, N, B, mpb);
        }
    });
    return rc == 0 ? g : nullptr;
}

void ref_grid_destroy(void *h) { delete static_cast<GridBase *>(h); }
int ref_max_blocks(void *h) { return static_cast<GridBase *>(h)->max_blocks(); }

int ref_initialize(void *h, const float *x, int32_t *perm, int32_t *offs, int32_t *info) {
    return guarded([&] { static_cast<GridBase *>(h)->initialize(x, perm, offs, info); });
}
int ref_bin_particles(void *h, const float *x, const float *s, const float *m, const int32_t *perm, float *xo,
                      float *so, float *mo, int C) {
    return guarded([&] { static_cast<GridBase *>(h)->bin(x, s, m, perm, xo, so, mo, C); });
}
int ref_density_forward(void *h, const float *x, const float *m, float *rho, const int32_t *offs, const int32_t *info) {
    return guarded([&] { static_cast<GridBase *>(h)->density_forward(x, m, rho, offs, info); });
}
int ref_blur_forward(void *h, const float *x, const float *rho, const float *m, const float *s, float *out, int C,
                     const int32_t *offs, const int32_t *info) {
    return guarded([&] { static_cast<GridBase *>(h)->blur_forward(x, rho, m, s, out, C, offs, info); });
}
int ref_gradient_forward(void *h, const float *x, const float *rho, const float *m, const float *s, float *out, int C,
                         const int32_t *offs, const int32_t *info) {
    return guarded([&] { static_cast<GridBase *>(h)->gradient_forward(x, rho, m, s, out, C, offs, info); });
}
int ref_density_backward(void *h, const float *x, const float *m, const float *g, float *gx, const int32_t *offs,
                         const int32_t *info) {
    return guarded([&] { static_cast<GridBase *>(h)->density_backward(x, m, g, gx, offs, info); });
}
int ref_blur_backward(void *h, const float *x, const float *rho, const float *m, const float *s, const float *g,
                      float *gx, float *gs, float *gr, int C, const int32_t *offs, const int32_t *info) {
    return guarded([&] { static_cast<GridBase *>(h)->blur_backward(x, rho, m, s, g, gx, gs, gr, C, offs, info); });
}
int ref_gradient_backward(void *h, const float *x, const float *rho, const float *m, const float *s, const float *g,
                          float *gx, float *gs, float *gr, int C, const int32_t *offs, const int32_t *info) {
    return guarded([&] { static_cast<GridBase *>(h)->gradient_backward(x, rho, m, s, g, gx, gs, gr, C, offs, info); });
}

}  // extern "C"
