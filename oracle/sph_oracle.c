/*
 * TEST INFRASTRUCTURE -- CPU restatement of the SPH perception operators.
 *
 * This file is the parity oracle for the CUDA kernels.  It is never part of
 * the product path: only tests/, __graft_entry__.smoke() and the cpu_baseline /
 * --impl reference legs of bench.py may load it.
 *
 * It restates, in plain C with double accumulation, the algorithm of the
 * reference's pure-torch oracle sphops/torch_sph.py (every function below names
 * the lines it follows).  torch_sph.py is a brute-force O(N^2) pairwise sum; the
 * sums here run over a private cell list (cell size = h) and therefore visit
 * exactly the pairs with |x_j - x_i| < h + (cell slack), applying the same
 * cut-off masks, so the result is the same sum.  Parity is pinned: the fixtures
 * under tests/golden/ were produced by importing torch_sph.py itself (fp32 and
 * fp64, forward and autograd backward) and tests/test_oracle_golden.py checks
 * this file against them.
 *
 * The cell list is private to the oracle (bounding box of the data when
 * clamped, the periodic box when periodic); it does not depend on the binning
 * under test.
 *
 * Build: gcc -O2 -fopenmp -shared -fPIC (see oracle/build.py, oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* Arithmetic type of the sums.  The default build accumulates in double (the parity truth).
 * Built with -DORACLE_FP32 every product, sum, square root and wrap below runs in float, in the
 * same order: a plain fp32 evaluation of the same formulas, the stand-in for the reference's own
 * fp32 run (torch_sph.py on float tensors) where no stored fp32 output exists.  Outputs are
 * handed back as double arrays in both builds. */
#ifdef ORACLE_FP32
typedef float real;
#define R_SQRT sqrtf
#define R_FMOD fmodf
#define R_FLOOR floorf
#else
typedef double real;
#define R_SQRT sqrt
#define R_FMOD fmod
#define R_FLOOR floor
#endif
#define RC(x) ((real)(x))

typedef struct oracle_cfg {
    int32_t dim;        /* 2 or 3 */
    int32_t pos_stride; /* floats per position in memory: 2, 3 or 4 */
    int32_t periodic;   /* torch_sph `periodic` flag */
    int32_t batch;      /* B */
    int32_t particles;  /* N */
    int32_t channels;   /* C (0 when no feature operator is requested) */
    double h;           /* smoothing length = eps */
    double box[3];      /* torch_sph `box_size` per axis (periodic only) */
} oracle_cfg;

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* torch_sph.py:96-104 smoothing_poly6_normalization */
static real poly6_norm(double h, int dim) {
    return RC(dim == 2 ? 4.0 / (M_PI * pow(h, 8.0)) : 315.0 / (64.0 * M_PI * pow(h, 9.0)));
}
/* torch_sph.py:130-138 gradient_spiky_normalization */
static real spiky_norm(double h, int dim) {
    return RC(dim == 2 ? 10.0 / (M_PI * pow(h, 5.0)) : 15.0 / (M_PI * pow(h, 6.0)));
}

/* torch.remainder(r + L/2, L) - L/2, torch_sph.py:41-52 */
static real wrap(real r, real L) {
    const real half = RC(0.5) * L;
    real t = R_FMOD(r + half, L);
    if (t < RC(0.0)) t += L;
    return t - half;
}

/* ---- private cell list --------------------------------------------------- */
typedef struct {
    int n[3];       /* cells per axis */
    double lo[3];   /* lower corner */
    double inv[3];  /* 1 / cell size per axis; every cell is at least h wide */
    int *start;     /* [cells + 1] */
    int *items;     /* particle indices sorted by cell */
    int brute;      /* 1: a periodic axis has fewer than 3 cells, visit every particle */
} cell_list;

static int axis_cell(const cell_list *cl, const oracle_cfg *c, double x, int d) {
    double u = x - cl->lo[d];
    if (c->periodic) {
        u = fmod(u, c->box[d]);
        if (u < 0.0) u += c->box[d];
    }
    int k = (int)floor(u * cl->inv[d]);
    if (k < 0) k = 0;
    if (k >= cl->n[d]) k = cl->n[d] - 1;
    return k;
}

static void build_cells(cell_list *cl, const oracle_cfg *c, const float *x) {
    const int N = c->particles, D = c->dim;
    cl->brute = 0;
    for (int d = 0; d < 3; ++d) { cl->n[d] = 1; cl->lo[d] = 0.0; cl->inv[d] = 1.0 / c->h; }
    for (int d = 0; d < D; ++d) {
        double extent;
        if (c->periodic) {
            cl->lo[d] = -0.5 * c->box[d];
            extent = c->box[d];
        } else {
            double lo = 1e300, hi = -1e300;
            for (int i = 0; i < N; ++i) {
                double v = x[(size_t)i * c->pos_stride + d];
                if (v < lo) lo = v;
                if (v > hi) hi = v;
            }
            cl->lo[d] = lo;
            extent = (hi - lo) * (1.0 + 1e-9) + 1e-300;
        }
        long n = (long)floor(extent / c->h + 1e-9);
        if (n > 1024) n = 1024; /* wider cells only cost time */
        if (n < 1) n = 1;
        if (c->periodic && n < 3) cl->brute = 1;
        cl->n[d] = (int)n;
        cl->inv[d] = (double)n / extent; /* cell size extent / n >= h */
    }
    const long cells = (long)cl->n[0] * cl->n[1] * cl->n[2];
    cl->start = (int *)calloc((size_t)cells + 1, sizeof(int));
    cl->items = (int *)malloc(sizeof(int) * (size_t)(N > 0 ? N : 1));
    int *cell_of = (int *)malloc(sizeof(int) * (size_t)(N > 0 ? N : 1));
    for (int i = 0; i < N; ++i) {
        int k[3] = {0, 0, 0};
        for (int d = 0; d < D; ++d) k[d] = axis_cell(cl, c, x[(size_t)i * c->pos_stride + d], d);
        int id = (k[2] * cl->n[1] + k[1]) * cl->n[0] + k[0];
        cell_of[i] = id;
        cl->start[id + 1]++;
    }
    for (long k = 0; k < cells; ++k) cl->start[k + 1] += cl->start[k];
    int *cur = (int *)malloc(sizeof(int) * (size_t)cells);
    memcpy(cur, cl->start, sizeof(int) * (size_t)cells);
    for (int i = 0; i < N; ++i) cl->items[cur[cell_of[i]]++] = i;
    free(cur);
    free(cell_of);
}

static void free_cells(cell_list *cl) {
    free(cl->start);
    free(cl->items);
}

/* Candidate iterator: calls BODY with `j` for every particle in the 3^D cells around i (or all
 * particles in brute mode).  Cells visited once even on small periodic grids. */
#define FOR_EACH_CANDIDATE(cl, c, xi, ...)                                                         \
    do {                                                                                           \
        if ((cl)->brute) {                                                                         \
            for (int j = 0; j < (c)->particles; ++j) { __VA_ARGS__ }                                      \
        } else {                                                                                   \
            int kc[3] = {0, 0, 0};                                                                 \
            for (int d_ = 0; d_ < (c)->dim; ++d_) kc[d_] = axis_cell((cl), (c), (xi)[d_], d_);     \
            int zlo = (c)->dim == 3 ? -1 : 0, zhi = (c)->dim == 3 ? 1 : 0;                         \
            for (int oz = zlo; oz <= zhi; ++oz)                                                    \
                for (int oy = -1; oy <= 1; ++oy)                                                   \
                    for (int ox = -1; ox <= 1; ++ox) {                                             \
                        int k0 = kc[0] + ox, k1 = kc[1] + oy, k2 = kc[2] + oz;                     \
                        if ((c)->periodic) {                                                       \
                            k0 = (k0 + (cl)->n[0]) % (cl)->n[0];                                   \
                            k1 = (k1 + (cl)->n[1]) % (cl)->n[1];                                   \
                            k2 = (k2 + (cl)->n[2]) % (cl)->n[2];                                   \
                        } else if (k0 < 0 || k1 < 0 || k2 < 0 || k0 >= (cl)->n[0] ||               \
                                   k1 >= (cl)->n[1] || k2 >= (cl)->n[2])                           \
                            continue;                                                              \
                        int id_ = (k2 * (cl)->n[1] + k1) * (cl)->n[0] + k0;                        \
                        for (int p_ = (cl)->start[id_]; p_ < (cl)->start[id_ + 1]; ++p_) {         \
                            int j = (cl)->items[p_];                                               \
                            __VA_ARGS__                                                             \
                        }                                                                          \
                    }                                                                              \
        }                                                                                          \
    } while (0)

/* r = x_j - x_i (wrapped when periodic), torch_sph.py:24-53 */
static real pair_r(const oracle_cfg *c, const float *xi, const float *xj, real *r) {
    real q = RC(0.0);
    for (int d = 0; d < c->dim; ++d) {
        real v = RC(xj[d]) - RC(xi[d]);
        if (c->periodic) v = wrap(v, RC(c->box[d]));
        r[d] = v;
        q += v * v;
    }
    return q;
}

/* fp32 evaluation of r^2 exactly as torch does for float tensors: fp32 subtract, fp32 wrap
 * (torch.remainder), fp32 squares summed left to right. */
static float pair_q_f32(const oracle_cfg *c, const float *xi, const float *xj) {
    float q = 0.0f;
    for (int d = 0; d < c->dim; ++d) {
        volatile float v = xj[d] - xi[d];
        if (c->periodic) {
            const float L = (float)c->box[d];
            const float half = L * 0.5f;
            volatile float s = v + half;
            float t = fmodf(s, L);
            if (t != 0.0f && ((t < 0.0f) != (L < 0.0f))) t += L;
            volatile float w = t - half;
            v = w;
        }
        volatile float sq = v * v;
        volatile float acc = q + sq;
        q = acc;
    }
    return q;
}

/* spiky magnitude and its derivative, torch_sph.py:140-162:
 *   d = sqrt(q), d_safe = sqrt(q + 1e-12), mask = d < h && d > 0,
 *   mag = 3 clamp(h - d_safe, 0)^2 / d_safe                      */
static int spiky(real q, real h, real *phi, real *psi) {
    real d = R_SQRT(q);
    if (!(d < h) || !(d > RC(0.0))) return 0;
    real ds = R_SQRT(q + RC(1e-12));
    real t = h - ds;
    if (t < RC(0.0)) t = RC(0.0);
    *phi = RC(3.0) * t * t / ds;
    if (psi) *psi = RC(3.0) * t * (h + ds) / (ds * ds * ds); /* -(d phi / d ds) / ds */
    return 1;
}

/*
 * Forward of every operator (any output pointer may be NULL):
 *   count    [B,N]      float : torch_sph.count             (torch_sph.py:292-316, fp32 semantics)
 *   rho      [B,N]      double: torch_sph.density           (torch_sph.py:185-221)
 *   rho_grad [B,N,D]    double: torch_sph.density_gradient  (torch_sph.py:371-408)
 *   blur     [B,N,C]    double: torch_sph.blur              (torch_sph.py:319-368)
 *   grad     [B,N,C,D]  double: torch_sph.gradient          (torch_sph.py:248-289)
 *   moment   [B,N,D,D]  double: torch_sph.moment_matrix     (torch_sph.py:410-471)
 * rho_in [B,N] float is the density fed to blur / gradient / moment_matrix (their `rho` argument).
 * mass may be NULL (all ones, torch_sph.py:6-22).
 */
int oracle_forward(const oracle_cfg *c, const float *x, const float *mass, const float *s,
                   const float *rho_in, float *count, double *rho, double *rho_grad, double *blur,
                   double *grad, double *moment) {
    const int N = c->particles, D = c->dim, C = c->channels, P = c->pos_stride;
    const real h = RC(c->h), h2 = RC(c->h * c->h);
    const float h2f = (float)(c->h * c->h);
    const real cs = poly6_norm(c->h, D), cg = spiky_norm(c->h, D);
    if ((blur || grad || moment) && !rho_in) return -1;
    if ((blur || grad) && (!s || C <= 0)) return -1;
    for (int b = 0; b < c->batch; ++b) {
        const float *xb = x + (size_t)b * N * P;
        const float *mb = mass ? mass + (size_t)b * N : NULL;
        const float *sb = s ? s + (size_t)b * N * C : NULL;
        const float *rb = rho_in ? rho_in + (size_t)b * N : NULL;
        cell_list cl;
        build_cells(&cl, c, xb);
#pragma omp parallel for schedule(dynamic, 64)
        for (int i = 0; i < N; ++i) {
            const float *xi = xb + (size_t)i * P;
            const size_t gi = (size_t)b * N + i;
            real a_rho = RC(0.0), a_dg[3] = {0, 0, 0}, a_m[9] = {0};
            float a_cnt = 0.0f;
            real acc_b[C > 0 ? C : 1], acc_g[C > 0 ? C * D : 1]; /* sums of this particle */
            real *ob = blur ? acc_b : NULL;
            real *og = grad ? acc_g : NULL;
            if (ob) memset(ob, 0, sizeof(real) * C);
            if (og) memset(og, 0, sizeof(real) * C * D);
            FOR_EACH_CANDIDATE(&cl, c, xi, {
                const float *xj = xb + (size_t)j * P;
                real r[3] = {0, 0, 0};
                const real q = pair_r(c, xi, xj, r);
                if (count && pair_q_f32(c, xi, xj) < h2f) a_cnt += 1.0f;
                const real mj = mb ? RC(mb[j]) : RC(1.0);
                const real vj = rb ? mj / RC(rb[j]) : RC(0.0);
                if (q < h2) {
                    real t = h2 - q;
                    if (t < RC(0.0)) t = RC(0.0);
                    const real w = t * t * t;
                    a_rho += mj * w;
                    if (ob) {
                        const float *sj = sb + (size_t)j * C;
                        for (int f = 0; f < C; ++f) ob[f] += (w * vj) * RC(sj[f]);
                    }
                }
                real phi;
                if ((rho_grad || og || moment) && spiky(q, h, &phi, NULL)) {
                    for (int d = 0; d < D; ++d) a_dg[d] += mj * phi * r[d];
                    if (og) {
                        const float *sj = sb + (size_t)j * C;
                        const float *si = sb + (size_t)i * C;
                        for (int f = 0; f < C; ++f) {
                            const real df = RC(sj[f]) - RC(si[f]);
                            for (int d = 0; d < D; ++d) og[f * D + d] += df * (vj * phi * r[d]);
                        }
                    }
                    if (moment)
                        for (int p = 0; p < D; ++p)
                            for (int e = 0; e < D; ++e) a_m[p * D + e] += r[p] * (vj * phi * r[e]);
                }
            });
            if (count) count[gi] = a_cnt;
            if (rho) rho[gi] = cs * a_rho;
            if (rho_grad)
                for (int d = 0; d < D; ++d) rho_grad[gi * D + d] = cg * a_dg[d];
            if (ob)
                for (int f = 0; f < C; ++f) blur[gi * C + f] = cs * ob[f];
            if (og)
                for (int f = 0; f < C * D; ++f) grad[gi * C * D + f] = cg * og[f];
            if (moment)
                for (int p = 0; p < D * D; ++p) moment[gi * D * D + p] = cg * a_m[p];
        }
        free_cells(&cl);
    }
    return 0;
}

/*
 * Backward of the same operators as a gather, each operator differentiated as torch autograd
 * differentiates torch_sph.py (rho_in is an independent input of blur / gradient / moment_matrix).
 * Upstream gradients (float, any may be NULL = zero):
 *   g_rho [B,N], g_rho_grad [B,N,D], g_blur [B,N,C], g_grad [B,N,C,D], g_moment [B,N,D,D]
 * Outputs (real, any may be NULL): dx [B,N,D], ds [B,N,C], drho [B,N] (w.r.t. rho_in).
 * With r = x_j - x_i, W = (h^2-q)^3, E = 6 (h^2-q)^2, K = phi r, J = phi I - psi r r^T,
 * v = m / rho_in:
 *   density      dx_i += cs sum_j E (g_i m_j + g_j m_i) r
 *   density_grad dx_i += cg sum_j J (m_i g_j - m_j g_i)
 *   blur         ds_i += cs v_i sum_j W gB_j ;  drho_i -= cs v_i^2/m_i sum_j W (gB_j . s_i)
 *                dx_i += cs sum_j E r [v_j (gB_i . s_j) + v_i (gB_j . s_i)]
 *   gradient     ds_i -= cg sum_j sum_d K_d (v_j gG_i[f,d] + v_i gG_j[f,d])
 *                drho_i += cg v_i^2/m_i sum_j sum_fd gG_j[f,d] (s_i - s_j)[f] K_d
 *                dx_i += cg sum_j J u,  u_d = sum_f (s_i - s_j)[f] (v_j gG_i[f,d] + v_i gG_j[f,d])
 *   moment       Cm = v_j gM_i + v_i gM_j
 *                dx_i[c] -= cg sum_j [ sum_b Cm[c,b] K_b + (J w)_c ],  w_b = sum_a r_a Cm[a,b]
 *                drho_i -= cg v_i^2/m_i sum_j phi sum_ab gM_j[a,b] r_a r_b
 */
int oracle_backward(const oracle_cfg *c, const float *x, const float *mass, const float *s,
                    const float *rho_in, const float *g_rho, const float *g_rho_grad,
                    const float *g_blur, const float *g_grad, const float *g_moment, double *dx,
                    double *ds, double *drho) {
    const int N = c->particles, D = c->dim, C = c->channels, P = c->pos_stride;
    const real h = RC(c->h), h2 = RC(c->h * c->h);
    const real cs = poly6_norm(c->h, D), cg = spiky_norm(c->h, D);
    if ((g_blur || g_grad || g_moment) && !rho_in) return -1;
    if ((g_blur || g_grad) && (!s || C <= 0)) return -1;
    for (int b = 0; b < c->batch; ++b) {
        const float *xb = x + (size_t)b * N * P;
        const float *mb = mass ? mass + (size_t)b * N : NULL;
        const float *sb = s ? s + (size_t)b * N * C : NULL;
        const float *rb = rho_in ? rho_in + (size_t)b * N : NULL;
        const float *gr = g_rho ? g_rho + (size_t)b * N : NULL;
        const float *gd = g_rho_grad ? g_rho_grad + (size_t)b * N * D : NULL;
        const float *gb = g_blur ? g_blur + (size_t)b * N * C : NULL;
        const float *gg = g_grad ? g_grad + (size_t)b * N * C * D : NULL;
        const float *gm = g_moment ? g_moment + (size_t)b * N * D * D : NULL;
        cell_list cl;
        build_cells(&cl, c, xb);
#pragma omp parallel for schedule(dynamic, 64)
        for (int i = 0; i < N; ++i) {
            const float *xi = xb + (size_t)i * P;
            const size_t gi = (size_t)b * N + i;
            const real mi = mb ? RC(mb[i]) : RC(1.0);
            const real vi = rb ? mi / RC(rb[i]) : RC(0.0);
            real a_dx[3] = {0, 0, 0}, a_dr = RC(0.0);
            real acc_s[C > 0 ? C : 1];
            real *ods = ds ? acc_s : NULL;
            if (ods) memset(ods, 0, sizeof(real) * C);
            FOR_EACH_CANDIDATE(&cl, c, xi, {
                const float *xj = xb + (size_t)j * P;
                real r[3] = {0, 0, 0};
                const real q = pair_r(c, xi, xj, r);
                const real mj = mb ? RC(mb[j]) : RC(1.0);
                const real vj = rb ? mj / RC(rb[j]) : RC(0.0);
                if (q < h2) {
                    real t = h2 - q;
                    if (t < RC(0.0)) t = RC(0.0);
                    const real W = t * t * t, E = RC(6.0) * t * t;
                    if (gr)
                        for (int d = 0; d < D; ++d)
                            a_dx[d] += cs * E * (RC(gr[i]) * mj + RC(gr[j]) * mi) * r[d];
                    if (gb) {
                        const float *sj = sb + (size_t)j * C, *si = sb + (size_t)i * C;
                        const float *gbj = gb + (size_t)j * C, *gbi = gb + (size_t)i * C;
                        real A = RC(0.0), Bp = RC(0.0);
                        for (int f = 0; f < C; ++f) {
                            if (ods) ods[f] += cs * vi * W * RC(gbj[f]);
                            A += RC(gbi[f]) * RC(sj[f]);
                            Bp += RC(gbj[f]) * RC(si[f]);
                        }
                        for (int d = 0; d < D; ++d) a_dx[d] += cs * E * r[d] * (vj * A + vi * Bp);
                        a_dr -= cs * (vi * vi / mi) * W * Bp;
                    }
                }
                real phi, psi;
                if ((gd || gg || gm) && spiky(q, h, &phi, &psi)) {
                    if (gd) {
                        real u[3] = {0, 0, 0}, ru = RC(0.0);
                        for (int d = 0; d < D; ++d) {
                            u[d] = mi * RC(gd[(size_t)j * D + d]) - mj * RC(gd[(size_t)i * D + d]);
                            ru += r[d] * u[d];
                        }
                        for (int d = 0; d < D; ++d) a_dx[d] += cg * (phi * u[d] - psi * ru * r[d]);
                    }
                    if (gg) {
                        const float *sj = sb + (size_t)j * C, *si = sb + (size_t)i * C;
                        const float *ggj = gg + (size_t)j * C * D, *ggi = gg + (size_t)i * C * D;
                        real u[3] = {0, 0, 0}, ru = RC(0.0);
                        for (int f = 0; f < C; ++f) {
                            const real df = RC(si[f]) - RC(sj[f]);
                            real hk = RC(0.0), gk = RC(0.0);
                            for (int d = 0; d < D; ++d) {
                                const real hd = vj * RC(ggi[f * D + d]) + vi * RC(ggj[f * D + d]);
                                hk += phi * r[d] * hd;
                                u[d] += df * hd;
                                gk += RC(ggj[f * D + d]) * phi * r[d];
                            }
                            if (ods) ods[f] -= cg * hk;
                            a_dr += cg * (vi * vi / mi) * df * gk;
                        }
                        for (int d = 0; d < D; ++d) ru += r[d] * u[d];
                        for (int d = 0; d < D; ++d) a_dx[d] += cg * (phi * u[d] - psi * ru * r[d]);
                    }
                    if (gm) {
                        const float *gmj = gm + (size_t)j * D * D, *gmi = gm + (size_t)i * D * D;
                        real w[3] = {0, 0, 0}, rw = RC(0.0), rr = RC(0.0);
                        for (int p = 0; p < D; ++p) {
                            real kc = RC(0.0);
                            for (int e = 0; e < D; ++e) {
                                const real cm = vj * RC(gmi[p * D + e]) + vi * RC(gmj[p * D + e]);
                                kc += cm * phi * r[e];
                                w[e] += r[p] * cm;
                                rr += RC(gmj[p * D + e]) * r[p] * r[e];
                            }
                            a_dx[p] -= cg * kc;
                        }
                        for (int d = 0; d < D; ++d) rw += r[d] * w[d];
                        for (int d = 0; d < D; ++d) a_dx[d] -= cg * (phi * w[d] - psi * rw * r[d]);
                        a_dr -= cg * (vi * vi / mi) * phi * rr;
                    }
                }
            });
            if (dx)
                for (int d = 0; d < D; ++d) dx[gi * D + d] = a_dx[d];
            if (drho) drho[gi] = a_dr;
            if (ods)
                for (int f = 0; f < C; ++f) ds[gi * C + f] = ods[f];
        }
        free_cells(&cl);
    }
    return 0;
}

/* Inverse of symmetric DxD matrices with the identity fallback of the reference's
 * safe_inv_sym_mat (sphops/sph_cuda.cu:3095-3179): upper triangle read, |det| < tol -> I.
 * Evaluated in fp32 like the reference so the branch decision matches. */
void oracle_safe_inv_sym_mat(int dim, long n, const float *m, float *out, float tol) {
    for (long i = 0; i < n; ++i) {
        if (dim == 2) {
            const float *p = m + i * 4;
            float *o = out + i * 4;
            float det = p[0] * p[3] - p[1] * p[1];
            if (fabsf(det) < tol) { o[0] = 1; o[1] = 0; o[2] = 0; o[3] = 1; }
            else { float r = 1.0f / det; o[0] = p[3] * r; o[1] = -p[1] * r; o[2] = -p[1] * r; o[3] = p[0] * r; }
        } else {
            const float *p = m + i * 9;
            float *o = out + i * 9;
            float a = p[0], b = p[1], cc = p[2], d = p[4], e = p[5], f = p[8];
            float t1 = d * f - e * e, t2 = cc * e - b * f, t3 = b * e - cc * d;
            float det = a * t1 + b * t2 + cc * t3;
            if (fabsf(det) < tol) {
                for (int k = 0; k < 9; ++k) o[k] = (k % 4 == 0) ? 1.0f : 0.0f;
            } else {
                float r = 1.0f / det;
                o[0] = t1 * r; o[1] = t2 * r; o[2] = t3 * r;
                o[3] = t2 * r; o[4] = (a * f - cc * cc) * r; o[5] = (b * cc - a * e) * r;
                o[6] = t3 * r; o[7] = (b * cc - a * e) * r; o[8] = (a * d - b * b) * r;
            }
        }
    }
}
