// Differentiable 2D Gaussian splatting of particles into an image, forward and backward.
//
// Replaces splat_particles / splat_particles_batch of the reference (utils/splatting.py:6-113), the
// renderer of its splat loss (losses/splat_loss.py:71-86).  The reference materialises the
// (2r+1)^2 patch of every particle as [N, (2r+1)^2] index / weight tensors and scatter-adds them
// (atomics, run-to-run different sums).  Here both directions are gathers:
//   forward  : a CTA owns a 16x16 pixel tile.  The particles of the system are culled against the
//              tile 256 at a time (ordered ballot compaction into shared memory), then every pixel
//              thread adds the listed particles in particle order -- no atomics, deterministic;
//   backward : a warp owns a particle and walks its patch, reading the upstream image gradient
//              (L2 resident) and reducing the colour and position gradients with shuffles.
// Pixel of a particle: p = (x - lo) / (hi - lo) * (img - 1) (y flipped when y_up), base = floor(p),
// frac = p - base; weight of pixel base + (dx, dy): g = exp(-((dx - frac_x)^2 + (dy - frac_y)^2) / (2 sigma^2)),
// with normalisation w = g / (1e-8 + sum of g over the whole patch) * norm_scale; out = [sum c w | sum w].
// The patch sum factorises into two 1D sums (the weight is separable).
#include "common.cuh"

namespace npa {

constexpr int kSplatTile = 16;
constexpr int kSplatMaxRadius = 64;

struct SplatArgs {
    const float *x;      // [B, N, 2]
    const float *color;  // [B, N, 3]
    float *out;          // [B, img, img, 4]  (r, g, b, density)
    const float *g_out;  // backward: upstream of out
    float *g_x;          // backward: [B, N, 2]
    float *g_color;      // backward: [B, N, 3]
    float *wscale;       // [B, N] scratch: norm_scale / (1e-8 + patch sum) per particle (normalised mode)
    int B, N, img, radius, y_up, normalize;
    float lo, span, sigma, norm_scale;  // span = hi - lo; sigma in pixels
};

struct SplatPoint {
    int cx, cy;
    float fx, fy;
};

__device__ inline SplatPoint splat_point(const SplatArgs &a, long long n) {
    const float2 v = __ldg(reinterpret_cast<const float2 *>(a.x) + n);
    const float top = (float)(a.img - 1);
    float px = __fmul_rn(__fdiv_rn(v.x - a.lo, a.span), top);
    float py = __fmul_rn(__fdiv_rn(v.y - a.lo, a.span), top);
    if (a.y_up) py = top - py;
    const float bx = floorf(px), by = floorf(py);
    SplatPoint p;
    // far-away or non-finite positions touch no pixel: park them outside every tile
    const float lim = 1.0e8f;
    p.cx = (bx > -lim && bx < lim) ? (int)bx : -(1 << 30);
    p.cy = (by > -lim && by < lim) ? (int)by : -(1 << 30);
    p.fx = px - bx;
    p.fy = py - by;
    return p;
}

// sum over d = -r..r of exp(-(d - f)^2 / (2 sigma^2)), and of the same times (d - f)
__device__ inline void axis_sums(int r, float f, float inv2s2, float &s0, float &s1) {
    s0 = 0.f; s1 = 0.f;
    for (int d = -r; d <= r; ++d) {
        const float t = (float)d - f;
        const float g = expf(-(t * t) * inv2s2);
        s0 += g;
        s1 = fmaf(g, t, s1);
    }
}

// Normalised mode: the scale of every particle, once (the forward tiles would otherwise redo the
// 2 (2r+1) exponentials for every tile a particle touches).
__global__ void __launch_bounds__(256) splat_scale_kernel(SplatArgs a) {
    const long long n = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (n >= (long long)a.B * a.N) return;
    const SplatPoint p = splat_point(a, n);
    const float inv2s2 = 1.0f / (2.0f * a.sigma * a.sigma);
    float sx, sy, unused;
    axis_sums(a.radius, p.fx, inv2s2, sx, unused);
    axis_sums(a.radius, p.fy, inv2s2, sy, unused);
    a.wscale[n] = a.norm_scale / (1e-8f + sx * sy);
}

__global__ void __launch_bounds__(kSplatTile *kSplatTile) splat_forward_kernel(SplatArgs a) {
    constexpr int T = kSplatTile * kSplatTile;
    __shared__ int s_cx[T], s_cy[T];
    __shared__ float s_fx[T], s_fy[T], s_w[T], s_r[T], s_g[T], s_b[T];
    __shared__ int s_warp_count[T / 32];
    const int tiles = (a.img + kSplatTile - 1) / kSplatTile;
    const int tx0 = (blockIdx.x % tiles) * kSplatTile, ty0 = (blockIdx.x / tiles) * kSplatTile;
    const int b = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int px = tx0 + (tid % kSplatTile), py = ty0 + (tid / kSplatTile);
    const int r = a.radius;
    const float inv2s2 = 1.0f / (2.0f * a.sigma * a.sigma);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};

    for (int n0 = 0; n0 < a.N; n0 += T) {
        const int n = n0 + tid;
        bool hit = false;
        SplatPoint p = {0, 0, 0.f, 0.f};
        if (n < a.N) {
            p = splat_point(a, (long long)b * a.N + n);
            hit = p.cx + r >= tx0 && p.cx - r < tx0 + kSplatTile && p.cy + r >= ty0 && p.cy - r < ty0 + kSplatTile;
        }
        // ordered compaction: particles keep their index order in the list
        const unsigned bal = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) s_warp_count[warp] = __popc(bal);
        __syncthreads();
        int base = 0, total = 0;
        for (int w = 0; w < T / 32; ++w) {
            const int c = s_warp_count[w];
            if (w < warp) base += c;
            total += c;
        }
        if (hit) {
            const int slot = base + __popc(bal & ((1u << lane) - 1u));
            const float scale = a.normalize ? __ldg(a.wscale + (long long)b * a.N + n) : 1.0f;
            const float *c = a.color + ((long long)b * a.N + n) * 3;
            s_cx[slot] = p.cx; s_cy[slot] = p.cy; s_fx[slot] = p.fx; s_fy[slot] = p.fy; s_w[slot] = scale;
            s_r[slot] = __ldg(c); s_g[slot] = __ldg(c + 1); s_b[slot] = __ldg(c + 2);
        }
        __syncthreads();
        for (int e = 0; e < total; ++e) {
            const int dx = px - s_cx[e], dy = py - s_cy[e];
            if (dx < -r || dx > r || dy < -r || dy > r) continue;
            const float tx = (float)dx - s_fx[e], ty = (float)dy - s_fy[e];
            const float w = expf(-(tx * tx + ty * ty) * inv2s2) * s_w[e];
            acc[0] = fmaf(s_r[e], w, acc[0]);
            acc[1] = fmaf(s_g[e], w, acc[1]);
            acc[2] = fmaf(s_b[e], w, acc[2]);
            acc[3] += w;
        }
        __syncthreads();
    }
    if (px < a.img && py < a.img)
        reinterpret_cast<float4 *>(a.out)[((long long)b * a.img + py) * a.img + px] =
            make_float4(acc[0], acc[1], acc[2], acc[3]);
}

__device__ inline float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One warp per particle.  With A = c . g_rgb + g_density at a pixel and g the unnormalised weight:
//   dL/dc      = scale * sum g g_rgb
//   dL/dfrac_x = scale / sigma^2 * [ sum A g t_x  -  (sum A g) (T_x S_y) / (1e-8 + S) ]   (normalised)
//              =         1 / sigma^2 * sum A g t_x                                         (plain)
// sums over the pixels of the patch that lie inside the image; S = S_x S_y and T_x = sum g_x t_x over
// the whole patch axis; t_x = dx - frac_x.  floor() passes no gradient, so dL/dp = dL/dfrac.
__global__ void __launch_bounds__(256) splat_backward_kernel(SplatArgs a) {
    const int lane = threadIdx.x & 31;
    const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
    const long long total = (long long)a.B * a.N;
    if (warp >= total) return;
    const int b = (int)(warp / a.N);
    const SplatPoint p = splat_point(a, warp);
    const int r = a.radius, P = 2 * r + 1;
    const float inv2s2 = 1.0f / (2.0f * a.sigma * a.sigma);
    const float *c = a.color + warp * 3;
    const float cr = __ldg(c), cg = __ldg(c + 1), cb = __ldg(c + 2);
    float gr = 0.f, gg = 0.f, gb = 0.f, a0 = 0.f, ax = 0.f, ay = 0.f;
    const float4 *img = reinterpret_cast<const float4 *>(a.g_out) + (long long)b * a.img * a.img;
    for (int k = lane; k < P * P; k += 32) {
        const int dy = k / P - r, dx = k - (k / P) * P - r;
        const int px = p.cx + dx, py = p.cy + dy;
        if (px < 0 || px >= a.img || py < 0 || py >= a.img) continue;
        const float tx = (float)dx - p.fx, ty = (float)dy - p.fy;
        const float g = expf(-(tx * tx + ty * ty) * inv2s2);
        const float4 d = __ldg(img + (long long)py * a.img + px);
        const float A = fmaf(cr, d.x, fmaf(cg, d.y, fmaf(cb, d.z, d.w)));
        gr = fmaf(g, d.x, gr); gg = fmaf(g, d.y, gg); gb = fmaf(g, d.z, gb);
        const float Ag = A * g;
        a0 += Ag;
        ax = fmaf(Ag, tx, ax);
        ay = fmaf(Ag, ty, ay);
    }
    gr = warp_sum(gr); gg = warp_sum(gg); gb = warp_sum(gb);
    a0 = warp_sum(a0); ax = warp_sum(ax); ay = warp_sum(ay);
    float sx = 0.f, sy = 0.f, t_x = 0.f, t_y = 0.f;
    if (a.normalize) {  // the axis sums, spread over the lanes
        for (int d = -r + lane; d <= r; d += 32) {
            const float ux = (float)d - p.fx, uy = (float)d - p.fy;
            const float ex = expf(-(ux * ux) * inv2s2), ey = expf(-(uy * uy) * inv2s2);
            sx += ex; sy += ey;
            t_x = fmaf(ex, ux, t_x); t_y = fmaf(ey, uy, t_y);
        }
        sx = warp_sum(sx); sy = warp_sum(sy); t_x = warp_sum(t_x); t_y = warp_sum(t_y);
    }
    if (lane != 0) return;
    float scale = 1.0f, gfx = ax, gfy = ay;
    if (a.normalize) {
        const float inv = 1.0f / (1e-8f + sx * sy);
        scale = a.norm_scale * inv;
        gfx = ax - a0 * inv * (t_x * sy);
        gfy = ay - a0 * inv * (sx * t_y);
    }
    const float inv_s2 = 1.0f / (a.sigma * a.sigma);
    const float chain = (float)(a.img - 1) / a.span;
    if (a.g_color) {
        float *o = a.g_color + warp * 3;
        o[0] = scale * gr; o[1] = scale * gg; o[2] = scale * gb;
    }
    if (a.g_x) {
        const float sign_y = a.y_up ? -1.0f : 1.0f;
        reinterpret_cast<float2 *>(a.g_x)[warp] =
            make_float2(scale * inv_s2 * gfx * chain, sign_y * scale * inv_s2 * gfy * chain);
    }
}

static int check_splat(const char *name, const SplatArgs &a) {
    if (a.B <= 0 || a.N <= 0 || a.img <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: batch, particles and img_size must be positive", name);
    if (a.radius < 1 || a.radius > kSplatMaxRadius)
        return fail(NPA_ERR_UNSUPPORTED, "%s: patch radius %d is outside 1..%d", name, a.radius, kSplatMaxRadius);
    if (!(a.sigma > 0.f) || !(a.span != 0.f)) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: sigma must be positive and hi != lo", name);
    if (!a.x || !a.color) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: x and color must be non-NULL", name);
    if ((uintptr_t)a.x % 8) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: x must be 8-byte aligned", name);
    return NPA_OK;
}

}  // namespace npa

using namespace npa;

extern "C" {

int npa_splat_forward(const float *x, const float *color, int32_t batch, int32_t particles, int32_t img_size,
                      double sigma_pixels, int32_t radius, double lo, double hi, int32_t y_up, int32_t normalize,
                      double norm_scale, float *scale_scratch, float *out, void *stream) {
    SplatArgs a = {};
    a.x = x; a.color = color; a.out = out; a.wscale = scale_scratch; a.B = batch; a.N = particles; a.img = img_size; a.radius = radius;
    a.y_up = y_up; a.normalize = normalize; a.lo = (float)lo; a.span = (float)(hi - lo); a.sigma = (float)sigma_pixels;
    a.norm_scale = (float)norm_scale;
    int rc = check_splat("npa_splat_forward", a);
    if (rc != NPA_OK) return rc;
    if (!out || (uintptr_t)out % 16) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_splat_forward: out must be non-NULL and 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (normalize) {
        if (!scale_scratch) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_splat_forward: scale_scratch [B*N] is needed when normalize != 0");
        const long long n = (long long)batch * particles;
        splat_scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(a);
        if ((rc = check_launch("splat_scale_kernel")) != NPA_OK) return rc;
    }
    const int tiles = (img_size + kSplatTile - 1) / kSplatTile;
    splat_forward_kernel<<<dim3(tiles * tiles, batch), kSplatTile * kSplatTile, 0, st>>>(a);
    return check_launch("splat_forward_kernel");
}

int npa_splat_backward(const float *x, const float *color, const float *g_out, int32_t batch, int32_t particles,
                       int32_t img_size, double sigma_pixels, int32_t radius, double lo, double hi, int32_t y_up,
                       int32_t normalize, double norm_scale, float *g_x, float *g_color, void *stream) {
    SplatArgs a = {};
    a.x = x; a.color = color; a.g_out = g_out; a.g_x = g_x; a.g_color = g_color; a.B = batch; a.N = particles;
    a.img = img_size; a.radius = radius; a.y_up = y_up; a.normalize = normalize; a.lo = (float)lo; a.span = (float)(hi - lo);
    a.sigma = (float)sigma_pixels; a.norm_scale = (float)norm_scale;
    int rc = check_splat("npa_splat_backward", a);
    if (rc != NPA_OK) return rc;
    if (!g_out || (uintptr_t)g_out % 16) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_splat_backward: g_out must be non-NULL and 16-byte aligned");
    if (g_x && (uintptr_t)g_x % 8) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_splat_backward: g_x must be 8-byte aligned");
    const long long warps = (long long)batch * particles;
    const long long ctas = (warps * 32 + 255) / 256;
    if (ctas >= (1ll << 31)) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_splat_backward: too many particles");
    splat_backward_kernel<<<(unsigned)ctas, 256, 0, (cudaStream_t)stream>>>(a);
    return check_launch("splat_backward_kernel");
}

}  // extern "C"
