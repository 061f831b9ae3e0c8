// Gradient at the hidden layer of the per-particle MLP, with the ReLU mask applied:
//
//     dh [rows, 128] = (dy [rows, out] . W2 [out, 128])  where h > 0,  else 0
//
// (models/npa.py:63-75: the backward of Linear(128, out, bias=False) followed by the backward of the
// ReLU that produced h).  torch runs it as a thin fp32 GEMM (35 columns of dy) plus a masking pass over
// dh; here it is one pass on the CUDA cores in fp32: dh is written once and h is read once.  The
// product is too thin for the tensor cores to matter (out <= 48 multiply-adds per output element
// against 8 bytes of traffic).
//
// A warp takes eight rows at a time.  W2 (zero-padded to a multiple of four rows) stays in shared
// memory; the eight rows of dy are staged per warp; lane l owns hidden units 4 l .. 4 l + 3 of all eight
// rows, so every shared-memory load is either a conflict-free float4 of W2 or a broadcast float4 of dy,
// and 16 multiply-adds follow each broadcast.
#include "common.cuh"

namespace npa {

constexpr int kHgHidden = 128;
constexpr int kHgMaxOut = 48;
constexpr int kHgRows = 8;       // rows per warp pass
constexpr int kHgWarps = 8;
constexpr int kHgThreads = kHgWarps * 32;

struct HiddenGradArgs {
    const float *dy, *W2, *h;
    float *dh;
    long long rows, w_stride_out, w_stride_in;
    int out_dim, out4;  // out4 = out_dim rounded up to a multiple of 4
};

__global__ void __launch_bounds__(kHgThreads, 3) mlp_hidden_grad_kernel(HiddenGradArgs a) {
    __shared__ __align__(16) float w2s[kHgMaxOut][kHgHidden];
    __shared__ __align__(16) float dys[kHgWarps][kHgRows][kHgMaxOut];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int O = a.out_dim, O4 = a.out4;
    for (int e = threadIdx.x; e < O4 * kHgHidden; e += kHgThreads) {
        const int o = e / kHgHidden, j = e - o * kHgHidden;
        w2s[o][j] = o < O ? __ldg(a.W2 + o * a.w_stride_out + j * a.w_stride_in) : 0.f;
    }
    __syncthreads();

    const long long groups = (a.rows + kHgRows - 1) / kHgRows;
    for (long long g = (long long)blockIdx.x * kHgWarps + warp; g < groups; g += (long long)gridDim.x * kHgWarps) {
        const long long r0 = g * kHgRows;
        // the eight rows of dy are contiguous: r0 * O .. (r0 + 8) * O
        const long long first = r0 * O, limit = a.rows * O;
        {   // the next pass's rows of dy (at most 12 lines) and this pass's rows of h (32 lines) towards L1
            const long long nfirst = first + (long long)gridDim.x * kHgWarps * kHgRows * O;
            if (lane * 32 < kHgRows * O && nfirst + lane * 32 < limit) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.dy + nfirst + lane * 32));
            if (r0 + (lane >> 2) < a.rows) asm volatile("prefetch.global.L1 [%0];" ::"l"(a.h + r0 * kHgHidden + lane * 32));
        }
        for (int e = lane; e < kHgRows * O4; e += 32) {
            const int r = e / O4, o = e - r * O4;
            const long long at = first + (long long)r * O + o;
            dys[warp][r][o] = (o < O && at < limit) ? __ldg(a.dy + at) : 0.f;
        }
        __syncwarp();
        float4 acc[kHgRows];
#pragma unroll
        for (int r = 0; r < kHgRows; ++r) acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 2
        for (int o = 0; o < O4; o += 4) {
            const float4 w0 = *(const float4 *)&w2s[o][4 * lane], w1 = *(const float4 *)&w2s[o + 1][4 * lane];
            const float4 w2 = *(const float4 *)&w2s[o + 2][4 * lane], w3 = *(const float4 *)&w2s[o + 3][4 * lane];
#pragma unroll
            for (int r = 0; r < kHgRows; ++r) {
                const float4 d = *(const float4 *)&dys[warp][r][o];  // the same address in every lane: a broadcast
                acc[r].x = fmaf(d.x, w0.x, acc[r].x); acc[r].y = fmaf(d.x, w0.y, acc[r].y);
                acc[r].z = fmaf(d.x, w0.z, acc[r].z); acc[r].w = fmaf(d.x, w0.w, acc[r].w);
                acc[r].x = fmaf(d.y, w1.x, acc[r].x); acc[r].y = fmaf(d.y, w1.y, acc[r].y);
                acc[r].z = fmaf(d.y, w1.z, acc[r].z); acc[r].w = fmaf(d.y, w1.w, acc[r].w);
                acc[r].x = fmaf(d.z, w2.x, acc[r].x); acc[r].y = fmaf(d.z, w2.y, acc[r].y);
                acc[r].z = fmaf(d.z, w2.z, acc[r].z); acc[r].w = fmaf(d.z, w2.w, acc[r].w);
                acc[r].x = fmaf(d.w, w3.x, acc[r].x); acc[r].y = fmaf(d.w, w3.y, acc[r].y);
                acc[r].z = fmaf(d.w, w3.z, acc[r].z); acc[r].w = fmaf(d.w, w3.w, acc[r].w);
            }
        }
#pragma unroll
        for (int r = 0; r < kHgRows; ++r) {
            const long long row = r0 + r;
            if (row < a.rows) {
                const float4 hv = __ldg((const float4 *)(a.h + row * kHgHidden) + lane);
                float4 v = acc[r];
                if (!(hv.x > 0.f)) v.x = 0.f;
                if (!(hv.y > 0.f)) v.y = 0.f;
                if (!(hv.z > 0.f)) v.z = 0.f;
                if (!(hv.w > 0.f)) v.w = 0.f;
                *((float4 *)(a.dh + row * kHgHidden) + lane) = v;
            }
        }
        __syncwarp();  // the staged rows are overwritten by the next pass
    }
}

}  // namespace npa

using namespace npa;

extern "C" {

int npa_mlp_hidden_grad(const float *dy, const float *W2, const float *h, float *dh, int64_t rows, int32_t hidden,
                        int32_t out_dim, int64_t w_stride_out, int64_t w_stride_in, void *stream) {
    const char *me = "npa_mlp_hidden_grad";
    if (hidden != kHgHidden) return fail(NPA_ERR_UNSUPPORTED, "%s: hidden width must be %d, got %d", me, kHgHidden, hidden);
    if (out_dim <= 0 || out_dim > kHgMaxOut) return fail(NPA_ERR_UNSUPPORTED, "%s: supports out <= %d, got %d", me, kHgMaxOut, out_dim);
    if (rows <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: rows must be positive", me);
    if (!dy || !W2 || !h || !dh) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: every pointer must be non-NULL", me);
    if ((uintptr_t)dy % 4 || ((uintptr_t)h | (uintptr_t)dh) % 16)
        return fail(NPA_ERR_INVALID_ARGUMENT, "%s: dy must be float aligned, h and dh 16-byte aligned", me);
    HiddenGradArgs a = {dy, W2, h, dh, rows, w_stride_out, w_stride_in, out_dim, (out_dim + 3) / 4 * 4};
    const long long groups = (rows + kHgRows - 1) / kHgRows;
    const long long want = (groups + kHgWarps - 1) / kHgWarps;
    // three CTAs per SM, all resident (the launch bounds cap the kernel at 80 registers; at 84 only two fit
    // and a grid of 3 or 4 x 148 ran as two waves)
    const int ctas = (int)(want < 148 * 3 ? want : 148 * 3);
    mlp_hidden_grad_kernel<<<ctas, kHgThreads, 0, (cudaStream_t)stream>>>(a);
    return check_launch("mlp_hidden_grad_kernel");
}

}  // extern "C"
