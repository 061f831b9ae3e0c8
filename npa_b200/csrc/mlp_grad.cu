// Weight gradients of the per-particle MLP of an NPA model in one pass over the particles.
//
// The adaptation MLP (models/npa.py:63-75: Linear(in, 128) -> ReLU -> Linear(128, out, bias=False))
// is applied to every particle, so the gradients of its weights are reductions over all B*N rows:
//     dW1 [H, in]  = dh^T z        dW2 [out, H] = dy^T h        db1 [H] = sum_rows dh
// (z the perception rows, h the hidden activations, dh / dy the upstream gradients of the hidden
// and output layers).  torch computes them as three separate tall-skinny cuBLAS / reduce kernels
// that together take half of the MLP's forward + backward time.  Here every CTA walks slabs of 32
// rows (copied with cp.async into a double-buffered shared-memory tile), keeps its share of the
// three results in registers as outer-product accumulators, and writes them once at the end to a
// scratch array [CTAs, H*in + out*H + H]; a second kernel adds the CTA partials in a fixed order,
// so the sums are deterministic.  fp32 on the CUDA cores; H is fixed at 128 (the reference's
// default), in <= 176, out <= 48.
#include "common.cuh"

namespace npa {

constexpr int kMlpHidden = 128;
constexpr int kMlpRows = 32;        // rows per slab
constexpr int kMlpMaxIn = 176;      // 11 columns per thread, 16 threads across
constexpr int kMlpMaxOut = 48;      // 3 outputs per thread, 16 threads across
constexpr int kMlpThreads = 256;

struct MlpGradArgs {
    const float *z, *dh, *h, *dy;
    long long rows;
    int in_dim, out_dim;
    float *partial;  // [gridDim.x, total]
    float *dW1, *dW2, *db1;
    int ctas;
};

__device__ inline void slab_copy_async(float *dst, const float *src, int floats) {
    for (int q = threadIdx.x; q < floats / 4; q += blockDim.x) {
        const unsigned d = (unsigned)__cvta_generic_to_shared(dst + 4 * q);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src + 4 * q) : "memory");
    }
}

// Thread (ti, tj) of a 16 x 16 arrangement owns
//   dW1[i][j]  for i = 8 ti .. 8 ti + 7 and j = tj + 16 k (k < NJ, NJ >= ceil(in / 16)),
//   dW2[o][i'] for i' = 8 tj .. 8 tj + 7 and o = ti + 16 k (k < NO, NO >= ceil(out / 16)),
//   db1[i]     for its 8 i when tj == 0.
// Columns j >= in (o >= out) of the last k are read from whatever follows in the tile and never
// written out: the loads carry no bounds test (the tile is followed by 16 floats of padding).
template <int NJ, int NO>
__global__ void __launch_bounds__(kMlpThreads, 1) mlp_weight_grad_kernel(MlpGradArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int K = a.in_dim, O = a.out_dim, H = kMlpHidden;
    const int slab_floats = kMlpRows * (K + 2 * H + O) + 16;  // + padding read by the unguarded loads
    const int ti = threadIdx.x >> 4, tj = threadIdx.x & 15;
    float acc1[8][NJ], acc2[NO][8], accb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        accb[i] = 0.f;
#pragma unroll
        for (int k = 0; k < NJ; ++k) acc1[i][k] = 0.f;
#pragma unroll
        for (int k = 0; k < NO; ++k) acc2[k][i] = 0.f;
    }
    const long long slabs = (a.rows + kMlpRows - 1) / kMlpRows;
    auto rows_of = [&](long long s) {
        const long long left = a.rows - s * kMlpRows;
        return (int)(left < kMlpRows ? left : kMlpRows);
    };
    // a slab in shared memory: [z rows | dh rows | h rows | dy rows], each block contiguous
    auto fetch = [&](long long s, int buf) {
        float *base = smem + (size_t)buf * slab_floats;
        const int n = rows_of(s);
        const long long r0 = s * kMlpRows;
        if (n == kMlpRows) {  // whole slabs are multiples of 16 bytes at 16-byte aligned offsets
            slab_copy_async(base, a.z + r0 * K, n * K);
            slab_copy_async(base + kMlpRows * K, a.dh + r0 * H, n * H);
            slab_copy_async(base + kMlpRows * (K + H), a.h + r0 * H, n * H);
            slab_copy_async(base + kMlpRows * (K + 2 * H), a.dy + r0 * O, n * O);
        } else {              // the last, partial slab: plain loads
            for (int e = threadIdx.x; e < n * K; e += blockDim.x) base[e] = __ldg(a.z + r0 * K + e);
            for (int e = threadIdx.x; e < n * H; e += blockDim.x) {
                base[kMlpRows * K + e] = __ldg(a.dh + r0 * H + e);
                base[kMlpRows * (K + H) + e] = __ldg(a.h + r0 * H + e);
            }
            for (int e = threadIdx.x; e < n * O; e += blockDim.x) base[kMlpRows * (K + 2 * H) + e] = __ldg(a.dy + r0 * O + e);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    long long s = blockIdx.x;
    int buf = 0;
    if (s < slabs) fetch(s, 0);
    for (; s < slabs; s += gridDim.x, buf ^= 1) {
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();  // slab s is complete; every thread is done with the other buffer
        if (s + gridDim.x < slabs) fetch(s + gridDim.x, buf ^ 1);
        const float *zt = smem + (size_t)buf * slab_floats;
        const float *dht = zt + kMlpRows * K, *ht = dht + kMlpRows * H, *dyt = ht + kMlpRows * H;
        const int n = rows_of(s);
        for (int r = 0; r < n; ++r) {
            float dv[8], hv[8], zv[NJ], yv[NO];
            const float4 d0 = *reinterpret_cast<const float4 *>(dht + r * H + 8 * ti);
            const float4 d1 = *reinterpret_cast<const float4 *>(dht + r * H + 8 * ti + 4);
            dv[0] = d0.x; dv[1] = d0.y; dv[2] = d0.z; dv[3] = d0.w; dv[4] = d1.x; dv[5] = d1.y; dv[6] = d1.z; dv[7] = d1.w;
            const float4 h0 = *reinterpret_cast<const float4 *>(ht + r * H + 8 * tj);
            const float4 h1 = *reinterpret_cast<const float4 *>(ht + r * H + 8 * tj + 4);
            hv[0] = h0.x; hv[1] = h0.y; hv[2] = h0.z; hv[3] = h0.w; hv[4] = h1.x; hv[5] = h1.y; hv[6] = h1.z; hv[7] = h1.w;
#pragma unroll
            for (int k = 0; k < NJ; ++k) zv[k] = zt[r * K + tj + 16 * k];
#pragma unroll
            for (int k = 0; k < NO; ++k) yv[k] = dyt[r * O + ti + 16 * k];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int k = 0; k < NJ; ++k) acc1[i][k] = fmaf(dv[i], zv[k], acc1[i][k]);
#pragma unroll
                for (int k = 0; k < NO; ++k) acc2[k][i] = fmaf(yv[k], hv[i], acc2[k][i]);
                accb[i] += dv[i];
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");

    // this CTA's partial sums: [dW1 (H x K) | dW2 (O x H) | db1 (H)]
    float *out = a.partial + (size_t)blockIdx.x * ((size_t)H * K + (size_t)O * H + H);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int k = 0; k < NJ; ++k)
            if (tj + 16 * k < K) out[(size_t)(8 * ti + i) * K + tj + 16 * k] = acc1[i][k];
#pragma unroll
        for (int k = 0; k < NO; ++k)
            if (ti + 16 * k < O) out[(size_t)H * K + (size_t)(ti + 16 * k) * H + 8 * tj + i] = acc2[k][i];
        if (tj == 0) out[(size_t)H * K + (size_t)O * H + 8 * ti + i] = accb[i];
    }
}

// Adds the CTA partials in CTA order (deterministic) and writes the three gradients.
__global__ void __launch_bounds__(256) mlp_weight_grad_reduce_kernel(MlpGradArgs a) {
    const int K = a.in_dim, O = a.out_dim, H = kMlpHidden;
    const int total = H * K + O * H + H;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    float sum = 0.f;
    for (int c = 0; c < a.ctas; ++c) sum += a.partial[(size_t)c * total + e];
    if (e < H * K) a.dW1[e] = sum;
    else if (e < H * K + O * H) a.dW2[e - H * K] = sum;
    else a.db1[e - H * K - O * H] = sum;
}

static int mlp_grad_ctas(long long rows) {
    const long long slabs = (rows + kMlpRows - 1) / kMlpRows;
    return (int)(slabs < 148 ? (slabs > 0 ? slabs : 1) : 148);
}

}  // namespace npa

using namespace npa;

extern "C" {

int64_t npa_mlp_weight_grad_scratch_floats(int64_t rows, int32_t in_dim, int32_t out_dim) {
    if (rows <= 0 || in_dim <= 0 || out_dim <= 0) return 0;
    return (int64_t)mlp_grad_ctas(rows) * ((int64_t)kMlpHidden * in_dim + (int64_t)out_dim * kMlpHidden + kMlpHidden);
}

int npa_mlp_weight_grad(const float *z, const float *dh, const float *h, const float *dy, int64_t rows, int32_t in_dim,
                        int32_t hidden, int32_t out_dim, float *scratch, int64_t scratch_floats, float *dW1,
                        float *dW2, float *db1, void *stream) {
    if (hidden != kMlpHidden) return fail(NPA_ERR_UNSUPPORTED, "npa_mlp_weight_grad: hidden width must be %d, got %d", kMlpHidden, hidden);
    if (in_dim <= 0 || in_dim > kMlpMaxIn || out_dim <= 0 || out_dim > kMlpMaxOut)
        return fail(NPA_ERR_UNSUPPORTED, "npa_mlp_weight_grad: supports in <= %d and out <= %d, got %d and %d", kMlpMaxIn,
                    kMlpMaxOut, in_dim, out_dim);
    if (rows <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_mlp_weight_grad: rows must be positive");
    if (!z || !dh || !h || !dy || !scratch || !dW1 || !dW2 || !db1)
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_mlp_weight_grad: every pointer must be non-NULL");
    if (((uintptr_t)z | (uintptr_t)dh | (uintptr_t)h | (uintptr_t)dy) % 16)
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_mlp_weight_grad: z, dh, h and dy must be 16-byte aligned");
    const int64_t need = npa_mlp_weight_grad_scratch_floats(rows, in_dim, out_dim);
    if (scratch_floats < need)
        return fail(NPA_ERR_SCRATCH_TOO_SMALL, "npa_mlp_weight_grad: scratch has %lld floats, %lld needed", (long long)scratch_floats, (long long)need);
    MlpGradArgs a = {z, dh, h, dy, rows, in_dim, out_dim, scratch, dW1, dW2, db1, mlp_grad_ctas(rows)};
    const size_t smem = (size_t)2 * (kMlpRows * (in_dim + 2 * kMlpHidden + out_dim) + 16) * sizeof(float);
    cudaStream_t st = (cudaStream_t)stream;
    // columns per thread: the smallest instantiated widths that cover in_dim and out_dim
    const int nj = (in_dim + 15) / 16, no = (out_dim + 15) / 16;
    cudaError_t e = cudaSuccess;
#define NPA_MLP_LAUNCH(NJ, NO)                                                                                      \
    do {                                                                                                            \
        e = cudaFuncSetAttribute(mlp_weight_grad_kernel<NJ, NO>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                                 (int)smem);                                                                        \
        if (e == cudaSuccess) mlp_weight_grad_kernel<NJ, NO><<<a.ctas, kMlpThreads, smem, st>>>(a);                 \
    } while (0)
#define NPA_MLP_PICK_NO(NJ)                                                                                         \
    do {                                                                                                            \
        if (no <= 1) NPA_MLP_LAUNCH(NJ, 1);                                                                         \
        else if (no == 2) NPA_MLP_LAUNCH(NJ, 2);                                                                    \
        else NPA_MLP_LAUNCH(NJ, 3);                                                                                 \
    } while (0)
    // the limit belongs to the function on the current device; setting it on every call keeps no state
    if (nj <= 3) NPA_MLP_PICK_NO(3);
    else if (nj <= 5) NPA_MLP_PICK_NO(5);
    else if (nj <= 8) NPA_MLP_PICK_NO(8);
    else NPA_MLP_PICK_NO(11);
#undef NPA_MLP_PICK_NO
#undef NPA_MLP_LAUNCH
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "npa_mlp_weight_grad: raising the shared-memory limit: %s", cudaGetErrorString(e));
    int rc = check_launch("mlp_weight_grad_kernel");
    if (rc != NPA_OK) return rc;
    const int total = kMlpHidden * in_dim + out_dim * kMlpHidden + kMlpHidden;
    mlp_weight_grad_reduce_kernel<<<(total + 255) / 256, 256, 0, st>>>(a);
    return check_launch("mlp_weight_grad_reduce_kernel");
}

}  // extern "C"
