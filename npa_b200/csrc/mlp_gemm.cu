// Linear layers of the per-particle MLP on the tensor cores, at fp32 accuracy.
//
//     C[M, N] = act( A[M, K] . B[K, N] + bias[N] ),    B[k][n] = W[n * stride_n + k * stride_k]
//
// covers the four GEMMs of the adaptation MLP of an NPA model (models/npa.py:63-75) -- h = relu(z W1^T
// + b1), y = h W2^T, dh = dy W2, dz = dh W1 -- with M = B*N particles (hundreds of thousands) and
// K, N <= 176.  torch runs them as SIMT fp32 cuBLAS kernels (28-44 TFLOP/s on these thin shapes).
// Here each product is formed by three TF32 tensor-core MMAs on operands split into a TF32 head
// and a TF32 tail (a = a_hi + a_lo; a.b ~ a_lo b_hi + a_hi b_lo + a_hi b_hi, fp32 accumulation):
// the dropped a_lo b_lo term is 2^-22 of the product, so results match fp32 arithmetic to ~1e-6.
// mma.sync.m16n8k8 is the tensor-core instruction used; it runs at ~278 TFLOP/s on a B200.
//
// A CTA of 16 warps keeps the whole weight matrix B in shared memory and streams tiles of 64 rows
// of A (cp.async, double buffered); warp w owns rows 16 (w % 4) .. +15 of the tile and one quarter
// of the column tiles.  Operands are split into head and tail on the fly (a mask and a subtraction);
// per k-step a warp first loads and splits its B fragments, then issues the MMAs term by term so that
// consecutive MMAs go to different accumulators.  Row pitches of the shared arrays are chosen so
// that the fragment loads of a warp hit 32 different banks (pitch of A = 4 mod 32, of B = 8 mod 32).
#include "common.cuh"

namespace npa {

constexpr int kGemmRows = 64;      // rows of A per tile
constexpr int kGemmThreads = 512;
constexpr int kGemmMaxDim = 176;   // K and N
constexpr int kGemmMaxNt = 6;      // column tiles (of 8) per warp

struct GemmArgs {
    const float *A;      // [M, K], row pitch K
    const float *W;      // weights, addressed through the two strides
    const float *bias;   // [N] or NULL
    const float *gate;   // [M, N] or NULL: the output is zero where gate <= 0 (ReLU backward)
    float *C;            // [M, N], row pitch N
    long long M;
    int K, N, stride_n, stride_k, relu;
    int Kp, lda, ldb, nt_warp;  // K rounded up to 8, shared pitches, column tiles per warp
};

// TF32 head of x by truncation (the MMA reads only the upper 19 bits of an operand anyway); the tail
// x - head is exact in fp32.  A mask and a subtraction run at full rate, unlike cvt.rna.tf32.
__device__ inline unsigned tf32_head(float x) { return __float_as_uint(x) & 0xffffe000u; }
__device__ inline unsigned tf32_tail(float x, unsigned head) { return __float_as_uint(x - __uint_as_float(head)); }

__device__ inline void mma_tf32(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kGemmThreads, 1) linear_tf32x3_kernel(GemmArgs a) {
    extern __shared__ __align__(16) float smem[];
    float *Bs = smem;                                  // [Kp][ldb]
    float *As = smem + (size_t)a.Kp * a.ldb;           // 2 x [kGemmRows][lda]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int K = a.K, N = a.N, lda = a.lda, ldb = a.ldb;

    // weights, once per CTA; padding rows and columns are zero
    for (int e = tid; e < a.Kp * ldb; e += kGemmThreads) {
        const int k = e / ldb, n = e - k * ldb;
        Bs[e] = (k < K && n < N) ? __ldg(a.W + (long long)n * a.stride_n + (long long)k * a.stride_k) : 0.f;
    }
    // padding columns of both A buffers (never written by the tile copies)
    for (int e = tid; e < 2 * kGemmRows * (lda - K); e += kGemmThreads) {
        const int r = e / (lda - K), c = K + e - r * (lda - K);
        As[(size_t)r * lda + c] = 0.f;
    }

    const long long tiles = (a.M + kGemmRows - 1) / kGemmRows;
    auto fetch = [&](long long tile, int buf) {  // rows of the tile, 4 bytes at a time into padded rows
        float *dst = As + (size_t)buf * kGemmRows * lda;
        const long long r0 = tile * kGemmRows;
        for (int r = warp; r < kGemmRows; r += kGemmThreads / 32) {
            if (r0 + r >= a.M) break;
            const float *src = a.A + (r0 + r) * K;
            for (int c = lane; c < K; c += 32) {
                const unsigned d = (unsigned)__cvta_generic_to_shared(dst + (size_t)r * lda + c);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(src + c) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    const int m0 = 16 * (warp & 3);            // rows of this warp inside the tile
    const int nt0 = (warp >> 2) * a.nt_warp;   // first column tile of this warp (four column groups)
    long long tile = blockIdx.x;
    int buf = 0;
    if (tile < tiles) fetch(tile, 0);
    for (; tile < tiles; tile += gridDim.x, buf ^= 1) {
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();  // the tile (and, first time, B) is complete; everyone has left the other buffer
        if (tile + gridDim.x < tiles) fetch(tile + gridDim.x, buf ^ 1);
        const float *At = As + (size_t)buf * kGemmRows * lda;

        float acc[kGemmMaxNt][4];
#pragma unroll
        for (int j = 0; j < kGemmMaxNt; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

#pragma unroll 2
        for (int k0 = 0; k0 < a.Kp; k0 += 8) {
            float af[4];
            af[0] = At[(m0 + g) * lda + k0 + t];
            af[1] = At[(m0 + g + 8) * lda + k0 + t];
            af[2] = At[(m0 + g) * lda + k0 + t + 4];
            af[3] = At[(m0 + g + 8) * lda + k0 + t + 4];
            unsigned ah[4], al[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                ah[q] = tf32_head(af[q]);
                al[q] = tf32_tail(af[q], ah[q]);
            }
            const float *b_row0 = Bs + (size_t)(k0 + t) * ldb + g;
            const float *b_row1 = Bs + (size_t)(k0 + t + 4) * ldb + g;
            // all column tiles of this warp: load and split first, then issue the MMAs term by term, so
            // that consecutive MMAs go to different accumulators (no dependent chain stalls the pipe)
            unsigned bh0[kGemmMaxNt], bh1[kGemmMaxNt], bl0[kGemmMaxNt], bl1[kGemmMaxNt];
#pragma unroll
            for (int j = 0; j < kGemmMaxNt; ++j) {
                if (j < a.nt_warp) {  // warp-uniform
                    const int n0 = 8 * (nt0 + j);
                    const float b0 = b_row0[n0], b1 = b_row1[n0];
                    bh0[j] = tf32_head(b0);
                    bh1[j] = tf32_head(b1);
                    bl0[j] = tf32_tail(b0, bh0[j]);
                    bl1[j] = tf32_tail(b1, bh1[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < kGemmMaxNt; ++j)
                if (j < a.nt_warp) mma_tf32(acc[j], al, bh0[j], bh1[j]);
#pragma unroll
            for (int j = 0; j < kGemmMaxNt; ++j)
                if (j < a.nt_warp) mma_tf32(acc[j], ah, bl0[j], bl1[j]);
#pragma unroll
            for (int j = 0; j < kGemmMaxNt; ++j)
                if (j < a.nt_warp) mma_tf32(acc[j], ah, bh0[j], bh1[j]);
        }

        // epilogue: bias, activation, store (c0, c1: row g; c2, c3: row g + 8; columns 2t, 2t + 1)
        const long long row_a = tile * kGemmRows + m0 + g, row_b = row_a + 8;
#pragma unroll
        for (int j = 0; j < kGemmMaxNt; ++j) {
            if (j < a.nt_warp) {
                const int col = 8 * (nt0 + j) + 2 * t;
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int c = col + q;
                    if (c < N) {
                        const float bv = a.bias ? __ldg(a.bias + c) : 0.f;
                        float v0 = acc[j][q] + bv, v1 = acc[j][2 + q] + bv;
                        if (a.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); }
                        if (row_a < a.M) a.C[row_a * N + c] = (a.gate && !(__ldg(a.gate + row_a * N + c) > 0.f)) ? 0.f : v0;
                        if (row_b < a.M) a.C[row_b * N + c] = (a.gate && !(__ldg(a.gate + row_b * N + c) > 0.f)) ? 0.f : v1;
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

}  // namespace npa

using namespace npa;

extern "C" {

int npa_linear_tf32x3(const float *A, const float *W, const float *bias, const float *gate, float *C, int64_t rows,
                      int32_t in_dim, int32_t out_dim, int64_t w_stride_out, int64_t w_stride_in, int32_t relu,
                      void *stream) {
    if (rows <= 0 || in_dim <= 0 || out_dim <= 0)
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tf32x3: rows, in_dim and out_dim must be positive");
    if (in_dim > kGemmMaxDim || out_dim > kGemmMaxDim)
        return fail(NPA_ERR_UNSUPPORTED, "npa_linear_tf32x3: supports in_dim and out_dim up to %d, got %d and %d", kGemmMaxDim,
                    in_dim, out_dim);
    if (!A || !W || !C) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tf32x3: A, W and C must be non-NULL");
    if ((uintptr_t)A % 4 || (uintptr_t)C % 4) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tf32x3: A and C must be float aligned");
    GemmArgs a = {};
    a.A = A; a.W = W; a.bias = bias; a.gate = gate; a.C = C; a.M = rows; a.K = in_dim; a.N = out_dim;
    a.stride_n = (int)w_stride_out; a.stride_k = (int)w_stride_in; a.relu = relu;
    a.Kp = (in_dim + 7) / 8 * 8;
    a.lda = a.Kp + 4;
    while (a.lda % 32 != 4) a.lda += 4;  // Kp is a multiple of 8: 4 mod 32 is reached within 32
    const int nt = (out_dim + 7) / 8;
    a.nt_warp = (nt + 3) / 4;  // column tiles per warp: the 16 warps form 4 row groups x 4 column groups
    a.ldb = 4 * a.nt_warp * 8;
    while (a.ldb % 32 != 8) a.ldb += 8;
    const size_t smem = ((size_t)a.Kp * a.ldb + (size_t)2 * kGemmRows * a.lda) * sizeof(float);
    if (smem > 227 * 1024)
        return fail(NPA_ERR_UNSUPPORTED, "npa_linear_tf32x3: %d x %d weights need %zu bytes of shared memory", in_dim, out_dim, smem);
    cudaError_t e = cudaFuncSetAttribute(linear_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "npa_linear_tf32x3: raising the shared-memory limit: %s", cudaGetErrorString(e));
    const long long tiles = (rows + kGemmRows - 1) / kGemmRows;
    const int ctas = (int)(tiles < 148 ? tiles : 148);
    linear_tf32x3_kernel<<<ctas, kGemmThreads, smem, (cudaStream_t)stream>>>(a);
    return check_launch("linear_tf32x3_kernel");
}

}  // extern "C"
