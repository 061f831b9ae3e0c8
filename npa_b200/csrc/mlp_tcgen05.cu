// Wide linear layers of the per-particle MLP on the fifth-generation tensor cores (tcgen05.mma,
// accumulators in tensor memory), at fp32 accuracy.
//
//     C[M, N] = act( A[M, K] . B[K, N] + bias[N] ),    B[k][n] = W[n * stride_n + k * stride_k]
//
// the same contract as npa_linear_tf32x3 (mlp_gemm.cu) for the wide products of the adaptation MLP of
// an NPA model (models/npa.py:63-75): h = relu(z W1^T + b1) and dz = dh W1 with M = B*N particles.
// Each product is three TF32 MMAs on operands split into a TF32 head and tail (a = a_hi + a_lo;
// a.b ~ a_lo b_hi + a_hi b_lo + a_hi b_hi, fp32 accumulation): the dropped a_lo b_lo term is 2^-22
// of the product.
//
// One persistent CTA per SM, warp-specialised, tiles of 128 rows, K walked in chunks of 32 floats
// (one 128-byte swizzle row):
//
//   * 16 producer warps read the rows of A from global memory (coalesced 128-byte row segments, three
//     chunks in flight in registers), split every element and write head and tail into the stage's
//     two K-major 128-byte-swizzled operand tiles;
//   * one lane streams the matching chunk of the weights -- split and swizzled once per call by
//     weight_image_kernel into an image that is copied verbatim -- with one bulk copy per stage;
//   * one lane issues the MMAs (M = 128, N = out_dim rounded up to 16, K = 8 per instruction) into
//     one of two accumulators in tensor memory and commits the stage back to the producers;
//   * eight epilogue warps read a finished accumulator (tcgen05.ld, lane = row, 16 columns at a time),
//     turn the blocks through shared memory and store rows with bias, ReLU and the optional gate
//     applied (float4 when out_dim is a multiple of 4).
//
// Every wait on an mbarrier is bounded in time; a wait that gives up raises a flag that ends all
// roles, the CTA frees its tensor memory and the host reads the reason from a status word.
#include <mutex>

#include "umma.cuh"

namespace npa {

constexpr int kUmmaRows = 128;
constexpr int kUmmaChunk = 32;            // floats of K per stage
constexpr int kUmmaProducerWarps = 16;
constexpr int kUmmaEpilogueWarps = 8;     // two per quarter of the accumulator's lanes
constexpr int kUmmaWarpMma = 8, kUmmaWarpWeights = 9, kUmmaWarpProducer0 = 10;
constexpr int kUmmaThreads = (kUmmaWarpProducer0 + kUmmaProducerWarps) * 32;
constexpr int kUmmaMaxStages = 4;
constexpr int kUmmaTmemCols = 512;        // two accumulators of up to 256 columns
constexpr int kUmmaAccStride = 256;
constexpr int kUmmaTileABytes = kUmmaRows * kUmmaChunk * 4;  // one operand tile of A: 16 KB
constexpr int kUmmaEpiPitch = 20;         // floats per staged row of 16 columns: 16-byte aligned, conflict-free float4 writes
constexpr int kUmmaEpiFloats = kUmmaEpilogueWarps * 32 * kUmmaEpiPitch;

constexpr int kUmmaHloCol = 256, kUmmaYCol = 384, kUmmaY2Col = 448;  // two-layer mode: accumulators at 0 / 128, tail of h, the second layer's two accumulators

// D[tmem] (+)= A[tmem] . B[smem]^T: the A operand (128 lanes x 8 columns of 32-bit values) is read from tensor memory.
__device__ inline void umma_tf32_ts(unsigned d_tmem, unsigned a_tmem, uint64_t b_desc, unsigned idesc, int accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

enum { UMMA_STATUS_MMA = 1, UMMA_STATUS_WEIGHTS = 2, UMMA_STATUS_PRODUCER = 4, UMMA_STATUS_EPILOGUE = 8 };

struct UmmaShared {
    uint64_t full[kUmmaMaxStages], empty[kUmmaMaxStages], acc_full[2], acc_empty[2];
    uint64_t h_ready[2], y_full, w2_full, y_written, y_copied;  // two-layer mode only
    uint32_t tmem_base;
    int abort;
    alignas(16) float bias[256];
};

struct UmmaArgs {
    const float *A;      // [M, K], row pitch K
    const float *Wimg;   // [nchunks][head | tail][Np rows x 128 bytes, swizzled]
    const float *bias;   // [N] or NULL
    const float *gate;   // [M, N] or NULL: the output is zero where gate <= 0
    float *C;            // [M, N], row pitch N
    long long M;
    int K, N, Np, nchunks, last_ksteps, stages, stage_bytes, relu;
    unsigned *status;
    // two-layer mode (Y != NULL): Y [M, N2] = C . W2^T with C = the activated output of the first layer kept in
    // tensor memory; N = Np = 128, W2img = [4 chunks][head | tail][N2p rows x 128 bytes, swizzled]
    const float *W2img;
    float *Y;
    int N2, N2p;
};

__device__ unsigned g_umma_status;

// Head and tail images of the weights, chunk by chunk, in the layout the MMA reads.
__global__ void weight_image_kernel(const float *W, long long stride_n, long long stride_k, int K, int N, int Np, int nchunks,
                                    float *img) {
    const int total = nchunks * Np * kUmmaChunk;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < total; e += gridDim.x * blockDim.x) {
        const int c = e / (Np * kUmmaChunk), rem = e - c * Np * kUmmaChunk;
        const int n = rem / kUmmaChunk, kk = rem - n * kUmmaChunk;
        const int k = c * kUmmaChunk + kk;
        const float v = (n < N && k < K) ? __ldg(W + n * stride_n + k * stride_k) : 0.f;
        const float head = __uint_as_float(tf32_head_bits(v));
        float *chunk = img + (size_t)c * 2 * Np * kUmmaChunk;
        const int at = umma_swizzled(n, kk);
        chunk[at] = head;
        chunk[Np * kUmmaChunk + at] = v - head;
    }
}

template <bool FUSE>
__global__ void __launch_bounds__(kUmmaThreads, 1) linear_umma_kernel(const __grid_constant__ UmmaArgs args) {
    // every field is read into a register once: the role loops below must not go back to the parameter block
    const float *__restrict__ A = args.A;
    const float *__restrict__ Wimg = args.Wimg;
    const float *__restrict__ gate = args.gate;
    float *__restrict__ C = args.C;
    unsigned *status = args.status;
    const long long M = args.M;
    const int K = args.K, N = args.N, Np = args.Np, nchunks = args.nchunks, last_ksteps = args.last_ksteps;
    const int stages = args.stages, stage_bytes = args.stage_bytes;
    const bool relu = args.relu != 0;
    constexpr bool fuse = FUSE;  // two-layer mode
    const int N2 = args.N2, N2p = args.N2p;
    const int acc_stride = fuse ? 128 : kUmmaAccStride;
    extern __shared__ uint8_t umma_smem_raw[];
    uint8_t *base = umma_smem_raw + ((1024u - (smem_u32(umma_smem_raw) & 1023u)) & 1023u);
    uint8_t *w2s = base + (size_t)stages * stage_bytes;   // two-layer mode: the whole image of W2, resident
    const int w2_bytes = fuse ? 4 * 2 * N2p * 128 : 0;
    float *epi = (float *)(w2s + w2_bytes);
    float *ytile = epi + kUmmaEpiFloats;                  // two-layer mode: the second layer's tile, rows of N2 floats as in global memory
    UmmaShared *sh = (UmmaShared *)(ytile + (fuse ? ((kUmmaRows * N2 + 3) & ~3) : 0));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(&sh->full[s], kUmmaProducerWarps + 1);  // one arrival per producer warp + the weight copy
            mbar_init(&sh->empty[s], 1);                      // the commit of the stage's MMAs
        }
        for (int q = 0; q < 2; ++q) {
            mbar_init(&sh->acc_full[q], 1);
            // free again: when every epilogue warp has read it and (two layers) the second layer's MMAs have as well
            mbar_init(&sh->acc_empty[q], fuse ? 1 + kUmmaEpilogueWarps : kUmmaEpilogueWarps);
            mbar_init(&sh->h_ready[q], kUmmaEpilogueWarps);
        }
        mbar_init(&sh->y_full, 1);
        mbar_init(&sh->w2_full, 1);
        mbar_init(&sh->y_written, kUmmaEpilogueWarps);
        mbar_init(&sh->y_copied, kUmmaEpilogueWarps);
        sh->abort = 0;
        mbar_fence_init();
    }
    for (int c = threadIdx.x; c < 256; c += kUmmaThreads) sh->bias[c] = (args.bias && c < N) ? __ldg(args.bias + c) : 0.f;
    if (warp == kUmmaWarpMma) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)),
                     "r"(kUmmaTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = sh->tmem_base;

    const long long tiles = (M + kUmmaRows - 1) / kUmmaRows;
    const int ntile = (int)((tiles - blockIdx.x + gridDim.x - 1) / gridDim.x);  // tiles blockIdx.x, + gridDim.x, ...
    const int total = ntile * nchunks;
    bool ok = true;

    if (warp == kUmmaWarpMma) {
        // One lane runs the whole role; stage, phase and descriptors advance by additions only.
        if (lane == 0) {
            // M = 128, N = Np, TF32 x TF32 -> F32, both operands K-major
            const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(Np >> 3) << 17) | ((unsigned)(kUmmaRows >> 4) << 24);
            const uint64_t desc0 = umma_desc(smem_u32(base));
            const uint64_t stage16 = (uint64_t)(stage_bytes >> 4), alo16 = kUmmaTileABytes >> 4, bhi16 = (2 * kUmmaTileABytes) >> 4;
            const uint64_t blo16 = bhi16 + (uint64_t)((Np * 128) >> 4);
            int s = 0;
            unsigned ph = 0;
            // second layer of tile t (two-layer mode): Y tile = h . W2^T with h (in place, activated) and its tail in
            // tensor memory; it runs after the first layer of tile t + 1 has been issued, so that the epilogue of
            // tile t overlaps those MMAs
            const unsigned idesc2 = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(N2p >> 3) << 17) | ((unsigned)(kUmmaRows >> 4) << 24);
            const uint64_t w2desc = umma_desc(smem_u32(w2s));
            auto second_layer = [&](int t) -> bool {
                const int a = t & 1;
                if (t == 0 && !umma_wait(&sh->w2_full, 0, &sh->abort)) return false;
                if (!umma_wait(&sh->h_ready[a], (t >> 1) & 1, &sh->abort)) return false;
                tc_fence_after();
                // two accumulators (the epilogue adds them): consecutive MMAs into one accumulator wait for each other,
                // and at 48 columns that wait is longer than the MMA
                const unsigned dy = tmem + kUmmaYCol, dy2 = tmem + kUmmaY2Col, ah = tmem + a * 128, al = tmem + kUmmaHloCol;
#pragma unroll 1
                for (int ks = 0; ks < 16; ++ks) {
                    const uint64_t b_hi = w2desc + (uint64_t)(((ks >> 2) * 2 * N2p * 128) >> 4) + 2ull * (ks & 3);
                    const uint64_t b_lo = b_hi + (uint64_t)((N2p * 128) >> 4);
                    umma_tf32_ts(dy, al + 8 * ks, b_hi, idesc2, ks != 0);
                    umma_tf32_ts(dy2, ah + 8 * ks, b_hi, idesc2, ks != 0);
                    umma_tf32_ts(dy, ah + 8 * ks, b_lo, idesc2, 1);
                }
                umma_commit(&sh->y_full);
                umma_commit(&sh->acc_empty[a]);  // the accumulator that held h is free when these MMAs are done
                return true;
            };
#pragma unroll 1
            for (int it = 0; it < ntile; ++it) {
                const int acc = it & 1;
                if (!(ok = umma_wait(&sh->acc_empty[acc], ((it >> 1) & 1) ^ 1, &sh->abort))) break;
                tc_fence_after();
                const unsigned d = tmem + acc * acc_stride;
#pragma unroll 1
                for (int c = 0; c < nchunks; ++c) {
                    if (!(ok = umma_wait(&sh->full[s], ph, &sh->abort))) break;
                    tc_fence_after();
                    const uint64_t a_hi = desc0 + stage16 * s, a_lo = a_hi + alo16, b_hi = a_hi + bhi16, b_lo = a_hi + blo16;
                    const int ksteps = c == nchunks - 1 ? last_ksteps : kUmmaChunk / 8;
#pragma unroll
                    for (int ks = 0; ks < kUmmaChunk / 8; ++ks) {
                        if (ks >= ksteps) break;
                        const uint64_t o = 2ull * ks;  // 8 floats = 32 bytes further along K, in 16-byte units
                        umma_tf32(d, a_lo + o, b_hi + o, idesc, (c | ks) != 0);
                        umma_tf32(d, a_hi + o, b_lo + o, idesc, 1);
                        umma_tf32(d, a_hi + o, b_hi + o, idesc, 1);
                    }
                    umma_commit(&sh->empty[s]);
                    if (c == nchunks - 1) umma_commit(&sh->acc_full[acc]);
                    if (++s == stages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
                if (fuse && it >= 1 && !(ok = second_layer(it - 1))) break;
            }
            if (ok && fuse && ntile > 0) ok = second_layer(ntile - 1);
            if (!ok) atomicOr(status, UMMA_STATUS_MMA);
        }
        __syncwarp();
    } else if (warp == kUmmaWarpWeights) {
        if (lane == 0) {
            const unsigned bytes = 2u * Np * 128u;
            const size_t chunk_floats = (size_t)2 * Np * kUmmaChunk;
            int s = 0, c = 0;
            unsigned ph = 1;  // the first pass over the stages finds them free
            if (fuse) {
                mbar_arrive_expect(&sh->w2_full, (unsigned)w2_bytes);
                bulk_copy_g2s(w2s, args.W2img, (unsigned)w2_bytes, &sh->w2_full);
            }
#pragma unroll 1
            for (int q = 0; q < total; ++q) {
                if (!(ok = umma_wait(&sh->empty[s], ph, &sh->abort))) break;
                mbar_arrive_expect(&sh->full[s], bytes);
                bulk_copy_g2s(base + (size_t)s * stage_bytes + 2 * kUmmaTileABytes, Wimg + chunk_floats * c, bytes, &sh->full[s]);
                if (++s == stages) {
                    s = 0;
                    ph ^= 1;
                }
                if (++c == nchunks) c = 0;
            }
            if (!ok) {
                atomicOr(status, UMMA_STATUS_WEIGHTS);
                __nanosleep(20000);  // a copy issued just before the flag was seen lands before the CTA leaves
            }
        }
    } else if (warp >= kUmmaWarpProducer0) {
        const int pw = warp - kUmmaWarpProducer0;  // rows 8 pw .. 8 pw + 7 of every tile
        // the load stream runs two chunks ahead of the store stream; both advance by additions only
        long long l_row0 = (long long)blockIdx.x * kUmmaRows + pw * 8;
        int l_c = 0;
        auto load = [&](float (&v)[8]) {
            const int k = l_c * kUmmaChunk + lane;
            const float *p = A + l_row0 * K + k;
            if (l_row0 + 8 <= M && l_c * kUmmaChunk + kUmmaChunk <= K) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __ldg(p + (long long)j * K);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = (l_row0 + j < M && k < K) ? __ldg(p + (long long)j * K) : 0.f;
            }
            if (++l_c == nchunks) {
                l_c = 0;
                l_row0 += (long long)gridDim.x * kUmmaRows;
            }
        };
        int s = 0;
        unsigned ph = 1;
        auto store = [&](const float (&v)[8]) -> bool {
            if (!umma_wait(&sh->empty[s], ph, &sh->abort)) return false;
            float *hi = (float *)(base + (size_t)s * stage_bytes), *lo = hi + kUmmaRows * kUmmaChunk;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int at = umma_swizzled(pw * 8 + j, lane);
                const float head = __uint_as_float(tf32_head_bits(v[j]));
                hi[at] = head;
                lo[at] = v[j] - head;
            }
            fence_proxy_async();  // the MMA reads these through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->full[s]);
            if (++s == stages) {
                s = 0;
                ph ^= 1;
            }
            return true;
        };
        // Three chunks in flight in three register sets that take turns (no register is copied: a copy
        // would wait for the load it reads and end the overlap).
        float v0[8], v1[8], v2[8];
        if (0 < total) load(v0);
        if (1 < total) load(v1);
#pragma unroll 1
        for (int q = 0; q < total; q += 3) {
            if (q + 2 < total) load(v2);
            if (!(ok = store(v0))) break;
            if (q + 1 >= total) break;
            if (q + 3 < total) load(v0);
            if (!(ok = store(v1))) break;
            if (q + 2 >= total) break;
            if (q + 4 < total) load(v1);
            if (!(ok = store(v2))) break;
        }
        if (!ok && lane == 0) atomicOr(status, UMMA_STATUS_PRODUCER);
    } else {
        // epilogue: warp w reads lanes 32 (w % 4) .. + 31 of the accumulator (= rows of the tile) and every
        // second block of 16 columns; a block goes through shared memory so that rows leave coalesced.
        // Two-layer mode: pass 0 activates the first layer's tile and writes it back in place together with its
        // TF32 tail (the A operand of the second layer; nothing else, so that the second layer can start early),
        // pass 1 stores the activated tile, pass 2 stores the second layer's tile.
        float *stg = epi + warp * 32 * kUmmaEpiPitch;
        const int quarter = warp & 3, first_block = warp >> 2;
        const float neg_inf = -__int_as_float(0x7f800000);
        const unsigned tlane = tmem + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
        for (int it = 0; it < ntile && ok; ++it) {
            const int acc = it & 1;
            const long long row0 = ((long long)blockIdx.x + (long long)it * gridDim.x) * kUmmaRows + quarter * 32;
            const int nrows = M - row0 < 32 ? (int)(M - row0) : 32;  // may be <= 0 in the last tile
#pragma unroll 1
            for (int pass = fuse ? 0 : 1; pass < (fuse ? 3 : 2); ++pass) {
                // what this pass reads and where it goes
                const bool act_here = fuse && pass == 0;           // bias and activation in registers, written back
                const bool post = !fuse;                            // bias and activation while storing
                float *const out = pass == 2 ? args.Y : C;
                const int ncol = pass == 2 ? N2 : N;
                const int nblocks = (pass == 2 ? N2p : Np) >> 4;
                const unsigned taddr0 = tlane + (pass == 2 ? kUmmaYCol : acc * acc_stride);
                const float lo = (post && relu) ? 0.f : neg_inf;
                const float *gt0 = (post && gate) ? gate : nullptr;
                const bool vec4 = (ncol & 3) == 0 && ((uintptr_t)out & 15) == 0 && (!gt0 || ((uintptr_t)gt0 & 15) == 0);
                if (pass != 1 || !fuse) {  // pass 1 of the two-layer mode reads what pass 0 of the same thread wrote
                    if (!(ok = umma_wait(pass == 2 ? &sh->y_full : &sh->acc_full[acc], pass == 2 ? it & 1 : (it >> 1) & 1, &sh->abort))) break;
                    tc_fence_after();
                }
                // the previous tile's rows have left the shared-memory tile
                if (fuse && pass == 2 && !(ok = umma_wait(&sh->y_copied, (it & 1) ^ 1, &sh->abort))) break;
                int last_block = first_block;
                while (last_block + 2 < nblocks) last_block += 2;
#pragma unroll 1
                for (int b = first_block; b < nblocks; b += 2) {
                    const int c0 = b << 4;
                    unsigned r[16];
                    tmem_ld16(taddr0 + c0, r);
                    tc_wait_ld();
                    if (pass == 1 && b == last_block) {  // this warp has read its last block: hand its share of the accumulator back
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
                    }
                    if (fuse && pass == 2) {
                        // the second layer's tile: the sum of its two accumulators goes into a shared-memory tile laid out
                        // like the tile's rows in global memory (they are contiguous there), copied out linearly below
                        unsigned r2[16];
                        tmem_ld16(tlane + kUmmaY2Col + c0, r2);
                        tc_wait_ld();
                        float *yrow = ytile + (quarter * 32 + lane) * ncol + c0;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < ncol) yrow[j] = __uint_as_float(r[j]) + __uint_as_float(r2[j]);
                        continue;
                    }
                    if (act_here) {
                        unsigned tail[16];
                        float bj[16];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 b4 = *(const float4 *)(sh->bias + c0 + 4 * j);
                            bj[4 * j] = b4.x; bj[4 * j + 1] = b4.y; bj[4 * j + 2] = b4.z; bj[4 * j + 3] = b4.w;
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            float v = __uint_as_float(r[j]) + bj[j];
                            if (relu) v = fmaxf(v, 0.f);
                            r[j] = __float_as_uint(v);
                            tail[j] = __float_as_uint(v - __uint_as_float(tf32_head_bits(v)));
                        }
                        tmem_st16(taddr0 + c0, r);                 // the MMA reads the head of these by truncation
                        tmem_st16(tlane + kUmmaHloCol + c0, tail);
                        continue;
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        *(float4 *)(stg + lane * kUmmaEpiPitch + 4 * j) = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                                     __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    __syncwarp();
                    if (vec4) {
                        // eight rows x four float4 per instruction; the two rows of a quarter-warp are four staged
                        // rows apart (4 x 20 floats = 16 banks), so that its eight float4 cover all 32 banks
                        const int c4 = 4 * (lane & 3), t = lane >> 2, sub = (t >> 1) + 4 * (t & 1);
                        if (c0 + c4 < ncol) {
                            const float4 bv = post ? *(const float4 *)(sh->bias + c0 + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int rr = 8 * i + sub;
                                if (rr < nrows) {
                                    float4 v = *(const float4 *)(stg + rr * kUmmaEpiPitch + c4);
                                    v.x = fmaxf(v.x + bv.x, lo); v.y = fmaxf(v.y + bv.y, lo);
                                    v.z = fmaxf(v.z + bv.z, lo); v.w = fmaxf(v.w + bv.w, lo);
                                    const long long at = (row0 + rr) * ncol + c0 + c4;
                                    if (gt0) {
                                        const float4 gv = __ldg((const float4 *)(gt0 + at));
                                        if (!(gv.x > 0.f)) v.x = 0.f;
                                        if (!(gv.y > 0.f)) v.y = 0.f;
                                        if (!(gv.z > 0.f)) v.z = 0.f;
                                        if (!(gv.w > 0.f)) v.w = 0.f;
                                    }
                                    *(float4 *)(out + at) = v;
                                }
                            }
                        }
                    } else {
                        const int cc = lane & 15, sub = lane >> 4;  // two rows x sixteen columns per instruction
                        if (c0 + cc < ncol) {
                            const float bv = post ? sh->bias[c0 + cc] : 0.f;
                            float *dst = out + (row0 + sub) * ncol + c0 + cc;
                            const float *gt = gt0 ? gt0 + (row0 + sub) * ncol + c0 + cc : nullptr;
                            const float *src = stg + sub * kUmmaEpiPitch + cc;
#pragma unroll 4
                            for (int rr = sub; rr < nrows; rr += 2) {
                                float v = fmaxf(*src + bv, lo);
                                if (gt) {
                                    if (!(__ldg(gt) > 0.f)) v = 0.f;
                                    gt += 2 * ncol;
                                }
                                *dst = v;
                                dst += 2 * ncol;
                                src += 2 * kUmmaEpiPitch;
                            }
                        }
                    }
                    __syncwarp();
                }
                if (fuse && pass == 2) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->y_written);
                    if (!(ok = umma_wait(&sh->y_written, it & 1, &sh->abort))) break;
                    // all eight warps copy the tile: (rows that exist) x N2 floats, contiguous and 16-byte aligned in global memory
                    const long long tile_row0 = ((long long)blockIdx.x + (long long)it * gridDim.x) * kUmmaRows;
                    const int rows_here = M - tile_row0 < kUmmaRows ? (int)(M - tile_row0) : kUmmaRows;
                    const int total = rows_here * ncol, e = warp * 32 + lane;
                    float *dst = out + tile_row0 * ncol;
                    if (((uintptr_t)out & 15) == 0) {
                        for (int q = e; q < total / 4; q += kUmmaEpilogueWarps * 32) ((float4 *)dst)[q] = ((const float4 *)ytile)[q];
                        for (int q = (total & ~3) + e; q < total; q += kUmmaEpilogueWarps * 32) dst[q] = ytile[q];
                    } else {
                        for (int q = e; q < total; q += kUmmaEpilogueWarps * 32) dst[q] = ytile[q];
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->y_copied);
                }
                if (act_here) {  // h and its tail are in tensor memory: the second layer (and pass 1) may read them
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->h_ready[acc]);
                }
            }
        }
        if (!ok && lane == 0) atomicOr(status, UMMA_STATUS_EPILOGUE);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kUmmaWarpMma) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kUmmaTmemCols) : "memory");
    }
}

// Self-test of the bounded waits: warp 0 waits, with a short limit, on an mbarrier that nothing completes
// and raises the flag; warp 1 waits with the full limit on another one and must leave through the flag.
// result[0] = 1 when warp 0 gave up, result[1] = 1 when warp 1 left because of the flag.
__global__ void umma_wait_selftest_kernel(unsigned long long limit_ns, int *result) {
    __shared__ uint64_t bar[2];
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar[0], 1);
        mbar_init(&bar[1], 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    const unsigned long long t0 = global_timer_ns();
    const bool completed = warp == 0 ? umma_wait(&bar[0], 0u, &abort_flag, limit_ns) : umma_wait(&bar[1], 0u, &abort_flag);
    const bool by_flag = global_timer_ns() - t0 < kUmmaWaitNs / 2;
    if ((threadIdx.x & 31) == 0) result[warp] = completed ? 0 : (warp == 0 || by_flag ? 1 : 2);
}

// Per-device set-up done once: the address of the status word and the shared-memory limit of the kernel.
struct UmmaDevice {
    unsigned *status = nullptr;
    int smem_limit[2] = {0, 0};  // per kernel instantiation
};
static std::mutex g_umma_mutex;
static UmmaDevice g_umma_device[64];

static int umma_device_setup(int smem, bool fuse, unsigned **status) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(NPA_ERR_CUDA, "npa_linear_tcgen05: cudaGetDevice: %s", cudaGetErrorString(e));
    std::lock_guard<std::mutex> lock(g_umma_mutex);
    UmmaDevice &d = g_umma_device[dev];
    if (!d.status) {
        e = cudaGetSymbolAddress((void **)&d.status, g_umma_status);
        if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "npa_linear_tcgen05: status word: %s", cudaGetErrorString(e));
    }
    if (smem > d.smem_limit[fuse]) {
        e = fuse ? cudaFuncSetAttribute(linear_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
                 : cudaFuncSetAttribute(linear_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "npa_linear_tcgen05: raising the shared-memory limit: %s", cudaGetErrorString(e));
        d.smem_limit[fuse] = smem;
    }
    *status = d.status;
    return NPA_OK;
}

// Device address of the status word on the current device (also used by mlp_grad_tcgen05.cu).
unsigned *umma_status_word() {
    unsigned *p = nullptr;
    return cudaGetSymbolAddress((void **)&p, g_umma_status) == cudaSuccess ? p : nullptr;
}

static int umma_round16(int v) { return (v + 15) / 16 * 16; }
static int umma_chunks(int k) { return (k + kUmmaChunk - 1) / kUmmaChunk; }

}  // namespace npa

using namespace npa;

extern "C" {

int64_t npa_linear_tcgen05_scratch_bytes(int32_t in_dim, int32_t out_dim) {
    if (in_dim <= 0 || out_dim <= 0) return 0;
    return (int64_t)umma_chunks(in_dim) * 2 * umma_round16(out_dim) * kUmmaChunk * (int64_t)sizeof(float);
}

int npa_linear_tcgen05(const float *A, const float *W, const float *bias, const float *gate, float *C, int64_t rows,
                       int32_t in_dim, int32_t out_dim, int64_t w_stride_out, int64_t w_stride_in, int32_t relu, void *scratch,
                       int64_t scratch_bytes, void *stream) {
    if (rows <= 0 || in_dim <= 0 || out_dim <= 0)
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tcgen05: rows, in_dim and out_dim must be positive");
    if (out_dim > 256 || in_dim > 1024)
        return fail(NPA_ERR_UNSUPPORTED, "npa_linear_tcgen05: supports in_dim <= 1024 and out_dim <= 256, got %d and %d", in_dim, out_dim);
    if (!A || !W || !C || !scratch) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tcgen05: A, W, C and scratch must be non-NULL");
    if ((uintptr_t)A % 4 || (uintptr_t)C % 4 || (uintptr_t)scratch % 16)
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tcgen05: A and C must be float aligned, scratch 16-byte aligned");
    if (scratch_bytes < npa_linear_tcgen05_scratch_bytes(in_dim, out_dim))
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tcgen05: scratch holds %lld bytes, %lld needed", (long long)scratch_bytes,
                    (long long)npa_linear_tcgen05_scratch_bytes(in_dim, out_dim));
    UmmaArgs a = {};
    a.A = A; a.Wimg = (const float *)scratch; a.bias = bias; a.gate = gate; a.C = C; a.M = rows; a.K = in_dim; a.N = out_dim;
    a.Np = umma_round16(out_dim);
    a.nchunks = umma_chunks(in_dim);
    a.last_ksteps = (in_dim - (a.nchunks - 1) * kUmmaChunk + 7) / 8;
    a.stage_bytes = 2 * kUmmaTileABytes + 2 * a.Np * 128;
    a.relu = relu;
    const int fixed = 1024 + kUmmaEpiFloats * 4 + (int)sizeof(UmmaShared);
    a.stages = (227 * 1024 - fixed) / a.stage_bytes;
    if (a.stages > kUmmaMaxStages) a.stages = kUmmaMaxStages;
    if (a.stages < 2) return fail(NPA_ERR_UNSUPPORTED, "npa_linear_tcgen05: out_dim %d leaves room for fewer than two stages", out_dim);
    const size_t smem = (size_t)fixed + (size_t)a.stages * a.stage_bytes;
    int rc = umma_device_setup((int)smem, false, &a.status);
    if (rc != NPA_OK) return rc;
    const int total = a.nchunks * a.Np * kUmmaChunk;
    weight_image_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(W, w_stride_out, w_stride_in, in_dim, out_dim, a.Np,
                                                                                 a.nchunks, (float *)scratch);
    rc = check_launch("weight_image_kernel");
    if (rc != NPA_OK) return rc;
    const long long tiles = (rows + kUmmaRows - 1) / kUmmaRows;
    const int ctas = (int)(tiles < 148 ? tiles : 148);
    linear_umma_kernel<false><<<ctas, kUmmaThreads, smem, (cudaStream_t)stream>>>(a);
    return check_launch("linear_umma_kernel");
}

int64_t npa_mlp_forward_tcgen05_scratch_bytes(int32_t in_dim, int32_t out_dim) {
    if (in_dim <= 0 || out_dim <= 0) return 0;
    return npa_linear_tcgen05_scratch_bytes(in_dim, kUmmaRows) + (int64_t)4 * 2 * umma_round16(out_dim) * kUmmaChunk * (int64_t)sizeof(float);
}

int npa_mlp_forward_tcgen05(const float *z, const float *W1, const float *b1, const float *W2, float *h, float *y, int64_t rows,
                            int32_t in_dim, int32_t out_dim, int64_t w1_stride_out, int64_t w1_stride_in, int64_t w2_stride_out,
                            int64_t w2_stride_in, void *scratch, int64_t scratch_bytes, void *stream) {
    const char *me = "npa_mlp_forward_tcgen05";
    if (rows <= 0 || in_dim <= 0 || out_dim <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: rows, in_dim and out_dim must be positive", me);
    if (in_dim > 1024 || out_dim > 64)
        return fail(NPA_ERR_UNSUPPORTED, "%s: supports in_dim <= 1024 and out_dim <= 64 (hidden width 128), got %d and %d", me, in_dim, out_dim);
    if (!z || !W1 || !W2 || !h || !y || !scratch) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: z, W1, W2, h, y and scratch must be non-NULL", me);
    if ((uintptr_t)z % 4 || (uintptr_t)h % 4 || (uintptr_t)y % 4 || (uintptr_t)scratch % 16)
        return fail(NPA_ERR_INVALID_ARGUMENT, "%s: z, h and y must be float aligned, scratch 16-byte aligned", me);
    if (scratch_bytes < npa_mlp_forward_tcgen05_scratch_bytes(in_dim, out_dim))
        return fail(NPA_ERR_INVALID_ARGUMENT, "%s: scratch holds %lld bytes, %lld needed", me, (long long)scratch_bytes,
                    (long long)npa_mlp_forward_tcgen05_scratch_bytes(in_dim, out_dim));
    UmmaArgs a = {};
    a.A = z; a.Wimg = (const float *)scratch; a.bias = b1; a.gate = nullptr; a.C = h; a.M = rows; a.K = in_dim; a.N = kUmmaRows;
    a.Np = kUmmaRows;  // hidden width 128
    a.nchunks = umma_chunks(in_dim);
    a.last_ksteps = (in_dim - (a.nchunks - 1) * kUmmaChunk + 7) / 8;
    a.stage_bytes = 2 * kUmmaTileABytes + 2 * a.Np * 128;
    a.relu = 1;
    a.Y = y; a.N2 = out_dim; a.N2p = umma_round16(out_dim);
    a.W2img = (const float *)((const char *)scratch + npa_linear_tcgen05_scratch_bytes(in_dim, kUmmaRows));
    const int w2_bytes = 4 * 2 * a.N2p * 128;
    const int fixed = 1024 + kUmmaEpiFloats * 4 + (int)sizeof(UmmaShared) + w2_bytes + ((kUmmaRows * out_dim + 3) & ~3) * 4;
    a.stages = (227 * 1024 - fixed) / a.stage_bytes;
    if (a.stages > kUmmaMaxStages) a.stages = kUmmaMaxStages;
    if (a.stages < 2) return fail(NPA_ERR_UNSUPPORTED, "%s: no room for two stages", me);
    const size_t smem = (size_t)fixed + (size_t)a.stages * a.stage_bytes;
    int rc = umma_device_setup((int)smem, true, &a.status);
    if (rc != NPA_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int total1 = a.nchunks * a.Np * kUmmaChunk, total2 = 4 * a.N2p * kUmmaChunk;
    weight_image_kernel<<<(total1 + 255) / 256, 256, 0, st>>>(W1, w1_stride_out, w1_stride_in, in_dim, kUmmaRows, a.Np, a.nchunks, (float *)scratch);
    if ((rc = check_launch("weight_image_kernel")) != NPA_OK) return rc;
    weight_image_kernel<<<(total2 + 255) / 256, 256, 0, st>>>(W2, w2_stride_out, w2_stride_in, kUmmaRows, out_dim, a.N2p, 4, (float *)a.W2img);
    if ((rc = check_launch("weight_image_kernel")) != NPA_OK) return rc;
    const long long tiles = (rows + kUmmaRows - 1) / kUmmaRows;
    const int ctas = (int)(tiles < 148 ? tiles : 148);
    linear_umma_kernel<true><<<ctas, kUmmaThreads, smem, st>>>(a);
    return check_launch("linear_umma_kernel (two layers)");
}

int npa_linear_tcgen05_wait_selftest(int32_t limit_us, int32_t *device_result, void *stream) {
    if (!device_result) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tcgen05_wait_selftest: device_result is NULL");
    if (limit_us <= 0 || limit_us > 1000000)
        return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tcgen05_wait_selftest: limit_us must be in (0, 1000000]");
    umma_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>((unsigned long long)limit_us * 1000ull, device_result);
    return check_launch("umma_wait_selftest_kernel");
}

/* Status word of the bounded waits of linear_umma_kernel on the current device (synchronises). */
int npa_linear_tcgen05_status(uint32_t *host_status, int32_t reset) {
    if (!host_status) return fail(NPA_ERR_INVALID_ARGUMENT, "npa_linear_tcgen05_status: host_status must be non-NULL");
    cudaError_t e = cudaMemcpyFromSymbol(host_status, g_umma_status, sizeof(unsigned));
    if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "npa_linear_tcgen05_status: %s", cudaGetErrorString(e));
    if (reset) {
        const unsigned zero = 0;
        e = cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(unsigned));
        if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "npa_linear_tcgen05_status: %s", cudaGetErrorString(e));
    }
    return NPA_OK;
}

}  // extern "C"
