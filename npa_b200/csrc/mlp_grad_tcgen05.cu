// Weight gradients of the per-particle MLP on the fifth-generation tensor cores.
//
//     dW1 [128, in] = dh^T z,   db1 [128] = sum over rows of dh,   dW2 [out, 128] = dy^T h
//
// (models/npa.py:63-75; the contract of npa_mlp_weight_grad, mlp_grad.cu) as two products whose
// reduction index is the row (particle) index:
//
//     D1 [128, in + 1] = dh^T [z | 1]        D2 [128, out] = h^T dy       (dW2 = D2^T)
//
// with tcgen05.mma kind::tf32, M = 128, K = 8 rows per instruction, both operands MN-major (a row of
// the row-major inputs is contiguous along M / N; 128-byte swizzle on 32-byte units), every product as three TF32 MMAs on operands split
// into head and tail, fp32 accumulators in tensor memory.  The tensor cores truncate when they add
// into the accumulator, and a chain of hundreds of accumulations drifts; so a chain is at most one
// segment of 128 rows (48 accumulations): after each segment the epilogue warps add the accumulators,
// rounding to nearest, into running sums kept in a second region of tensor memory, and the MMAs
// start the next segment from zero.  At the end each CTA writes its sums to global memory and a
// second kernel adds the CTAs' partial sums in a fixed order: results are deterministic.
//
// One persistent CTA per SM with a contiguous slab of rows; stages of 16 rows:
//   * one lane brings the 16 rows of dh, h, z and dy of a stage into a ring of raw stages with four bulk
//     copies (each input's 16 rows are one contiguous, 16-byte aligned block of global memory);
//   * 16 producer warps, one row of the stage each, read the raw row, split it and store head and tail
//     into the stage's swizzled operand tiles (a last, partial stage is read from global memory);
//   * one lane issues the 12 MMAs of a stage and commits the stage back to the producers;
//   * eight epilogue warps drain a finished accumulator set (tcgen05.ld, lane = hidden unit).
// Every wait on an mbarrier is bounded in time; a wait that gives up raises a flag that ends all roles,
// the CTA frees its tensor memory, and the host reads the reason from the status word of
// npa_linear_tcgen05_status (bits 16, 32, 64: MMA lane, producers, epilogue of this kernel).
#include <mutex>

#include "umma.cuh"

namespace npa {

constexpr int kGradHidden = 128;
constexpr int kGradStageRows = 16;                 // two k-groups of eight rows
constexpr int kGradSegmentStages = 8;              // 128 rows per accumulation chain
constexpr int kGradProducerWarps = 16;
constexpr int kGradEpilogueWarps = 8;
constexpr int kGradWarpMma = 8, kGradWarpCopy = 9, kGradWarpProducer0 = 10;
constexpr int kGradThreads = (kGradWarpProducer0 + kGradProducerWarps) * 32;
constexpr int kGradAtomBytes = 512;                // 4 rows x 128 bytes (32 columns)
constexpr int kGradAtomsH = 4, kGradAtomsZ = 6, kGradAtomsY = 2;  // atoms of 32 columns: dh / h, [z | 1], dy
// byte offsets inside a stage: [k-group of 8 rows][4-row half][atom] per operand part
constexpr int kGradOffDhHi = 0, kGradOffDhLo = 8192, kGradOffHHi = 16384, kGradOffHLo = 24576;
constexpr int kGradOffZHi = 32768, kGradOffZLo = 45056, kGradOffYHi = 57344, kGradOffYLo = 61440;
constexpr int kGradStageBytes = 65536;
constexpr int kGradStages = 2;                     // operand stages
constexpr int kGradRawStages = 3;                  // raw input rows, as the bulk copies deliver them
// a raw stage: 16 rows of dh | h | z | dy, each block contiguous as in global memory
constexpr int kGradRawDh = 0, kGradRawH = 8192, kGradRawZ = 16384, kGradRawY = 16384 + 11264, kGradRawBytes = 16384 + 11264 + 3072;
constexpr int kGradTmemCols = 512, kGradSumCol = 256, kGradD2Col = 192;  // accumulators at 0 / 192, running sums 256 columns up
constexpr int kGradMaxIn = 175, kGradMaxOut = 48;  // in + 1 <= 192 columns of D1 (six atoms), out <= 64 of D2

enum { GRAD_STATUS_MMA = 16, GRAD_STATUS_PRODUCER = 32, GRAD_STATUS_EPILOGUE = 64 };

struct GradShared {
    uint64_t full[kGradStages], empty[kGradStages], acc_full, acc_empty;
    uint64_t raw_full[kGradRawStages], raw_empty[kGradRawStages];
    uint32_t tmem_base;
    int abort;
};

struct GradArgs {
    const float *z, *dh, *h, *dy;
    float *partial;          // [ctas][128][N1p + N2p]
    float *dW1, *dW2, *db1;
    long long M;
    int in_dim, out_dim, N1p, N2p, stages_per_cta, ctas;
    unsigned *status;
};

unsigned *umma_status_word();  // mlp_tcgen05.cu: device address of the status word on the current device

__global__ void __launch_bounds__(kGradThreads, 1) mlp_grad_umma_kernel(const __grid_constant__ GradArgs args) {
    const float *__restrict__ Z = args.z;
    const float *__restrict__ DH = args.dh;
    const float *__restrict__ H = args.h;
    const float *__restrict__ DY = args.dy;
    const long long M = args.M;
    const int K1 = args.in_dim, O = args.out_dim, N1p = args.N1p, N2p = args.N2p;
    unsigned *status = args.status;
    extern __shared__ uint8_t grad_smem_raw[];
    uint8_t *base = grad_smem_raw + ((1024u - (smem_u32(grad_smem_raw) & 1023u)) & 1023u);
    uint8_t *raw = base + kGradStages * kGradStageBytes;
    GradShared *sh = (GradShared *)(raw + kGradRawStages * kGradRawBytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGradStages; ++s) {
            mbar_init(&sh->full[s], kGradProducerWarps);
            mbar_init(&sh->empty[s], 1);
        }
        for (int s = 0; s < kGradRawStages; ++s) {
            mbar_init(&sh->raw_full[s], 1);                    // the copy lane's arrival + the bytes of four copies
            mbar_init(&sh->raw_empty[s], kGradProducerWarps);  // every producer warp has read its row
        }
        mbar_init(&sh->acc_full, 1);
        mbar_init(&sh->acc_empty, kGradEpilogueWarps);
        sh->abort = 0;
        mbar_fence_init();
    }
    if (warp == kGradWarpMma) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)),
                     "r"(kGradTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = sh->tmem_base;

    // this CTA's slab: stages first_stage .. first_stage + nstage - 1 of 16 rows
    const long long stages_total = (M + kGradStageRows - 1) / kGradStageRows;
    const long long first_stage = (long long)blockIdx.x * args.stages_per_cta;
    const int nstage = (int)(stages_total - first_stage < args.stages_per_cta ? stages_total - first_stage : args.stages_per_cta);
    const int nseg = (nstage + kGradSegmentStages - 1) / kGradSegmentStages;
    // stages whose 16 rows all exist come in by bulk copy; a last, partial stage is read row by row
    const long long rows_left = M - first_stage * kGradStageRows;
    const int nraw = (int)(rows_left / kGradStageRows < nstage ? rows_left / kGradStageRows : nstage);
    bool ok = true;

    if (warp == kGradWarpMma) {
        if (lane == 0) {
            // M = 128, TF32 x TF32 -> F32, both operands MN-major
            const unsigned idesc0 = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (1u << 16) | ((unsigned)(kGradHidden >> 4) << 24);
            const unsigned idesc1 = idesc0 | ((unsigned)(N1p >> 3) << 17), idesc2 = idesc0 | ((unsigned)(N2p >> 3) << 17);
            const unsigned sbase = smem_u32(base);
            int s = 0, done = 0;
            unsigned ph = 0;
#pragma unroll 1
            for (int seg = 0; seg < nseg; ++seg) {
                if (!(ok = umma_wait(&sh->acc_empty, (seg & 1) ^ 1, &sh->abort))) break;  // the epilogue has read segment seg - 1
                tc_fence_after();
                const unsigned d1 = tmem, d2 = tmem + kGradD2Col;
                const int nst = nstage - done < kGradSegmentStages ? nstage - done : kGradSegmentStages;
#pragma unroll 1
                for (int st = 0; st < nst; ++st) {
                    if (!(ok = umma_wait(&sh->full[s], ph, &sh->abort))) break;
                    tc_fence_after();
                    const unsigned sa = sbase + s * kGradStageBytes;
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        const unsigned oh = kk * 2 * kGradAtomsH * kGradAtomBytes, oz = kk * 2 * kGradAtomsZ * kGradAtomBytes;
                        const unsigned oy = kk * 2 * kGradAtomsY * kGradAtomBytes;
                        const uint64_t a1h = umma_desc_mn32(sa + kGradOffDhHi + oh, kGradAtomBytes, kGradAtomsH * kGradAtomBytes);
                        const uint64_t a1l = umma_desc_mn32(sa + kGradOffDhLo + oh, kGradAtomBytes, kGradAtomsH * kGradAtomBytes);
                        const uint64_t b1h = umma_desc_mn32(sa + kGradOffZHi + oz, kGradAtomBytes, kGradAtomsZ * kGradAtomBytes);
                        const uint64_t b1l = umma_desc_mn32(sa + kGradOffZLo + oz, kGradAtomBytes, kGradAtomsZ * kGradAtomBytes);
                        const uint64_t a2h = umma_desc_mn32(sa + kGradOffHHi + oh, kGradAtomBytes, kGradAtomsH * kGradAtomBytes);
                        const uint64_t a2l = umma_desc_mn32(sa + kGradOffHLo + oh, kGradAtomBytes, kGradAtomsH * kGradAtomBytes);
                        const uint64_t b2h = umma_desc_mn32(sa + kGradOffYHi + oy, kGradAtomBytes, kGradAtomsY * kGradAtomBytes);
                        const uint64_t b2l = umma_desc_mn32(sa + kGradOffYLo + oy, kGradAtomBytes, kGradAtomsY * kGradAtomBytes);
                        const int acc = (st | kk) != 0;
                        umma_tf32(d1, a1l, b1h, idesc1, acc);
                        umma_tf32(d1, a1h, b1l, idesc1, 1);
                        umma_tf32(d1, a1h, b1h, idesc1, 1);
                        umma_tf32(d2, a2l, b2h, idesc2, acc);
                        umma_tf32(d2, a2h, b2l, idesc2, 1);
                        umma_tf32(d2, a2h, b2h, idesc2, 1);
                    }
                    umma_commit(&sh->empty[s]);
                    if (++s == kGradStages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
                umma_commit(&sh->acc_full);
                done += nst;
            }
            if (!ok) atomicOr(status, GRAD_STATUS_MMA);
        }
        __syncwarp();
    } else if (warp == kGradWarpCopy) {
        if (lane == 0) {
            // four bulk copies per stage: the 16 rows of each input are one contiguous, 16-byte aligned block
            const unsigned bz = kGradStageRows * K1 * 4, by = kGradStageRows * O * 4;
            int rs = 0;
            unsigned rphase = 1;  // the first pass finds the raw stages free
#pragma unroll 1
            for (int q = 0; q < nraw; ++q) {
                if (!(ok = umma_wait(&sh->raw_empty[rs], rphase, &sh->abort))) break;
                const long long row = (first_stage + q) * kGradStageRows;
                uint8_t *dst = raw + rs * kGradRawBytes;
                mbar_arrive_expect(&sh->raw_full[rs], 2u * 8192u + bz + by);
                bulk_copy_g2s(dst + kGradRawDh, DH + row * kGradHidden, 8192u, &sh->raw_full[rs]);
                bulk_copy_g2s(dst + kGradRawH, H + row * kGradHidden, 8192u, &sh->raw_full[rs]);
                bulk_copy_g2s(dst + kGradRawZ, Z + row * K1, bz, &sh->raw_full[rs]);
                bulk_copy_g2s(dst + kGradRawY, DY + row * O, by, &sh->raw_full[rs]);
                if (++rs == kGradRawStages) {
                    rs = 0;
                    rphase ^= 1;
                }
            }
            if (!ok) {
                atomicOr(status, GRAD_STATUS_PRODUCER);
                __nanosleep(20000);  // copies issued just before the flag was seen land before the CTA leaves
            }
        }
    } else if (warp >= kGradWarpProducer0) {
        const int pw = warp - kGradWarpProducer0;  // this warp owns row pw of every stage
        const int kk = pw >> 3;                    // its k-group of eight rows
        const int half4 = (pw >> 2) & 1;           // its group of four rows inside the k-group
        const int at = umma_mn32_offset(pw & 3, lane);  // float offset of (row, lane) inside an atom of 32 columns
        int s = 0, rs = 0;
        unsigned phase = 1, rphase = 0;  // operand stages start free; raw stages start empty of data
#pragma unroll 1
        for (int q = 0; q < nstage; ++q) {
            // v[0..3] dh, v[4..7] h, v[8..13] [z | 1 | 0...], v[14..15] dy: column 32 t + lane of this warp's row
            float v[16];
            if (q < nraw) {
                if (!(ok = umma_wait(&sh->raw_full[rs], rphase, &sh->abort))) break;
                const float *r = (const float *)(raw + rs * kGradRawBytes);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    v[t] = r[kGradRawDh / 4 + pw * kGradHidden + 32 * t + lane];
                    v[4 + t] = r[kGradRawH / 4 + pw * kGradHidden + 32 * t + lane];
                }
#pragma unroll
                for (int t = 0; t < 6; ++t) {
                    const int col = 32 * t + lane;
                    v[8 + t] = col < K1 ? r[kGradRawZ / 4 + pw * K1 + col] : (col == K1 ? 1.f : 0.f);  // the ones column gives db1
                }
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const int col = 32 * t + lane;
                    v[14 + t] = col < O ? r[kGradRawY / 4 + pw * O + col] : 0.f;
                }
            } else {
                const long long row = (first_stage + q) * kGradStageRows + pw;
                if (row < M) {
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        v[t] = __ldg(DH + row * kGradHidden + 32 * t + lane);
                        v[4 + t] = __ldg(H + row * kGradHidden + 32 * t + lane);
                    }
#pragma unroll
                    for (int t = 0; t < 6; ++t) {
                        const int col = 32 * t + lane;
                        v[8 + t] = col < K1 ? __ldg(Z + row * K1 + col) : (col == K1 ? 1.f : 0.f);
                    }
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        const int col = 32 * t + lane;
                        v[14 + t] = col < O ? __ldg(DY + row * O + col) : 0.f;
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < 16; ++t) v[t] = 0.f;  // rows behind the end add nothing, not even to db1
                }
            }
            if (!(ok = umma_wait(&sh->empty[s], phase, &sh->abort))) break;
            float *stage = (float *)(base + s * kGradStageBytes);
            auto put = [&](int off_hi, int off_lo, int natoms, int atom, float x) {
                const int f = ((kk * 2 + half4) * natoms + atom) * (kGradAtomBytes / 4) + at;
                const float head = __uint_as_float(tf32_head_bits(x));
                stage[off_hi / 4 + f] = head;
                stage[off_lo / 4 + f] = x - head;
            };
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                put(kGradOffDhHi, kGradOffDhLo, kGradAtomsH, t, v[t]);
                put(kGradOffHHi, kGradOffHLo, kGradAtomsH, t, v[4 + t]);
            }
#pragma unroll
            for (int t = 0; t < 6; ++t) put(kGradOffZHi, kGradOffZLo, kGradAtomsZ, t, v[8 + t]);
#pragma unroll
            for (int t = 0; t < 2; ++t) put(kGradOffYHi, kGradOffYLo, kGradAtomsY, t, v[14 + t]);
            fence_proxy_async();  // the MMA reads these through the async proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&sh->full[s]);
                if (q < nraw) mbar_arrive(&sh->raw_empty[rs]);  // the raw row has been consumed
            }
            if (q < nraw && ++rs == kGradRawStages) {
                rs = 0;
                rphase ^= 1;
            }
            if (++s == kGradStages) {
                s = 0;
                phase ^= 1;
            }
        }
        if (!ok && lane == 0) atomicOr(status, GRAD_STATUS_PRODUCER);
    } else {
        // epilogue: warp w owns lanes 32 (w % 4) .. + 31 of tensor memory (= hidden units) and every second
        // block of 16 columns.  After each segment it adds the accumulators, rounding to nearest, into running
        // sums that stay in tensor memory (the same thread reads and writes the same cells every time);
        // after the last segment the sums go to this CTA's partial sums in global memory.
        const int quarter = warp & 3, half = warp >> 2;
        const int nb1 = N1p >> 4, nb = nb1 + (N2p >> 4);
        float *prow = args.partial + ((long long)blockIdx.x * kGradHidden + quarter * 32 + lane) * (N1p + N2p);
        const unsigned taddr0 = tmem + ((unsigned)(quarter * 32) << 16);
        int last_block = half;
        while (last_block + 2 < nb) last_block += 2;
#pragma unroll 1
        for (int seg = 0; seg < nseg; ++seg) {
            if (!(ok = umma_wait(&sh->acc_full, seg & 1, &sh->abort, kUmmaWaitNs, 200))) break;
            tc_fence_after();
#pragma unroll 1
            for (int b = half; b < nb; b += 2) {
                const int col = b < nb1 ? b * 16 : kGradD2Col + (b - nb1) * 16;  // column in tensor memory
                unsigned r[16], sum[16];
                tmem_ld16(taddr0 + col, r);
                if (seg > 0) tmem_ld16(taddr0 + kGradSumCol + col, sum);
                tc_wait_ld();
                if (b == last_block) {  // this warp has read its share of the accumulators: hand them back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sh->acc_empty);
                }
                if (seg > 0) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(sum[j]));
                }
                if (seg + 1 < nseg) {
                    tmem_st16(taddr0 + kGradSumCol + col, r);
                } else {
                    float4 *p = (float4 *)(prow + b * 16);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        p[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                           __uint_as_float(r[4 * j + 3]));
                }
            }
            tc_wait_st();  // the sums are in place before this thread reads them again
        }
        if (!ok && lane == 0) atomicOr(status, GRAD_STATUS_EPILOGUE);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kGradWarpMma) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGradTmemCols) : "memory");
    }
}

// dW1, db1 and dW2 from the CTAs' partial sums, added in CTA order.
__global__ void mlp_grad_umma_reduce_kernel(GradArgs a) {
    const int K1 = a.in_dim, O = a.out_dim, Wp = a.N1p + a.N2p;
    const int n1 = kGradHidden * K1, total = n1 + kGradHidden + O * kGradHidden;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    int j, col;
    float *out;
    if (e < n1) {
        j = e / K1;
        col = e - j * K1;
        out = a.dW1 + e;
    } else if (e < n1 + kGradHidden) {
        j = e - n1;
        col = K1;  // the ones column
        out = a.db1 + j;
    } else {
        const int idx = e - n1 - kGradHidden, o = idx / kGradHidden;
        j = idx - o * kGradHidden;
        col = a.N1p + o;
        out = a.dW2 + idx;
    }
    const float *p = a.partial + (long long)j * Wp + col;
    const long long step = (long long)kGradHidden * Wp;
    float sum = 0.f;
    int c = 0;
    for (; c + 8 <= a.ctas; c += 8) {  // eight loads in flight, added in CTA order
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldg(p + (c + u) * step);
#pragma unroll
        for (int u = 0; u < 8; ++u) sum += v[u];
    }
    for (; c < a.ctas; ++c) sum += __ldg(p + c * step);
    *out = sum;
}

static int grad_round16(int v) { return (v + 15) / 16 * 16; }

struct GradDevice {
    unsigned *status = nullptr;
    bool smem_set = false;
};
static std::mutex g_grad_mutex;
static GradDevice g_grad_device[64];
constexpr int kGradSmemBytes = 1024 + kGradStages * kGradStageBytes + kGradRawStages * kGradRawBytes + (int)sizeof(GradShared);

}  // namespace npa

using namespace npa;

extern "C" {

int64_t npa_mlp_weight_grad_tcgen05_scratch_floats(int64_t rows, int32_t in_dim, int32_t out_dim) {
    if (rows <= 0 || in_dim <= 0 || out_dim <= 0) return 0;
    return (int64_t)148 * kGradHidden * (grad_round16(in_dim + 1) + grad_round16(out_dim));
}

int npa_mlp_weight_grad_tcgen05(const float *z, const float *dh, const float *h, const float *dy, int64_t rows, int32_t in_dim,
                                int32_t hidden, int32_t out_dim, float *scratch, int64_t scratch_floats, float *dW1,
                                float *dW2, float *db1, void *stream) {
    const char *me = "npa_mlp_weight_grad_tcgen05";
    if (hidden != kGradHidden) return fail(NPA_ERR_UNSUPPORTED, "%s: hidden width must be %d, got %d", me, kGradHidden, hidden);
    if (in_dim <= 0 || in_dim > kGradMaxIn || out_dim <= 0 || out_dim > kGradMaxOut)
        return fail(NPA_ERR_UNSUPPORTED, "%s: supports in <= %d and out <= %d, got %d and %d", me, kGradMaxIn, kGradMaxOut, in_dim, out_dim);
    if (rows <= 0) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: rows must be positive", me);
    if (!z || !dh || !h || !dy || !scratch || !dW1 || !dW2 || !db1) return fail(NPA_ERR_INVALID_ARGUMENT, "%s: every pointer must be non-NULL", me);
    if (((uintptr_t)z | (uintptr_t)dh | (uintptr_t)h | (uintptr_t)dy | (uintptr_t)scratch) % 16)
        return fail(NPA_ERR_INVALID_ARGUMENT, "%s: z, dh, h, dy and scratch must be 16-byte aligned", me);
    const int64_t need = npa_mlp_weight_grad_tcgen05_scratch_floats(rows, in_dim, out_dim);
    if (scratch_floats < need)
        return fail(NPA_ERR_SCRATCH_TOO_SMALL, "%s: scratch has %lld floats, %lld needed", me, (long long)scratch_floats, (long long)need);

    GradArgs a = {};
    a.z = z; a.dh = dh; a.h = h; a.dy = dy; a.partial = scratch; a.dW1 = dW1; a.dW2 = dW2; a.db1 = db1;
    a.M = rows; a.in_dim = in_dim; a.out_dim = out_dim;
    a.N1p = grad_round16(in_dim + 1);
    a.N2p = grad_round16(out_dim);
    const long long stages_total = (rows + kGradStageRows - 1) / kGradStageRows;
    int ctas = (int)(stages_total < 148 ? stages_total : 148);
    a.stages_per_cta = (int)((stages_total + ctas - 1) / ctas);
    a.ctas = (int)((stages_total + a.stages_per_cta - 1) / a.stages_per_cta);

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(NPA_ERR_CUDA, "%s: cudaGetDevice: %s", me, cudaGetErrorString(e));
    {
        std::lock_guard<std::mutex> lock(g_grad_mutex);
        GradDevice &d = g_grad_device[dev];
        if (!d.status && !(d.status = umma_status_word())) return fail(NPA_ERR_CUDA, "%s: no status word", me);
        if (!d.smem_set) {
            e = cudaFuncSetAttribute(mlp_grad_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGradSmemBytes);
            if (e != cudaSuccess) return fail(NPA_ERR_CUDA, "%s: raising the shared-memory limit: %s", me, cudaGetErrorString(e));
            d.smem_set = true;
        }
        a.status = d.status;
    }
    cudaStream_t st = (cudaStream_t)stream;
    mlp_grad_umma_kernel<<<a.ctas, kGradThreads, kGradSmemBytes, st>>>(a);
    int rc = check_launch("mlp_grad_umma_kernel");
    if (rc != NPA_OK) return rc;
    const int total = kGradHidden * in_dim + kGradHidden + out_dim * kGradHidden;
    mlp_grad_umma_reduce_kernel<<<(total + 63) / 64, 64, 0, st>>>(a);
    return check_launch("mlp_grad_umma_reduce_kernel");
}

}  // extern "C"
