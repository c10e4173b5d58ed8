// The projections either side of attention on the Blackwell tensor pipe (tcgen05 + TMEM) with fp32-grade results:
//   C[M][K] = A[M][N] B[N][K] (+ bias[K]),  the reference's argument order, N the inner dimension
// (HipGPT launch_matmul / launch_matmul_add_bias, src/hip_kernels.cpp:69-154; callers src/transformer_layer.cpp:217,220).
// The exact mode (one accumulator per output, inner index ascending, FMA: bit-identical to the reference's order) is
// hipgpt_matmul in layer_ops.cu; this is the fast mode: same operands, same output, 1e-5 instead of identical bits.
//
// Arithmetic (the scheme of the tiled attention kernel): every fp32 operand x is scaled by a power of two (exact) and cut
// into hi (its 11 leading bits, exact in fp16) and lo = x - hi (rounded to fp16's 11 bits); a*b = a_hi*b_hi + a_hi*b_lo +
// a_lo*b_hi as kind::f16 products with fp32 accumulation in the tensor core, the dropped a_lo*b_lo is 2^-22 relative.
// Scales: one per row of A (range_scale of the row's largest magnitude) and one for the whole of B; both leave in the
// epilogue.  An element of B more than 2^-20 below B's largest magnitude keeps fewer bits (its lo part becomes a
// subnormal fp16); the exact mode is there for such operands.
//
// Four kernels per call:
//   gemm_amax_kernel     largest |B|  (B is at most a few MB here: one pass)
//   gemm_pack_a_kernel   A -> per (128-row tile, 64-deep slice) the shared-memory image of a K-major operand stage with
//                        128-byte swizzle: a block of A_hi rows and a block of A_lo rows (fp16); row scales to a vector
//   gemm_pack_b_kernel   B -> per (64-deep slice, 128-column tile) the image of an N-major operand stage without
//                        swizzle, columns [B_hi (128) | B_lo (128)]
//   gemm_tc_kernel       one block per SM, 128 x 128 output tiles in turn: a producer warp fetches whole stages with bulk
//                        copies (three stages of 64 KB in flight, running on into the next tile), an issuing warp forms
//                        A_hi [B_hi | B_lo] (N = 256) and A_lo B_hi (N = 128, onto the second half) for every slice, 8
//                        instructions per slice, into one of two accumulators of 256 TMEM columns; four warps (thread =
//                        output row = TMEM lane) add the halves, take the scales out, add the bias and store one tile
//                        while the products of the next one run.
// Rows, columns and depth beyond the matrices are zeros in the images; stores are bounded by M and K.
// Every wait is bounded: on expiry the block records a status code, skips its stores, frees its TMEM and returns.
#include "tc_primitives.cuh"

#include <math.h>

#include <mutex>
#include <vector>

namespace hipgpt {
namespace {

constexpr int kTM = 128, kTN = 128, kTK = 64;     // output tile and depth of a slice
constexpr int kStages = 3;
constexpr int kABlk = kTM * 128;                  // bytes of one block of an A stage: 128 rows of 64 fp16
constexpr int kAStage = 2 * kABlk;                // [A_hi | A_lo]
constexpr int kBStage = kTK * 2 * kTN * 2;        // 64 deep x [B_hi (128) | B_lo (128)] fp16
constexpr int kGroupStride = 2 * kTN * 16;        // bytes between groups of 8 reduction rows of a B stage (32 column blocks of 128 bytes)
constexpr int kGemmThreads = 192;                 // 4 epilogue warps, a producer warp, an issuing warp
constexpr int kTmemCols = 512;                    // two accumulators of [A_hi B_hi (128) | corrections (128)]
constexpr size_t kGemmSmem = (size_t)kStages * (kAStage + kBStage) + 1024;

__device__ int g_gemm_status = 0;

__device__ __forceinline__ float pow2_scale(float amax)
{
    // the power of two that brings `amax` into [2^14, 2^15); 1 for zero, infinite or NaN input
    if (!(amax > 0.0f && amax <= 3.0e38f)) return 1.0f;
    const int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
    int sh = 14 - e;
    sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
    return __uint_as_float((uint32_t)(127 + sh) << 23);
}
__device__ __forceinline__ float pow2_inverse(float p) { return __uint_as_float(0x7F000000u - __float_as_uint(p)); }

// largest |x| of n floats -> *out (zeroed before the launch; non-negative floats order like their bit patterns)
__global__ void __launch_bounds__(256) gemm_amax_kernel(const float *__restrict__ x, size_t n, float *out)
{
    dependents_may_start();
    float m = 0.0f;
    const size_t tid = (size_t)blockIdx.x * 256 + threadIdx.x, nthr = (size_t)gridDim.x * 256;
    if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const size_t n4 = n / 4;
        for (size_t i = tid; i < n4; i += nthr) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(x) + i);
            m = fmaxf(m, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
        }
        for (size_t i = 4 * n4 + tid; i < n; i += nthr) m = fmaxf(m, fabsf(__ldg(x + i)));
    } else {
        for (size_t i = tid; i < n; i += nthr) m = fmaxf(m, fabsf(__ldg(x + i)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(reinterpret_cast<unsigned *>(out), __float_as_uint(m));
}

// One warp per row of A (rows up to the padded count: rows past M are zeros).  A lane owns runs of 8 consecutive values
// (one 16-byte chunk of fp16).  Image: stage (mt, kt) at ((mt * KT + kt) * kAStage); block 0 = hi, block 1 = lo; row r,
// chunk c at r * 128 + ((c ^ (r & 7)) * 16).
// With ln_g / ln_b given, the row is layer-normalised first (mean and variance over its N values, eps 1e-5, times gamma
// plus beta: launch_layer_norm_forward, src/hip_kernels.cpp:757-848, to rounding), so that LN + projection of the
// reference's block (src/transformer_layer.cpp:240-241, 246-247) need no pass over memory of their own.
__global__ void __launch_bounds__(128) gemm_pack_a_kernel(const float *__restrict__ A, uint8_t *__restrict__ img, float *__restrict__ row_inv,
                                                           int M, int N, int KT, const float *__restrict__ ln_g, const float *__restrict__ ln_b)
{
    // overlapped launch: placed while the kernel before it drains; waiting for it here also orders the product kernel,
    // which waits for this one, after everything before
    dependency_wait();
    dependents_may_start();
    const int lane = threadIdx.x & 31;
    const int m = blockIdx.x * 4 + (threadIdx.x >> 5);
    const bool live = m < M;
    const float *row = A + (size_t)(live ? m : 0) * N;
    const bool vec = (N & 3) == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0;
    auto raw8 = [&](int k0, float (&v)[8]) {
        if (live && vec && k0 + 8 <= N) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(row + k0)), b = __ldg(reinterpret_cast<const float4 *>(row + k0) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (live && k0 + j < N) ? __ldg(row + k0 + j) : 0.0f;
        }
    };
    const int depth = KT * kTK;
    float mean = 0.0f, rstd = 1.0f;
    if (ln_g) {
        float sum = 0.0f;
        for (int k0 = lane * 8; k0 < depth; k0 += 256) {
            float v[8];
            raw8(k0, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) sum += v[j];             // values past N are zeros
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        mean = sum / (float)N;
        float var = 0.0f;
        for (int k0 = lane * 8; k0 < depth; k0 += 256) {
            float v[8];
            raw8(k0, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) { const float d = (k0 + j < N) ? v[j] - mean : 0.0f; var = fmaf(d, d, var); }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
        rstd = 1.0f / sqrtf(var / (float)N + 1e-5f);
    }
    auto load8 = [&](int k0, float (&v)[8]) {
        raw8(k0, v);
        if (ln_g) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                v[j] = (live && k0 + j < N) ? __ldg(ln_g + k0 + j) * (v[j] - mean) * rstd + __ldg(ln_b + k0 + j) : 0.0f;
        }
    };
    float amax = 0.0f;
    for (int k0 = lane * 8; k0 < depth; k0 += 256) {
        float v[8];
        load8(k0, v);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = pow2_scale(amax);
    if (lane == 0) row_inv[m] = pow2_inverse(s);
    const int mt = m / kTM, r = m % kTM;
    for (int k0 = lane * 8; k0 < depth; k0 += 256) {             // the row is read again: it is in L1 / L2
        float v[8];
        load8(k0, v);
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = v[2 * j] * s, b = v[2 * j + 1] * s;
            const float ah = tf32_hi(a), bh = tf32_hi(b);
            hi[j] = pack_f16(ah, bh);
            lo[j] = pack_f16(a - ah, b - bh);
        }
        const int kt = k0 / kTK, c = (k0 % kTK) >> 3;
        uint8_t *stage = img + ((size_t)mt * KT + kt) * kAStage;
        *reinterpret_cast<uint4 *>(stage + sw128(r, c)) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4 *>(stage + kABlk + sw128(r, c)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

// One block per 8 reduction rows of a (64-deep slice kt, 128-column tile nt) of B [N][K] (N inner, K the output width).
// A thread owns 8 consecutive columns of one reduction row.  Image: stage (nt, kt) at ((nt * KT + kt) * kBStage); reduction row r,
// column block cb (8 columns of [B_hi (128) | B_lo (128)]) at (r / 8) * kGroupStride + cb * 128 + (r % 8) * 16.
__global__ void __launch_bounds__(128) gemm_pack_b_kernel(const float *__restrict__ B, const float *__restrict__ amax, uint8_t *__restrict__ img,
                                                           int N, int K, int KT)
{
    dependency_wait();                               // the largest magnitude has been found
    dependents_may_start();
    const int kt = blockIdx.x >> 3, pass = blockIdx.x & 7, nt = blockIdx.y;
    const float s = pow2_scale(*amax);
    const int cb = threadIdx.x & 15, r0 = threadIdx.x >> 4;      // 16 threads cover the 128 columns of a row, 8 rows per block
    const bool vec = (K & 3) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0;
    uint8_t *stage = img + ((size_t)nt * KT + kt) * kBStage;
    {
        const int r = r0 + 8 * pass;
        const int n = kt * kTK + r, c0 = nt * kTN + 8 * cb;
        float v[8];
        if (n < N && vec && c0 + 8 <= K) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(B + (size_t)n * K + c0)), b = __ldg(reinterpret_cast<const float4 *>(B + (size_t)n * K + c0) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (n < N && c0 + j < K) ? __ldg(B + (size_t)n * K + c0 + j) : 0.0f;
        }
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float a = v[2 * j] * s, b = v[2 * j + 1] * s;
            const float ah = tf32_hi(a), bh = tf32_hi(b);
            hi[j] = pack_f16(ah, bh);
            lo[j] = pack_f16(a - ah, b - bh);
        }
        uint8_t *dst = stage + (r >> 3) * kGroupStride + (r & 7) * 16;
        *reinterpret_cast<uint4 *>(dst + cb * 128) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4 *>(dst + (16 + cb) * 128) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

__device__ __noinline__ void gemm_wait_slow(uint64_t *bar, uint32_t parity, int site, volatile int *abort_flag)
{
    if (!mbar_wait(bar, parity)) {
        *abort_flag = 1;
        atomicCAS(&g_gemm_status, 0, site);
    }
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const uint8_t *__restrict__ aimg, const uint8_t *__restrict__ bimg, const float *__restrict__ row_inv, const float *__restrict__ b_amax,
               const float *__restrict__ bias, float *__restrict__ C, int M, int K, int KT, int NT, int ntiles)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *a_s = base;                              // [stage][A_hi block | A_lo block]
    uint8_t *b_s = base + kStages * kAStage;          // [stage][64 deep][B_hi | B_lo]
    __shared__ uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2];
    __shared__ __align__(16) float epi[4][32 * 32];  // per epilogue warp: a 32 x 32 piece of the output on its way out
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int abort_flag;

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);      // warp-uniform for the compiler

    if (tid == 0) {
        abort_flag = 0;
        for (int i = 0; i < kStages; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    }
    __syncthreads();
    // site codes in the status word: 1 stage landed, 2 stage free, 3 accumulator complete, 4 accumulator drained
    auto wait = [&](uint64_t *bar, uint32_t parity, int site) {
        if (abort_flag || mbar_test(bar, parity)) return;
        gemm_wait_slow(bar, parity, site, &abort_flag);
    };
    // The block takes output tiles blockIdx.x, + gridDim.x, ... (column tile fastest: blocks that run side by side share
    // the rows of A).  Stages are counted through all tiles (g), accumulators alternate between two halves of TMEM, so
    // the copies of the next tile and its products run while the four epilogue warps drain the tile before it.

    if (warp == 4) {
        // ---- producer: whole stages by bulk copies ----
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        dependents_may_start();
        dependency_wait();                            // the pack kernels have completed
        tc_fence_before();
        __syncthreads();                              // TMEM allocated
        int g = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
            const int nt = t % NT, mt = t / NT;
            for (int kt = 0; kt < KT; ++kt, ++g) {
                const int s = g % kStages;
                if (g >= kStages) wait(&empty[s], (uint32_t)((g / kStages - 1) & 1), 2);     // the products that read the stage have completed
                if (lane == 0) {
                    mbar_arrive_expect_tx(&full[s], (uint32_t)(kAStage + kBStage));
                    const uint8_t *asrc = aimg + ((size_t)mt * KT + kt) * kAStage, *bsrc = bimg + ((size_t)nt * KT + kt) * kBStage;
                    bulk_load(a_s + s * kAStage, asrc, kABlk, &full[s]);
                    bulk_load(a_s + s * kAStage + kABlk, asrc + kABlk, kABlk, &full[s]);
                    bulk_load(b_s + s * kBStage, bsrc, kBStage / 2, &full[s]);
                    bulk_load(b_s + s * kBStage + kBStage / 2, bsrc + kBStage / 2, kBStage / 2, &full[s]);
                }
                __syncwarp();
            }
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();                              // the last output has been read from TMEM
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_slot), "r"(kTmemCols) : "memory");
        return;
    }
    if (warp == 5) {
        // ---- issuing warp: stays converged, elects the lane per instruction ----
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
        const uint32_t tmem = tmem_base_slot;
        constexpr uint32_t id_wide = idesc_f16(kTM, 2 * kTN) | (1u << 16);       // A_hi x [B_hi | B_lo], B N-major
        constexpr uint32_t id_half = idesc_f16(kTM, kTN) | (1u << 16);           // A_lo x B_hi
        int g = 0, i = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++i) {
            const uint32_t acc = tmem + (uint32_t)((i & 1) * 2 * kTN);
            if (i >= 2) wait(&acc_empty[i & 1], (uint32_t)((i / 2 - 1) & 1), 4);             // the epilogue has read this half's previous tile
            tc_fence_after();
            for (int kt = 0; kt < KT; ++kt, ++g) {
                const int s = g % kStages;
                wait(&full[s], (uint32_t)((g / kStages) & 1), 1);
                tc_fence_after();
                const uint64_t da_hi = make_desc(smem_u32(a_s + s * kAStage), 16, 1024, 2);
                const uint64_t da_lo = make_desc(smem_u32(a_s + s * kAStage + kABlk), 16, 1024, 2);
                // N-major B without swizzle: lbo = bytes between groups of 8 reduction rows, sbo = bytes between blocks of 8 columns
                const uint64_t db = make_desc(smem_u32(b_s + s * kBStage), kGroupStride, 128, 0);
#pragma unroll
                for (int k = 0; k < kTK / 16; ++k)    // 16 deep = 32 bytes of an A row = two groups of B
                    if (elect_one()) mma_h_ss(acc, da_hi + (uint64_t)(2 * k), db + (uint64_t)(k * 2 * (kGroupStride >> 4)), id_wide, (kt | k) ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < kTK / 16; ++k)
                    if (elect_one()) mma_h_ss(acc + kTN, da_lo + (uint64_t)(2 * k), db + (uint64_t)(k * 2 * (kGroupStride >> 4)), id_half, 1u);
                if (elect_one()) tc_commit(&empty[s]);
            }
            if (elect_one()) tc_commit(&acc_full[i & 1]);
        }
        __syncwarp();
        tc_fence_before();
        __syncthreads();
        return;
    }

    // ---- epilogue warps: thread = output row = TMEM lane ----
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const float b_inv = pow2_inverse(pow2_scale(__ldg(b_amax)));
    const bool vec = (K & 3) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0;
    int i = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++i) {
        const int nt = t % NT, mt = t / NT;
        const int r = warp * 32 + lane, m = mt * kTM + r;
        const uint32_t lane_base = tmem_base_slot + ((uint32_t)(warp * 32) << 16) + (uint32_t)((i & 1) * 2 * kTN);
        const float unscale = (m < M ? __ldg(row_inv + m) : 0.0f) * b_inv;
        wait(&acc_full[i & 1], (uint32_t)((i / 2) & 1), 3);
        tc_fence_after();
        const int c_base = nt * kTN;
        const bool live = !abort_flag;
        // 32 columns at a time; the warp turns its 32 x 32 piece through shared memory (16-byte chunk c of row r at
        // r * 128 + ((c ^ (r & 7)) * 16)) so that a store instruction writes four rows of 128 contiguous bytes instead
        // of 32 rows of 16
        uint8_t *tb = reinterpret_cast<uint8_t *>(epi[warp]);
#pragma unroll 1
        for (int c0 = 0; c0 < kTN; c0 += 32) {
            float a[32], b[32];
            tmem_ld32(lane_base + c0, a);             // A_hi B_hi
            tmem_ld32(lane_base + kTN + c0, b);       // the correction terms
            tmem_wait_ld();
            if (c_base + c0 >= K) continue;           // warp-uniform: a tile past the last column
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
                float o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int c = c_base + c0 + 4 * j4 + j;
                    o[j] = (a[4 * j4 + j] + b[4 * j4 + j]) * unscale + ((bias && c < K) ? __ldg(bias + c) : 0.0f);
                }
                *reinterpret_cast<float4 *>(tb + lane * 128 + ((j4 ^ (lane & 7)) << 4)) = make_float4(o[0], o[1], o[2], o[3]);
            }
            __syncwarp();
            const int ch = lane & 7;
            const int col = c_base + c0 + 4 * ch;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int rr = 4 * i + (lane >> 3);
                const int mrow = mt * kTM + warp * 32 + rr;
                const float4 val = *reinterpret_cast<const float4 *>(tb + rr * 128 + ((ch ^ (rr & 7)) << 4));
                if (live && mrow < M) {
                    float *dst = C + (size_t)mrow * K + col;
                    if (vec && col + 4 <= K) {
                        *reinterpret_cast<float4 *>(dst) = val;
                    } else {
                        if (col < K) dst[0] = val.x;
                        if (col + 1 < K) dst[1] = val.y;
                        if (col + 2 < K) dst[2] = val.z;
                        if (col + 3 < K) dst[3] = val.w;
                    }
                }
            }
            __syncwarp();                             // the piece is out before the next one is staged
        }
        // this half of TMEM may take the tile after next
        tc_fence_before();
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[i & 1])) : "memory");
    }
    tc_fence_before();
    __syncthreads();
}

// The packed operands of a call live in a buffer of the library, one per device and stream; it grows to the largest call.
struct GemmScratch {
    std::mutex mu;
    struct Entry { int dev; cudaStream_t st; uint8_t *buf; size_t cap; };
    std::vector<Entry> entries;
    int get(int dev, cudaStream_t st, size_t need, uint8_t **out)
    {
        std::lock_guard<std::mutex> lock(mu);
        Entry *e = nullptr;
        for (auto &x : entries) if (x.dev == dev && x.st == st) e = &x;
        if (!e) { entries.push_back({dev, st, nullptr, 0}); e = &entries.back(); }
        if (e->cap < need) {
            if (e->buf) cudaFree(e->buf);            // waits for the kernels that read it
            e->buf = nullptr;
            e->cap = 0;
            const cudaError_t err = cudaMalloc(&e->buf, need);
            if (err != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMalloc(%zu) for the packed operands: %s", need, cudaGetErrorString(err));
            e->cap = need;
        }
        *out = e->buf;
        return HIPGPT_OK;
    }
    void release()
    {
        std::lock_guard<std::mutex> lock(mu);
        for (auto &x : entries) if (x.buf) cudaFree(x.buf);
        entries.clear();
    }
};
GemmScratch g_gemm;

}  // namespace

void gemm_tc_release_scratch() { g_gemm.release(); }

int gemm_tc_status_fetch(int *status)
{
    int v = 0;
    const cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(v));
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (v) { const int zero = 0; cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(zero)); }
    *status = v;
    return HIPGPT_OK;
}

namespace {

int set_gemm_attr()
{
    static bool attr_set = false;
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        attr_set = true;
    }
    return HIPGPT_OK;
}

// B -> its stage images and its largest magnitude (three launches on `st`; the first is a plain one, so everything
// enqueued before has completed when the images are written)
int pack_b(const float *B, int N, int K, uint8_t *bimg, float *b_amax, cudaStream_t st)
{
    const int NT = (K + kTN - 1) / kTN, KT = (N + kTK - 1) / kTK;
    cudaError_t e = cudaMemsetAsync(b_amax, 0, sizeof(float), st);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    const size_t nb = (size_t)N * K;
    size_t ablocks = (nb + 256 * 4 - 1) / (256 * 4);
    if (ablocks > 1184) ablocks = 1184;
    gemm_amax_kernel<<<(unsigned)ablocks, 256, 0, st>>>(B, nb, b_amax);
    int rc = check_launch("gemm_amax_kernel");
    if (rc != HIPGPT_OK) return rc;
    e = launch_overlapped(gemm_pack_b_kernel, dim3((unsigned)(KT * (kTK / 8)), (unsigned)NT), dim3(128), 0, st, B, (const float *)b_amax, bimg, N, K, KT);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "gemm_pack_b_kernel launch: %s", cudaGetErrorString(e));
    return check_launch("gemm_pack_b_kernel");
}

// A -> its stage images, then the product kernel, with B's images given
int pack_a_and_multiply(const float *A, const uint8_t *bimg, const float *b_amax, const float *bias, float *C, int M, int N, int K,
                        uint8_t *aimg, float *row_inv, bool first_is_plain, int dev, cudaStream_t st, const float *ln_g = nullptr, const float *ln_b = nullptr)
{
    const int MT = (M + kTM - 1) / kTM, NT = (K + kTN - 1) / kTN, KT = (N + kTK - 1) / kTK;
    cudaError_t e;
    if (first_is_plain) {
        // nothing of this call precedes the pack kernel: a plain launch, so that the product kernel, which waits for the
        // pack kernel only, is ordered after everything before the call (the kernel's own wait then returns at once)
        gemm_pack_a_kernel<<<(unsigned)(MT * kTM / 4), 128, 0, st>>>(A, aimg, row_inv, M, N, KT, ln_g, ln_b);
    } else {
        e = launch_overlapped(gemm_pack_a_kernel, dim3((unsigned)(MT * kTM / 4)), dim3(128), 0, st, A, aimg, row_inv, M, N, KT, ln_g, ln_b);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "gemm_pack_a_kernel launch: %s", cudaGetErrorString(e));
    }
    int rc = check_launch("gemm_pack_a_kernel");
    if (rc != HIPGPT_OK) return rc;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    const long long ntiles = (long long)MT * NT;
    if (ntiles > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "%lld output tiles are too many", ntiles);
    const unsigned grid = (unsigned)(ntiles < sms ? ntiles : sms);           // one block per SM, each takes tiles in turn
    e = launch_overlapped(gemm_tc_kernel, dim3(grid), dim3(kGemmThreads), kGemmSmem, st, (const uint8_t *)aimg, bimg,
                          (const float *)row_inv, b_amax, bias, C, M, K, KT, NT, (int)ntiles);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "gemm_tc_kernel launch: %s", cudaGetErrorString(e));
    return check_launch("gemm_tc_kernel");
}

}  // namespace

// C[M][K] = A[M][N] B[N][K] (+ bias), fp32-grade on the tensor pipe.  C must not alias A or B.
int launch_matmul_tc(const float *A, const float *B, const float *bias, float *C, int M, int N, int K, cudaStream_t st, const float *ln_g, const float *ln_b)
{
    const int MT = (M + kTM - 1) / kTM, NT = (K + kTN - 1) / kTN, KT = (N + kTK - 1) / kTK;
    if (MT > 65535) return fail(HIPGPT_ERR_BAD_ARG, "M = %d is beyond %d rows per call", M, 65535 * kTM);
    if (KT == 0) return fail(HIPGPT_ERR_BAD_ARG, "an inner dimension of 0");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    const size_t abytes = (size_t)MT * KT * kAStage, bbytes = (size_t)NT * KT * kBStage, rbytes = ((size_t)MT * kTM * sizeof(float) + 255) & ~(size_t)255;
    uint8_t *scratch = nullptr;
    int rc = g_gemm.get(dev, st, abytes + bbytes + rbytes + 256, &scratch);
    if (rc != HIPGPT_OK) return rc;
    uint8_t *aimg = scratch, *bimg = scratch + abytes;
    float *row_inv = reinterpret_cast<float *>(scratch + abytes + bbytes), *b_amax = reinterpret_cast<float *>(scratch + abytes + bbytes + rbytes);
    rc = set_gemm_attr();
    if (rc == HIPGPT_OK) rc = pack_b(B, N, K, bimg, b_amax, st);
    if (rc != HIPGPT_OK) return rc;
    return pack_a_and_multiply(A, bimg, b_amax, bias, C, M, N, K, aimg, row_inv, false, dev, st, ln_g, ln_b);
}

// ---- a right-hand side packed once (the weights of a layer) and used by many products ---------------------------
struct PackedB {
    int dev, N, K;
    uint8_t *bimg;
    float *b_amax;
};

int matmul_tc_prepare(const float *B, int N, int K, PackedB **out, cudaStream_t st)
{
    const int NT = (K + kTN - 1) / kTN, KT = (N + kTK - 1) / kTK;
    if (KT == 0 || NT == 0) return fail(HIPGPT_ERR_BAD_ARG, "an empty right-hand side: N=%d K=%d", N, K);
    PackedB *p = new PackedB{0, N, K, nullptr, nullptr};
    cudaError_t e = cudaGetDevice(&p->dev);
    const size_t bbytes = (size_t)NT * KT * kBStage;
    if (e == cudaSuccess) e = cudaMalloc(&p->bimg, bbytes + 256);
    if (e != cudaSuccess) { delete p; return fail(HIPGPT_ERR_CUDA, "cudaMalloc(%zu) for the packed right-hand side: %s", bbytes + 256, cudaGetErrorString(e)); }
    p->b_amax = reinterpret_cast<float *>(p->bimg + bbytes);
    const int rc = pack_b(B, N, K, p->bimg, p->b_amax, st);
    if (rc != HIPGPT_OK) { cudaFree(p->bimg); delete p; return rc; }
    *out = p;
    return HIPGPT_OK;
}

void matmul_tc_release(PackedB *p)
{
    if (!p) return;
    cudaFree(p->bimg);                               // waits for the kernels that read it
    delete p;
}

int launch_matmul_tc_prepared(const float *A, const PackedB *b, const float *bias, float *C, int M, cudaStream_t st, const float *ln_g, const float *ln_b)
{
    const int N = b->N, K = b->K;
    const int MT = (M + kTM - 1) / kTM, KT = (N + kTK - 1) / kTK;
    if (MT > 65535) return fail(HIPGPT_ERR_BAD_ARG, "M = %d is beyond %d rows per call", M, 65535 * kTM);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev != b->dev) return fail(HIPGPT_ERR_BAD_ARG, "the right-hand side was packed on device %d, the current device is %d", b->dev, dev);
    const size_t abytes = (size_t)MT * KT * kAStage, rbytes = ((size_t)MT * kTM * sizeof(float) + 255) & ~(size_t)255;
    uint8_t *scratch = nullptr;
    int rc = g_gemm.get(dev, st, abytes + rbytes, &scratch);
    if (rc != HIPGPT_OK) return rc;
    rc = set_gemm_attr();
    if (rc != HIPGPT_OK) return rc;
    return pack_a_and_multiply(A, b->bimg, b->b_amax, bias, C, M, N, K, scratch, reinterpret_cast<float *>(scratch + abytes), true, dev, st, ln_g, ln_b);
}

}  // namespace hipgpt
