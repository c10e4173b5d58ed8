// Fused attention forward on the Blackwell tensor pipe (tcgen05 + TMEM), fp32-grade results.
//
// Replaces, like the FFMA rows kernel, the two kernels behind HipGPT's
// launch_multihead_attention (src/hip_kernels.cpp:263-325 and :329-402).
//
// The contraction runs as split-TF32 ("3xTF32"): every fp32 operand x is cut into
//   hi = x with the 13 low mantissa bits cleared (exactly a TF32 number), lo = x - hi (exact),
// and a product a*b is accumulated as a_hi*b_hi + a_hi*b_lo + a_lo*b_hi in the tensor core's
// fp32 accumulator.  The dropped a_lo*b_lo term and the truncation of lo are below 2^-21
// relative, so scores and outputs agree with fp32 FFMA arithmetic to about 1e-6.
//
// One thread block = 128 query rows of one (batch, head), 128 threads, thread t owns row t:
//   stage   Q (scaled by log2(e)/sqrt(D)), then per tile of 64 keys K and V, are read from
//           global with coalesced 128-bit loads, split into hi / lo and written to shared memory
//           in the tensor core's canonical 128-byte-swizzled layout (rows of 32 floats);
//   S       = Q K^T for the tile: tcgen05.mma kind::tf32, M=128 N=64, both operands K-major
//           from shared memory, accumulator in TMEM (3 passes x D/8 instructions);
//   softmax thread t reads its row of S with tcgen05.ld (TMEM lane t), applies the causal / tail
//           mask, keeps the running maximum and sum (log2 domain, one ex2 per score), splits
//           P into hi / lo and writes both back to TMEM with tcgen05.st;
//   O_tile  = P V: tcgen05.mma with A = P from TMEM and B = V from shared memory, N-major
//           (3 passes x 8 instructions), fresh accumulator per tile;
//   update  thread t reads its row of O_tile and adds it to its register accumulator, which
//           it rescaled when the running maximum moved.
// Completion of each batch of MMAs is signalled by tcgen05.commit on an mbarrier.  Every wait
// on it is bounded: on expiry the block records a status code, skips its stores, frees its
// TMEM and returns.  No probabilities are written by this kernel; callers that want them get
// the FFMA rows kernel.
#include "attn_common.cuh"

#include <math.h>

namespace hipgpt {
namespace {

constexpr int kM = 128;          // query rows per block
constexpr int kN = 64;           // keys per tile
constexpr int kThreads = 128;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColPhi = 64, kColPlo = 128, kColO = 192;
constexpr long long kSpinLimit = 1LL << 22;

__device__ int g_tc_status = 0;   // 0 ok; 1 = an mbarrier wait ran out

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Bounded wait for the phase with the given parity; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    const uint32_t addr = smem_u32(bar);
    for (long long i = 0; i < kSpinLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Shared-memory matrix descriptor for a tile made of 128-byte rows.
//   K-major operands (Q, K): layout 2 = SWIZZLE_128B, rows grouped by 8 (1024 bytes); sbo = bytes
//     between groups, lbo unused (16).
//   N-major operand (V): 32-bit operands that are contiguous along N must use layout 1,
//     SWIZZLE_128B with a 32-byte base: reduction rows grouped by 4 (512 bytes); sbo = bytes
//     between groups, lbo = bytes between 32-float column blocks.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;          // descriptor version of sm_100
    d |= (uint64_t)layout_type << 61;   // 2 = SWIZZLE_128B, 1 = SWIZZLE_128B with 32-byte base
    return d;
}

// Instruction descriptor: fp32 accumulator, TF32 operands, A K-major, B K- or N-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int b_n_major)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)b_n_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld32(uint32_t addr, float (&v)[32])
{
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr) : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t addr, const float (&v)[32])
{
    const uint32_t *r = reinterpret_cast<const uint32_t *>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }

// Writes one 16-byte chunk of a row, split into hi and lo, at its swizzled place:
// chunk c of row r of a [rows][128 B] block lands at r*128 + ((c ^ (r & 7)) * 16).
__device__ __forceinline__ void store_split(float *hi_blk, float *lo_blk, int row, int chunk, float4 x)
{
    const int off = row * 32 + ((chunk ^ (row & 7)) << 2);
    const float4 h = make_float4(tf32_hi(x.x), tf32_hi(x.y), tf32_hi(x.z), tf32_hi(x.w));
    *reinterpret_cast<float4 *>(hi_blk + off) = h;
    *reinterpret_cast<float4 *>(lo_blk + off) = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
}

// The same for the N-major operand: 32-byte pieces of a row are permuted by the row index
// modulo 4; the 16-byte half inside a piece keeps its place.
__device__ __forceinline__ void store_split_nmajor(float *hi_blk, float *lo_blk, int row, int chunk, float4 x)
{
    const int piece = (chunk >> 1) ^ (row & 3);
    const int off = row * 32 + (((piece << 1) | (chunk & 1)) << 2);
    const float4 h = make_float4(tf32_hi(x.x), tf32_hi(x.y), tf32_hi(x.z), tf32_hi(x.w));
    *reinterpret_cast<float4 *>(hi_blk + off) = h;
    *reinterpret_cast<float4 *>(lo_blk + off) = make_float4(x.x - h.x, x.y - h.y, x.z - h.z, x.w - h.w);
}

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kThreads)
mha_tc_kernel(const float *__restrict__ Q, const float *__restrict__ K, const float *__restrict__ V,
              float *__restrict__ O, int S, int E, int H, int BH, int nqblk, float qscale)
{
    constexpr int DB = D / 32;                   // 32-float column blocks per row
    constexpr int QBLK = kM * 32;                // floats per [128][32] block
    constexpr int KBLK = kN * 32;                // floats per [64][32] block
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment is what the swizzled layout assumes
    float *base = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float *q_hi = base, *q_lo = q_hi + DB * QBLK;
    float *k_hi = q_lo + DB * QBLK, *k_lo = k_hi + DB * KBLK;
    float *v_hi = k_lo + DB * KBLK, *v_lo = v_hi + DB * KBLK;
    __shared__ uint64_t mbar;
    __shared__ uint32_t tmem_base_slot;

    const int tid = threadIdx.x, warp = tid >> 5;
    const int bh = blockIdx.x % BH;
    const int qblk = CAUSAL ? (nqblk - 1 - blockIdx.x / BH) : (blockIdx.x / BH);   // heaviest first
    const int b = bh / H, h = bh % H;
    const size_t tok0 = (size_t)b * S;
    const size_t hcol = (size_t)h * D;
    const int q0 = qblk * kM;
    const int row = q0 + tid;                    // this thread's query

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) mbar_init(&mbar, 1);

    // ---- stage Q: thread t owns row t -------------------------------------------------------
    {
        const bool ok = row < S;
        const float4 *src = reinterpret_cast<const float4 *>(Q + (tok0 + (ok ? row : 0)) * (size_t)E + hcol);
#pragma unroll
        for (int c = 0; c < D / 4; ++c) {
            float4 x = ok ? __ldg(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            x.x *= qscale; x.y *= qscale; x.z *= qscale; x.w *= qscale;
            store_split(q_hi + (c >> 3) * QBLK, q_lo + (c >> 3) * QBLK, tid, c & 7, x);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_slot;
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);   // this warp's 32 TMEM lanes

    float o[D];
#pragma unroll
    for (int d = 0; d < D; ++d) o[d] = 0.0f;
    float m = -1e30f, l = 0.0f;
    uint32_t phase = 0;
    bool failed = false;

    const int kend = CAUSAL ? min(S, q0 + kM) : S;
    const int ntiles = (kend + kN - 1) / kN;
    constexpr uint32_t idesc_qk = make_idesc(kM, kN, 0);
    constexpr uint32_t idesc_pv = make_idesc(kM, D, 1);

    for (int t = 0; t < ntiles && !failed; ++t) {
        const int j0 = t * kN;
        // ---- stage K and V of this tile: 8 (or 16) threads per row, coalesced 128-bit loads --
        {
            constexpr int CPR = D / 4;                       // 16-byte chunks per row
            constexpr int RPP = kThreads / CPR;              // rows per pass
            const int c = tid % CPR, r0 = tid / CPR;
#pragma unroll
            for (int p = 0; p < kN / RPP; ++p) {
                const int r = r0 + p * RPP;
                const int j = j0 + r;
                const bool ok = j < S;
                const size_t g = (tok0 + (ok ? j : 0)) * (size_t)E + hcol + c * 4;
                const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 kx = ok ? __ldg(reinterpret_cast<const float4 *>(K + g)) : zero;
                const float4 vx = ok ? __ldg(reinterpret_cast<const float4 *>(V + g)) : zero;
                store_split(k_hi + (c >> 3) * KBLK, k_lo + (c >> 3) * KBLK, r, c & 7, kx);
                store_split_nmajor(v_hi + (c >> 3) * KBLK, v_lo + (c >> 3) * KBLK, r, c & 7, vx);
            }
        }
        proxy_fence();                 // generic-proxy writes -> visible to the tensor core's reads
        tc_fence_before();
        __syncthreads();

        // ---- S = Q K^T -------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after();
            uint32_t acc = 0;
#pragma unroll
            for (int pass = 0; pass < 3; ++pass) {
                // the two correction terms first: the accumulator is still tiny while they are
                // added, so the tensor core's truncating adds cost no accuracy there
                const float *qa = pass == 0 ? q_lo : q_hi;
                const float *kb = pass == 1 ? k_lo : k_hi;
#pragma unroll
                for (int db = 0; db < DB; ++db) {
                    const uint64_t da = make_desc(smem_u32(qa + db * QBLK), 16, 1024, 2);
                    const uint64_t dk = make_desc(smem_u32(kb + db * KBLK), 16, 1024, 2);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {            // 8 floats = 32 bytes per instruction
                        mma_ss(tmem + kColS, da + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), idesc_qk, acc);
                        acc = 1;
                    }
                }
            }
            tc_commit(&mbar);
        }
        // every tcgen05.ld / st below is warp-wide (.sync.aligned): keep the outcome warp-uniform
        failed = __any_sync(0xffffffffu, !mbar_wait(&mbar, phase));
        phase ^= 1;
        tc_fence_after();

        // ---- softmax of this thread's row ------------------------------------------------
        float alpha = 1.0f;
        if (!failed) {
            float s[kN];
            float lo[kN];
            float(&s0)[32] = *reinterpret_cast<float(*)[32]>(&s[0]);
            float(&s1)[32] = *reinterpret_cast<float(*)[32]>(&s[32]);
            float(&l0)[32] = *reinterpret_cast<float(*)[32]>(&lo[0]);
            float(&l1)[32] = *reinterpret_cast<float(*)[32]>(&lo[32]);
            if (CAUSAL && j0 > q0 + warp * 32 + 31) {
                // the whole tile lies above the diagonal for every row of this warp: P = 0
#pragma unroll
                for (int c = 0; c < kN; ++c) { s[c] = 0.0f; lo[c] = 0.0f; }
            } else {
                tmem_ld32(lane_base + kColS, s0);
                tmem_ld32(lane_base + kColS + 32, s1);
                tmem_wait_ld();
                if ((CAUSAL && j0 + kN - 1 > q0 + warp * 32) || j0 + kN > S) {
#pragma unroll
                    for (int c = 0; c < kN; ++c) {
                        const int j = j0 + c;
                        if (j >= S || (CAUSAL && j > row)) s[c] = -INFINITY;
                    }
                }
                float mx = s[0];
#pragma unroll
                for (int c = 1; c < kN; ++c) mx = fmaxf(mx, s[c]);
                const float mn = fmaxf(m, mx);       // m is finite (-1e30f at worst), so is mn
                alpha = ex2_approx(m - mn);
                m = mn;
                float psum = 0.0f;
#pragma unroll
                for (int c = 0; c < kN; ++c) {
                    const float p = ex2_approx(s[c] - mn);   // masked scores give exactly 0
                    psum += p;
                    const float ph = tf32_hi(p);
                    s[c] = ph;
                    lo[c] = p - ph;
                }
                l = fmaf(l, alpha, psum);
            }
            tmem_st32(lane_base + kColPhi, s0);
            tmem_st32(lane_base + kColPhi + 32, s1);
            tmem_st32(lane_base + kColPlo, l0);
            tmem_st32(lane_base + kColPlo + 32, l1);
            tmem_wait_st();
        }
        tc_fence_before();
        if (__syncthreads_or(failed ? 1 : 0)) { failed = true; break; }

        // ---- O_tile = P V ------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after();
            uint32_t acc = 0;
#pragma unroll
            for (int pass = 0; pass < 3; ++pass) {
                const uint32_t pa = tmem + (pass == 0 ? kColPlo : kColPhi);
                const float *vb = pass == 1 ? v_lo : v_hi;
                // N-major B: 8 reduction rows (keys) of 128 bytes per instruction = 1024 bytes
                const uint64_t dv = make_desc(smem_u32(vb), KBLK * 4, 512, 1);
#pragma unroll
                for (int k = 0; k < kN / 8; ++k) {
                    mma_ts(tmem + kColO, pa + (uint32_t)(k * 8), dv + (uint64_t)(k * 64), idesc_pv, acc);
                    acc = 1;
                }
            }
            tc_commit(&mbar);
        }
        failed = __any_sync(0xffffffffu, !mbar_wait(&mbar, phase));
        phase ^= 1;
        tc_fence_after();
        if (!failed) {
#pragma unroll
            for (int db = 0; db < DB; ++db) {
                float ot[32];
                tmem_ld32(lane_base + kColO + db * 32, ot);
                tmem_wait_ld();

#pragma unroll
                for (int d = 0; d < 32; ++d) o[db * 32 + d] = fmaf(o[db * 32 + d], alpha, ot[d]);
            }
        }
        tc_fence_before();
        if (__syncthreads_or(failed ? 1 : 0)) { failed = true; break; }
    }

    if (failed) {
        if (tid == 0) atomicExch(&g_tc_status, 1);
    } else if (row < S) {
        const float inv = 1.0f / fmaxf(l, 1e-20f);
        float4 *dst = reinterpret_cast<float4 *>(O + (tok0 + row) * (size_t)E + hcol);
#pragma unroll
        for (int c = 0; c < D / 4; ++c)
            dst[c] = make_float4(o[c * 4 + 0] * inv, o[c * 4 + 1] * inv, o[c * 4 + 2] * inv, o[c * 4 + 3] * inv);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

template <int D, bool CAUSAL>
int launch_tc_cfg(const float *q, const float *k, const float *v, float *out, int B, int S, int E, int H, cudaStream_t st)
{
    auto kern = mha_tc_kernel<D, CAUSAL>;
    constexpr int DB = D / 32;
    // operands + alignment slack; never less than 100 KB, so that at most two blocks share an
    // SM and their two 256-column TMEM allocations always fit in the 512 columns
    size_t smem = (size_t)(2 * DB * kM * 32 + 4 * DB * kN * 32) * sizeof(float) + 1024;
    if (smem < 100 * 1024) smem = 100 * 1024;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    const int nqblk = (S + kM - 1) / kM;
    const long long blocks = (long long)B * H * nqblk;
    if (blocks > 2147483647LL) return fail(HIPGPT_ERR_BAD_ARG, "grid of %lld blocks is too large", blocks);
    const float qscale = (1.0f / sqrtf((float)D)) * kLog2e;
    kern<<<(unsigned)blocks, kThreads, smem, st>>>(q, k, v, out, S, E, H, B * H, nqblk, qscale);
    return check_launch("mha_tc_kernel");
}

}  // namespace

bool mha_tc_supports(int D) { return D == 32 || D == 64; }

int launch_mha_tc(const float *q, const float *k, const float *v, float *out,
                  int B, int S, int E, int H, int causal, cudaStream_t st)
{
    const int D = E / H;
    if (D == 32) return causal ? launch_tc_cfg<32, true>(q, k, v, out, B, S, E, H, st)
                               : launch_tc_cfg<32, false>(q, k, v, out, B, S, E, H, st);
    if (D == 64) return causal ? launch_tc_cfg<64, true>(q, k, v, out, B, S, E, H, st)
                               : launch_tc_cfg<64, false>(q, k, v, out, B, S, E, H, st);
    return fail(HIPGPT_ERR_UNSUPPORTED, "tensor-core kernel: head_dim %d is not 32 or 64", D);
}

// Reads and clears the status word of the tensor-core kernels (synchronises the device).
int tc_status_fetch(int *status)
{
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(status, g_tc_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
    if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "status fetch: %s", cudaGetErrorString(e));
    return HIPGPT_OK;
}

}  // namespace hipgpt
